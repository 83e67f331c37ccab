/*
 * kipp_b200: a small, whole inference engine for one GPU.  This is its C interface: open a
 * model folder (config.json + safetensors), feed batches of (request, next tokens) through
 * kipp_engine_step, read logits, sample, or let the scheduler generate.  The Python package
 * is a thin ctypes face of these functions.
 *
 * The vocabulary follows the reference's C interface (src/kipp.h: open / close / info
 * :109-145, session create / reset / truncate / destroy / info / eval :172-200, batch eval
 * :238-255, sample :264-295, error names :297).  A "request" here is what the reference
 * calls a session: one timeline of tokens with its pages of the cache.  Where the reference
 * evaluates one session or a batch of whole items, kipp_engine_step takes any mixture of
 * prompt portions and single decoded tokens and returns logits at the wanted places only.
 *
 * Every function that can fail returns a kipp_result; the text of the last failure of an
 * engine is kept in the engine (kipp_engine_last_error), of a call without an engine in
 * thread-local storage (kipp_last_error).  Nothing changes in an engine when a call fails.
 * An engine may be used by one host thread at a time.
 */
#ifndef KIPP_B200_H
#define KIPP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    KIPP_OK = 0,
    KIPP_E_ARGUMENT = 1,      /* a value outside what the call takes */
    KIPP_E_CONFIG = 2,        /* config.json: a key missing, of a wrong type, or an option not built */
    KIPP_E_WEIGHTS = 3,       /* checkpoint and model disagree (the message lists every difference) */
    KIPP_E_IO = 4,            /* a file is missing or cannot be read */
    KIPP_E_UNSUPPORTED = 5,   /* unknown architecture or part kind */
    KIPP_E_OUT_OF_PAGES = 6,  /* the cache cannot hold the step; every request is as it was */
    KIPP_E_OUT_OF_SLOTS = 7,  /* max_requests requests are live already */
    KIPP_E_MEMORY = 8,        /* weights, cache and workspace do not fit the device */
    KIPP_E_KERNEL = 9,        /* a kernel refused its sizes, or reported a refused access or a wait that ran out */
    KIPP_E_CUDA = 10,         /* a CUDA runtime call failed */
    KIPP_E_STATE = 11,        /* the call does not fit the engine's or the request's state */
    KIPP_E_BUILD = 12         /* a kernel library is missing */
} kipp_result;

const char* kipp_result_name(int code);
/* Text of the last failure of a call made without an engine (open, create, plan and weights calls). */
const char* kipp_last_error(void);

#define KIPP_DTYPE_F32 0
#define KIPP_DTYPE_BF16 1
#define KIPP_DTYPE_F16 2
#define KIPP_DTYPE_I32 3
#define KIPP_DTYPE_I64 4
#define KIPP_DTYPE_I16 5
#define KIPP_DTYPE_I8 6
#define KIPP_DTYPE_U8 7

typedef struct kipp_engine kipp_engine;

typedef struct {
    int dtype;                 /* KIPP_DTYPE_BF16: the serving kernels; KIPP_DTYPE_F32: everything in true 32-bit */
    int device;                /* CUDA device ordinal */
    int page_size;             /* tokens per cache page */
    long long cache_tokens;    /* tokens every cache group can hold; 0: sized from the free device memory */
    int max_requests;          /* live requests (state slots) */
    int max_batch_tokens;      /* tokens of one step (activation workspace) */
    int max_logit_rows;        /* wanted rows of one step (logits buffer); 0: a default from the vocabulary */
    int cuda_graphs;           /* capture decode steps and repeating prompt shapes (bfloat16 path) */
    int kv_round_bf16;         /* 32-bit path only: round keys and values to bfloat16 when stored, the
                                  reference's storage contract (src/kipp.c:2806-2811) */
    int own_length_splits;     /* decode attention splits from each token's own context only, so that a
                                  token's bfloat16 result does not depend on its neighbours in the batch */
} kipp_engine_options;

void kipp_engine_default_options(kipp_engine_options* options);

/*
 * Kernel libraries are found beside this library (lib<name>.so).  A resolver, if set, is
 * asked first: it returns the path of the library `name` (building it if it has to) or NULL.
 */
typedef const char* (*kipp_library_resolver)(const char* name);
void kipp_set_library_resolver(kipp_library_resolver resolver);

/* ---- a model's description ------------------------------------------------------------ */

/*
 * The plan of a model: its parts with their sizes and tensor names, and the order in which
 * its layers run, as JSON.  kipp_plan_from_config builds it from the text of a config.json
 * with the builder registered for architectures[0]; a caller may also write one itself out
 * of the registered part kinds.  The returned text is owned by the library and stays valid
 * until the thread's next plan call.
 */
int kipp_plan_from_config(const char* config_json, const char** plan_json);
/* The config.json keys of a registered architecture after defaults and checks, as JSON. */
int kipp_config_normalize(const char* config_json, const char** normalized_json);
/* The checkpoint tensors a plan needs: a JSON list of {name, shape, init, optional, alias_of}. */
int kipp_plan_tensor_specs(const char* plan_json, const char** specs_json);
/* The same for one part of a plan (its JSON object) under a name prefix. */
int kipp_part_tensor_specs(const char* part_json, const char* prefix, const char** specs_json);
/* Keys per split that the paged attention's planner chooses for `decoded` tokens whose longest
   context is `longest` keys (own_length: for one token of that context alone). */
int kipp_attention_split_length(int decoded, int longest, int kv_heads, int sm_count, int own_length);
int kipp_attention_stream_pays(int decoded, const int* keys, int kv_heads, int sm_count);
/* Names of the registered architectures and part kinds, as a JSON object of two lists. */
const char* kipp_registered(void);

/* ---- checkpoints ------------------------------------------------------------------------ */

typedef struct kipp_weights kipp_weights;
typedef struct {
    const char* name;
    int dtype;                 /* KIPP_DTYPE_* of the stored elements */
    int ndim;
    const int64_t* shape;
    const void* data;          /* the mapped bytes */
    size_t bytes;
} kipp_tensor_info;

/* Maps the safetensors files of a folder (model.safetensors, or the shards its index names). */
int kipp_weights_open(const char* folder, kipp_weights** out);
void kipp_weights_close(kipp_weights* weights);
int kipp_weights_count(const kipp_weights* weights);
int kipp_weights_tensor(const kipp_weights* weights, int index, kipp_tensor_info* out);
int kipp_weights_find(const kipp_weights* weights, const char* name, kipp_tensor_info* out);
/* Compares a checkpoint with a list of tensor specs (JSON, as kipp_plan_tensor_specs writes it);
   on KIPP_E_WEIGHTS the message lists every missing, unexpected, misshapen and mistyped tensor. */
int kipp_weights_check(const kipp_weights* weights, const char* specs_json);
/* The same comparison as a JSON object {missing, unexpected, wrong_shape: [[name, is, expected]],
   wrong_dtype: [[name, stored type]], message}; it succeeds whether or not they match. */
int kipp_weights_compare(const kipp_weights* weights, const char* specs_json, const char** report_json);

/* ---- parts defined outside the library ---------------------------------------------------- */

/*
 * A plan may name parts of kind "external": parts whose forward pass the caller supplies.
 * What such a part sees of a step (device pointers unless a name says host):
 */
typedef struct {
    int role;                        /* 0 embedding stage, 1 norm, 2 mixer, 3 feed-forward */
    int tokens, entries;
    int layer, cache, writes_cache;  /* the run it is called for (mixers) */
    const int* token_ids;            /* [tokens] */
    const int* positions;            /* [tokens] absolute position of each token */
    const int* entry_of_token;       /* [tokens] */
    const int* q_start;              /* [entries + 1] first token of each entry */
    const int* context_len;          /* [entries] tokens cached before the step */
    const int* slots;                /* [entries] state slot of each entry */
    const int* host_q_lens;          /* host copies for control flow */
    const int* host_context_len;
    const int* host_slots;
    const void* input;               /* [tokens, input_cols] activations in the compute dtype, or NULL */
    int input_dtype;
    long long input_cols;
    float* residual;                 /* [tokens, hidden] float32 residual stream (roles 0, 2, 3: update in place) */
    long long hidden;
    void* output;                    /* role 1: [tokens or rows, hidden] in the compute dtype */
    const int* rows;                 /* role 1: token rows to normalise, or NULL for all */
    int n_rows;
    void* state;                     /* [max_requests, state_bytes] state of the run's cache id, or NULL */
    long long state_bytes;
    int max_requests;
    void* stream;                    /* the engine's CUDA stream: enqueue the work there */
} kipp_external_call;

typedef struct {
    void* user;
    int (*forward)(void* user, const kipp_external_call* call);   /* 0 on success */
} kipp_external_part;

/* ---- where tensors come from when a model is created from a plan ---------------------------- */

typedef struct {
    const void* data;          /* host or device memory holding the tensor, row-major */
    int on_device;
    int dtype;
    int ndim;
    int64_t shape[8];
} kipp_tensor_view;

/* Returns 0 and fills `out` (valid until the next call) or nonzero when it has no such tensor. */
typedef int (*kipp_tensor_provider)(void* user, const char* name, kipp_tensor_view* out);

/* ---- engines ---------------------------------------------------------------------------------- */

/* A model folder: config.json selects the architecture, the safetensors are bound by name. */
int kipp_engine_open(const char* model_dir, const kipp_engine_options* options, kipp_engine** out);
/*
 * A model from a plan.  Tensors come from `model_dir` (if not NULL) or from `provider`.
 * `external[i]` stands behind the plan's parts of kind "external" with index i.
 */
int kipp_engine_create(const char* plan_json, const char* model_dir, kipp_tensor_provider provider,
                       void* provider_user, const kipp_external_part* external, int n_external,
                       const kipp_engine_options* options, kipp_engine** out);
void kipp_engine_close(kipp_engine* engine);
const char* kipp_engine_last_error(const kipp_engine* engine);
/* What is loaded and what it may hold, as JSON (owned by the engine, valid until the next info call). */
const char* kipp_engine_info(kipp_engine* engine);
void* kipp_engine_stream(kipp_engine* engine);
/* The engine's cache manager (cache_core.h), for looking at its bookkeeping; not to be destroyed. */
void* kipp_engine_cache_manager(kipp_engine* engine);

/* Requests are named by 64-bit numbers chosen by the caller. */
int kipp_engine_add_request(kipp_engine* engine, int64_t request);
int kipp_engine_finish(kipp_engine* engine, int64_t request);            /* pages and slot go back */
int kipp_engine_truncate(kipp_engine* engine, int64_t request, int new_length);
int kipp_engine_is_live(kipp_engine* engine, int64_t request);
int kipp_engine_length(kipp_engine* engine, int64_t request);            /* tokens cached, or -1 */

typedef struct {
    int64_t request;
    const int32_t* tokens;     /* the request's next tokens */
    int n_tokens;
    const int32_t* want;       /* indices among these tokens whose logits are wanted (may be empty) */
    int n_want;
} kipp_step_entry;

/*
 * One step: all entries run as one batch against the cache that earlier steps left.  A
 * request that is not live is admitted.  On success *logits points at float32
 * [*n_rows, vocab] on the device (engine memory: read or copy it before the next step;
 * NULL when nothing is wanted) in the order of the entries and of their want lists.  The
 * work is enqueued on the engine's stream; kipp_engine_read_logits and
 * kipp_engine_synchronize wait for it.  KIPP_E_OUT_OF_PAGES leaves every request as it was.
 */
int kipp_engine_step(kipp_engine* engine, const kipp_step_entry* entries, int n_entries,
                     const float** logits, int* n_rows);
/* Copies the last step's logits to host memory [n_rows, vocab] and checks the kernels' status words. */
int kipp_engine_read_logits(kipp_engine* engine, float* host_out, size_t capacity_floats);
/* Writes a value into one of the engine's four status words, as a kernel that refused an access or
   gave up a bounded wait does (tests of the error path). */
int kipp_engine_debug_set_status(kipp_engine* engine, int word, int value);
/* Rows of logits the last step left (0 when it wanted none). */
int kipp_engine_last_rows(kipp_engine* engine);
/* Waits for the engine's stream and checks the kernels' status words. */
int kipp_engine_synchronize(kipp_engine* engine);
/* Where a step's time goes.  Between kipp_engine_profile(e, 1) and kipp_engine_profile(e, 0) steps
 * run without CUDA graphs and every kernel launch is followed by an event; afterwards
 * kipp_engine_profile_json gives {"kernel name": milliseconds, ...} (time between consecutive
 * events, so the gaps between launches are inside: read the figures as shares). */
int kipp_engine_profile(kipp_engine* engine, int on);
const char* kipp_engine_profile_json(kipp_engine* engine);

/*
 * Greedy decoding of `steps` tokens for every listed live request without the host in the
 * loop: tokens[i] is the next token of requests[i]; out_host receives int32 [steps, n].
 */
int kipp_engine_decode_burst(kipp_engine* engine, const int64_t* requests, const int32_t* tokens, int n,
                             int steps, int32_t* out_host);

/* Sampling options of one row, with the reference's names and defaults (src/kipp.h:278-291). */
typedef struct {
    float temperature;         /* <= 0: argmax, the generator state is not touched */
    float top_p;               /* (0, 1]; 1 disables */
    int top_k;                 /* 0 disables */
    float min_p;               /* [0, 1]; 0 disables */
    float frequency_penalty, presence_penalty, repetition_penalty;
    const int32_t* recent_tokens;
    int recent_count;
    const int32_t* logit_bias_tokens;
    const float* logit_bias_values;
    int logit_bias_count;
} kipp_sample_params;

void kipp_sample_default_params(kipp_sample_params* params);
/*
 * One token for each row of the last step's logits, on the device, drawing what the
 * reference's host sampler draws (src/kipp.c:3433-3559).  rng_states[i] (xorshift64*,
 * nonzero) advances for rows with temperature > 0 only.
 */
int kipp_engine_sample(kipp_engine* engine, const kipp_sample_params* params, uint64_t* rng_states, int n_rows,
                       int32_t* out_tokens_host);

/* ---- generation: the scheduler above the step ------------------------------------------------- */

typedef struct {
    int max_batch_tokens;      /* token budget of one step; 0: the engine's */
    int chunk;                 /* largest prompt portion of one request in one step; 0: the budget */
    int max_running;           /* 0: the engine's max_requests */
    int max_positions;         /* most tokens one request may hold; 0: the model's */
    int preempt;               /* 0: admit only what can never run out of pages (the reference's rule,
                                  src/kipp_server.c:1736-1777); 1: admit early, put the youngest back */
} kipp_scheduler_options;

typedef struct {
    int64_t id;
    const int32_t* prompt;
    int n_prompt;
    int max_new_tokens;
    kipp_sample_params sampling;
    uint64_t seed;             /* nonzero when temperature > 0 */
    const int32_t* stop_tokens;
    int n_stop_tokens;
} kipp_generation_request;

typedef struct {
    int64_t id;
    int finished;              /* 0 waiting or running */
    int reason;                /* 1 stop token, 2 length, 3 aborted */
    int n_tokens;              /* generated so far */
    int preemptions;
} kipp_generation_state;

/*
 * The scheduler by itself: its decisions need the cache manager's bookkeeping only, so it can
 * be driven without a device (tests do).  kipp_scheduler_schedule plans the next step and keeps
 * the plan until kipp_scheduler_complete records the tokens sampled for it; between the two the
 * caller runs the step (kipp_engine_run does both halves itself).
 */
typedef struct kipp_scheduler kipp_scheduler;
typedef struct {
    int64_t id;
    int first;                 /* index of the entry's first token in prompt + output */
    int n_tokens;
    int want_last;             /* the logits of its last token are sampled */
} kipp_plan_entry;

/* Over a cache manager of cache_core.h; admitting and releasing requests are that manager's own calls. */
int kipp_scheduler_create(void* cache_manager, int n_groups, const int* pages, const int* windows, int page_size,
                          int max_requests, const kipp_scheduler_options* options, kipp_scheduler** out);
void kipp_scheduler_destroy(kipp_scheduler* scheduler);
const char* kipp_scheduler_last_error(const kipp_scheduler* scheduler);
int kipp_scheduler_submit(kipp_scheduler* scheduler, const kipp_generation_request* request);
int kipp_scheduler_has_work(const kipp_scheduler* scheduler);
int kipp_scheduler_schedule(kipp_scheduler* scheduler, kipp_plan_entry* entries, int capacity, int* n);
int kipp_scheduler_tokens(kipp_scheduler* scheduler, int64_t id, int first, int n, int32_t* out);
int kipp_scheduler_complete(kipp_scheduler* scheduler, const int32_t* sampled, int n);
int kipp_scheduler_poll(kipp_scheduler* scheduler, int64_t id, kipp_generation_state* state);
int kipp_scheduler_output(kipp_scheduler* scheduler, int64_t id, int32_t* tokens, int capacity, int* n);
int kipp_scheduler_abort(kipp_scheduler* scheduler, int64_t id);
int kipp_scheduler_forget(kipp_scheduler* scheduler, int64_t id);
/* Ids of the requests that are waiting (0), running (1) or finished (2), in the scheduler's order. */
int kipp_scheduler_list(kipp_scheduler* scheduler, int which, int64_t* ids, int capacity, int* n);
uint64_t kipp_scheduler_rng_state(kipp_scheduler* scheduler, int64_t id);
/* preemptions, steps planned, requests admitted, tokens fed, tokens sampled */
void kipp_scheduler_stats(const kipp_scheduler* scheduler, long long out[5]);

/* The engine's own scheduler (made with default options at first use, or by configure). */
int kipp_engine_scheduler_configure(kipp_engine* engine, const kipp_scheduler_options* options);
kipp_scheduler* kipp_engine_scheduler(kipp_engine* engine);
int kipp_engine_submit(kipp_engine* engine, const kipp_generation_request* request);
/* Runs scheduled steps until no request is waiting or running (max_steps > 0 limits them). */
int kipp_engine_run(kipp_engine* engine, int max_steps, int* steps_run);
int kipp_engine_poll(kipp_engine* engine, int64_t id, kipp_generation_state* state);
/* Copies the tokens generated so far; returns their number through *n. */
int kipp_engine_output(kipp_engine* engine, int64_t id, int32_t* tokens, int capacity, int* n);
int kipp_engine_abort(kipp_engine* engine, int64_t id);
/* Forgets a finished request's record. */
int kipp_engine_forget(kipp_engine* engine, int64_t id);

/*
 * One part of one run alone, on a step of its own (tests of the parts): `which` is
 * "embedding", "input_norm", "mixer", "post_norm", "feed_forward", "block", "final_norm" or
 * "head"; `input` the activations a mixer, feed-forward or head reads (compute dtype),
 * `residual` the float32 stream the part reads or updates, `output` what a norm or the head
 * writes.  All device pointers.  The requests' lengths advance as after a step.
 */
int kipp_engine_debug_part(kipp_engine* engine, const kipp_step_entry* entries, int n_entries, int run_index,
                           const char* which, const void* input, float* residual, void* output);

#ifdef __cplusplus
}
#endif
#endif
