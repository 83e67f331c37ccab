// The C interface of the host core (kipp_b200.h): every function catches what the C++ below
// throws, keeps its text, and returns a kipp_result.
#include "engine.hpp"
#include "scheduler.hpp"

using namespace kipp;

struct kipp_scheduler {
    std::unique_ptr<Scheduler> scheduler;
    StepPlan plan;                       // planned, not yet completed
    std::string error;
};

struct kipp_engine {
    std::unique_ptr<Engine> engine;
    kipp_scheduler sched;
    std::string error;
};

struct kipp_weights {
    Checkpoint checkpoint;
    explicit kipp_weights(const std::string& folder) : checkpoint(folder) {}
};

namespace {
thread_local std::string g_error;
thread_local std::string g_text;

template <typename F> int guarded(std::string& error, F&& body) {
    try {
        body();
        return KIPP_OK;
    } catch (const Error& e) {
        error = e.what();
        return e.code;
    } catch (const JsonError& e) {
        error = e.what();
        return KIPP_E_CONFIG;
    } catch (const std::bad_alloc&) {
        error = "out of host memory";
        return KIPP_E_MEMORY;
    } catch (const std::exception& e) {
        error = e.what();
        return KIPP_E_STATE;
    }
}

void fill_info(const StoredTensor& t, kipp_tensor_info* out) {
    out->name = t.name.c_str();
    out->dtype = t.dtype;
    out->ndim = (int)t.shape.size();
    out->shape = t.shape.data();
    out->data = t.data;
    out->bytes = t.bytes;
}

std::vector<TensorSpec> specs_from_json(const char* specs_json) {
    Json j = Json::parse(specs_json);
    std::vector<TensorSpec> specs;
    for (auto& s : j.items()) specs.push_back(TensorSpec::from_json(s));
    return specs;
}

kipp_engine* make_engine(const Json& plan_json, TensorSource& source, const kipp_external_part* external, int n_external,
                         const kipp_engine_options* options) {
    kipp_engine_options opt;
    if (options) opt = *options;
    else kipp_engine_default_options(&opt);
    BuildContext ctx;
    ctx.external = external;
    ctx.n_external = n_external;
    auto plan = build_plan(plan_json, ctx);
    auto holder = std::make_unique<kipp_engine>();
    holder->engine = std::make_unique<Engine>(std::move(plan), source, opt);
    return holder.release();
}
}  // namespace

extern "C" {

const char* kipp_result_name(int code) {
    static const char* names[] = {"ok", "argument", "config", "weights", "io", "unsupported", "out_of_pages",
                                  "out_of_slots", "memory", "kernel", "cuda", "state", "build"};
    return code >= 0 && code <= KIPP_E_BUILD ? names[code] : "unknown";
}
const char* kipp_last_error(void) { return g_error.c_str(); }

void kipp_engine_default_options(kipp_engine_options* o) {
    if (!o) return;
    o->dtype = KIPP_DTYPE_BF16;
    o->device = 0;
    o->page_size = 16;
    o->cache_tokens = 0;
    o->max_requests = 64;
    o->max_batch_tokens = 8192;
    o->max_logit_rows = 0;
    o->cuda_graphs = 1;
    o->kv_round_bf16 = 0;
    o->own_length_splits = 0;
}

void kipp_set_library_resolver(kipp_library_resolver resolver) { KernelLibraries::get().set_resolver(resolver); }

int kipp_plan_from_config(const char* config_json, const char** plan_json) {
    return guarded(g_error, [&] {
        g_text = plan_from_config(Json::parse(config_json)).dump();
        *plan_json = g_text.c_str();
    });
}

int kipp_config_normalize(const char* config_json, const char** normalized_json) {
    return guarded(g_error, [&] {
        ensure_registered();
        Json config = Json::parse(config_json);
        g_text = Registry::get().architecture(architecture_of(config)).normalize(config).dump();
        *normalized_json = g_text.c_str();
    });
}

int kipp_plan_tensor_specs(const char* plan_json, const char** specs_json) {
    return guarded(g_error, [&] {
        // external parts are not called here: a stand-in serves every index the plan names
        static kipp_external_part stand_in[256];
        for (auto& s : stand_in)
            s.forward = [](void*, const kipp_external_call*) { return 1; };
        BuildContext ctx;
        ctx.external = stand_in;
        ctx.n_external = 256;
        auto plan = build_plan(Json::parse(plan_json), ctx);
        Json out = Json::array();
        for (auto& s : plan->tensor_specs()) out.push(s.to_json());
        g_text = out.dump();
        *specs_json = g_text.c_str();
    });
}

int kipp_part_tensor_specs(const char* part_json, const char* prefix, const char** specs_json) {
    return guarded(g_error, [&] {
        ensure_registered();
        static kipp_external_part stand_in[256];
        for (auto& s : stand_in)
            s.forward = [](void*, const kipp_external_call*) { return 1; };
        BuildContext ctx;
        ctx.external = stand_in;
        ctx.n_external = 256;
        auto part = Registry::get().make(Json::parse(part_json), ctx);
        std::vector<TensorSpec> specs;
        part->tensor_specs(prefix ? prefix : "", specs);
        Json out = Json::array();
        for (auto& s : specs) out.push(s.to_json());
        g_text = out.dump();
        *specs_json = g_text.c_str();
    });
}

// The decode-split rule of the paged attention's planner, for tests that lay the device's
// choice against the host's.
int kipp_attention_split_length(int decoded, int longest, int kv_heads, int sm_count, int own_length) {
    if (own_length) return AttentionPlanner::own_split_length(longest);
    return AttentionPlanner(kv_heads, sm_count, false).step_split_length(decoded, longest);
}

// Whether the planner deals a step of `decoded` single tokens with these numbers of keys out as a
// stream over one wave of CTAs (1) or cuts each into splits of the step's length (0).
int kipp_attention_stream_pays(int decoded, const int* keys, int kv_heads, int sm_count) {
    StepShape s;
    s.entries = decoded;
    for (int i = 0; i < decoded; ++i) {
        s.q_lens.push_back(1);
        s.starts.push_back(keys[i] - 1);
    }
    s.tokens = decoded;
    return AttentionPlanner(kv_heads, sm_count, false).stream_pays(s) ? 1 : 0;
}

const char* kipp_registered(void) {
    ensure_registered();
    Json j = Json::object();
    Json a = Json::array(), k = Json::array();
    for (auto& n : Registry::get().architectures()) a.push(n);
    for (auto& n : Registry::get().part_kinds()) k.push(n);
    j.set("architectures", std::move(a));
    j.set("part_kinds", std::move(k));
    g_text = j.dump();
    return g_text.c_str();
}

// ---- checkpoints ---------------------------------------------------------------------------
int kipp_weights_open(const char* folder, kipp_weights** out) {
    return guarded(g_error, [&] { *out = new kipp_weights(folder); });
}
void kipp_weights_close(kipp_weights* w) { delete w; }
int kipp_weights_count(const kipp_weights* w) { return (int)w->checkpoint.tensors().size(); }
int kipp_weights_tensor(const kipp_weights* w, int index, kipp_tensor_info* out) {
    return guarded(g_error, [&] {
        if (index < 0 || index >= (int)w->checkpoint.tensors().size()) fail(KIPP_E_ARGUMENT, "no such tensor index");
        fill_info(w->checkpoint.tensors()[(size_t)index], out);
    });
}
int kipp_weights_find(const kipp_weights* w, const char* name, kipp_tensor_info* out) {
    return guarded(g_error, [&] {
        const StoredTensor* t = w->checkpoint.find(name);
        if (!t) fail(KIPP_E_WEIGHTS, std::string("the checkpoint has no tensor ") + name);
        fill_info(*t, out);
    });
}
int kipp_weights_check(const kipp_weights* w, const char* specs_json) {
    return guarded(g_error, [&] { w->checkpoint.check(specs_from_json(specs_json)); });
}
int kipp_weights_compare(const kipp_weights* w, const char* specs_json, const char** report_json) {
    return guarded(g_error, [&] {
        const Checkpoint::Report r = w->checkpoint.compare(specs_from_json(specs_json));
        Json j = r.to_json();
        j.set("message", r.clean() ? Json("") : Json(w->checkpoint.describe(r)));
        g_text = j.dump();
        *report_json = g_text.c_str();
    });
}

// ---- engines --------------------------------------------------------------------------------
int kipp_engine_open(const char* model_dir, const kipp_engine_options* options, kipp_engine** out) {
    return guarded(g_error, [&] {
        const std::string dir = model_dir;
        const std::string config_path = dir + "/config.json";
        if (!file_exists(config_path)) fail(KIPP_E_CONFIG, dir + ": no config.json");
        Json config;
        try {
            config = Json::parse(read_text_file(config_path));
        } catch (const JsonError& e) {
            fail(KIPP_E_CONFIG, config_path + ": " + e.what());
        }
        Json plan = plan_from_config(config);
        CheckpointSource source(dir);
        *out = make_engine(plan, source, nullptr, 0, options);
    });
}

int kipp_engine_create(const char* plan_json, const char* model_dir, kipp_tensor_provider provider,
                       void* provider_user, const kipp_external_part* external, int n_external,
                       const kipp_engine_options* options, kipp_engine** out) {
    return guarded(g_error, [&] {
        Json plan = Json::parse(plan_json);
        if (model_dir) {
            CheckpointSource source(model_dir);
            *out = make_engine(plan, source, external, n_external, options);
        } else if (provider) {
            ProviderSource source(provider, provider_user);
            *out = make_engine(plan, source, external, n_external, options);
        } else {
            fail(KIPP_E_ARGUMENT, "a model folder or a tensor provider is needed");
        }
    });
}

void kipp_engine_close(kipp_engine* e) { delete e; }
const char* kipp_engine_last_error(const kipp_engine* e) { return e ? e->error.c_str() : g_error.c_str(); }
const char* kipp_engine_info(kipp_engine* e) {
    static thread_local std::string text;
    if (guarded(e->error, [&] { text = e->engine->info_json(); }) != KIPP_OK) text = "{}";
    return text.c_str();
}
void* kipp_engine_stream(kipp_engine* e) { return e->engine->stream(); }
void* kipp_engine_cache_manager(kipp_engine* e) { return e->engine->cache_manager(); }

int kipp_engine_add_request(kipp_engine* e, int64_t request) {
    return guarded(e->error, [&] { e->engine->add_request(request); });
}
int kipp_engine_finish(kipp_engine* e, int64_t request) {
    return guarded(e->error, [&] { e->engine->finish(request); });
}
int kipp_engine_truncate(kipp_engine* e, int64_t request, int new_length) {
    return guarded(e->error, [&] { e->engine->truncate(request, new_length); });
}
int kipp_engine_is_live(kipp_engine* e, int64_t request) { return e->engine->is_live(request) ? 1 : 0; }
int kipp_engine_length(kipp_engine* e, int64_t request) { return e->engine->length(request); }

int kipp_engine_step(kipp_engine* e, const kipp_step_entry* entries, int n_entries, const float** logits,
                     int* n_rows) {
    return guarded(e->error, [&] {
        if (n_entries <= 0 || !entries) fail(KIPP_E_ARGUMENT, "a step needs at least one entry");
        std::vector<StepEntryView> views((size_t)n_entries);
        for (int i = 0; i < n_entries; ++i)
            views[(size_t)i] = {entries[i].request, entries[i].tokens, entries[i].n_tokens, entries[i].want,
                                entries[i].n_want};
        int rows = 0;
        const float* out = e->engine->step(views.data(), n_entries, &rows);
        if (logits) *logits = out;
        if (n_rows) *n_rows = rows;
    });
}
int kipp_engine_read_logits(kipp_engine* e, float* host_out, size_t capacity_floats) {
    return guarded(e->error, [&] { e->engine->read_logits(host_out, capacity_floats); });
}
// Writes a value into one of the engine's status words, as a kernel that refused an access or gave
// up a wait does (tests of the error path; no kernel is made to fail for it).
int kipp_engine_debug_set_status(kipp_engine* e, int word, int value) {
    return guarded(e->error, [&] { e->engine->debug_set_status(word, value); });
}
int kipp_engine_last_rows(kipp_engine* e) { return e->engine->last_rows(); }
int kipp_engine_profile(kipp_engine* e, int on) {
    return guarded(e->error, [&] { e->engine->profile(on != 0); });
}
const char* kipp_engine_profile_json(kipp_engine* e) { return e->engine->profile_json().c_str(); }
int kipp_engine_synchronize(kipp_engine* e) {
    return guarded(e->error, [&] { e->engine->synchronize(); });
}
int kipp_engine_decode_burst(kipp_engine* e, const int64_t* requests, const int32_t* tokens, int n, int steps,
                             int32_t* out_host) {
    return guarded(e->error, [&] { e->engine->decode_burst(requests, tokens, n, steps, out_host); });
}

void kipp_sample_default_params(kipp_sample_params* p) {
    if (!p) return;
    *p = kipp_sample_params{};
    p->temperature = 0.f;
    p->top_p = 1.f;
    p->repetition_penalty = 1.f;
}
int kipp_engine_sample(kipp_engine* e, const kipp_sample_params* params, uint64_t* rng_states, int n_rows,
                       int32_t* out_tokens_host) {
    return guarded(e->error, [&] { e->engine->sample(params, rng_states, n_rows, out_tokens_host); });
}

// One part of one run alone, on a step of its own (tests of the parts): `which` is "input_norm",
// "mixer", "post_norm", "feed_forward", "block", "embedding", "final_norm" or "head"; `input` the
// activations a mixer, feed-forward or head reads (compute dtype), `residual` the float32 stream
// the part reads or updates, `output` what a norm or the head writes.  All device pointers.
int kipp_engine_debug_part(kipp_engine* e, const kipp_step_entry* entries, int n_entries, int run_index,
                           const char* which, const void* input, float* residual, void* output) {
    return guarded(e->error, [&] {
        std::vector<StepEntryView> views((size_t)n_entries);
        for (int i = 0; i < n_entries; ++i)
            views[(size_t)i] = {entries[i].request, entries[i].tokens, entries[i].n_tokens, entries[i].want,
                                entries[i].n_want};
        e->engine->debug_part(views.data(), n_entries, run_index, which, input, residual, output);
    });
}

// ---- generation -------------------------------------------------------------------------------
int kipp_scheduler_create(void* cache_manager, int n_groups, const int* pages, const int* windows, int page_size,
                          int max_requests, const kipp_scheduler_options* options, kipp_scheduler** out) {
    return guarded(g_error, [&] {
        if (!cache_manager || n_groups < 0 || page_size <= 0 || max_requests <= 0)
            fail(KIPP_E_ARGUMENT, "a cache manager, a page size and a number of requests are needed");
        SchedulerHost h;
        h.cm = cache_manager;
        h.page_size = page_size;
        for (int g = 0; g < n_groups; ++g) {
            h.group_pages.push_back(pages[g]);
            h.group_windows.push_back(windows[g] > 0 ? windows[g] : 0);
        }
        h.max_requests = max_requests;
        kipp_scheduler_options o = options ? *options : kipp_scheduler_options{};
        h.max_batch_tokens = o.max_batch_tokens;
        h.admit = [cache_manager, max_requests](int64_t rid) {
            const int rc = kipp_cm_admit(cache_manager, rid);
            if (rc == KIPP_CM_OUT_OF_SLOTS) fail(KIPP_E_OUT_OF_SLOTS, format("all %d request slots are in use", max_requests));
            if (rc < 0) fail(KIPP_E_STATE, format("admit: error %d", rc));
        };
        h.release = [cache_manager](int64_t rid) {
            const int rc = kipp_cm_release(cache_manager, rid);
            if (rc) fail(KIPP_E_STATE, format("release: error %d", rc));
        };
        auto s = std::make_unique<kipp_scheduler>();
        s->scheduler = std::make_unique<Scheduler>(std::move(h), o);
        *out = s.release();
    });
}
void kipp_scheduler_destroy(kipp_scheduler* s) { delete s; }
const char* kipp_scheduler_last_error(const kipp_scheduler* s) { return s->error.c_str(); }
int kipp_scheduler_submit(kipp_scheduler* s, const kipp_generation_request* r) {
    return guarded(s->error, [&] { s->scheduler->submit(*r); });
}
int kipp_scheduler_has_work(const kipp_scheduler* s) { return s->scheduler->has_work() ? 1 : 0; }
int kipp_scheduler_schedule(kipp_scheduler* s, kipp_plan_entry* entries, int capacity, int* n) {
    return guarded(s->error, [&] {
        s->plan = s->scheduler->schedule();
        const int count = (int)s->plan.entries.size();
        if (count > capacity) fail(KIPP_E_ARGUMENT, format("the plan has %d entries, room was given for %d", count, capacity));
        for (int i = 0; i < count; ++i) {
            const PlanEntry& e = s->plan.entries[(size_t)i];
            entries[i] = {e.request->id, e.first, e.n_tokens, e.want_last ? 1 : 0};
        }
        *n = count;
    });
}
int kipp_scheduler_tokens(kipp_scheduler* s, int64_t id, int first, int n, int32_t* out) {
    return guarded(s->error, [&] {
        GenRequest* r = s->scheduler->find(id);
        if (first < 0 || n < 0 || first + n > r->known()) fail(KIPP_E_ARGUMENT, "tokens outside the request");
        for (int i = 0; i < n; ++i) out[i] = r->token_at(first + i);
    });
}
int kipp_scheduler_complete(kipp_scheduler* s, const int32_t* sampled, int n) {
    return guarded(s->error, [&] {
        s->scheduler->complete(s->plan, sampled, n);
        s->plan = StepPlan{};
    });
}
int kipp_scheduler_poll(kipp_scheduler* s, int64_t id, kipp_generation_state* state) {
    return guarded(s->error, [&] { s->scheduler->poll(id, state); });
}
int kipp_scheduler_output(kipp_scheduler* s, int64_t id, int32_t* tokens, int capacity, int* n) {
    return guarded(s->error, [&] { s->scheduler->output(id, tokens, capacity, n); });
}
int kipp_scheduler_abort(kipp_scheduler* s, int64_t id) {
    return guarded(s->error, [&] { s->scheduler->abort(id); });
}
int kipp_scheduler_forget(kipp_scheduler* s, int64_t id) {
    return guarded(s->error, [&] { s->scheduler->forget(id); });
}
int kipp_scheduler_list(kipp_scheduler* s, int which, int64_t* ids, int capacity, int* n) {
    return guarded(s->error, [&] {
        std::vector<int64_t> v;
        if (which == 0) for (GenRequest* r : s->scheduler->waiting()) v.push_back(r->id);
        else if (which == 1) for (GenRequest* r : s->scheduler->running()) v.push_back(r->id);
        else if (which == 2) for (GenRequest* r : s->scheduler->finished()) v.push_back(r->id);
        else fail(KIPP_E_ARGUMENT, "which: 0 waiting, 1 running, 2 finished");
        *n = (int)v.size();
        for (int i = 0; i < (int)v.size() && i < capacity; ++i) ids[i] = v[(size_t)i];
    });
}
uint64_t kipp_scheduler_rng_state(kipp_scheduler* s, int64_t id) {
    uint64_t out = 0;
    guarded(s->error, [&] { out = s->scheduler->find(id)->rng_state; });
    return out;
}
void kipp_scheduler_stats(const kipp_scheduler* s, long long out[5]) {
    out[0] = s->scheduler->stat_preemptions;
    out[1] = s->scheduler->stat_steps;
    out[2] = s->scheduler->stat_admitted;
    out[3] = s->scheduler->stat_tokens_fed;
    out[4] = s->scheduler->stat_tokens_sampled;
}

int kipp_engine_scheduler_configure(kipp_engine* e, const kipp_scheduler_options* options) {
    return guarded(e->error, [&] {
        if (e->sched.scheduler && e->sched.scheduler->has_work()) fail(KIPP_E_STATE, "the scheduler still has requests");
        e->sched.scheduler = std::make_unique<Scheduler>(engine_scheduler_host(*e->engine),
                                                         options ? *options : kipp_scheduler_options{});
        e->sched.plan = StepPlan{};
    });
}
kipp_scheduler* kipp_engine_scheduler(kipp_engine* e) {
    if (!e->sched.scheduler)
        e->sched.scheduler = std::make_unique<Scheduler>(engine_scheduler_host(*e->engine), kipp_scheduler_options{});
    return &e->sched;
}
int kipp_engine_submit(kipp_engine* e, const kipp_generation_request* request) {
    return guarded(e->error, [&] { kipp_engine_scheduler(e)->scheduler->submit(*request); });
}
int kipp_engine_run(kipp_engine* e, int max_steps, int* steps_run) {
    return guarded(e->error, [&] {
        const int n = run_scheduler(*e->engine, *kipp_engine_scheduler(e)->scheduler, max_steps);
        if (steps_run) *steps_run = n;
    });
}
int kipp_engine_poll(kipp_engine* e, int64_t id, kipp_generation_state* state) {
    return guarded(e->error, [&] { kipp_engine_scheduler(e)->scheduler->poll(id, state); });
}
int kipp_engine_output(kipp_engine* e, int64_t id, int32_t* tokens, int capacity, int* n) {
    return guarded(e->error, [&] { kipp_engine_scheduler(e)->scheduler->output(id, tokens, capacity, n); });
}
int kipp_engine_abort(kipp_engine* e, int64_t id) {
    return guarded(e->error, [&] { kipp_engine_scheduler(e)->scheduler->abort(id); });
}
int kipp_engine_forget(kipp_engine* e, int64_t id) {
    return guarded(e->error, [&] { kipp_engine_scheduler(e)->scheduler->forget(id); });
}

}  // extern "C"
