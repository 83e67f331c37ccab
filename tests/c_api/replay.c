/* A C program on the library's C interface alone (no Python in the process): it opens a model
 * folder, replays a trace of steps through kipp_engine_step, writes the logits of every step that
 * wants some as <out>/<step>.f32, then generates a few greedy tokens for one prompt with the
 * scheduler (kipp_engine_submit / kipp_engine_run) and prints them.
 *
 *   replay MODEL_DIR bfloat16|float32 MAX_TOKENS PAGE_SIZE TRACE.bin OUT_DIR
 *
 * TRACE.bin is a stream of little-endian int32: n_steps; per step: id, n_entries; per entry:
 * request, n_tokens, tokens..., n_want, want...; then n_end, the requests that end after the
 * step; at last n_prompt, prompt..., n_decode for the generation.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "kipp_b200.h"

static int32_t next_int(FILE* f) {
    int32_t v;
    if (fread(&v, sizeof v, 1, f) != 1) {
        fprintf(stderr, "replay: the trace ends early\n");
        exit(3);
    }
    return v;
}

static void die(kipp_engine* e, const char* what, int rc) {
    fprintf(stderr, "replay: %s failed (%s): %s\n", what, kipp_result_name(rc),
            e ? kipp_engine_last_error(e) : kipp_last_error());
    exit(1);
}

int main(int argc, char** argv) {
    if (argc != 7) {
        fprintf(stderr, "usage: replay MODEL_DIR bfloat16|float32 MAX_TOKENS PAGE_SIZE TRACE.bin OUT_DIR\n");
        return 2;
    }
    kipp_engine_options opt;
    kipp_engine_default_options(&opt);
    opt.dtype = strcmp(argv[2], "float32") == 0 ? KIPP_DTYPE_F32 : KIPP_DTYPE_BF16;
    opt.cache_tokens = atoll(argv[3]);
    opt.page_size = atoi(argv[4]);
    opt.max_requests = 8;
    opt.max_batch_tokens = opt.cache_tokens > 64 ? (int)opt.cache_tokens : 64;
    kipp_engine* engine = NULL;
    int rc = kipp_engine_open(argv[1], &opt, &engine);
    if (rc) die(NULL, "kipp_engine_open", rc);

    FILE* f = fopen(argv[5], "rb");
    if (!f) {
        fprintf(stderr, "replay: cannot open %s\n", argv[5]);
        return 2;
    }
    const int n_steps = next_int(f);
    int vocab = 0;
    {   /* the vocabulary from the engine's own description */
        const char* info = kipp_engine_info(engine);
        const char* at = strstr(info, "\"vocab_size\": ");
        if (at) vocab = atoi(at + strlen("\"vocab_size\": "));
    }
    if (vocab <= 0) {
        fprintf(stderr, "replay: the engine did not tell its vocabulary\n");
        return 1;
    }
    float* host = NULL;
    size_t host_floats = 0;
    for (int s = 0; s < n_steps; ++s) {
        const int id = next_int(f), n = next_int(f);
        kipp_step_entry* entries = calloc((size_t)n, sizeof *entries);
        int32_t** owned = calloc((size_t)2 * n, sizeof *owned);
        for (int i = 0; i < n; ++i) {
            entries[i].request = next_int(f);
            entries[i].n_tokens = next_int(f);
            int32_t* tokens = malloc(sizeof(int32_t) * (size_t)(entries[i].n_tokens + 1));
            for (int t = 0; t < entries[i].n_tokens; ++t) tokens[t] = next_int(f);
            entries[i].n_want = next_int(f);
            int32_t* want = malloc(sizeof(int32_t) * (size_t)(entries[i].n_want + 1));
            for (int w = 0; w < entries[i].n_want; ++w) want[w] = next_int(f);
            entries[i].tokens = tokens;
            entries[i].want = want;
            owned[2 * i] = tokens;
            owned[2 * i + 1] = want;
        }
        const float* logits = NULL;
        int rows = 0;
        rc = kipp_engine_step(engine, entries, n, &logits, &rows);
        if (rc) die(engine, "kipp_engine_step", rc);
        if (rows > 0) {
            const size_t need = (size_t)rows * (size_t)vocab;
            if (need > host_floats) {
                host = realloc(host, need * sizeof(float));
                host_floats = need;
            }
            rc = kipp_engine_read_logits(engine, host, host_floats);
            if (rc) die(engine, "kipp_engine_read_logits", rc);
            char path[4096];
            snprintf(path, sizeof path, "%s/%d.f32", argv[6], id);
            FILE* out = fopen(path, "wb");
            if (!out || fwrite(host, sizeof(float), need, out) != need) {
                fprintf(stderr, "replay: cannot write %s\n", path);
                return 1;
            }
            fclose(out);
        } else {
            rc = kipp_engine_synchronize(engine);
            if (rc) die(engine, "kipp_engine_synchronize", rc);
        }
        const int n_end = next_int(f);
        for (int i = 0; i < n_end; ++i) {
            const int64_t request = next_int(f);
            if (kipp_engine_is_live(engine, request)) {
                rc = kipp_engine_finish(engine, request);
                if (rc) die(engine, "kipp_engine_finish", rc);
            }
        }
        for (int i = 0; i < 2 * n; ++i) free(owned[i]);
        free(owned);
        free(entries);
        printf("done %d\n", id);
        fflush(stdout);
    }

    /* generation: one prompt, greedy, through the scheduler */
    const int n_prompt = next_int(f);
    int32_t* prompt = malloc(sizeof(int32_t) * (size_t)(n_prompt + 1));
    for (int i = 0; i < n_prompt; ++i) prompt[i] = next_int(f);
    const int n_decode = next_int(f);
    fclose(f);
    kipp_generation_request request;
    memset(&request, 0, sizeof request);
    request.id = 1000;
    request.prompt = prompt;
    request.n_prompt = n_prompt;
    request.max_new_tokens = n_decode;
    kipp_sample_default_params(&request.sampling);
    request.seed = 1;
    rc = kipp_engine_submit(engine, &request);
    if (rc) die(engine, "kipp_engine_submit", rc);
    int steps = 0;
    rc = kipp_engine_run(engine, 0, &steps);
    if (rc) die(engine, "kipp_engine_run", rc);
    kipp_generation_state state;
    rc = kipp_engine_poll(engine, 1000, &state);
    if (rc) die(engine, "kipp_engine_poll", rc);
    int32_t* generated = malloc(sizeof(int32_t) * (size_t)(n_decode + 1));
    int n = 0;
    rc = kipp_engine_output(engine, 1000, generated, n_decode, &n);
    if (rc) die(engine, "kipp_engine_output", rc);
    printf("generated");
    for (int i = 0; i < n; ++i) printf(" %d", generated[i]);
    printf("\nfinished %d reason %d steps %d\n", state.finished, state.reason, steps);
    free(generated);
    free(prompt);
    free(host);
    kipp_engine_close(engine);
    return 0;
}
