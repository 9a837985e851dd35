/* A C program on the library's C API (plm.h), used by tests/test_capi.py:
 *
 *   plm_demo config DIR                  print the typed configuration as JSON
 *   plm_demo missing DIR                 try to load DIR; print the code and the error text
 *   plm_demo run DIR DTYPE OUT           BASELINE's Tiny-A workload: three prompts of 5, 11 and 17 tokens
 *                                        in one step (logits of every token), then 8 tokens each, one step per
 *                                        token (token t of sequence s is (7 s + 3 t + 1) mod vocab); the
 *                                        logits go to OUT as float32, [33 + 24, vocab].  Then the slots are
 *                                        emptied and plm_generate runs the three prompts greedily for 6 tokens;
 *                                        the tokens are printed, one line per prompt.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "plm.h"

#define CHECK(call)                                                                   \
    do {                                                                              \
        int rc_ = (call);                                                             \
        if (rc_ != 0) {                                                               \
            fprintf(stderr, "%s failed with %d: %s\n", #call, rc_, plm_last_error()); \
            return 1;                                                                 \
        }                                                                             \
    } while (0)

static int token(int s, int t, int vocab) { return (7 * s + 3 * t + 1) % vocab; }

int main(int argc, char** argv) {
    if (argc >= 3 && strcmp(argv[1], "config") == 0) {
        static char text[8192];
        CHECK(plm_config_from_json(argv[2], text, sizeof(text)));
        printf("%s\n", text);
        return 0;
    }
    if (argc >= 3 && strcmp(argv[1], "missing") == 0) {
        plm_model* m = NULL;
        int rc = plm_model_load(argv[2], "float32", &m);
        printf("%d %s\n", rc, plm_last_error());
        return m == NULL ? 0 : 1;
    }
    if (argc < 5 || strcmp(argv[1], "run") != 0) {
        fprintf(stderr, "usage: plm_demo config DIR | missing DIR | run DIR DTYPE OUT\n");
        return 2;
    }
    plm_model* model = NULL;
    plm_ctx* ctx = NULL;
    int vocab = 0;
    CHECK(plm_model_load(argv[2], argv[3], &model));
    CHECK(plm_model_vocab_size(model, &vocab));
    CHECK(plm_ctx_create(model, 3, 0, &ctx));

    const int lens[3] = {5, 11, 17}, slots[3] = {0, 1, 2};
    int prompts[3][17], flat[33], rows[33], n = 0;
    for (int s = 0; s < 3; ++s)
        for (int t = 0; t < lens[s]; ++t) {
            prompts[s][t] = token(s, t, vocab);
            rows[n] = n;
            flat[n++] = prompts[s][t];
        }
    float* logits = (float*)malloc(sizeof(float) * (size_t)(33 + 24) * (size_t)vocab);
    CHECK(plm_step(ctx, 3, slots, lens, flat, 33, rows, logits));
    const int one[3] = {1, 1, 1};
    for (int step = 0; step < 8; ++step) {
        int next[3];
        for (int s = 0; s < 3; ++s) next[s] = token(s, lens[s] + step, vocab);
        /* logit_rows NULL: the last token of every sequence */
        CHECK(plm_step(ctx, 3, slots, one, next, 0, NULL, logits + (size_t)(33 + 3 * step) * (size_t)vocab));
    }
    int length = 0;
    CHECK(plm_slot_length(ctx, 2, &length));
    if (length != 17 + 8) {
        fprintf(stderr, "slot 2 holds %d tokens, expected 25\n", length);
        return 1;
    }
    FILE* f = fopen(argv[4], "wb");
    if (f == NULL || fwrite(logits, sizeof(float), (size_t)(33 + 24) * (size_t)vocab, f) != (size_t)(33 + 24) * (size_t)vocab) {
        fprintf(stderr, "cannot write %s\n", argv[4]);
        return 1;
    }
    fclose(f);

    /* a greedy pick through plm_sample agrees with the largest logit of the row */
    plm_sampling greedy = plm_sampling_default();
    greedy.temperature = 0.0f;
    int picked[3];
    CHECK(plm_sample(ctx, logits + (size_t)(33 + 21) * (size_t)vocab, 3, &greedy, NULL, picked));
    for (int s = 0; s < 3; ++s) {
        const float* row = logits + (size_t)(33 + 21 + s) * (size_t)vocab;
        int best = 0;
        for (int v = 1; v < vocab; ++v)
            if (row[v] > row[best]) best = v;
        if (picked[s] != best) {
            fprintf(stderr, "plm_sample picked %d, the largest logit is at %d\n", picked[s], best);
            return 1;
        }
    }

    /* a step that does not fit changes nothing: slot 0 cannot take more tokens than its context */
    {
        int ctx_len = 0, too_many = 100000, rc;
        int* big = (int*)calloc((size_t)too_many, sizeof(int));
        CHECK(plm_slot_length(ctx, 0, &ctx_len));
        rc = plm_step(ctx, 1, slots, &too_many, big, 0, rows, NULL);
        free(big);
        if (rc != PLM_API_CACHE_FULL) {
            fprintf(stderr, "a step beyond the context returned %d (%s)\n", rc, plm_last_error());
            return 1;
        }
        CHECK(plm_slot_length(ctx, 0, &length));
        if (length != ctx_len) return 1;
    }

    for (int s = 0; s < 3; ++s) CHECK(plm_slot_reset(ctx, s));
    const int* ptrs[3] = {prompts[0], prompts[1], prompts[2]};
    int out[3][6], out_lens[3];
    int* outs[3] = {out[0], out[1], out[2]};
    const int no_stop[1] = {0};                     /* a list of no stop tokens (NULL would mean the model's own) */
    CHECK(plm_generate(ctx, 3, ptrs, lens, 6, &greedy, no_stop, 0, outs, out_lens));
    for (int s = 0; s < 3; ++s) {
        for (int t = 0; t < out_lens[s]; ++t) printf("%d ", out[s][t]);
        printf("\n");
    }
    CHECK(plm_ctx_free(ctx));
    CHECK(plm_model_free(model));
    free(logits);
    return 0;
}
