/* picolm_b200: the C face of the library, in the manner of whoreson/picolm's model.h
 * (picolm/model.h:504-582: model_load, model_forward, model_forward_prefill, model_free, with the
 * caller holding the position).  Where the reference has one sequence per model and the caller's `pos`,
 * this API has a context with `n_slots` cache slots, one per live sequence, and ONE step function that
 * takes the next tokens of any number of them: model_forward(token, pos) is plm_step with one slot and
 * one token, model_forward_prefill(tokens, n, start_pos) is plm_step with one slot and n tokens.
 *
 * The engine behind these calls is the library's one engine (the parts are put together by configuration
 * and registered by name, which is why its host side is Python): this library starts an interpreter inside
 * the calling process the first time it is used (or joins the one that is running, if the caller is a
 * Python process) and forwards every call to it.  There is no second forward pass behind this header.
 * Hot loops do not pay for that: a decode step is one replay of a captured CUDA graph, and plm_generate
 * runs whole batches per call.
 *
 * Every function returns 0 on success and a non-zero code otherwise; plm_last_error() then gives the
 * reason in words (per thread).  Token ids and logits are host memory owned by the caller.
 */
#ifndef PICOLM_B200_PLM_H
#define PICOLM_B200_PLM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct plm_model plm_model; /* weights on the device, built from config.json by the architecture registry */
typedef struct plm_ctx plm_ctx;     /* a cache (slots, pages, per-sequence state) and the step function over it */

enum {
    PLM_API_OK = 0,
    PLM_API_ERROR = 1,       /* see plm_last_error() */
    PLM_API_CACHE_FULL = 2,  /* the step needs more pages or positions than the context has; nothing was changed */
    PLM_API_BAD_ARGUMENT = 3
};

/* The reference's sampler options with its defaults (picolm/picolm.c:774-776, :1230): temperature <= 0 is
 * greedy; top_k <= 0, top_p >= 1 and min_p <= 0 switch the respective filter off. */
typedef struct plm_sampling {
    float temperature; /* 0.8 */
    int top_k;         /* 40 */
    float top_p;       /* 0.9 */
    float min_p;       /* 0.05 */
    uint64_t seed;     /* 42; request i draws from the xorshift64 stream seeded seed + i */
} plm_sampling;

plm_sampling plm_sampling_default(void);

/* The reason of the calling thread's last failure ("" if none). */
const char* plm_last_error(void);

/* Read and validate `path` (a model folder or a config.json) through the architecture registry and write
 * the typed configuration, with every default filled in, as JSON text into `out` (NUL-terminated).
 * Needs no GPU. */
int plm_config_from_json(const char* path, char* out, size_t out_capacity);

/* Load a model folder (config.json + safetensors).  `dtype`: "bfloat16" (the serving kernels) or "float32"
 * (everything in true 32-bit). */
int plm_model_load(const char* model_dir, const char* dtype, plm_model** out);

/* A model with random weights from a config.json and a seed: the folder `out_dir` is written
 * (config.json, model.safetensors) and loaded. */
int plm_model_random(const char* config_json, uint64_t seed, const char* dtype, const char* out_dir, plm_model** out);

int plm_model_free(plm_model* model);
int plm_model_vocab_size(const plm_model* model, int* out);

/* A context of `n_slots` sequences of up to `max_context` tokens each (0: the model's own limit). */
int plm_ctx_create(plm_model* model, int n_slots, int max_context, plm_ctx** out);
int plm_ctx_free(plm_ctx* ctx);

/* Empty a slot: length 0, its pages given back, its fixed-size state zeroed.  A slot that was never used
 * is empty already. */
int plm_slot_reset(plm_ctx* ctx, int slot);
int plm_slot_length(plm_ctx* ctx, int slot, int* out);

/* One step.  Sequence i lives in `slots[i]` (distinct, each in [0, n_slots)) and brings `n_new[i]` >= 1
 * tokens, all sequences' tokens flattened in `tokens`; its new tokens take the positions after what its
 * slot holds.  `logit_rows`: indices into the flattened tokens whose logits are wanted (NULL: the last
 * token of every sequence, n_logit_rows is then ignored); `logits_out` receives [rows, vocab] floats.
 * With n_logit_rows == 0 and logit_rows != NULL nothing is computed beyond the cache. */
int plm_step(plm_ctx* ctx, int n_seqs, const int* slots, const int* n_new, const int* tokens, int n_logit_rows,
             const int* logit_rows, float* logits_out);

/* Choose one token per row of `logits` [rows, vocab] (host memory).  `rng_states` holds one xorshift64
 * state per row and is advanced in place (ignored when greedy; seed a stream with plm_sampling.seed + i). */
int plm_sample(plm_ctx* ctx, const float* logits, int rows, const plm_sampling* sampling, uint64_t* rng_states,
               int* tokens_out);

/* Generate up to `max_new` tokens for each of `n_prompts` prompts: batches of unequal prompts in one step,
 * then one token each; a sequence ends with a stop token (recorded, not fed), at max_new, or when its
 * context is full; as many batches one after another as the slots and the cache allow.  `stop_ids` NULL:
 * the model's own end-of-sequence ids (a non-NULL pointer with n_stop 0: no stop tokens).  `out_tokens[i]` must have room for max_new ints; `out_lens[i]`
 * receives how many were generated.  All slots of the context must be empty. */
int plm_generate(plm_ctx* ctx, int n_prompts, const int* const* prompts, const int* prompt_lens, int max_new,
                 const plm_sampling* sampling, const int* stop_ids, int n_stop, int* const* out_tokens, int* out_lens);

#ifdef __cplusplus
}
#endif
#endif
