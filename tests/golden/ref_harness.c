/* Drives whoreson/picolm's own CPU model code (compiled from its sources,
 * untouched) on a tiny Llama whose fp32 weights arrive in a flat file, and writes
 * the logits of every position: token by token through model_forward, and the
 * last position once more through model_forward_prefill.
 *
 * It only fills the reference's structs and calls its functions; the file
 * layout is this harness's own (see make_golden.py, which writes it).
 * The reference's CLI does not link without its GPU backend, so the timer that
 * model_core.c expects from picolm.c is defined here. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "model.h"
#include "tensor.h"
#include "quant.h"

double get_time_ms(void) { return 0.0; }

static void *read_block(FILE *f, size_t bytes) {
    void *p = malloc(bytes ? bytes : 1);
    if (fread(p, 1, bytes, f) != bytes) { fprintf(stderr, "short read\n"); exit(2); }
    return p;
}

int main(int argc, char **argv) {
    if (argc != 3) { fprintf(stderr, "usage: ref_harness <in.bin> <out.bin>\n"); return 1; }
    FILE *f = fopen(argv[1], "rb");
    if (!f) { perror(argv[1]); return 1; }
    int hdr[12];
    float fl[2];
    if (fread(hdr, sizeof(int), 12, f) != 12 || fread(fl, sizeof(float), 2, f) != 2) return 2;
    int d = hdr[0], F = hdr[1], H = hdr[2], G = hdr[3], L = hdr[4], V = hdr[5], S = hdr[6], hd = hdr[7];
    int rope_type = hdr[8], tied = hdr[9], n_tok = hdr[10], has_table = hdr[11];

    static model_t m;
    memset(&m, 0, sizeof(m));
    model_config_t *c = &m.config;
    c->n_embd = d; c->n_ffn = F; c->n_heads = H; c->n_kv_heads = G; c->n_layers = L; c->vocab_size = V;
    c->max_seq_len = S; c->head_dim = hd; c->rope_freq_base = fl[0]; c->rms_norm_eps = fl[1];
    c->rope_type = rope_type; c->rope_dim = hd; c->weight_type = GGUF_TYPE_F32;

    int *tokens = (int *)read_block(f, sizeof(int) * (size_t)n_tok);
    model_weights_t *w = &m.weights;
    w->token_embd = read_block(f, sizeof(float) * (size_t)V * d); w->type_token_embd = GGUF_TYPE_F32;
    for (int l = 0; l < L; l++) {
        layer_weights_t *lw = &w->layers[l];
        lw->is_attn_layer = 1;
        lw->attn_norm = read_block(f, sizeof(float) * d);                      lw->type_attn_norm = GGUF_TYPE_F32;
        lw->attn_q = read_block(f, sizeof(float) * (size_t)H * hd * d);        lw->type_attn_q = GGUF_TYPE_F32;
        lw->attn_k = read_block(f, sizeof(float) * (size_t)G * hd * d);        lw->type_attn_k = GGUF_TYPE_F32;
        lw->attn_v = read_block(f, sizeof(float) * (size_t)G * hd * d);        lw->type_attn_v = GGUF_TYPE_F32;
        lw->attn_output = read_block(f, sizeof(float) * (size_t)d * H * hd);   lw->type_attn_output = GGUF_TYPE_F32;
        lw->post_attn_norm = read_block(f, sizeof(float) * d);                 lw->type_post_attn_norm = GGUF_TYPE_F32;
        lw->ffn_gate = read_block(f, sizeof(float) * (size_t)F * d);           lw->type_ffn_gate = GGUF_TYPE_F32;
        lw->ffn_up = read_block(f, sizeof(float) * (size_t)F * d);             lw->type_ffn_up = GGUF_TYPE_F32;
        lw->ffn_down = read_block(f, sizeof(float) * (size_t)d * F);           lw->type_ffn_down = GGUF_TYPE_F32;
    }
    w->output_norm = read_block(f, sizeof(float) * d); w->type_output_norm = GGUF_TYPE_F32;
    w->output = tied ? w->token_embd : read_block(f, sizeof(float) * (size_t)V * d);
    w->type_output = GGUF_TYPE_F32;

    fp16_table_init();
    if (allocate_run_state(&m, KV_CACHE_F16, KV_CACHE_F16, 0, 0, 1) != 0) { fprintf(stderr, "allocate_run_state failed\n"); return 3; }
    tensor_set_threads(1);
    if (has_table) {                       /* a rotary table that the reference cannot build itself (llama3 scaling) */
        size_t n = (size_t)S * (hd / 2);
        float *cs = (float *)read_block(f, sizeof(float) * n), *sn = (float *)read_block(f, sizeof(float) * n);
        memcpy(m.state.rope_cos, cs, sizeof(float) * n);
        memcpy(m.state.rope_sin, sn, sizeof(float) * n);
    }
    fclose(f);

    FILE *o = fopen(argv[2], "wb");
    if (!o) { perror(argv[2]); return 1; }
    for (int t = 0; t < n_tok; t++) {
        float *logits = model_forward(&m, tokens[t], t);
        if (!logits) { fprintf(stderr, "model_forward failed at %d\n", t); return 4; }
        fwrite(logits, sizeof(float), (size_t)V, o);
    }
    float *last = model_forward_prefill(&m, tokens, n_tok, 0, NULL);
    if (!last) { fprintf(stderr, "model_forward_prefill failed\n"); return 5; }
    fwrite(last, sizeof(float), (size_t)V, o);
    fclose(o);
    return 0;
}
