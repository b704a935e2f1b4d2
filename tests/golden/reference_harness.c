/* Drives the reference's own float32 forward pass (st_qwen_model_forward,
 * src/model/vllm_safetensors.c:16356) on weights read from a flat file, one token at a time,
 * and writes the logits after every token.  Used once by make_reference_golden.py to anchor
 * tests/plain_qwen3.py on the reference's code; nothing in the engine uses it.
 *
 * Input file (little-endian): int32 L, d, nh, nkv, hd, ff, V, T; float32 theta, eps;
 * int32 tokens[T]; then float32 arrays in this order: token_embed[V*d], lm_head[V*d],
 * final_norm[d], attn_norm[L*d], ffn_norm[L*d], q[L*q_out*d], k[L*kv*d], v[L*kv*d],
 * o[L*d*q_out], q_norm[L*hd], k_norm[L*hd], gate[L*ff*d], up[L*ff*d], down[L*d*ff].
 * Output file: float32 logits[T*V].
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "vllm_safetensors.h"

int g_bench_seqlen = 0;

static float *rd(FILE *f, size_t n) {
    float *p = (float *)malloc(n * sizeof(float));
    if (!p || fread(p, sizeof(float), n, f) != n) { fprintf(stderr, "short read\n"); exit(2); }
    return p;
}

int main(int argc, char **argv) {
    if (argc < 3) return 1;
    FILE *f = fopen(argv[1], "rb");
    if (!f) return 1;
    int h[8];
    float fl[2];
    if (fread(h, 4, 8, f) != 8 || fread(fl, 4, 2, f) != 2) return 2;
    int L = h[0], d = h[1], nh = h[2], nkv = h[3], hd = h[4], ff = h[5], V = h[6], T = h[7];
    int *tok = (int *)malloc(sizeof(int) * T);
    if (fread(tok, 4, T, f) != (size_t)T) return 2;
    size_t q_out = (size_t)nh * hd, kv = (size_t)nkv * hd;
    static STModelWeights w;
    memset(&w, 0, sizeof(w));
    w.cfg.dim = d; w.cfg.n_layers = L; w.cfg.n_heads = nh; w.cfg.n_kv_heads = nkv;
    w.cfg.head_dim = hd; w.cfg.head_dim_full = hd; w.cfg.ffn_dim = ff; w.cfg.vocab_size = V;
    w.cfg.max_seq_len = 256; w.cfg.rope_theta = fl[0]; w.cfg.norm_eps = fl[1];
    w.cfg.has_q_norm = true;
    w.token_embed = rd(f, (size_t)V * d);
    w.lm_head = rd(f, (size_t)V * d);
    w.final_norm = rd(f, d);
    w.attn_norm = rd(f, (size_t)L * d);
    w.ffn_norm = rd(f, (size_t)L * d);
    w.q_weight = rd(f, L * q_out * d);
    w.k_weight = rd(f, L * kv * d);
    w.v_weight = rd(f, L * kv * d);
    w.o_weight = rd(f, L * d * q_out);
    w.q_norm = rd(f, (size_t)L * hd);
    w.k_norm = rd(f, (size_t)L * hd);
    w.gate_weight = rd(f, (size_t)L * ff * d);
    w.up_weight = rd(f, (size_t)L * ff * d);
    w.down_weight = rd(f, (size_t)L * d * ff);
    fclose(f);
    w.n_layers_allocated = L;
    w.is_allocated = 1;
    w.weights_loaded = ~0;

    static STQwenInferenceState st;
    if (st_qwen_inference_init(&st, &w) != 0) { fprintf(stderr, "init failed\n"); return 3; }
    FILE *o = fopen(argv[2], "wb");
    for (int t = 0; t < T; t++) {
        st_qwen_model_forward(&st, tok[t]);
        fwrite(st.logits, sizeof(float), V, o);
    }
    fclose(o);
    return 0;
}
