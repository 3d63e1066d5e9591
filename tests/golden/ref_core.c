/* Harness TU 1: the reference's scalar kernels, included in place from its
 * source tree (never copied), with thin exported wrappers.  Built only by
 * make_golden.py; not part of the package. */
#include "backend/cpu/scalar/core.c"

void gold_attention(const float *k, const float *v, const float *q, float *out, int head_dim, int n_pos,
                    float scale, int flash) {
	/* keys/values go through the reference's fp16 cache format */
	uint16_t *kh = malloc((size_t)n_pos * head_dim * 2), *vh = malloc((size_t)n_pos * head_dim * 2);
	float *scores = malloc((size_t)n_pos * sizeof(float));
	for (int i = 0; i < n_pos * head_dim; i++) {
		kh[i] = f32_to_f16(k[i]);
		vh[i] = f32_to_f16(v[i]);
	}
	cpu_attention_inner(kh, vh, head_dim, q, out, head_dim, n_pos, scale, flash, scores);
	free(kh); free(vh); free(scores);
}

void gold_f16_round(const float *in, float *out, int n) {
	for (int i = 0; i < n; i++) out[i] = f16_to_f32(f32_to_f16(in[i]));
}

void gold_swiglu(const float *g, const float *u, float *o, int n, int rows) {
	cpu_ffn_act_batch_job job = {.g = g, .u = u, .o = o, .n = n, .activation = 0};
	cpu_ffn_act_batch_chunk(0, rows, 0, &job);
}

void gold_rope_neox(float *v, int n_heads, int head_dim, int rope_dim, const float *c, const float *s) {
	rope_rotate_neox(v, n_heads, head_dim, rope_dim, c, s);
}
