/* Harness TU 3: norms (scalar/quants.c), the rope table (compute.c) and the sampler, included in place. */
#include "backend/cpu/scalar/quants.c"
#include "sampler.c"

void gold_rmsnorm(const float *x, const float *w, float *y, int n, float eps) { rmsnorm(x, w, y, n, eps); }
void gold_rmsnorm_per_head(const float *x, const float *w, float *y, int n_heads, int head_dim, float eps) {
	rmsnorm_per_head(x, w, y, n_heads, head_dim, eps);
}
/* one draw: a fresh sampler seeded with `seed`; returns the token and the uniform it used */
int gold_sample(const float *logits, int vocab, unsigned long long seed, float temp, int top_k, float top_p,
                float min_p, float *u_out) {
	sampler s, t;
	sampler_init(&s, seed);
	sampler_init(&t, seed);
	*u_out = rng_uniform(&t.rng);
	sampler_set_params(&s, temp, top_k, top_p, min_p, 1.0f, 64);
	sampler_set_vocab(&s, vocab);
	int tok = sampler_sample(&s, logits, vocab);
	sampler_free(&s); sampler_free(&t);
	return tok;
}
int gold_argmax(const float *logits, int vocab) { return sampler_argmax(logits, vocab); }
