/* Harness TU 4: the reference's rope table builder (static in compute.c), included in place. */
#include "compute.c"

void gold_rope_table(float *cos_out, float *sin_out, int n_ctx, int head_dim, float theta) {
	rope_table_job job = {.cos_out = cos_out, .sin_out = sin_out, .n_ctx = n_ctx, .half = head_dim / 2,
	                      .theta_scale = pow(theta, -2.0 / (double)head_dim)};
	rope_table_chunk(0, head_dim / 2, -1, &job);
}
