/* Harness TU 2: the reference's gated short convolution (a static function of
 * backend/cpu/common.c), included in place. */
#include "backend/cpu/common.c"

void gold_shortconv(const float *mixed, const float *conv_w, float *state, float *out, int n_rows, int dim,
                    int kernel) {
	shortconv_desc d = {0};
	d.mixed = mixed; d.conv_w = conv_w; d.state = state; d.out = out;
	d.n_rows = n_rows; d.dim = dim; d.kernel = kernel; d.in_stride = 3 * dim; d.out_stride = dim;
	shortconv_causal_chunk(0, dim, 0, &d);
}
