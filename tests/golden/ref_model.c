/* Harness TU 5: a whole LFM2 model through the reference's own loader, recipe and CPU backend.
 * It is linked with the reference's sources compiled in place from its tree (never copied): see
 * make_golden.py, which also gives a two-line stand-in for the json-c header that model.c includes but this
 * path never uses.  The model comes from a GGUF file that make_golden.py writes from the same tensors the plain
 * implementation reads. */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "backend/backend.h"
#include "compute.h"
#include "kvcache.h"
#include "model.h"

/* Logits of a sequence fed in portions: portion i is tokens[cuts[i] .. cuts[i+1]) (cuts[0] = 0,
 * cuts[n_cuts] = n); out gets one row of `vocab` floats per portion, the logits behind its last token
 * (compute_forward_batch gives those of a chunk's last row).  flash: the reference's --flash-attn.
 * Returns 0, or the first failing status code (negative: set-up failed). */
int gold_model_logits(const char *gguf_path, const int32_t *tokens, const int *cuts, int n_cuts, int n_ctx,
                      int flash, float *out, int vocab) {
	backend *be = NULL;
	model m;
	kvcache kv;
	compute_scratch s;
	memset(&m, 0, sizeof(m));
	memset(&kv, 0, sizeof(kv));
	if (backend_create("cpu", 0, &be) != OK) return -1;
	if (model_load_backend_ex_repack(&m, gguf_path, be, 0, NULL) != OK) return -2;
	if (m.vocab_size != vocab) return -3;
	if (kvcache_init(&kv, &m, n_ctx, KV_QUANT_F16) != OK) return -4;
	compute_scratch_init(&s);
	if (compute_scratch_ensure(&s, &m, n_ctx) != OK) return -5;
	int rc = 0;
	for (int i = 0; i < n_cuts && rc == 0; i++) {
		const int a = cuts[i], n = cuts[i + 1] - cuts[i];
		status_code st = compute_forward_batch(&m, &kv, &s, tokens + a, n, a, flash, out + (size_t)i * vocab);
		kv.n_pos += n;
		if (st != OK) rc = (int)st ? (int)st : 99;
	}
	compute_scratch_free(&s);
	kvcache_free(&kv);
	model_free(&m);
	backend_destroy(be);
	return rc;
}
