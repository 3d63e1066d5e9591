"""Tolerances of the engine-versus-plain comparisons, stated once.

float32 path: the engine sums in float32 in another order than the float64
plain implementation; logits of the tiny models are O(1), so 2e-5 absolute is
about a hundred float32 roundings.

bfloat16 path: weights are the same bfloat16 values on both sides; the engine
rounds activations to bfloat16 (relative 2^-9) before each matrix product and
keeps keys and values in bfloat16.  With a dozen such roundings a layer the
logits move by a few per cent of their spread; the bound is 5 % of the
standard deviation of the plain logits of the request.
"""
import numpy as np

FP32_ATOL = 2e-5
BF16_REL_STD = 0.05


def tol_for(dtype, expected):
    if dtype == "float32":
        return FP32_ATOL
    return BF16_REL_STD * float(np.std(expected))


def fp32_tol_at_width(width):
    """The float32 bound at another width.  FP32_ATOL was set at widths of 64 to 128; a sum of K float32
    products strays from its exact value like sqrt(K) roundings, so the bound grows with the square root of
    the width (2048: 5.7 x 2e-5 = 1.1e-4)."""
    return FP32_ATOL * float(np.sqrt(max(width, 64) / 64.0))


BF16_RMS_REL_STD = BF16_REL_STD / 3.53          # the same bound as a root-mean-square error: see below


def bf16_bounds_for(n_layers, vocab):
    """The bfloat16 bounds for a model of ``n_layers`` and a vocabulary of ``vocab``, as fractions of the
    standard deviation of a row of logits: (bound on the largest error of the row, bound on its
    root-mean-square error).

    Every layer adds two branch outputs to the float32 residual, each computed from operands rounded to
    bfloat16 (relative 2^-9 each, about six roundings a branch); the errors of the branches are independent,
    so the error of a logit grows like the square root of the number of layers.  The errors of a row's logits
    are close to Gaussian, and the largest of V Gaussians lies near sqrt(2 ln V) standard deviations: 3.53 for
    the 512 logits of the six-layer test model, where BF16_REL_STD (5 %) is the bound on the largest error, so
    its root-mean-square error is bounded by 5 % / 3.53 = 1.42 %; 4.71 for 65536 logits.  Sixteen layers and
    65536 logits: rms 1.42 % x sqrt(16 / 6) = 2.3 %, largest 2.3 % x 4.71 = 10.9 %."""
    rms = BF16_RMS_REL_STD * float(np.sqrt(max(n_layers, 6) / 6.0))
    return rms * float(np.sqrt(2.0 * np.log(max(vocab, 512)))), rms
