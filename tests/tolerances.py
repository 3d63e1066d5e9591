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


BF16_IDEAL_FACTOR = 1.5


def bf16_bounds_from_ideal(exact, emulated):
    """The bfloat16 bounds at sizes other than the tiny models', measured instead of guessed: ``exact`` are
    the plain implementation's logits of a request, ``emulated`` the same with every value that the engine's
    bfloat16 mode stores in 16 bits rounded to bfloat16 (``PlainLfm2(storage="bfloat16")``), everything else
    exact: the error that an ideal implementation with the engine's storage points makes.  Rounding errors grow
    with the depth, the widths and the vocabulary (the largest of V errors), and two correct implementations
    that sum in different orders round differently and end up as far from each other as from the exact
    result; so the engine is held to BF16_IDEAL_FACTOR times the ideal error, row by row, both as a
    root-mean-square and as the largest error of a row, each as a fraction of the standard deviation of the row's
    exact logits.  Returns (largest-error bound, rms bound).  At the LFM2-1.2B shape, 16 layers, the ideal error
    was measured at 3.1 % rms (worst row 3.9 %) and 14 % largest (worst row 19 %); the engine's at 3.1 % / 4.0 %
    and 14 % / 19 %."""
    std = exact.std(axis=1)
    err = emulated - exact
    rms = float((np.sqrt((err ** 2).mean(axis=1)) / std).max())
    big = float((np.abs(err).max(axis=1) / std).max())
    return BF16_IDEAL_FACTOR * big, BF16_IDEAL_FACTOR * rms
