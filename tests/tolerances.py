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
