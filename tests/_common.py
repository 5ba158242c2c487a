"""Helpers shared by the test modules: seeded inputs per dtype and the error statistics the tolerances
are stated in."""
import numpy as np

import oracle
from numkong_b200 import synthetic as syn

TENSOR_DTYPES = ["i8", "u8", "bf16", "f16", "e4m3", "e5m2", "e2m3", "e3m2"]
ALL_DTYPES = TENSOR_DTYPES + ["f32"]
MINIFLOATS = ("e4m3", "e5m2", "e2m3", "e3m2")

# Odd shapes in the spirit of the reference's Python suite (test/test_base.py:36-95): (height, width, depth)
SMALL_SHAPES = [(1, 1, 1), (1, 8, 3), (3, 1, 7), (7, 5, 3), (33, 17, 65), (17, 63, 127), (129, 257, 129), (130, 300, 1000)]

# Sanity bound for floating-point dots on odd shapes, stated as  max |c - c_exact| / sum_l |a_l||b_l|  where c_exact is the
# f64 accumulation of the exactly decoded inputs (the statistic recommended for signed inputs, because plain relative
# error explodes near zero). This is NOT the acceptance gate: that is tests/test_gpu_error_envelope.py, which holds bf16 /
# f16 products and distances to the error of the reference's own worst back end on the same inputs. The bound here only
# has to cover the worst single cell of tiny problems: the tensor cores truncate instead of rounding, so even a 3-term dot
# can be off by one f32 ulp of the result (1.2e-7 in this statistic); long dots measure 1e-8 (8/6-bit) to 5e-8 (16-bit).
DOT_TOLERANCE = {"bf16": 2.5e-7, "f16": 2.5e-7, "e4m3": 1.5e-7, "e5m2": 1.5e-7, "e2m3": 1.5e-7, "e3m2": 1.5e-7, "f32": 1e-15}

# Batched distances: absolute tolerance on the result (angular lives in [0, 2], so this is ~4 ulp of 1.0),
# relative for euclidean. The reference's back ends differ from each other by up to 1 ulp / 4 ulp here.
ANGULAR_ATOL = 5e-7
EUCLIDEAN_RTOL = 2e-6


def make_matrix(rows, cols, dtype, seed, kind="normal"):
    if kind == "codes" and dtype in MINIFLOATS:
        return syn.finite_codes_matrix(rows, cols, dtype, seed)
    if kind == "lognormal":
        return syn.lognormal_matrix(rows, cols, dtype, seed)
    return syn.normal_matrix(rows, cols, dtype, seed)


def normalized_error(c, a, b, dtype):
    """max |c - exact| / sum|a||b| with exact = f64 accumulation of the decoded inputs."""
    exact = oracle.exact_dots_f64(a, b, dtype)
    fa = np.abs(oracle.decode(a, dtype)).astype(np.float64)
    fb = np.abs(oracle.decode(b, dtype)).astype(np.float64)
    denom = fa @ fb.T
    denom[denom == 0] = 1.0
    return float(np.max(np.abs(np.asarray(c, dtype=np.float64) - exact) / denom))


def ones_matrix(rows, cols, dtype):
    """A matrix of ones in the storage format of `dtype` (reference KAT: rust/matrix.rs:4610-4643)."""
    return syn.encode(np.ones((rows, cols), dtype=np.float32), dtype)
