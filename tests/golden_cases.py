"""Case list and seeded input generator shared by tests/golden/make_golden.py
(which runs the reference) and the tests (which run the oracle and the CUDA
library).  Inputs follow the reference's own benchmark distributions:
x ~ N(0,1) (src/ksmm_py/benchmark/ksmm_time.py:143-146) and
W ~ U(-1/sqrt(c), 1/sqrt(c)) (interface.py:30,67), drawn from the frozen
``numpy.random.RandomState`` stream so that they are identical everywhere.
"""
from __future__ import annotations

import math

import numpy as np

_ALL = ["dense", "einsum", "bmm"]


def _case(name, patterns, batch, bs_last, dtype="float32", seed=0, bias=False,
          algos=None, lead=None, **kw):
    d = dict(name=name, patterns=[tuple(p) for p in patterns], batch=batch, bs_last=bs_last,
             dtype=dtype, seed=seed, bias=bias, algos=algos or _ALL, lead=lead)
    d.update(kw)
    return d


CASES = [
    # single factors, every structural regime: a=1/d=1, a>1, d>1, both, b!=c, odd sizes
    _case("f_1_16_16_1_last", [(1, 16, 16, 1)], 24, True, seed=1, store_kernel_format=True),
    _case("f_1_16_16_1_first", [(1, 16, 16, 1)], 24, False, seed=2),
    _case("f_2_3_5_4_last", [(2, 3, 5, 4)], 17, True, seed=3, store_kernel_format=True),
    _case("f_2_3_5_4_first", [(2, 3, 5, 4)], 17, False, seed=4),
    _case("f_4_8_8_1_last", [(4, 8, 8, 1)], 32, True, seed=5),
    _case("f_1_48_24_3_first", [(1, 48, 24, 3)], 20, False, seed=6),
    _case("f_1_24_48_3_last", [(1, 24, 48, 3)], 20, True, seed=7),
    _case("f_3_7_9_2_last", [(3, 7, 9, 2)], 33, True, seed=8),
    _case("f_3_7_9_2_first", [(3, 7, 9, 2)], 33, False, seed=9),
    _case("f_1_64_64_16_last", [(1, 64, 64, 16)], 16, True, seed=10),
    _case("f_4_64_64_4_first", [(4, 64, 64, 4)], 16, False, seed=11),
    _case("f_1_1_1_8_last", [(1, 1, 1, 8)], 12, True, seed=12, algos=["dense", "einsum"]),
    _case("f_2_128_32_2_last_h", [(2, 128, 32, 2)], 40, True, dtype="float16", seed=13,
          algos=["dense", "einsum"]),
    _case("f_2_32_128_2_first_h", [(2, 32, 128, 2)], 40, False, dtype="float16", seed=14,
          algos=["dense", "einsum"]),
    # chains named by the benchmark configurations
    _case("c_readme_last", [(6, 64, 64, 1), (1, 768, 192, 2)], 16, True, seed=20),
    _case("c_readme_first", [(6, 64, 64, 1), (1, 768, 192, 2)], 16, False, seed=21),
    _case("c_vit_fc1_first", [(4, 192, 192, 1), (1, 768, 192, 4)], 8, False, seed=22),
    _case("c_vit_fc2_first", [(1, 192, 768, 4), (4, 192, 192, 1)], 8, False, seed=23),
    _case("c_vit_fc1_last", [(4, 192, 192, 1), (1, 768, 192, 4)], 8, True, seed=24),
    _case("c_three_last", [(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)], 8, True, seed=25),
    _case("c_three_first_h", [(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)], 8, False,
          dtype="float16", seed=26, algos=["dense", "einsum"]),
    # bias (added once, after the chain) and extra batch dimensions
    _case("c_bias_first", [(2, 8, 4, 2), (4, 6, 4, 2)], 10, False, seed=30, bias=True),
    _case("c_bias_last", [(2, 8, 4, 2), (4, 6, 4, 2)], 10, True, seed=31, bias=True),
    _case("c_lead_first", [(2, 8, 4, 2), (4, 6, 4, 2)], 12, False, seed=32, bias=True, lead=(3, 4)),
    _case("c_lead_last", [(2, 8, 4, 2), (4, 6, 4, 2)], 12, True, seed=33, bias=True, lead=(4, 3)),
]

CASES_BY_NAME = {c["name"]: c for c in CASES}


def make_weights(patterns, rng, dtype=np.float32):
    ws = []
    for (a, b, c, d) in patterns:
        s = 1.0 / math.sqrt(c)
        ws.append(rng.uniform(-s, s, size=(a, b, c, d)).astype(dtype))
    return ws


def make_inputs(case):
    """Returns (x, [W_f (a,b,c,d) ...], bias or None) as numpy arrays in the
    case's dtype.  ``x`` is (in, *lead) for batch-last, (*lead, in) for
    batch-first; ``lead`` defaults to (batch,)."""
    rng = np.random.RandomState(case["seed"])
    npdt = np.dtype(case["dtype"])
    pats = case["patterns"]
    a, b, c, d = pats[0]
    n_in = a * c * d
    lead = tuple(case["lead"]) if case.get("lead") else (case["batch"],)
    shape = (n_in, *lead) if case["bs_last"] else (*lead, n_in)
    x = rng.standard_normal(size=shape).astype(npdt)
    ws = make_weights(pats, rng, npdt)
    bias = None
    if case.get("bias"):
        a2, b2, c2, d2 = pats[-1]
        bound = 1.0 / math.sqrt(n_in)
        bias = rng.uniform(-bound, bound, size=(a2 * b2 * d2,)).astype(npdt)
    return x, ws, bias
