"""Every pattern of the reference's tuning list through the default dispatch.

``tests/golden/patterns_in.txt`` holds the 728 distinct (a,b,c,d) rows of the
reference's ``patterns.in`` (odd b and c, d up to 14336, a up to 4096, blocks
from 1 x 2 to 1024 x 1024).  Each one runs in fp32 and fp16, batch-last and
batch-first, through ``ksmm_cu_forward`` with whatever kernel the library
picks; a refusal is a failure.  One fp64 oracle result per pattern (on the fp32
inputs) serves the four runs: the fp16 runs see the inputs rounded to fp16, an
error of about 7e-4 against a tolerance of 1e-2.

* all patterns at batch 64 (the tensor-core kernels' alignment rules hold);
* every ninth pattern at batch 40 (fp32 batch-last then leaves the tensor-core family);
* a stratified subset at the benchmark batch 25088 on sampled columns: every distinct d,
  the odd-sized rows, the largest a, the largest d, the largest blocks.
"""
import os

import numpy as np
import pytest
import torch

import ksmm_b200 as kb
from oracle import ksmm_oracle as ko

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 1e-5, torch.float16: 1e-2}
HERE = os.path.dirname(os.path.abspath(__file__))


def load_patterns():
    rows = []
    for ln in open(os.path.join(HERE, "golden", "patterns_in.txt")):
        ln = ln.strip()
        if ln and not ln.startswith("#"):
            rows.append(tuple(int(v) for v in ln.split(",")))
    return rows


PATTERNS = load_patterns()


def _draw(pattern, batch, seed):
    """x ~ N(0,1) of shape (a*c*d, batch) and W ~ U(+-1/sqrt(c)) of shape (a,b,c,d), fp32, drawn on
    the device (the list holds 3.5e9 weights in all) from a seeded generator."""
    a, b, c, d = pattern
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn((a * c * d, batch), generator=g, device=DEV)
    w = (torch.rand((a, b, c, d), generator=g, device=DEV) * 2 - 1) / (c ** 0.5)
    return x, w


def _check_all_four(pattern, x, w, ref_last, cols=None):
    """x: (in, batch) fp32 on the device; ref_last: oracle (out, batch or len(cols))."""
    a, b, c, d = pattern
    for dtype in (torch.float32, torch.float16):
        xd = x.to(dtype)
        wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
        for bs_last in (True, False):
            xin = xd if bs_last else xd.t().contiguous()
            y = kb.Kernel.forward(xin, wk, bs_last, a, b, c, d, dtype)      # raises on a refusal
            if cols is not None:
                y = y[:, cols] if bs_last else y[cols]
            y = y.float().cpu().numpy()
            if not bs_last:
                y = y.T
            assert not np.isnan(y).any(), (pattern, dtype, bs_last)
            err = ko.rel_fro_error(y, ref_last)
            assert err < TOL[dtype], (pattern, dtype, bs_last, err)
            del xin, y
        del xd, wk


def test_patterns_file_is_the_reference_list():
    assert len(PATTERNS) == 728 and len(set(PATTERNS)) == 728
    assert PATTERNS[0] == (1, 48, 48, 1)
    assert max(p[3] for p in PATTERNS) == 14336 and max(p[0] for p in PATTERNS) == 4096
    assert any(p[1] % 2 for p in PATTERNS) and any(p[2] % 8 for p in PATTERNS)


@pytest.mark.parametrize("part", range(8))
def test_every_pattern_at_a_small_batch(part):
    for pi in range(part, len(PATTERNS), 8):
        pattern = PATTERNS[pi]
        batches = (64, 40) if pi % 9 == 0 else (64,)
        for batch in batches:
            x, w = _draw(pattern, batch, seed=1000 + pi)
            ref = ko.factor_apply(x.cpu().numpy(), w.cpu().numpy(), True)
            _check_all_four(pattern, x, w, ref)
            del x, w
    kb.check_device()


def stratified_subset():
    chosen = []
    by_d = {}
    for p in PATTERNS:
        by_d.setdefault(p[3], []).append(p)
    for d, ps in sorted(by_d.items()):
        chosen.append(max(ps, key=lambda p: (p[1] * p[2], p[0])))        # largest block of every d
    odd = [p for p in PATTERNS if p[1] % 8 or p[2] % 8]
    chosen += odd[::6]
    chosen.append(max(PATTERNS, key=lambda p: p[0]))
    chosen.append(max(PATTERNS, key=lambda p: p[0] * max(p[1], p[2]) * p[3]))   # most features
    chosen.append(max(PATTERNS, key=lambda p: p[0] * p[1] * p[2] * p[3]))       # most weights
    out = []
    for p in chosen:
        if p not in out:
            out.append(p)
    return out


FULL_B = 25088


@pytest.mark.parametrize("part", range(4))
def test_stratified_subset_at_the_benchmark_batch(part):
    subset = stratified_subset()
    assert len(subset) >= 30
    cols = np.unique(np.concatenate([np.arange(0, 4), np.arange(FULL_B - 4, FULL_B),
                                     np.random.RandomState(5).randint(0, FULL_B, 40)]))
    cols_t = torch.from_numpy(cols).to(DEV)
    for pi in range(part, len(subset), 4):
        pattern = subset[pi]
        x, w = _draw(pattern, FULL_B, seed=5000 + pi)
        ref = ko.factor_apply(x[:, cols_t].cpu().numpy(), w.cpu().numpy(), True)
        _check_all_four(pattern, x, w, ref, cols=cols_t)
        del x, w
        torch.cuda.empty_cache()
    kb.check_device()
