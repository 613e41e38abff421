"""Parity of the CUDA library (through its C ABI) with the CPU oracle and with
the reference's own outputs.  Tolerances are the relative Frobenius errors of
the benchmark specification: 1e-5 fp32, 1e-2 fp16/bf16, 5e-2 fp8."""
import ctypes
import math
import os

import numpy as np
import pytest
import torch

import ksmm_b200 as kb
from golden_cases import CASES, make_inputs, make_weights
from ksmm_b200 import _lib
from oracle import ksmm_oracle as ko

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "ksmm_golden.npz"))
TOL = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-2}
TDT = {"float32": torch.float32, "float16": torch.float16}
DEV = "cuda:0"


def _inputs(pattern, batch, dtype, bs_last, seed):
    rng = np.random.RandomState(seed)
    a, b, c, d = pattern
    shape = (a * c * d, batch) if bs_last else (batch, a * c * d)
    x = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dtype)
    w = torch.from_numpy(make_weights([pattern], rng)[0]).to(dtype)
    return x, w


def _oracle(x, w, bs_last):
    """fp64 oracle on the values the GPU actually sees (already rounded to dtype)."""
    return ko.factor_apply(x.float().numpy(), w.float().numpy(), bs_last)


def _run(x, w, pattern, bs_last, algo=_lib.KSMM_ALGO_AUTO, config=-1, poison=True, **kw):
    wk = kb.generate_factor(*pattern, "kernel", w, x.dtype, DEV)
    xg = x.to(DEV)
    a, b, c, d = pattern
    batch = x.shape[1] if bs_last else x.shape[0]
    shape = (a * b * d, batch) if bs_last else (batch, a * b * d)
    out = None
    if poison:
        out = torch.full(shape, float("nan"), dtype=kw.get("out_dtype", x.dtype), device=DEV)
    y = kb.forward_ex(xg, wk, bs_last, a, b, c, d, algo=algo, config=config, out=out, **kw)
    return y.float().cpu().numpy()


# ---------------------------------------------------------------------------
# 1. the reference's own outputs, through KSLinear
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_kslinear_matches_reference_golden(case):
    x, ws, bias = make_inputs(case)
    dt = TDT[case["dtype"]]
    layer = kb.KSLinear(case["patterns"], weights=[torch.from_numpy(w) for w in ws],
                        bias=bias is not None, algo="kernel", dtype=dt, bs_last=case["bs_last"],
                        device=DEV)
    if bias is not None:
        layer.bias.data.copy_(torch.from_numpy(bias).to(dt).reshape(layer.bias.shape))
    y = layer(torch.from_numpy(x).to(DEV))
    ref = GOLDEN[case["name"] + "/y"]
    assert tuple(y.shape) == ref.shape
    err = ko.rel_fro_error(y.float().cpu().numpy(), ref)
    assert err < TOL[dt], (case["name"], err)
    # per-factor execution gives the same answer as the single chain call
    layer.fuse_chain = False
    y2 = layer(torch.from_numpy(x).to(DEV))
    assert ko.rel_fro_error(y2.float().cpu().numpy(), ref) < TOL[dt]


def test_state_dict_layout_is_the_reference_kernel_format():
    case = next(c for c in CASES if c["name"] == "f_2_3_5_4_last")
    _, ws, _ = make_inputs(case)
    layer = kb.KSLinear(case["patterns"], weights=[torch.from_numpy(w) for w in ws], bias=True,
                        algo="kernel", dtype=torch.float32, bs_last=True, device=DEV)
    sd = layer.state_dict()
    assert set(sd) == {"factors.0", "bias"}
    assert np.array_equal(sd["factors.0"].cpu().numpy(), GOLDEN["f_2_3_5_4_last/kernel_format0"])
    assert tuple(sd["bias"].shape) == (layer.out_size, 1)
    dense = layer.get_dense_product().cpu().numpy()
    assert np.array_equal(dense, GOLDEN["f_2_3_5_4_last/dense_from_kernel0"])


# ---------------------------------------------------------------------------
# 2. FFMA family: every tile configuration, ragged shapes, every element type
# ---------------------------------------------------------------------------
SIMT_PATTERNS = [(2, 3, 5, 4), (1, 16, 16, 1), (3, 7, 9, 2), (1, 48, 24, 3), (2, 130, 20, 1),
                 (1, 64, 64, 2), (1, 1, 1, 8), (4, 8, 8, 1)]


@pytest.mark.parametrize("config", range(6))
@pytest.mark.parametrize("bs_last", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_simt_family_every_config(config, bs_last, dtype):
    for pi, pattern in enumerate(SIMT_PATTERNS):
        for batch in (33, 256):
            x, w = _inputs(pattern, batch, dtype, bs_last, seed=100 + pi)
            y = _run(x, w, pattern, bs_last, algo=_lib.KSMM_ALGO_SIMT, config=config)
            assert not np.isnan(y).any(), (pattern, batch)
            err = ko.rel_fro_error(y, _oracle(x, w, bs_last))
            assert err < TOL[dtype], (pattern, batch, err)


@pytest.mark.parametrize("config", [6, 7])
def test_ffma_tma_staged_fp32_batch_last(config):
    """fp32 batch-last kernel with TMA-staged operands (FFMA family, configurations 6 and 7)."""
    pats = [(2, 12, 8, 1), (1, 16, 16, 1), (2, 132, 20, 1), (1, 64, 64, 2), (4, 8, 8, 1),
            (1, 768, 192, 2), (3, 72, 45, 3), (1, 4, 100, 2)]
    for pi, pattern in enumerate(pats):
        for batch in (36, 256, 388):
            x, w = _inputs(pattern, batch, torch.float32, True, seed=150 + pi)
            y = _run(x, w, pattern, True, algo=_lib.KSMM_ALGO_SIMT, config=config)
            assert not np.isnan(y).any(), (pattern, batch)
            err = ko.rel_fro_error(y, _oracle(x, w, True))
            assert err < 1e-5, (pattern, batch, err)
    # outside its envelope (odd batch, batch-first, 16-bit) the configuration is refused
    x, w = _inputs((1, 16, 16, 1), 33, torch.float32, True, seed=1)
    with pytest.raises(kb.KsmmError):
        _run(x, w, (1, 16, 16, 1), True, algo=_lib.KSMM_ALGO_SIMT, config=config)
    x, w = _inputs((1, 16, 16, 1), 32, torch.float32, False, seed=1)
    with pytest.raises(kb.KsmmError):
        _run(x, w, (1, 16, 16, 1), False, algo=_lib.KSMM_ALGO_SIMT, config=config)
    kb.check_device()


def test_ffma_tma_staged_fp32_batch_first():
    """fp32 batch-first kernel with TMA-staged operands (FFMA family, configuration 8):
    d = 1, d = 2 and d = 4 take three different thread tilings."""
    pats = [(2, 12, 8, 1), (1, 64, 64, 1), (3, 72, 44, 1), (1, 768, 192, 1),        # d = 1
            (2, 12, 8, 2), (1, 64, 64, 2), (1, 132, 50, 2), (1, 768, 192, 2),       # d = 2
            (1, 64, 64, 4), (2, 12, 9, 4), (1, 768, 192, 4), (4, 64, 64, 4), (2, 72, 20, 4)]       # d = 4
    rng = np.random.RandomState(7)
    for pi, pattern in enumerate(pats):
        for batch in (37, 256, 390):
            x, w = _inputs(pattern, batch, torch.float32, False, seed=170 + pi)
            a, b, c, d = pattern
            bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32))
            y = _run(x, w, pattern, False, algo=_lib.KSMM_ALGO_SIMT, config=8, bias=bias.to(DEV),
                     alpha=2.0)
            assert not np.isnan(y).any(), (pattern, batch)
            ref = 2.0 * _oracle(x, w, False) + bias.numpy()[None, :]
            err = ko.rel_fro_error(y, ref)
            assert err < 1e-5, (pattern, batch, err)
    x, w = _inputs((1, 16, 16, 3), 32, torch.float32, False, seed=1)   # d = 3 is outside its envelope
    with pytest.raises(kb.KsmmError):
        _run(x, w, (1, 16, 16, 3), False, algo=_lib.KSMM_ALGO_SIMT, config=8)
    kb.check_device()


@pytest.mark.parametrize("bs_last", [True, False])
def test_simt_unaligned_pointers_take_the_scalar_path(bs_last):
    pattern, batch = (2, 12, 8, 1), 36
    x, w = _inputs(pattern, batch, torch.float32, bs_last, seed=5)
    a, b, c, d = pattern
    # views that start 4 bytes into an allocation: 16-byte vector accesses are illegal
    xs = torch.empty(x.numel() + 1, device=DEV)[1:].view(x.shape).copy_(x)
    wk = kb.generate_factor(*pattern, "kernel", w, torch.float32, DEV)
    ws = torch.empty(wk.numel() + 1, device=DEV)[1:].view(wk.shape).copy_(wk)
    out = torch.empty((a * b * d) * batch + 1, device=DEV)[1:].view(
        (a * b * d, batch) if bs_last else (batch, a * b * d))
    y = kb.forward_ex(xs, ws, bs_last, a, b, c, d, out=out)
    assert ko.rel_fro_error(y.cpu().numpy(), _oracle(x, w, bs_last)) < 1e-5


# ---------------------------------------------------------------------------
# 3. tensor-core family
# ---------------------------------------------------------------------------
TC_PATTERNS_LAST = [(1, 64, 64, 1), (2, 128, 32, 2), (1, 192, 192, 1), (4, 64, 64, 4),
                    (1, 768, 192, 2), (1, 192, 768, 4), (3, 48, 80, 2), (1, 136, 72, 3)]
TC_PATTERNS_FIRST = [(1, 64, 64, 1), (2, 128, 32, 1), (4, 192, 192, 1), (16, 64, 64, 1),
                     (1, 768, 192, 1), (3, 48, 80, 1), (1, 136, 72, 1)]


@pytest.mark.parametrize("config", range(5))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tc_family_batch_last(config, dtype):
    for pi, pattern in enumerate(TC_PATTERNS_LAST):
        for batch in (8, 136, 520):
            x, w = _inputs(pattern, batch, dtype, True, seed=200 + pi)
            y = _run(x, w, pattern, True, algo=_lib.KSMM_ALGO_TC, config=config)
            assert not np.isnan(y).any(), (pattern, batch)
            err = ko.rel_fro_error(y, _oracle(x, w, True))
            assert err < TOL[dtype], (pattern, batch, config, err)
    kb.check_device()


@pytest.mark.parametrize("config", range(5))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tc_family_batch_first(config, dtype):
    for pi, pattern in enumerate(TC_PATTERNS_FIRST):
        for batch in (8, 136, 520):
            x, w = _inputs(pattern, batch, dtype, False, seed=300 + pi)
            y = _run(x, w, pattern, False, algo=_lib.KSMM_ALGO_TC, config=config)
            assert not np.isnan(y).any(), (pattern, batch)
            err = ko.rel_fro_error(y, _oracle(x, w, False))
            assert err < TOL[dtype], (pattern, batch, config, err)
    kb.check_device()


TC_PATTERNS_FIRST_D = [(1, 64, 64, 2), (2, 128, 32, 4), (1, 768, 192, 4), (1, 192, 768, 4),
                       (1, 768, 192, 2), (3, 48, 80, 2), (1, 136, 72, 4), (4, 64, 64, 4), (2, 8, 200, 4)]


@pytest.mark.parametrize("config", [0, 1])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tc_family_batch_first_interleaved_blocks(dtype, config):
    """Batch-first with d = 2 or 4.  Configuration 0: in-kernel split of the interleaved input by
    block; configuration 1: a regrouping pass, then a kernel whose input tiles are plain TMA tiles."""
    for pi, pattern in enumerate(TC_PATTERNS_FIRST_D):
        for batch in (8, 136, 520):
            x, w = _inputs(pattern, batch, dtype, False, seed=400 + pi)
            y = _run(x, w, pattern, False, algo=_lib.KSMM_ALGO_TC, config=config)
            assert not np.isnan(y).any(), (pattern, batch)
            err = ko.rel_fro_error(y, _oracle(x, w, False))
            assert err < TOL[dtype], (pattern, batch, err)
    kb.check_device()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_batch_first_layout_conversion_path(dtype):
    """Batch-first factors with a d that no direct kernel covers (12, 6: neither 2, 4 nor a multiple of 8) run as
    transpose -> batch-last kernel -> transpose, with bias and scale in the kernel's epilogue."""
    rng = np.random.RandomState(3)
    for pi, pattern in enumerate([(1, 64, 64, 12), (2, 128, 32, 6), (1, 72, 48, 6)]):
        for batch in (40, 520):
            x, w = _inputs(pattern, batch, dtype, False, seed=500 + pi)
            a, b, c, d = pattern
            bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32)).to(dtype)
            before = kb.launch_count()
            y = _run(x, w, pattern, False, bias=bias.to(DEV), alpha=0.5)
            assert kb.launch_count() - before == 3          # transpose, kernel, transpose
            ref = 0.5 * _oracle(x, w, False) + bias.float().numpy()[None, :]
            assert ko.rel_fro_error(y, ref) < TOL[dtype], (pattern, batch)
    kb.check_device()


F32_TC_LAST = [(1, 64, 64, 1), (2, 128, 32, 4), (1, 768, 192, 4), (6, 64, 64, 1), (3, 96, 80, 2),
               (1, 160, 72, 4), (1, 64, 64, 16), (1, 192, 768, 2), (2, 32, 200, 3), (2, 96, 40, 2),
               (1, 128, 224, 2)]   # the last one takes the 128-column tile (operands from shared memory)
F32_TC_FIRST = [(1, 64, 64, 1), (4, 192, 192, 1), (3, 96, 80, 1), (2, 64, 48, 1), (6, 64, 64, 1),
                (1, 224, 100, 1), (1, 768, 192, 1), (2, 96, 40, 1)]


@pytest.mark.parametrize("bs_last", [True, False])
def test_tc_family_fp32_split_into_three_tf32_products(bs_last):
    """fp32 factors on the tensor cores (hi*hi + lo*hi + hi*lo in tf32, fp32 accumulate).  The
    specification's fp32 tolerance is 1e-5; the three-term split has to stay near fp32 rounding
    (a single tf32 product would sit at about 5e-4), so the test asks for 3e-6 (measured: 5e-7 to 8e-7
    for c <= 192, 2e-6 for c = 768, where the truncating accumulator shows)."""
    for pi, pattern in enumerate(F32_TC_LAST if bs_last else F32_TC_FIRST):
        for batch in ((32, 160, 544) if bs_last else (8, 136, 520)):   # batch-last: multiples of 32
            x, w = _inputs(pattern, batch, torch.float32, bs_last, seed=600 + pi)
            y = _run(x, w, pattern, bs_last, algo=_lib.KSMM_ALGO_TC, config=0)
            assert not np.isnan(y).any(), (pattern, batch)
            err = ko.rel_fro_error(y, _oracle(x, w, bs_last))
            assert err < 3e-6, (pattern, batch, err)
    kb.check_device()


@pytest.mark.parametrize("config", [1, 2, 3])
def test_tc_family_fp32_forced_j_tiles(config):
    """Configurations 1..3 of the fp32 tensor kernel force j tiles of 128, 96 and 64 columns (the
    tuner's candidates); every form has to give the result of configuration 0."""
    cases = [((1, 768, 192, 4), True, 544), ((1, 192, 768, 2), True, 160), ((2, 96, 40, 2), True, 96),
             ((4, 192, 192, 1), False, 136), ((1, 224, 100, 1), False, 520)]
    for pi, (pattern, bs_last, batch) in enumerate(cases):
        x, w = _inputs(pattern, batch, torch.float32, bs_last, seed=670 + pi)
        y = _run(x, w, pattern, bs_last, algo=_lib.KSMM_ALGO_TC, config=config)
        assert ko.rel_fro_error(y, _oracle(x, w, bs_last)) < 3e-6, (pattern, bs_last, config)
    kb.check_device()


def test_tc_family_fp32_resident_weights_across_block_changes():
    """Batch-last fp32 with short blocks keeps a block's weights in shared memory; with more
    (block, batch tile) pairs than CTAs, CTAs walk over block boundaries and reload them."""
    for pi, (pattern, batch) in enumerate([((8, 96, 32, 1), 5120), ((2, 192, 96, 3), 9600)]):
        x, w = _inputs(pattern, batch, torch.float32, True, seed=650 + pi)
        rng = np.random.RandomState(660 + pi)
        a, b, c, d = pattern
        bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32))
        y = _run(x, w, pattern, True, algo=_lib.KSMM_ALGO_TC, config=0, bias=bias.to(DEV), alpha=0.5)
        ref = 0.5 * _oracle(x, w, True) + bias.numpy()[:, None]
        assert ko.rel_fro_error(y, ref) < 3e-6, pattern
    kb.check_device()


def test_tc_refuses_what_it_cannot_run():
    x, w = _inputs((1, 64, 64, 3), 16, torch.float16, False, seed=1)  # batch-first with d = 3
    with pytest.raises(kb.KsmmError) as ei:
        _run(x, w, (1, 64, 64, 3), False, algo=_lib.KSMM_ALGO_TC, config=0)
    assert ei.value.status == _lib.KSMM_ERR_UNSUPPORTED
    x, w = _inputs((1, 64, 64, 2), 16, torch.float32, False, seed=1)  # fp32 batch-first with d = 2
    with pytest.raises(kb.KsmmError):
        _run(x, w, (1, 64, 64, 2), False, algo=_lib.KSMM_ALGO_TC, config=0)


@pytest.mark.parametrize("bs_last", [True, False])
def test_bias_and_alpha_epilogue(bs_last):
    for dtype, algo in ((torch.float32, _lib.KSMM_ALGO_SIMT), (torch.float32, _lib.KSMM_ALGO_TC),
                        (torch.float16, _lib.KSMM_ALGO_SIMT),
                        (torch.float16, _lib.KSMM_ALGO_TC), (torch.bfloat16, _lib.KSMM_ALGO_TC)):
        pattern, batch = (2, 96, 48, 1), 96
        x, w = _inputs(pattern, batch, dtype, bs_last, seed=9)
        rng = np.random.RandomState(10)
        bias = torch.from_numpy(rng.standard_normal(2 * 96).astype(np.float32)).to(dtype)
        y = _run(x, w, pattern, bs_last, algo=algo, bias=bias.to(DEV), alpha=0.5)
        ref = 0.5 * _oracle(x, w, bs_last)
        bf = bias.float().numpy()
        ref = ref + (bf[:, None] if bs_last else bf[None, :])
        assert ko.rel_fro_error(y, ref) < TOL[dtype], (dtype, algo)


# ---------------------------------------------------------------------------
# 4. fp8-e4m3 with per-tensor scales and fp32 accumulation
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("pattern", [(4, 192, 192, 1), (1, 768, 192, 4), (1, 192, 768, 4)])
@pytest.mark.parametrize("algo", [_lib.KSMM_ALGO_TC, _lib.KSMM_ALGO_SIMT])
def test_fp8_factor(pattern, algo):
    batch, bs_last = 512, True
    x, w = _inputs(pattern, batch, torch.float32, bs_last, seed=40)
    a, b, c, d = pattern
    wk = kb.generate_factor(a, b, c, d, "kernel", w, torch.float32, DEV)
    xq, sx = kb.quantize_e4m3(x.to(DEV))
    wq, sw = kb.quantize_e4m3(wk)
    ref_full = _oracle(x, w, bs_last)                       # unquantised fp32 dense result
    xq_f = xq.float().cpu().numpy()
    wq_abcd = ko.kernel_format_to_abcd(wq.float().cpu().numpy(), pattern)
    ref_q = sx * sw * ko.factor_apply(xq_f, wq_abcd, bs_last)  # exact result on the quantised values
    for out_dtype, tol_q in ((torch.bfloat16, 1e-2), (torch.float32, 1e-5)):
        y = kb.forward_fp8(xq, wq, bs_last, a, b, c, d, sx, sw, out_dtype=out_dtype, algo=algo)
        y = y.float().cpu().numpy()
        assert ko.rel_fro_error(y, ref_q) < tol_q, (pattern, out_dtype)
        assert ko.rel_fro_error(y, ref_full) < 5e-2, (pattern, out_dtype)
    kb.check_device()


def test_fp8_kslinear_chain():
    pats = [(4, 192, 192, 1), (1, 768, 192, 4)]
    rng = np.random.RandomState(41)
    ws = make_weights(pats, rng)
    x = rng.standard_normal((768, 256)).astype(np.float32)
    layer = kb.KSLinear(pats, weights=[torch.from_numpy(w) for w in ws], bias=False, algo="kernel",
                        dtype=torch.float8_e4m3fn, bs_last=True, device=DEV)
    y = layer(torch.from_numpy(x).to(DEV).to(torch.bfloat16))
    ref = ko.chain_apply(x, ws, True)
    assert ko.rel_fro_error(y.float().cpu().numpy(), ref) < 5e-2 * math.sqrt(2)


# ---------------------------------------------------------------------------
# 5. full benchmark batch (25088): size-independent properties
# ---------------------------------------------------------------------------
FULL_B = 25088
FULL_PATTERNS = [(6, 64, 64, 1), (1, 768, 192, 2), (4, 192, 192, 1), (1, 768, 192, 4),
                 (1, 192, 768, 4), (1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)]


@pytest.mark.parametrize("bs_last", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_full_batch_sampled_columns_against_oracle(dtype, bs_last):
    g = torch.Generator(device="cpu").manual_seed(77)
    cols = np.unique(np.concatenate([np.arange(0, 8), np.arange(FULL_B - 8, FULL_B),
                                     np.random.RandomState(1).randint(0, FULL_B, 48)]))
    for pattern in FULL_PATTERNS:
        a, b, c, d = pattern
        shape = (a * c * d, FULL_B) if bs_last else (FULL_B, a * c * d)
        x = torch.randn(shape, generator=g).to(dtype)
        w = torch.from_numpy(make_weights([pattern], np.random.RandomState(3))[0]).to(dtype)
        wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
        y = kb.Kernel.forward(x.to(DEV), wk, bs_last, a, b, c, d, dtype)
        ys = (y[:, cols] if bs_last else y[cols]).float().cpu().numpy()
        xs = (x[:, cols] if bs_last else x[cols]).float().numpy()
        err = ko.rel_fro_error(ys, ko.factor_apply(xs, w.float().numpy(), bs_last))
        assert err < TOL[dtype], (pattern, err)
    kb.check_device()


def test_full_batch_linearity_and_determinism_fp32():
    pattern = (1, 768, 192, 2)
    a, b, c, d = pattern
    g = torch.Generator(device="cpu").manual_seed(5)
    x1 = torch.randn((a * c * d, FULL_B), generator=g).to(DEV)
    x2 = torch.randn((a * c * d, FULL_B), generator=g).to(DEV)
    w = torch.from_numpy(make_weights([pattern], np.random.RandomState(4))[0])
    wk = kb.generate_factor(a, b, c, d, "kernel", w, torch.float32, DEV)
    f = lambda t: kb.Kernel.forward(t, wk, True, a, b, c, d, torch.float32)  # noqa: E731
    y1, y2, y12 = f(x1), f(x2), f(x1 + x2)
    rel = (torch.linalg.norm(y12 - (y1 + y2)) / torch.linalg.norm(y12)).item()
    assert rel < 1e-5
    assert torch.equal(f(x1), y1)  # bitwise repeatable


def test_full_batch_families_agree_fp16():
    g = torch.Generator(device="cpu").manual_seed(6)
    for pattern in [(1, 768, 192, 4), (4, 64, 64, 4)]:
        a, b, c, d = pattern
        x = torch.randn((a * c * d, FULL_B), generator=g).half().to(DEV)
        w = torch.from_numpy(make_weights([pattern], np.random.RandomState(4))[0]).half()
        wk = kb.generate_factor(a, b, c, d, "kernel", w, torch.float16, DEV)
        y_tc = kb.forward_ex(x, wk, True, a, b, c, d, algo=_lib.KSMM_ALGO_TC)
        y_ffma = kb.forward_ex(x, wk, True, a, b, c, d, algo=_lib.KSMM_ALGO_SIMT)
        rel = (torch.linalg.norm(y_tc.float() - y_ffma.float()) / torch.linalg.norm(y_ffma.float())).item()
        assert rel < 2e-3, (pattern, rel)   # both round one fp32 sum to fp16
    kb.check_device()


def test_readme_chain_full_batch_fp32():
    pats = [(6, 64, 64, 1), (1, 768, 192, 2)]
    rng = np.random.RandomState(8)
    ws = make_weights(pats, rng)
    g = torch.Generator(device="cpu").manual_seed(9)
    x = torch.randn((384, FULL_B), generator=g)
    layer = kb.KSLinear(pats, weights=[torch.from_numpy(w) for w in ws], bias=False, algo="kernel",
                        dtype=torch.float32, bs_last=True, device=DEV)
    y = layer(x.to(DEV))
    assert tuple(y.shape) == (1536, FULL_B)
    cols = np.random.RandomState(2).randint(0, FULL_B, 64)
    ref = ko.chain_apply(x[:, cols].numpy(), ws, True)
    assert ko.rel_fro_error(y[:, cols].cpu().numpy(), ref) < 1e-5


@pytest.mark.parametrize("bs_last", [True, False])
def test_vit_mlp_chains_full_batch_fp16(bs_last):
    rng = np.random.RandomState(12)
    g = torch.Generator(device="cpu").manual_seed(13)
    for pats in ([(4, 192, 192, 1), (1, 768, 192, 4)], [(1, 192, 768, 4), (4, 192, 192, 1)],
                 [(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)]):
        ws = [w.astype(np.float16) for w in make_weights(pats, rng)]
        n_in = pats[0][0] * pats[0][2] * pats[0][3]
        x = torch.randn((n_in, FULL_B) if bs_last else (FULL_B, n_in), generator=g).half()
        layer = kb.KSLinear(pats, weights=[torch.from_numpy(w) for w in ws], bias=True,
                            algo="kernel", dtype=torch.float16, bs_last=bs_last, device=DEV)
        y = layer(x.to(DEV))
        cols = np.random.RandomState(2).randint(0, FULL_B, 32)
        xs = (x[:, cols] if bs_last else x[cols]).float().numpy()
        ref = ko.chain_apply(xs, [w.astype(np.float64) for w in ws], bs_last,
                             bias=layer.bias.float().cpu().numpy(), round_to=np.float16)
        ys = (y[:, cols] if bs_last else y[cols]).float().cpu().numpy()
        assert ko.rel_fro_error(ys, ref) < 1e-2, pats
    kb.check_device()


# ---------------------------------------------------------------------------
# 6. C ABI called directly: host-buffer entry point, tuner, edge cases
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_chain_layout_fusion_batch_first(dtype):
    """Batch-first chains in which a d = 1 factor is followed by a d = 2 / 4 factor: the intermediate is
    stored regrouped by the next factor's blocks (no transposer stage, no regrouping pass), so the
    chain is one launch per factor.  Checked against the oracle, with a bias on the last factor."""
    chains = [[(4, 192, 192, 1), (1, 768, 192, 4)],
              [(2, 128, 64, 1), (1, 128, 128, 2)],
              [(1, 64, 64, 1), (1, 96, 16, 4)],
              [(2, 64, 64, 1), (1, 128, 32, 4), (4, 64, 128, 1)]]
    for ci, pats in enumerate(chains):
        for batch in (40, 520):
            rng = np.random.RandomState(700 + ci)
            ws = make_weights(pats, rng)
            n_in = pats[0][0] * pats[0][2] * pats[0][3]
            n_out = pats[-1][0] * pats[-1][1] * pats[-1][3]
            x = torch.from_numpy(rng.standard_normal((batch, n_in)).astype(np.float32)).to(dtype)
            bias = torch.from_numpy(rng.standard_normal(n_out).astype(np.float32)).to(dtype)
            wt = [torch.from_numpy(w).to(dtype) for w in ws]
            layer = kb.KSLinear(pats, weights=wt, bias=True, algo="kernel", dtype=dtype, bs_last=False,
                                device=DEV)
            with torch.no_grad():
                layer.bias.copy_(bias.to(DEV).reshape(layer.bias.shape))
            before = kb.launch_count()
            y = layer(x.to(DEV)).float().cpu().numpy()
            # one launch per factor; a plan that changes the layout at the chain's end adds a transpose
            assert len(pats) <= kb.launch_count() - before <= len(pats) + 1, (pats, kb.launch_count() - before)
            # oracle on the values the GPU sees (intermediates exact; the 16-bit storage of the
            # intermediates is well inside the tolerance)
            ref = ko.chain_apply(x.float().numpy(), [w.float().numpy() for w in wt], False)
            ref = ref + bias.float().numpy()[None, :]
            assert not np.isnan(y).any()
            assert ko.rel_fro_error(y, ref) < TOL[dtype], (pats, batch)
    kb.check_device()


def _act_ref(y, act):
    if act == "gelu":
        erf = np.vectorize(math.erf)
        return 0.5 * y * (1.0 + erf(y / math.sqrt(2.0)))
    return np.maximum(y, 0.0)


@pytest.mark.parametrize("act", ["gelu", "relu"])
def test_activation_in_the_epilogue(act):
    """act(alpha * K x + bias) on every kernel path: tensor kernels apply it in their epilogue, the
    FFMA family through an element-wise pass after the kernel."""
    cases = [((2, 96, 48, 1), torch.float16, True, _lib.KSMM_ALGO_TC), ((2, 96, 48, 1), torch.float16, False, _lib.KSMM_ALGO_TC),
             ((1, 128, 32, 4), torch.bfloat16, False, _lib.KSMM_ALGO_TC),       # interleaved batch-first kernel
             ((2, 96, 48, 1), torch.float32, True, _lib.KSMM_ALGO_TC), ((2, 96, 48, 1), torch.float32, False, _lib.KSMM_ALGO_TC),
             ((2, 72, 48, 2), torch.float32, True, _lib.KSMM_ALGO_SIMT), ((2, 72, 48, 2), torch.float16, False, _lib.KSMM_ALGO_SIMT),
             ((1, 64, 64, 16), torch.float16, False, _lib.KSMM_ALGO_AUTO)]    # layout-conversion path
    for ci, (pattern, dtype, bs_last, algo) in enumerate(cases):
        batch = 96
        x, w = _inputs(pattern, batch, dtype, bs_last, seed=800 + ci)
        rng = np.random.RandomState(810 + ci)
        a, b, c, d = pattern
        bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32)).to(dtype)
        y = _run(x, w, pattern, bs_last, algo=algo, bias=bias.to(DEV), alpha=0.5, activation=act)
        ref = 0.5 * _oracle(x, w, bs_last)
        bf = bias.float().numpy()
        ref = _act_ref(ref + (bf[:, None] if bs_last else bf[None, :]), act)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert ko.rel_fro_error(y, ref) < tol, (pattern, dtype, bs_last, algo, act)
    # a chain: the activation follows the last factor only
    pats = [(4, 192, 192, 1), (1, 768, 192, 4)]
    rng = np.random.RandomState(820)
    ws = make_weights(pats, rng)
    x = torch.from_numpy(rng.standard_normal((136, 768)).astype(np.float32)).half()
    wt = [torch.from_numpy(v).half() for v in ws]
    layer = kb.KSLinear(pats, weights=wt, bias=False, algo="kernel", dtype=torch.float16, bs_last=False,
                        device=DEV, activation=act)
    y = layer(x.to(DEV)).float().cpu().numpy()
    ref = _act_ref(ko.chain_apply(x.float().numpy(), [v.float().numpy() for v in wt], False), act)
    assert ko.rel_fro_error(y, ref) < 1e-2
    kb.check_device()


GRID = [16, 48, 64, 96, 128, 192, 384, 768]


@pytest.mark.parametrize("bs_last", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_synthetic_pattern_grid_through_the_default_dispatch(dtype, bs_last):
    """The synthetic patterns of the benchmark specification: b, c in {16, ..., 768} with a and d chosen
    so that a*c*d is 768 or 3072, both layouts, whatever kernel the default dispatch picks
    (tensor-core kernels, layout conversion, FFMA kernels), at a batch that the tensor-core
    kernels accept (96) and one that sends fp32 batch-last to the FFMA family (40)."""
    rng = np.random.RandomState(900)
    for c in GRID:
        for b in GRID:
            total = 3072 if (GRID.index(b) + GRID.index(c)) % 2 else 768
            if total % c:
                continue
            rest = total // c                      # a * d
            d = 4 if rest % 4 == 0 and (GRID.index(b) % 2 == 0) else (2 if rest % 2 == 0 and GRID.index(c) % 3 == 0 else 1)
            a = rest // d
            pattern = (a, b, c, d)
            for batch in (96, 40):
                shape = (a * c * d, batch) if bs_last else (batch, a * c * d)
                x = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dtype)
                w = torch.from_numpy(make_weights([pattern], rng)[0]).to(dtype)
                y = _run(x, w, pattern, bs_last)
                assert not np.isnan(y).any(), (pattern, batch)
                err = ko.rel_fro_error(y, _oracle(x, w, bs_last))
                assert err < TOL[dtype], (pattern, batch, err)
    kb.check_device()


def test_standalone_driver_writes_the_reference_row(tmp_path):
    """ksmm_cli: the stand-alone driver with the reference's sparse_mm flags times the library on one
    pattern, checks 1 % of the batch on the CPU and appends `batch a b c d ... ms std mse`."""
    import subprocess
    exe = os.path.join(os.path.dirname(_lib.LIB_PATH), "ksmm_cli")
    assert os.path.exists(exe), "ksmm_cli is built next to libksmm_cu.so by `make -C ksmm_b200/csrc`"
    for kernel, pat in (("kernel_bs_last_float", "2,64,32,2"), ("kernel_bs_first_half", "1,128,64,4"),
                        ("kernel_bs_last_bf16", "4,64,64,1")):
        out = tmp_path / (kernel + ".out")
        res = subprocess.run([exe, "-n", kernel, "-p", pat, "-b", "2048", "-r", "5", "-o", str(out)],
                             capture_output=True, text=True, cwd=str(tmp_path), timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        row = out.read_text().split()
        assert row[:5] == ["2048"] + pat.split(",") and len(row) == 14
        assert float(row[11]) > 0 and float(row[13]) < 1e-2


def test_chain_forward_host_buffers():
    lib = _lib.load()
    pats = [(2, 8, 4, 2), (4, 6, 4, 2)]
    rng = np.random.RandomState(21)
    ws = make_weights(pats, rng)
    # 50: one slice; 8500: four slices through the copy / compute / copy pipeline, ragged last slice
    for bs_last, batch in ((1, 50), (0, 50), (1, 8500), (0, 8500)):
        x = rng.standard_normal((16, batch) if bs_last else (batch, 16)).astype(np.float32)
        bias = rng.standard_normal(48).astype(np.float32)
        wk = [ko.abcd_to_kernel_format(w) for w in ws]
        y = np.full((48, batch) if bs_last else (batch, 48), np.nan, dtype=np.float32)
        vals = (ctypes.c_void_p * 2)(*[w.ctypes.data for w in wk])
        flat = _lib.int32_array([v for p in pats for v in p])
        for _ in range(2):  # second call reuses the library's device buffers
            st = lib.ksmm_cu_chain_forward_host(x.ctypes.data, vals, y.ctypes.data, bias.ctypes.data,
                                                batch, 2, flat, _lib.KSMM_F32, bs_last, 0)
            _lib.check(st)
            ref = ko.chain_apply(x, ws, bool(bs_last), bias=bias)
            assert ko.rel_fro_error(y, ref) < 1e-5


def test_tuner_picks_a_working_candidate():
    lib = _lib.load()
    pattern, batch = (2, 128, 64, 2), 2048
    a, b, c, d = pattern
    for dtype in (torch.float32, torch.float16):
        x, w = _inputs(pattern, batch, dtype, True, seed=31)
        xg = x.to(DEV)
        wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
        out = torch.empty((a * b * d, batch), dtype=dtype, device=DEV)
        code = kb.kernel.dtype_code(dtype)
        desc = _lib.ForwardDesc(input=xg.data_ptr(), values=wk.data_ptr(), output=out.data_ptr(),
                                bias=None, batch=batch, a=a, b=b, c=c, d=d, in_dtype=code,
                                out_dtype=code, bs_last=1, algo=0, config=-1, alpha=1.0)
        algo, cfg, ms = ctypes.c_int(), ctypes.c_int(), ctypes.c_float()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(lib.ksmm_cu_tune(ctypes.byref(desc), 5, stream, ctypes.byref(algo),
                                    ctypes.byref(cfg), ctypes.byref(ms)))
        assert algo.value in (_lib.KSMM_ALGO_SIMT, _lib.KSMM_ALGO_TC) and ms.value > 0
        ga, gc = ctypes.c_int(), ctypes.c_int()
        assert lib.ksmm_cu_get_choice(batch, a, b, c, d, code, code, 1, ctypes.byref(ga),
                                      ctypes.byref(gc)) == 0
        assert (ga.value, gc.value) == (algo.value, cfg.value)
        y = kb.Kernel.forward(xg, wk, True, a, b, c, d, dtype)  # now served by the cached choice
        assert ko.rel_fro_error(y.float().cpu().numpy(), _oracle(x, w, True)) < TOL[dtype]


def test_edge_batches():
    for dtype in (torch.float32, torch.float16):
        for bs_last in (True, False):
            pattern = (2, 16, 8, 1)
            a, b, c, d = pattern
            _, w = _inputs(pattern, 4, dtype, bs_last, seed=1)
            wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
            for batch in (0, 1, 2):
                shape = (a * c * d, batch) if bs_last else (batch, a * c * d)
                x = torch.randn(shape).to(dtype)
                y = kb.Kernel.forward(x.to(DEV), wk, bs_last, a, b, c, d, dtype)
                assert tuple(y.shape) == ((a * b * d, batch) if bs_last else (batch, a * b * d))
                if batch:
                    assert ko.rel_fro_error(y.float().cpu().numpy(), _oracle(x, w, bs_last)) < TOL[dtype]


def test_ffma_peak_probe_and_launch_counter():
    lib = _lib.load()
    before = kb.launch_count()
    x, w = _inputs((1, 16, 16, 1), 32, torch.float32, True, seed=2)
    _run(x, w, (1, 16, 16, 1), True)
    assert kb.launch_count() == before + 1
    tf = ctypes.c_float()
    _lib.check(lib.ksmm_cu_measure_ffma_peak(ctypes.byref(tf), None))
    assert 20.0 < tf.value < 120.0   # B200: 148 SMs x 128 lanes x 2 flop x ~1.9 GHz ~ 72
    kb.check_device()


# ---------------------------------------------------------------------------
# 7. fp8 / bf16 at the sizes of the benchmark specification; KS-ViT-B against dense factors
# ---------------------------------------------------------------------------
def test_fp8_batch_first_on_the_tensor_kernel():
    """fp8-e4m3 batch-first, d = 1, on the tcgen05 kernel (kind::f8f6f4, K-major input operand):
    every tile configuration that accepts 8-bit inputs, both output types."""
    for pi, pattern in enumerate([(4, 192, 192, 1), (1, 768, 192, 1), (16, 64, 64, 1), (3, 48, 80, 1)]):
        a, b, c, d = pattern
        for batch in (136, 520):
            x, w = _inputs(pattern, batch, torch.float32, False, seed=440 + pi)
            wk = kb.generate_factor(a, b, c, d, "kernel", w, torch.float32, DEV)
            xq, sx = kb.quantize_e4m3(x.to(DEV))
            wq, sw = kb.quantize_e4m3(wk)
            ref_full = _oracle(x, w, False)
            wq_abcd = ko.kernel_format_to_abcd(wq.float().cpu().numpy(), pattern)
            ref_q = sx * sw * ko.factor_apply(xq.float().cpu().numpy(), wq_abcd, False)
            for config in range(4):
                for out_dtype, tol_q in ((torch.bfloat16, 1e-2), (torch.float32, 1e-5)):
                    y = kb.forward_fp8(xq, wq, False, a, b, c, d, sx, sw, out_dtype=out_dtype,
                                       algo=_lib.KSMM_ALGO_TC, config=config).float().cpu().numpy()
                    assert ko.rel_fro_error(y, ref_q) < tol_q, (pattern, batch, config, out_dtype)
                    assert ko.rel_fro_error(y, ref_full) < 5e-2, (pattern, batch, config, out_dtype)
    kb.check_device()


@pytest.mark.parametrize("batch", [25088, 4096])
@pytest.mark.parametrize("pattern", [(4, 192, 192, 1), (1, 768, 192, 4), (1, 192, 768, 4)])
def test_fp8_and_bf16_at_the_specified_batches_against_the_oracle(pattern, batch):
    """Per-tensor scale amax / 448, values cast after scaling, fp32 accumulation; the error is
    measured against the fp64 oracle on the unquantised fp32 inputs (sampled columns): 5e-2 for
    fp8-e4m3, 1e-2 for bf16.  Batch-last for every pattern, batch-first as well where d = 1."""
    a, b, c, d = pattern
    g = torch.Generator(device=DEV).manual_seed(91)
    x = torch.randn((a * c * d, batch), generator=g, device=DEV)
    w = (torch.rand((a, b, c, d), generator=g, device=DEV) * 2 - 1) / math.sqrt(c)
    cols = np.unique(np.concatenate([np.arange(0, 4), np.arange(batch - 4, batch),
                                     np.random.RandomState(6).randint(0, batch, 56)]))
    cols_t = torch.from_numpy(cols).to(DEV)
    ref = ko.factor_apply(x[:, cols_t].cpu().numpy(), w.cpu().numpy(), True)
    wk32 = kb.generate_factor(a, b, c, d, "kernel", w, torch.float32, DEV)
    xq, sx = kb.quantize_e4m3(x)
    wq, sw = kb.quantize_e4m3(wk32)
    layouts = (True, False) if d == 1 else (True,)
    for bs_last in layouts:
        xin = xq if bs_last else xq.t().contiguous()
        y = kb.forward_fp8(xin, wq, bs_last, a, b, c, d, sx, sw, out_dtype=torch.bfloat16)
        ys = (y[:, cols_t] if bs_last else y[cols_t].t()).float().cpu().numpy()
        assert ko.rel_fro_error(ys, ref) < 5e-2, (pattern, batch, bs_last, "fp8")
    wkb = kb.generate_factor(a, b, c, d, "kernel", w, torch.bfloat16, DEV)
    xb = x.to(torch.bfloat16)
    for bs_last in (True, False):
        xin = xb if bs_last else xb.t().contiguous()
        y = kb.Kernel.forward(xin, wkb, bs_last, a, b, c, d, torch.bfloat16)
        ys = (y[:, cols_t] if bs_last else y[cols_t].t()).float().cpu().numpy()
        assert ko.rel_fro_error(ys, ref) < 1e-2, (pattern, batch, bs_last, "bf16")
    kb.check_device()


def _dense_twin(model):
    """The same KS-ViT-B with every KSLinear replaced by an nn.Linear holding the dense product of
    its factors (KSLinear.get_dense_product) and its bias."""
    import copy

    from ksmm_b200.ksvit import KSFeedForward
    twin = copy.deepcopy(model)
    for m in twin.modules():
        if isinstance(m, KSFeedForward):
            for name in ("fc1", "fc2"):
                ks = getattr(m, name)
                lin = torch.nn.Linear(ks.in_size, ks.out_size, bias=True, device=DEV, dtype=torch.float32)
                with torch.no_grad():
                    lin.weight.copy_(ks.get_dense_product())
                    lin.bias.copy_(ks.bias.float().reshape(-1))
                setattr(m, name, lin)
            m.fuse_gelu = False
            m.layout_plan = False
            m.dense = True
    return twin.float()


def test_ks_vit_b_block_and_forward_against_dense_factors():
    """KS-ViT-B/16 in fp16 against the same network in fp32 whose MLP projections are dense
    matrices built from the same factors: one encoder block at 25088 tokens (128 images) and the
    12-layer forward at 8 images, relative Frobenius error below 1e-2."""
    from ksmm_b200.ksvit import KSViTB
    torch.manual_seed(3)
    model = KSViTB(dtype=torch.float16, device=DEV).eval()
    twin = _dense_twin(model).eval()
    with torch.no_grad():
        x = torch.randn(128, 196, 768, device=DEV)
        attn, ff = model.layers[0]
        attn32, ff32 = twin.layers[0]
        h16 = attn(x.half()) + x.half()
        y16 = ff(h16) + h16
        h32 = attn32(x) + x
        y32 = ff32(h32) + h32
        err = (torch.linalg.norm(y16.float() - y32) / torch.linalg.norm(y32)).item()
        assert err < 1e-2, err
        # the MLP alone, on identical inputs
        m16 = ff(h16).float()
        m32 = ff32(h16.float())
        err = (torch.linalg.norm(m16 - m32) / torch.linalg.norm(m32)).item()
        assert err < 1e-2, err
        img = torch.randn(8, 3, 224, 224, device=DEV)
        l16 = model(img.half()).float()
        l32 = twin(img)
        err = (torch.linalg.norm(l16 - l32) / torch.linalg.norm(l32)).item()
        assert err < 1e-2, err
    kb.check_device()


# ---------------------------------------------------------------------------
# 8. robustness of the boundary
# ---------------------------------------------------------------------------
def test_bounded_wait_runs_out_and_is_reported():
    """A wait that nothing will ever satisfy gives up after its limit, the kernel returns, and the
    host reads KSMM_ERR_DEVICE_TIMEOUT from ksmm_cu_check_device; the context stays usable and the
    flag is cleared by the read."""
    lib = _lib.load()
    kb.check_device()                                           # clean start
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.ksmm_cu_debug_wait_probe(2_000_000, stream))  # about one millisecond of SM clock
    st = lib.ksmm_cu_check_device(stream)
    assert st == _lib.KSMM_ERR_DEVICE_TIMEOUT
    assert b"code 99" in lib.ksmm_cu_last_error()
    assert lib.ksmm_cu_check_device(stream) == _lib.KSMM_OK     # cleared
    x, w = _inputs((2, 96, 48, 1), 96, torch.float16, True, seed=3)
    y = _run(x, w, (2, 96, 48, 1), True)                        # the device still works
    assert ko.rel_fro_error(y, _oracle(x, w, True)) < 1e-2
    kb.check_device()


def test_tuner_times_the_conversion_path_and_unaligned_calls_fall_back():
    """Tuning a batch-first factor that no direct tensor kernel covers must not pin a slower kernel
    than the default (the conversion path is a candidate), and a choice tuned on aligned buffers
    must not make a later call on an unaligned buffer fail."""
    lib = _lib.load()
    pattern, batch, dtype = (1, 64, 64, 16), 8192, torch.float16
    a, b, c, d = pattern
    x, w = _inputs(pattern, batch, dtype, False, seed=33)
    xg = x.to(DEV)
    wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
    out = torch.empty((batch, a * b * d), dtype=dtype, device=DEV)
    code = kb.kernel.dtype_code(dtype)

    def timed(n=20):
        kb.forward_ex(xg, wk, False, a, b, c, d, out=out)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            kb.forward_ex(xg, wk, False, a, b, c, d, out=out)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / n

    t_default = timed()
    desc = _lib.ForwardDesc(input=xg.data_ptr(), values=wk.data_ptr(), output=out.data_ptr(), bias=None,
                            batch=batch, a=a, b=b, c=c, d=d, in_dtype=code, out_dtype=code, bs_last=0,
                            algo=0, config=-1, alpha=1.0)
    algo, cfg, ms = ctypes.c_int(), ctypes.c_int(), ctypes.c_float()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.ksmm_cu_tune(ctypes.byref(desc), 10, stream, ctypes.byref(algo), ctypes.byref(cfg),
                                ctypes.byref(ms)))
    t_tuned = timed()
    assert t_tuned < 1.25 * t_default, (t_tuned, t_default, algo.value, cfg.value)
    y = kb.forward_ex(xg, wk, False, a, b, c, d)
    assert ko.rel_fro_error(y.float().cpu().numpy(), _oracle(x, w, False)) < 1e-2
    # pin a TMA-based choice for a batch-last problem, then call with a pointer 2 bytes off 16-byte alignment
    pattern2, batch2 = (2, 64, 32, 1), 256
    a, b, c, d = pattern2
    assert lib.ksmm_cu_set_choice(batch2, a, b, c, d, code, code, 1, _lib.KSMM_ALGO_TC, 1) == 0
    x2, w2 = _inputs(pattern2, batch2, dtype, True, seed=34)
    wk2 = kb.generate_factor(a, b, c, d, "kernel", w2, dtype, DEV)
    xs = torch.empty(x2.numel() + 1, dtype=dtype, device=DEV)[1:].view(x2.shape).copy_(x2)
    y2 = kb.forward_ex(xs, wk2, True, a, b, c, d)
    assert ko.rel_fro_error(y2.float().cpu().numpy(), _oracle(x2, w2, True)) < 1e-2
    kb.check_device()


def test_layout_scratch_from_the_caller_and_per_stream():
    """A batch-first d = 16 factor through the conversion path: with the scratch passed in the
    descriptor the library allocates nothing; without it, calls on two streams get a buffer each
    and may overlap."""
    lib = _lib.load()
    pattern, batch, dtype = (1, 64, 64, 12), 1000, torch.float16
    a, b, c, d = pattern
    x, w = _inputs(pattern, batch, dtype, False, seed=35)
    ref = _oracle(x, w, False)
    xg = x.to(DEV)
    wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
    code = kb.kernel.dtype_code(dtype)
    out = torch.full((batch, a * b * d), float("nan"), dtype=dtype, device=DEV)
    desc = _lib.ForwardDesc(input=xg.data_ptr(), values=wk.data_ptr(), output=out.data_ptr(), bias=None,
                            batch=batch, a=a, b=b, c=c, d=d, in_dtype=code, out_dtype=code, bs_last=0,
                            algo=0, config=-1, alpha=1.0)
    need = lib.ksmm_cu_layout_scratch_bytes(ctypes.byref(desc))
    if need:
        scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
        desc.scratch, desc.scratch_bytes = scratch.data_ptr(), need
    torch.cuda.synchronize()
    allocs = lib.ksmm_cu_alloc_count()
    _lib.check(lib.ksmm_cu_forward_ex(ctypes.byref(desc), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert lib.ksmm_cu_alloc_count() == allocs
    assert ko.rel_fro_error(out.float().cpu().numpy(), ref) < 1e-2
    # two streams, library-owned scratch: interleaved calls, each correct
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for rep in range(4):
        for s in (s1, s2):
            with torch.cuda.stream(s):
                outs.append(kb.forward_ex(xg, wk, False, a, b, c, d))
    torch.cuda.synchronize()
    for y in outs:
        assert ko.rel_fro_error(y.float().cpu().numpy(), ref) < 1e-2
    _lib.check(lib.ksmm_cu_release_scratch())
    kb.check_device()


def test_chain_forward_host_async_tickets():
    """Several host-buffer calls in flight: each is enqueued at once, results are complete after
    the wait on its ticket, in any waiting order, and equal the synchronous call's."""
    lib = _lib.load()
    pats = [(2, 8, 4, 2), (4, 6, 4, 2)]
    rng = np.random.RandomState(23)
    ws = make_weights(pats, rng)
    wk = [ko.abcd_to_kernel_format(w) for w in ws]
    vals = (ctypes.c_void_p * 2)(*[w.ctypes.data for w in wk])
    flat = _lib.int32_array([v for p in pats for v in p])
    calls = []
    for ci, (bs_last, batch) in enumerate(((1, 9000), (0, 50), (0, 17000), (1, 300), (0, 8200), (1, 64))):
        x = torch.from_numpy(rng.standard_normal((16, batch) if bs_last else (batch, 16)).astype(np.float32)).pin_memory()
        y = torch.full((48, batch) if bs_last else (batch, 48), float("nan")).pin_memory()
        calls.append((bs_last, batch, x, y))
    for rep in range(2):
        tickets = []
        for bs_last, batch, x, y in calls:
            y.fill_(float("nan"))
            t = ctypes.c_uint64(0)
            _lib.check(lib.ksmm_cu_chain_forward_host_async(x.data_ptr(), vals, y.data_ptr(), None, batch, 2,
                                                            flat, _lib.KSMM_F32, bs_last, 0, ctypes.byref(t)))
            assert t.value > 0
            tickets.append(t.value)
        assert tickets == sorted(tickets)
        for idx in (reversed(range(len(calls))) if rep else range(len(calls))):
            _lib.check(lib.ksmm_cu_host_wait(tickets[idx]))
            bs_last, batch, x, y = calls[idx]
            ref = ko.chain_apply(x.numpy(), ws, bool(bs_last))
            assert ko.rel_fro_error(y.numpy(), ref) < 1e-5, (rep, idx)
    t = ctypes.c_uint64(7)
    x0 = calls[1][2]
    _lib.check(lib.ksmm_cu_chain_forward_host_async(x0.data_ptr(), vals, calls[1][3].data_ptr(), None, 0, 2, flat,
                                                    _lib.KSMM_F32, 0, 0, ctypes.byref(t)))
    assert t.value == 0 and lib.ksmm_cu_host_wait(0) == _lib.KSMM_OK          # empty batch
    assert lib.ksmm_cu_host_wait(1 << 40) == _lib.KSMM_ERR_BAD_ARGUMENT       # never issued


# ---------------------------------------------------------------------------
# 9. grouped calls: several weight sets of one pattern on one input (q, k, v projections)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bs_last", [True, False])
def test_grouped_forward_shared_and_stacked_inputs(dtype, bs_last):
    lib = _lib.load()
    G = 3
    code = kb.kernel.dtype_code(dtype)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for pi, pattern in enumerate([(1, 768, 768, 1), (6, 128, 128, 1), (2, 96, 48, 2), (1, 64, 64, 4)]):
        a, b, c, d = pattern
        for batch in (512, 136):
            for shared in (1, 0):
                rng = np.random.RandomState(1200 + pi)
                ws = [torch.from_numpy(make_weights([pattern], rng)[0]).to(dtype) for _ in range(G)]
                wk = torch.cat([kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV) for w in ws]).contiguous()
                shape = (a * c * d, batch) if bs_last else (batch, a * c * d)
                xs = [torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dtype)
                      for _ in range(1 if shared else G)]
                xg = torch.stack(xs).contiguous().to(DEV) if not shared else xs[0].to(DEV)
                bias = torch.from_numpy(rng.standard_normal(G * a * b * d).astype(np.float32)).to(dtype)
                oshape = (G, a * b * d, batch) if bs_last else (G, batch, a * b * d)
                out = torch.full(oshape, float("nan"), dtype=dtype, device=DEV)
                before = kb.launch_count()
                _lib.check(lib.ksmm_cu_grouped_forward(xg.data_ptr(), wk.data_ptr(), out.data_ptr(),
                                                       bias.to(DEV).data_ptr(), batch, a, b, c, d, code,
                                                       int(bs_last), G, shared, stream))
                launches = kb.launch_count() - before
                one_launch = dtype != torch.float32 and (bs_last or (d == 1 and batch % 32 == 0))
                if one_launch and b >= 32 and c >= 16:
                    assert launches == 1, (pattern, batch, shared, launches)
                for g in range(G):
                    xq = xs[0] if shared else xs[g]
                    bf = bias.float().numpy()[g * a * b * d:(g + 1) * a * b * d]
                    ref = _oracle(xq, ws[g], bs_last) + (bf[:, None] if bs_last else bf[None, :])
                    y = out[g].float().cpu().numpy()
                    assert not np.isnan(y).any(), (pattern, batch, shared, g)
                    assert ko.rel_fro_error(y, ref) < TOL[dtype], (pattern, batch, shared, g)
    kb.check_device()


@pytest.mark.parametrize("bs_last", [True, False])
def test_kslinear_group_matches_separate_layers(bs_last):
    """q, k, v as one KSLinearGroup: same results as the three layers called one by one, one launch
    per factor instead of three, and the stacked weights follow an in-place update of a layer."""
    pats = [(6, 128, 128, 1), (1, 768, 128, 6)]
    dtype = torch.float16
    torch.manual_seed(5)
    layers = [kb.KSLinear(pats, bias=True, algo="kernel", dtype=dtype, bs_last=bs_last, device=DEV) for _ in range(3)]
    group = kb.KSLinearGroup(layers)
    x = torch.randn((768, 4, 160) if bs_last else (4, 160, 768), device=DEV).to(dtype)
    before = kb.launch_count()
    q, k, v = group(x)
    fused_launches = kb.launch_count() - before
    singles = [l(x) for l in layers]
    for y, ref in zip((q, k, v), singles):
        assert y.shape == ref.shape and y.is_contiguous()
        rel = (torch.linalg.norm(y.float() - ref.float()) / torch.linalg.norm(ref.float())).item()
        assert rel < 2e-3, rel
    if bs_last:
        assert fused_launches == len(pats)           # batch-first: the d = 6 factor runs group by group
    dense = layers[1].get_dense_product()
    xf = x.float().reshape(768, -1) if bs_last else x.float().reshape(-1, 768)
    ref = (dense @ xf + layers[1].bias.float().reshape(-1, 1)) if bs_last else (xf @ dense.t() + layers[1].bias.float())
    rel = (torch.linalg.norm(k.float().reshape(ref.shape) - ref) / torch.linalg.norm(ref)).item()
    assert rel < 1e-2, rel
    with torch.no_grad():
        layers[2].factors[0].mul_(0.5)
    v2 = group(x)[2]
    ref2 = layers[2](x)
    rel = (torch.linalg.norm(v2.float() - ref2.float()) / torch.linalg.norm(ref2.float())).item()
    assert rel < 2e-3, rel
    with pytest.raises(ValueError):
        kb.KSLinearGroup([layers[0], kb.KSLinear([(1, 768, 768, 1)], dtype=dtype, bs_last=bs_last, device=DEV)])
    kb.check_device()


# ---------------------------------------------------------------------------
# 10. backward of one factor
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bs_last", [True, False])
def test_factor_backward_against_the_oracle(dtype, bs_last):
    """dX (the forward kernels on transposed blocks) and dW (tensor-core kernel with the batch
    split over CTAs for 16-bit batch-last and batch-first d = 1; FFMA kernel otherwise)."""
    pats = [(2, 96, 48, 2), (1, 768, 192, 4), (4, 192, 192, 1), (3, 40, 24, 3), (1, 64, 64, 16), (6, 64, 64, 1),
            (1, 200, 136, 1), (2, 8, 300, 1)]
    for pi, pattern in enumerate(pats):
        a, b, c, d = pattern
        for batch in (136, 4104):
            rng = np.random.RandomState(1300 + pi)
            x, w = _inputs(pattern, batch, dtype, bs_last, seed=1300 + pi)
            gshape = (a * b * d, batch) if bs_last else (batch, a * b * d)
            g = torch.from_numpy(rng.standard_normal(gshape).astype(np.float32)).to(dtype)
            wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
            dx = kb.backward_input(g.to(DEV), wk, bs_last, a, b, c, d).float().cpu().numpy()
            ref_dx = ko.factor_grad_input(g.float().numpy(), w.float().numpy(), bs_last)
            assert ko.rel_fro_error(dx, ref_dx) < TOL[dtype], (pattern, batch, "dX")
            dwk = kb.backward_weights(x.to(DEV), g.to(DEV), bs_last, a, b, c, d)
            assert tuple(dwk.shape) == (a * d * c, b) and dwk.dtype == dtype
            ref_dw = ko.abcd_to_kernel_format(ko.factor_grad_weights(x.float().numpy(), g.float().numpy(), pattern, bs_last))
            assert ko.rel_fro_error(dwk.float().cpu().numpy(), ref_dw) < TOL[dtype], (pattern, batch, "dW")
            # repeatable bit for bit (partial sums are added in a fixed order)
            assert torch.equal(dwk, kb.backward_weights(x.to(DEV), g.to(DEV), bs_last, a, b, c, d))
    kb.check_device()


@pytest.mark.parametrize("bs_last", [True, False])
def test_kslinear_trains_through_autograd(bs_last):
    """A two-factor KSLinear with trainable factors and bias: gradients of a scalar loss against torch
    autograd on the dense matrices of the same factors (fp32)."""
    pats = [(4, 192, 192, 1), (1, 768, 192, 4)]
    torch.manual_seed(11)
    layer = kb.KSLinear(pats, bias=True, algo="kernel", dtype=torch.float32, bs_last=bs_last, device=DEV,
                        requires_grad=True)
    x = torch.randn((768, 256) if bs_last else (256, 768), device=DEV, requires_grad=True)
    gy = torch.randn((3072, 256) if bs_last else (256, 3072), device=DEV)
    y = layer(x)
    (y * gy).sum().backward()
    # reference: dense factors rebuilt from 4-D leaves so that autograd reaches (a,b,c,d) weights
    leaves = [kb.from_kernel_format_to_abcd(f.detach(), p).clone().requires_grad_(True)
              for f, p in zip(layer.factors, pats)]
    xr = x.detach().clone().requires_grad_(True)
    br = layer.bias.detach().clone().requires_grad_(True)
    h = xr
    for wl, (a, b, c, d) in zip(leaves, pats):
        blocks = torch.diag_embed(wl).permute(0, 1, 3, 2, 4).reshape(a, b * d, c * d)
        dense = torch.block_diag(*torch.unbind(blocks, dim=0))
        h = dense @ h if bs_last else h @ dense.t()
    yr = h + (br.reshape(-1, 1) if bs_last else br.reshape(1, -1))
    (yr * gy).sum().backward()
    rel = lambda u, v: (torch.linalg.norm(u - v) / torch.linalg.norm(v)).item()  # noqa: E731
    assert rel(y.detach(), yr.detach()) < 1e-5
    assert rel(x.grad, xr.grad) < 1e-5
    assert rel(layer.bias.grad, br.grad) < 1e-5
    for f, wl, p in zip(layer.factors, leaves, pats):
        a, b, c, d = p
        ref = wl.grad.permute(0, 3, 2, 1).reshape(a * d * c, b)
        assert rel(f.grad, ref) < 1e-5, p
    kb.check_device()


# ---------------------------------------------------------------------------
# 11. layouts: factors that read one layout and write the other, planned chains
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("in_last", [True, False])
def test_layout_changing_factor(dtype, in_last):
    """A 16-bit factor with d = 1 as a one-factor chain whose output layout is the other one: the
    tensor kernel reads batch-first rows and writes batch-last rows (or the reverse) in one launch."""
    pats = [(4, 192, 192, 1), (1, 768, 192, 1), (16, 64, 64, 1), (1, 64, 768, 1), (3, 48, 80, 1), (2, 136, 72, 1),
            (1, 32, 16, 1)]
    rng = np.random.RandomState(1400)
    for pi, pattern in enumerate(pats):
        a, b, c, d = pattern
        for batch in (8, 136, 520, 4104):
            x, w = _inputs(pattern, batch, dtype, in_last, seed=1400 + pi)
            bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32)).to(dtype)
            wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, DEV)
            before = kb.launch_count()
            y = kb.chain_forward(x.to(DEV), [wk], [pattern], in_last, bias=bias.to(DEV), out_bs_last=not in_last)
            assert kb.launch_count() - before == 1, (pattern, batch)
            assert tuple(y.shape) == ((batch, a * b * d) if in_last else (a * b * d, batch))
            ref = _oracle(x, w, in_last)
            bf = bias.float().numpy()
            ref = (ref + (bf[:, None] if in_last else bf[None, :])).T
            yy = y.float().cpu().numpy()
            assert not np.isnan(yy).any()
            assert ko.rel_fro_error(yy, ref) < TOL[dtype], (pattern, batch)
    kb.check_device()


@pytest.mark.parametrize("in_last", [True, False])
def test_layout_changing_factor_fp32(in_last):
    """The fp32 tensor kernel's layout-changing forms (d = 1, b a multiple of 32, c of 4, batch of 32):
    one launch, the 96- and 64-column tiles, blocks of one and of many 32-row chunks."""
    pats = [(4, 192, 192, 1), (1, 768, 192, 1), (16, 64, 64, 1), (1, 64, 768, 1), (3, 32, 20, 1), (2, 160, 72, 1),
            (1, 1024, 1024, 1)]
    rng = np.random.RandomState(1450)
    for pi, pattern in enumerate(pats):
        a, b, c, d = pattern
        for batch in (32, 160, 544, 4128):
            x, w = _inputs(pattern, batch, torch.float32, in_last, seed=1450 + pi)
            bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32))
            wk = kb.generate_factor(a, b, c, d, "kernel", w, torch.float32, DEV)
            before = kb.launch_count()
            y = kb.chain_forward(x.to(DEV), [wk], [pattern], in_last, bias=bias.to(DEV), out_bs_last=not in_last,
                                 activation="relu")
            assert kb.launch_count() - before == 1, (pattern, batch)
            assert tuple(y.shape) == ((batch, a * b * d) if in_last else (a * b * d, batch))
            ref = _oracle(x, w, in_last)
            bf = bias.numpy()
            ref = np.maximum(ref + (bf[:, None] if in_last else bf[None, :]), 0.0).T
            yy = y.cpu().numpy()
            assert not np.isnan(yy).any()
            assert ko.rel_fro_error(yy, ref) < 1e-5, (pattern, batch)
    kb.check_device()


def test_planned_chains_mixed_layouts():
    """Chains whose output layout differs from the input's, and batch-first chains that run their
    d > 1 factors batch-last inside: KS-ViT-B's fc1 (batch-first tokens -> batch-last 3072 features,
    GELU fused), fc2 (back), the 3-factor chain (input transposed once, last factor writes
    batch-first), and fp32 chains (a d = 2 factor last: transposed at the end; the MLP layers)."""
    cases = [([(4, 192, 192, 1), (1, 768, 192, 4)], torch.float16, False, True, "gelu", 2),
             ([(1, 192, 768, 4), (4, 192, 192, 1)], torch.float16, True, False, None, 2),
             ([(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)], torch.float16, False, False, None, 4),
             ([(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)], torch.bfloat16, True, False, "relu", 3),
             ([(6, 64, 64, 1), (1, 768, 192, 2)], torch.float32, True, False, None, 3),
             ([(2, 96, 48, 2)], torch.float16, False, True, None, 2),
             # fp32: fc1 / fc2 of the KS-ViT-B MLP between batch-first tokens (first factor changes the
             # layout, the d = 4 factor runs batch-last, one transpose at the end / at the start)
             ([(4, 192, 192, 1), (1, 768, 192, 4)], torch.float32, False, False, "gelu", 3),
             ([(1, 192, 768, 4), (4, 192, 192, 1)], torch.float32, False, False, None, 3),
             ([(4, 192, 192, 1), (1, 768, 192, 4)], torch.float32, False, True, None, 2)]
    for ci, (pats, dtype, in_last, out_last, act, launches) in enumerate(cases):
        for batch in (520, 25088):
            rng = np.random.RandomState(1500 + ci)
            ws = make_weights(pats, rng)
            n_in = pats[0][0] * pats[0][2] * pats[0][3]
            n_out = pats[-1][0] * pats[-1][1] * pats[-1][3]
            x = torch.from_numpy(rng.standard_normal((n_in, batch) if in_last else (batch, n_in)).astype(np.float32)).to(dtype)
            bias = torch.from_numpy(rng.standard_normal(n_out).astype(np.float32)).to(dtype)
            wt = [torch.from_numpy(w).to(dtype) for w in ws]
            wk = [kb.generate_factor(*p, "kernel", w, dtype, DEV) for p, w in zip(pats, wt)]
            before = kb.launch_count()
            y = kb.chain_forward(x.to(DEV), wk, pats, in_last, bias=bias.to(DEV), activation=act,
                                 out_bs_last=out_last)
            used = kb.launch_count() - before
            assert tuple(y.shape) == ((n_out, batch) if out_last else (batch, n_out))
            if batch == 25088:
                assert used == launches, (pats, dtype, used)
            cols = np.arange(batch) if batch <= 520 else np.random.RandomState(3).randint(0, batch, 48)
            xs = (x[:, cols] if in_last else x[cols]).float().numpy()
            ref = ko.chain_apply(xs, [w.float().numpy() for w in wt], in_last, bias=bias.float().numpy(),
                                 round_to=None if dtype == torch.float32 else np.float32)
            if act:
                ref = _act_ref(ref, act)
            if in_last != out_last:
                ref = ref.T
            ct = torch.from_numpy(np.asarray(cols)).to(DEV)
            ys = (y[:, ct] if out_last else y[ct]).float().cpu().numpy()
            assert not np.isnan(ys).any()
            assert ko.rel_fro_error(ys, ref) < TOL[dtype], (pats, dtype, batch)
    kb.check_device()


def test_kslinear_out_layout_option():
    torch.manual_seed(9)
    fc1 = kb.KSLinear([(4, 192, 192, 1), (1, 768, 192, 4)], bias=True, dtype=torch.float16, bs_last=False,
                      device=DEV, out_bs_last=True, activation="gelu")
    fc2 = kb.KSLinear([(1, 192, 768, 4), (4, 192, 192, 1)], bias=True, dtype=torch.float16, bs_last=True,
                      device=DEV, out_bs_last=False)
    x = torch.randn(4, 98, 768, device=DEV).half()
    h = fc1(x)
    assert tuple(h.shape) == (3072, 392)
    y = fc2(h)
    assert tuple(y.shape) == (392, 768)
    d1, d2 = fc1.get_dense_product(), fc2.get_dense_product()
    xr = x.float().reshape(-1, 768)
    hr = torch.nn.functional.gelu(xr @ d1.t() + fc1.bias.float())
    yr = hr @ d2.t() + fc2.bias.float().reshape(-1)
    rel = (torch.linalg.norm(y.float() - yr) / torch.linalg.norm(yr)).item()
    assert rel < 1e-2, rel
    kb.check_device()


def test_residual_in_the_epilogue_and_as_a_pass():
    """out = act(alpha K x + bias) + residual: in the epilogue of the 16-bit tensor kernel (both
    layouts, layout-changing factors included), as a pass after every other kernel."""
    cases = [((2, 96, 48, 1), torch.float16, True, _lib.KSMM_ALGO_TC), ((2, 96, 48, 1), torch.float16, False, _lib.KSMM_ALGO_TC),
             ((1, 200, 72, 3), torch.bfloat16, True, _lib.KSMM_ALGO_TC), ((4, 192, 192, 1), torch.bfloat16, False, _lib.KSMM_ALGO_TC),
             ((1, 128, 32, 4), torch.float16, False, _lib.KSMM_ALGO_TC),      # interleaved batch-first kernel: pass
             ((2, 96, 48, 1), torch.float32, True, _lib.KSMM_ALGO_TC), ((2, 72, 48, 2), torch.float32, False, _lib.KSMM_ALGO_SIMT),
             ((1, 64, 64, 16), torch.float16, False, _lib.KSMM_ALGO_AUTO)]    # layout conversion: pass
    for ci, (pattern, dtype, bs_last, algo) in enumerate(cases):
        for batch in (96, 544):     # (multiples of 32: the fp32 tensor kernel's batch-last rule)
            x, w = _inputs(pattern, batch, dtype, bs_last, seed=1600 + ci)
            rng = np.random.RandomState(1610 + ci)
            a, b, c, d = pattern
            oshape = (a * b * d, batch) if bs_last else (batch, a * b * d)
            bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32)).to(dtype)
            res = torch.from_numpy(rng.standard_normal(oshape).astype(np.float32)).to(dtype)
            y = _run(x, w, pattern, bs_last, algo=algo, bias=bias.to(DEV), alpha=0.5, activation="relu",
                     residual=res.to(DEV))
            bf = bias.float().numpy()
            ref = np.maximum(0.5 * _oracle(x, w, bs_last) + (bf[:, None] if bs_last else bf[None, :]), 0.0)
            ref = ref + res.float().numpy()
            tol = 1e-5 if dtype == torch.float32 else 1e-2
            assert ko.rel_fro_error(y, ref) < tol, (pattern, dtype, bs_last, batch)
    # chains: fc2 of the KS-ViT-B MLP reads batch-last activations and adds the batch-first residual
    pats = [(1, 192, 768, 4), (4, 192, 192, 1)]
    rng = np.random.RandomState(1650)
    ws = make_weights(pats, rng)
    wt = [torch.from_numpy(v).half() for v in ws]
    wk = [kb.generate_factor(*p, "kernel", v, torch.float16, DEV) for p, v in zip(pats, wt)]
    for in_last, out_last in ((True, False), (False, False), (True, True), (False, True)):
        batch = 520
        x = torch.from_numpy(rng.standard_normal((3072, batch) if in_last else (batch, 3072)).astype(np.float32)).half()
        res = torch.from_numpy(rng.standard_normal((768, batch) if out_last else (batch, 768)).astype(np.float32)).half()
        before = kb.launch_count()
        y = kb.chain_forward(x.to(DEV), wk, pats, in_last, out_bs_last=out_last, residual=res.to(DEV))
        if in_last and not out_last:
            assert kb.launch_count() - before == 2          # nothing but the two factors
        ref = ko.chain_apply(x.float().numpy(), [v.float().numpy() for v in wt], in_last)
        ref = (ref.T if in_last != out_last else ref) + res.float().numpy()
        assert ko.rel_fro_error(y.float().cpu().numpy(), ref) < 1e-2, (in_last, out_last)
    kb.check_device()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tc_family_batch_first_groups_of_eight_blocks(dtype):
    """Batch-first with d a multiple of 8 and b <= 64 (tc_bsfirst_g.cu): eight blocks per CTA, 16-byte
    pieces of l through TMA, 8 x 8 de-interleave in the transposer warps, interleaving epilogue.
    One launch, every shape regime: several l groups, several block rows, ragged batch, b and c
    that do not fill a tile, bias / scale / activation."""
    pats = [(1, 64, 64, 16), (2, 64, 32, 8), (1, 64, 64, 8), (3, 48, 80, 24), (1, 56, 72, 32), (4, 64, 64, 64),
            (1, 32, 40, 16), (2, 32, 16, 128), (1, 48, 192, 8),
            (1, 136, 72, 32), (1, 768, 192, 8)]   # wider than one j tile: the default path converts the layout
    rng = np.random.RandomState(1700)
    for pi, pattern in enumerate(pats):
        a, b, c, d = pattern
        for batch in (8, 136, 520):
            x, w = _inputs(pattern, batch, dtype, False, seed=1700 + pi)
            ref = _oracle(x, w, False)
            before = kb.launch_count()
            y = _run(x, w, pattern, False)
            # the default takes this kernel up to d = 16; beyond, the layout conversion is faster
            assert kb.launch_count() - before == (1 if b <= 64 and d <= 16 else 3), pattern
            assert not np.isnan(y).any(), (pattern, batch)
            err = ko.rel_fro_error(y, ref)
            assert err < TOL[dtype], (pattern, batch, err)
            if b <= 64 and d > 16:
                before = kb.launch_count()
                y = _run(x, w, pattern, False, algo=_lib.KSMM_ALGO_TC, config=0)   # the kernel by name
                assert kb.launch_count() - before == 1, pattern
                assert ko.rel_fro_error(y, ref) < TOL[dtype], (pattern, batch)
        bias = torch.from_numpy(rng.standard_normal(a * b * d).astype(np.float32)).to(dtype)
        x, w = _inputs(pattern, 200, dtype, False, seed=1750 + pi)
        y = _run(x, w, pattern, False, bias=bias.to(DEV), alpha=0.5, activation="gelu")
        ref = _act_ref(0.5 * _oracle(x, w, False) + bias.float().numpy()[None, :], "gelu")
        assert ko.rel_fro_error(y, ref) < TOL[dtype], pattern
    kb.check_device()
