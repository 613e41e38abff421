"""The allocation-free chain call (ksmm_cu_chain_forward_static).

Some hosts of this library may not allocate device memory at call time: a
plugin running on a latency-critical stream where cudaMalloc would stall the
whole device, or an embedding process that fixes every plugin's memory budget
at start-up.  For them the chain call exists in a variant whose scratch (the
intermediate activations and, for batch-first factors that go through a layout
conversion, the transposed copies) is a fixed array inside the library.

Two tests drive it through the C ABI with raw pointers:

* in a fresh child process, as the very first library call, so that no earlier
  call can have grown a library-owned buffer: the library's own allocation
  counter must not move and the free device memory must not drop by anything
  near the size of the scratch, over batch-last and batch-first chains in fp32
  and fp16, including factors that take the layout-conversion path;
* in this process, after every other test: the same check against the ordinary
  entry point with a caller-owned workspace, twice in a row (the array keeps
  the previous call's contents), plus the refusal of a chain that does not fit.

Collected last on purpose: a failure here stops a `-x` run only after every
other test has run.
"""
import ctypes
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import ksmm_b200 as kb
from golden_cases import make_weights
from ksmm_b200 import _lib
from oracle import ksmm_oracle as ko

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HERE = os.path.dirname(os.path.abspath(__file__))


def test_static_chain_first_call_of_a_fresh_process_allocates_nothing():
    env = dict(os.environ)
    env["CUDA_MODULE_LOADING"] = "EAGER"   # kernel images load at start-up, not at the first launch
    res = subprocess.run([sys.executable, os.path.join(HERE, "no_alloc_child.py")], capture_output=True,
                         text=True, timeout=900, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("NO_ALLOC_RESULT ")][-1]
    results = json.loads(line[len("NO_ALLOC_RESULT "):])
    assert len(results) == 14
    for idx, r in enumerate(results):
        assert r["status"] == 0, r
        assert r["allocs"] == 0, r                      # no cudaMalloc inside the library
        # Free device memory: the first call on a device makes the driver load the part of the library
        # image that holds the array (its 40 MiB and some code), once, whatever the chain; after that
        # nothing may move, although every case here needs more than 4 MiB of scratch (intermediates,
        # and from the second case on transposed copies that no earlier call has ever needed).
        limit = _lib.STATIC_SCRATCH_BYTES + 16 * 1024 * 1024 if idx == 0 else 4 * 1024 * 1024
        assert r["free_delta"] < limit, (idx, r, [q["free_delta"] for q in results])
        assert not r["nan"], r
        tol = 1e-2 if r["half"] else 1e-5
        assert r["err_vs_ordinary"] < tol, r
        assert r["err_vs_oracle"] < tol, r


def _chain_case(pats, batch, dtype, bs_last, seed):
    rng = np.random.RandomState(seed)
    ws = make_weights(pats, rng)
    n_in = pats[0][0] * pats[0][2] * pats[0][3]
    n_out = pats[-1][0] * pats[-1][1] * pats[-1][3]
    x = torch.from_numpy(rng.standard_normal((n_in, batch) if bs_last else (batch, n_in)).astype(np.float32))
    xg = x.to(dtype).to(DEV)
    wk = [kb.generate_factor(*p, "kernel", torch.from_numpy(w), dtype, DEV) for p, w in zip(pats, ws)]
    bias = torch.from_numpy(rng.standard_normal(n_out).astype(np.float32)).to(dtype).to(DEV)
    return xg, wk, bias, ws, n_out


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 1e-2)])
@pytest.mark.parametrize("bs_last", [True, False])
def test_static_scratch_chain_matches_workspace_chain(dtype, tol, bs_last):
    lib = _lib.load()
    pats = [(4, 192, 192, 1), (1, 768, 192, 4)]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flat = _lib.int32_array([v for p in pats for v in p])
    code = kb.kernel.dtype_code(dtype)
    for call, batch in enumerate((1024, 1536)):   # two calls in a row, different sizes
        xg, wk, bias, ws, n_out = _chain_case(pats, batch, dtype, bs_last, seed=50 + call)
        out = torch.full((n_out, batch) if bs_last else (batch, n_out), float("nan"), dtype=dtype, device=DEV)
        vals = (ctypes.c_void_p * len(wk))(*[w.data_ptr() for w in wk])
        torch.cuda.synchronize()
        allocs_before = lib.ksmm_cu_alloc_count()
        st = lib.ksmm_cu_chain_forward_static(xg.data_ptr(), vals, out.data_ptr(), bias.data_ptr(),
                                              batch, len(pats), flat, code, int(bs_last), stream)
        _lib.check(st)
        torch.cuda.synchronize()
        assert lib.ksmm_cu_alloc_count() == allocs_before
        assert not torch.isnan(out.float()).any()
        ref = kb.chain_forward(xg, wk, pats, bs_last, bias=bias)       # caller-owned workspace
        # same kernels, same order: the two entry points agree far inside the tolerance
        err = ko.rel_fro_error(out.float().cpu().numpy(), ref.float().cpu().numpy())
        assert err < tol, (call, err)
        half = dtype == torch.float16
        w_seen = [w.astype(np.float16).astype(np.float32) if half else w for w in ws]
        oracle = ko.chain_apply(xg.float().cpu().numpy(), w_seen, bs_last,
                                bias=bias.float().cpu().numpy(),
                                round_to=np.float16 if half else None)
        assert ko.rel_fro_error(out.float().cpu().numpy(), oracle) < tol
    kb.check_device()


def test_static_scratch_rejects_oversized_chains():
    lib = _lib.load()
    pats = [(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)]   # needs two 1024-feature intermediates
    flat = _lib.int32_array([v for p in pats for v in p])
    batch = 25088
    need = lib.ksmm_cu_chain_workspace_bytes(3, flat, batch, _lib.KSMM_F16)
    assert need > _lib.STATIC_SCRATCH_BYTES
    x = torch.zeros(1024, batch, dtype=torch.float16, device=DEV)
    y = torch.zeros(1024, batch, dtype=torch.float16, device=DEV)
    wk = [torch.zeros(p[0] * p[3] * p[2], p[1], dtype=torch.float16, device=DEV) for p in pats]
    vals = (ctypes.c_void_p * 3)(*[w.data_ptr() for w in wk])
    st = lib.ksmm_cu_chain_forward_static(x.data_ptr(), vals, y.data_ptr(), None, batch, 3, flat,
                                          _lib.KSMM_F16, 1, None)
    assert st == _lib.KSMM_ERR_WORKSPACE
    assert b"built-in scratch" in lib.ksmm_cu_last_error()
    # a single batch-last factor needs no scratch at all and always goes through
    one = _lib.int32_array(list(pats[0]))
    st = lib.ksmm_cu_chain_forward_static(x.data_ptr(), vals, y.data_ptr(), None, batch, 1, one,
                                          _lib.KSMM_F16, 1, None)
    _lib.check(st)
    # A batch-first factor whose dispatch goes through a layout conversion needs its two transposed
    # copies in the array as well.  When they do not fit, the call is refused before anything is
    # launched; it never allocates behind the caller's back.
    before = lib.ksmm_cu_launch_count()
    allocs = lib.ksmm_cu_alloc_count()
    xf = x.t().contiguous()
    for pat in ((1, 64, 64, 16), (1, 64, 64, 3)):
        one = _lib.int32_array(list(pat))
        n_feat = pat[0] * pat[2] * pat[3]
        need = lib.ksmm_cu_chain_workspace_bytes_ex(1, one, batch, _lib.KSMM_F16, 0)
        w1 = torch.zeros(pat[0] * pat[3] * pat[2], pat[1], dtype=torch.float16, device=DEV)
        v1 = (ctypes.c_void_p * 1)(w1.data_ptr())
        launches = lib.ksmm_cu_launch_count()
        st = lib.ksmm_cu_chain_forward_static(xf[:, :n_feat].contiguous().data_ptr(), v1, y.data_ptr(), None,
                                              batch, 1, one, _lib.KSMM_F16, 0, None)
        if need > _lib.STATIC_SCRATCH_BYTES:
            assert st == _lib.KSMM_ERR_WORKSPACE, pat
            assert lib.ksmm_cu_launch_count() == launches
        else:
            _lib.check(st)
    assert lib.ksmm_cu_launch_count() >= before and lib.ksmm_cu_alloc_count() == allocs
    kb.check_device()
