"""Per-pattern tuner with a persistent table.

Replaces the reference's offline search (src/ksmm_cu/long_run.sh:178-229: one
nvcc build and one process per candidate, hours per kernel) and its ``.best``
tables (e.g. kernel_bs_last_float.best: ``batch a b c d TILEX TILEK TILEY TX TY
VSIZE ms std mse``): every candidate tile configuration is compiled into
libksmm_cu.so, ``tune_factor`` times the ones that can run a problem in-process
with CUDA events (``ksmm_cu_tune``) and the winners are kept in a JSON table
keyed by (sm, dtype, layout, a, b, c, d, batch) that ``load`` pushes back into
the library (``ksmm_cu_set_choice``) without re-timing.  Any pattern and batch
size works; an untuned problem runs with the library's heuristic default.
"""
from __future__ import annotations

import ctypes
import json
import math

import torch

from . import _lib
from .kernel import dtype_code

_DT_NAME = {_lib.KSMM_F32: "f32", _lib.KSMM_F16: "f16", _lib.KSMM_BF16: "bf16", _lib.KSMM_F8E4M3: "f8e4m3"}
_DT_CODE = {v: k for k, v in _DT_NAME.items()}
_ALGO_NAME = {_lib.KSMM_ALGO_SIMT: "ffma", _lib.KSMM_ALGO_TC: "tensor"}
_ALGO_CODE = {v: k for k, v in _ALGO_NAME.items()}

# entries tuned or loaded in this process: key -> dict
_table = {}


def _key(batch, pattern, in_dtype, out_dtype, bs_last):
    a, b, c, d = (int(v) for v in pattern)
    return (int(batch), a, b, c, d, int(in_dtype), int(out_dtype), int(bool(bs_last)))


def tune_factor(pattern, batch, dtype=torch.float16, bs_last=True, out_dtype=None, nrepeats=20,
                device="cuda"):
    """Time every kernel candidate for one factor on scratch buffers of the real
    size and remember the fastest.  Returns the table entry."""
    lib = _lib.load()
    a, b, c, d = (int(v) for v in pattern)
    out_dtype = dtype if out_dtype is None else out_dtype
    dev = torch.device(device)
    shape_in = (a * c * d, batch) if bs_last else (batch, a * c * d)
    shape_out = (a * b * d, batch) if bs_last else (batch, a * b * d)
    work = torch.float32 if dtype == torch.float8_e4m3fn else dtype
    x = torch.randn(shape_in, device=dev, dtype=work).to(dtype)
    w = (torch.rand(a * d * c, b, device=dev, dtype=work) * 2 - 1).mul_(1.0 / math.sqrt(c)).to(dtype)
    y = torch.empty(shape_out, device=dev, dtype=out_dtype)
    ic, oc = dtype_code(dtype), dtype_code(out_dtype)
    desc = _lib.ForwardDesc(input=x.data_ptr(), values=w.data_ptr(), output=y.data_ptr(), bias=None,
                            batch=batch, a=a, b=b, c=c, d=d, in_dtype=ic, out_dtype=oc,
                            bs_last=int(bool(bs_last)), algo=0, config=-1, alpha=1.0)
    algo, cfg, ms = ctypes.c_int(), ctypes.c_int(), ctypes.c_float()
    with torch.cuda.device(dev):
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(lib.ksmm_cu_tune(ctypes.byref(desc), int(nrepeats), stream, ctypes.byref(algo),
                                    ctypes.byref(cfg), ctypes.byref(ms)))
        cap = torch.cuda.get_device_capability(dev)
    entry = {"sm": cap[0] * 10 + cap[1], "dtype": _DT_NAME[ic], "out_dtype": _DT_NAME[oc],
             "bs_last": bool(bs_last), "pattern": [a, b, c, d], "batch": int(batch),
             "family": _ALGO_NAME[algo.value], "config": int(cfg.value), "ms": float(ms.value)}
    _table[_key(batch, pattern, ic, oc, bs_last)] = entry
    return entry


def entries():
    """Entries tuned or loaded in this process."""
    return list(_table.values())


def save(path):
    with open(path, "w") as f:
        json.dump({"format": "ksmm_b200.tuner/1", "entries": entries()}, f, indent=1)


def load(path, sm=None):
    """Push a saved table into the library.  Entries for another GPU generation
    (``sm``) or that the current build cannot run are skipped; returns the count applied."""
    lib = _lib.load()
    with open(path) as f:
        doc = json.load(f)
    if doc.get("format") != "ksmm_b200.tuner/1":
        raise ValueError(f"{path}: not a ksmm_b200 tuner table")
    applied = 0
    for e in doc["entries"]:
        if sm is not None and e.get("sm") != sm:
            continue
        a, b, c, d = e["pattern"]
        ic, oc = _DT_CODE[e["dtype"]], _DT_CODE[e["out_dtype"]]
        st = lib.ksmm_cu_set_choice(e["batch"], a, b, c, d, ic, oc, int(e["bs_last"]),
                                    _ALGO_CODE[e["family"]], e["config"])
        if st == _lib.KSMM_OK:
            _table[_key(e["batch"], e["pattern"], ic, oc, e["bs_last"])] = e
            applied += 1
    return applied


def export_best_rows(path):
    """Write the table in the column order of the reference's ``.best`` files
    (``batch a b c d TILEX TILEK TILEY TX TY VSIZE ms std mse``).  The tile columns
    of the reference have no counterpart here: TILEX carries the configuration
    index, TILEK the kernel family (1 = ffma, 2 = tensor), the rest are zero."""
    with open(path, "w") as f:
        for e in entries():
            a, b, c, d = e["pattern"]
            f.write(f"{e['batch']} {a} {b} {c} {d} {e['config']} {_ALGO_CODE[e['family']]} 0 0 0 0 "
                    f"{e['ms']:.6f} 0.000000 0.000000e+00\n")
