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
import os

import torch

from . import _lib
from .kernel import dtype_code

_DT_NAME = {_lib.KSMM_F32: "f32", _lib.KSMM_F16: "f16", _lib.KSMM_BF16: "bf16", _lib.KSMM_F8E4M3: "f8e4m3"}
_DT_CODE = {v: k for k, v in _DT_NAME.items()}
_ALGO_NAME = {_lib.KSMM_ALGO_SIMT: "ffma", _lib.KSMM_ALGO_TC: "tensor", _lib.KSMM_ALGO_CONVERT: "convert"}
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
    (``batch a b c d TILEX TILEK TILEY TX TY VSIZE ms std mse``), header line included, so that
    tooling written for those files keeps reading it.  The tile columns of the reference have no
    counterpart here: TILEX carries the configuration index, TILEK the kernel family (1 = ffma,
    2 = tensor, 3 = layout conversion), the rest are zero."""
    with open(path, "w") as f:
        f.write(BEST_HEADER + "\n")
        for e in entries():
            a, b, c, d = e["pattern"]
            f.write(f"{e['batch']} {a} {b} {c} {d} {e['config']} {_ALGO_CODE[e['family']]} 0 0 0 0 "
                    f"{e['ms']:.6f} 0.000000 0.000000e+00\n")


# ---------------------------------------------------------------------------
# The reference's tables as priors
# ---------------------------------------------------------------------------
BEST_HEADER = "batch_size a b c d TILEX TILEK TILEY TX TY VSIZE ms std mse"
# output-tile height (j) of the register-staged FFMA configurations 0..5 and their batch tile
_FFMA_TILES = {0: (128, 128), 1: (64, 128), 2: (32, 128), 3: (16, 128), 4: (64, 256), 5: (8, 128)}


def read_best_rows(path):
    """Parse a ``.best`` table of the reference (kernel_bs_last_float.best and its siblings; the
    reference scans them line by line in kernel.py:151-169).  Returns one dict per row:
    ``batch, pattern, tile = (TILEX, TILEK, TILEY, TX, TY, VSIZE), ms``.  Malformed lines raise."""
    rows = []
    with open(path) as f:
        lines = [ln.strip() for ln in f if ln.strip()]
    if not lines or lines[0].split()[:5] != BEST_HEADER.split()[:5]:
        raise ValueError(f"{path}: not a .best table (header line missing)")
    for ln in lines[1:]:
        t = ln.split()
        if len(t) != 14:
            raise ValueError(f"{path}: expected 14 columns, got {len(t)}: {ln!r}")
        rows.append({"batch": int(t[0]), "pattern": [int(v) for v in t[1:5]],
                     "tile": tuple(int(v) for v in t[5:11]), "ms": float(t[11])})
    return rows


def ffma_config_from_tile(tilex, tiley):
    """The register-staged FFMA configuration whose output tile is nearest to the reference's
    (TILEX = output rows j per CTA, TILEY = batch entries per CTA)."""
    import math as _m
    return min(_FFMA_TILES, key=lambda q: (abs(_m.log2(_FFMA_TILES[q][0] / max(tilex, 1))),
                                           abs(_m.log2(_FFMA_TILES[q][1] / max(tiley, 1)))))


def import_best_rows(path, dtype, bs_last, apply=True):
    """Use a reference ``.best`` table as priors: every row names a problem the reference was tuned
    for.  Returns the list of ``(pattern, batch)`` it holds (what ``tune_factor`` should be run on),
    and, with ``apply``, seeds the library's choice cache for the rows that only the FFMA family can
    run (no tensor-core kernel and no layout conversion for that problem) with the configuration
    whose tile is nearest to the reference's winner.  Problems the heuristic already sends to a
    tensor-core kernel are left to it: the reference's tiles say nothing about those kernels.
    ``dtype``/``bs_last`` are what the table's file name encodes (``kernel_bs_{first,last}_{float,half}``)."""
    from .kernel import default_choice
    lib = _lib.load()
    code = dtype_code(dtype)
    known, seeded = [], 0
    for r in read_best_rows(path):
        a, b, c, d = r["pattern"]
        known.append((tuple(r["pattern"]), r["batch"]))
        if not apply:
            continue
        family, _, conv = default_choice(r["pattern"], r["batch"], dtype, bs_last)
        algo, cfg = ctypes.c_int(), ctypes.c_int()
        cached = lib.ksmm_cu_get_choice(r["batch"], a, b, c, d, code, code, int(bool(bs_last)),
                                        ctypes.byref(algo), ctypes.byref(cfg)) == _lib.KSMM_OK
        if family != "ffma" or conv or cached:
            continue
        config = ffma_config_from_tile(r["tile"][0], r["tile"][2])
        if lib.ksmm_cu_set_choice(r["batch"], a, b, c, d, code, code, int(bool(bs_last)),
                                  _lib.KSMM_ALGO_SIMT, config) == _lib.KSMM_OK:
            _table[_key(r["batch"], r["pattern"], code, code, bs_last)] = {
                "sm": None, "dtype": _DT_NAME[code], "out_dtype": _DT_NAME[code], "bs_last": bool(bs_last),
                "pattern": list(r["pattern"]), "batch": r["batch"], "family": "ffma", "config": config,
                "ms": float("nan"), "prior": {"tile": list(r["tile"]), "reference_ms": r["ms"]}}
            seeded += 1
    return known, seeded


# ---------------------------------------------------------------------------
# The shipped table
# ---------------------------------------------------------------------------
import os as _os

DEFAULT_TABLE = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "tuned_sm100.json")
# the factor patterns of the benchmark specification (README layer, KS-ViT-B MLP, 3-factor chain)
BENCHMARK_PATTERNS = [(6, 64, 64, 1), (1, 768, 192, 2), (4, 192, 192, 1), (1, 768, 192, 4),
                      (1, 192, 768, 4), (1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)]


def _time_default(pattern, batch, dtype, bs_last, reps=30):
    """Milliseconds per launch of whatever KSMM_ALGO_AUTO runs for this problem right now."""
    from .kernel import forward_ex
    a, b, c, d = pattern
    dev = torch.device("cuda")
    x = torch.randn((a * c * d, batch) if bs_last else (batch, a * c * d), device=dev).to(dtype)
    w = (torch.rand(a * d * c, b, device=dev) * 2 - 1).mul_(1.0 / math.sqrt(c)).to(dtype)
    y = torch.empty((a * b * d, batch) if bs_last else (batch, a * b * d), device=dev, dtype=dtype)
    for _ in range(3):
        forward_ex(x, w, bs_last, a, b, c, d, out=y)
    # every timed launch starts with a cold L2 (a buffer larger than the cache is overwritten
    # before it, outside the timed interval), like ksmm_cu_tune's own timing
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for e0, e1 in pairs:
        flush.zero_()
        e0.record()
        forward_ex(x, w, bs_last, a, b, c, d, out=y)
        e1.record()
    torch.cuda.synchronize()
    return sum(e0.elapsed_time(e1) for e0, e1 in pairs) / reps


def tune_set(patterns=BENCHMARK_PATTERNS, batch=25088, dtypes=(torch.float32, torch.float16, torch.bfloat16),
             layouts=(True, False), min_gain=0.03, nrepeats=30, time_budget_s=None, log=None):
    """Tune every (pattern, dtype, layout) and keep a choice only where it beats the heuristic by
    more than `min_gain` when both are timed the same way; everything else is left to the
    heuristic (a cached choice also switches off the layout fusion of chains for that factor, so
    an entry has to earn its place).  Returns the kept entries.  With `time_budget_s` the loop
    goes pattern by pattern (all types and layouts of one pattern together) and stops once the
    budget is spent; `log` (a callable) receives one line per tuned case."""
    import time
    lib = _lib.load()
    kept = []
    t_start = time.time()
    for pattern in patterns:
        if time_budget_s is not None and time.time() - t_start > time_budget_s:
            break
        for dtype in dtypes:
            code = dtype_code(dtype)
            for bs_last in layouts:
                a, b, c, d = pattern
                lib.ksmm_cu_clear_choice(batch, a, b, c, d, code, code, int(bs_last))
                _table.pop(_key(batch, pattern, code, code, bs_last), None)
                from .kernel import default_choice
                fam0, cfg0, conv0 = default_choice(pattern, batch, dtype, bs_last)
                t_default = _time_default(pattern, batch, dtype, bs_last, nrepeats)
                entry = tune_factor(pattern, batch, dtype, bs_last, nrepeats=nrepeats)
                t_tuned = _time_default(pattern, batch, dtype, bs_last, nrepeats)
                entry["ms"], entry["ms_heuristic"] = t_tuned, t_default
                same = (entry["family"] == "convert" and conv0) or \
                    (not conv0 and entry["family"] == fam0 and (entry["config"] == cfg0 or cfg0 < 0))
                keep = (not same) and t_tuned < (1.0 - min_gain) * t_default
                if keep:
                    # a second look at both: single timings wander by several per cent
                    lib.ksmm_cu_clear_choice(batch, a, b, c, d, code, code, int(bs_last))
                    t_default = min(t_default, _time_default(pattern, batch, dtype, bs_last, nrepeats))
                    lib.ksmm_cu_set_choice(batch, a, b, c, d, code, code, int(bs_last),
                                           _ALGO_CODE[entry["family"]], entry["config"])
                    t_tuned = max(t_tuned, _time_default(pattern, batch, dtype, bs_last, nrepeats))
                    entry["ms"], entry["ms_heuristic"] = t_tuned, t_default
                    keep = t_tuned < (1.0 - min_gain) * t_default
                if log is not None:
                    log(f"{pattern} {str(dtype)[6:]} {'bs_last' if bs_last else 'bs_first'}: heuristic "
                        f"{fam0}/{cfg0}{' via transposes' if conv0 else ''} {t_default * 1e3:.1f} us, tuned "
                        f"{entry['family']}/{entry['config']} {t_tuned * 1e3:.1f} us{' KEPT' if keep else ''}")
                if keep:
                    kept.append(entry)
                else:
                    lib.ksmm_cu_clear_choice(batch, a, b, c, d, code, code, int(bs_last))
                    _table.pop(_key(batch, pattern, code, code, bs_last), None)
    return kept


def load_default():
    """Push the table shipped with the package (if any) into the library; returns the count applied.
    Set KSMM_NO_TUNED_TABLE=1 to start from the heuristic alone."""
    if _os.environ.get("KSMM_NO_TUNED_TABLE") or not _os.path.exists(DEFAULT_TABLE):
        return 0
    return load(DEFAULT_TABLE)


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="tune the benchmark patterns and write the shipped table")
    ap.add_argument("--out", default=DEFAULT_TABLE)
    ap.add_argument("--batch", type=int, default=25088)
    ap.add_argument("--patterns-file", default=None,
                    help="text file with one a,b,c,d row per line (# comments allowed), tuned as well")
    ap.add_argument("--every", type=int, default=1, help="take every n-th row of --patterns-file")
    ap.add_argument("--offset", type=int, default=0, help="first row of --patterns-file to take")
    ap.add_argument("--time-budget", type=float, default=None,
                    help="stop after this many seconds and write what has been tuned so far")
    ap.add_argument("--dtypes", default="fp32,fp16,bf16")
    ap.add_argument("--keep-existing", action="store_true", help="start from the table already at --out")
    args = ap.parse_args()
    pats = [] if args.patterns_file and args.offset else list(BENCHMARK_PATTERNS)
    if args.patterns_file:
        rows = [tuple(int(v) for v in ln.split(",")) for ln in open(args.patterns_file)
                if ln.strip() and not ln.startswith("#")]
        pats += [r for r in rows[max(0, args.offset)::max(1, args.every)] if r not in pats]
    names = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}
    if args.keep_existing and os.path.exists(args.out):
        load(args.out)
    for e in tune_set(patterns=pats, batch=args.batch, dtypes=tuple(names[n] for n in args.dtypes.split(",")),
                      time_budget_s=args.time_budget, log=lambda ln: print(ln, flush=True)):
        print(e)
    save(args.out)
    print(f"{len(entries())} entries -> {args.out}")
