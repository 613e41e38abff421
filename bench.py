#!/usr/bin/env python
"""Benchmark of the KSMM hot path.

One *step* is one pass of the single-factor sweep: every benchmark pattern at
batch 25088 in fp32 and fp16, batch-last and batch-first (one kernel launch per
case).  Inputs are synthetic (x ~ N(0,1), W ~ U(+-1/sqrt(c)), seeded), resident
in device memory for `value`, and in pinned host memory for `e2e`, which goes
through the C ABI's host-buffer entry point (host->device copy, kernel,
device->host copy inside the timed call).

    python bench.py --gpus N --steps K --warmup W          # this library
    python bench.py --impl reference ...                   # the reference's CPU algorithm

With N > 1 (launched by torch.distributed.run) every rank runs the same sweep
on its own batch shard of 25088 columns: weak scaling, no collective on the
data path; the time is the maximum over ranks.

Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH = 25088
# the patterns the benchmark specification names (README layer, KS-ViT-B MLP, 3-factor chain)
PATTERNS = [(6, 64, 64, 1), (1, 768, 192, 2), (4, 192, 192, 1), (1, 768, 192, 4),
            (1, 192, 768, 4), (1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)]
DTYPES = ["fp32", "fp16"]
TORCH_DT = {"fp32": torch.float32, "fp16": torch.float16}
ESIZE = {"fp32": 4, "fp16": 2}


# (dtype, batch-last, pattern) -> DRAM bytes of one launch under ncu, the summary it comes from and
# the (family, configuration, via_transpose) that capture ran
NCU_TRAFFIC = {
    ("fp32", True, (1, 768, 192, 4)): {"bytes": 332.4e6, "profile": "profiles/tc_f32x3_kernel_fp32.md",
                                       "choice": ("tensor", 0, False)},
    ("fp32", True, (1, 192, 768, 4)): {"bytes": 369.7e6, "profile": "profiles/tc_f32x3_kernel_fp32.md",
                                       "choice": ("tensor", 0, False)},
    ("fp16", True, (1, 768, 192, 4)): {"bytes": 135.8e6, "profile": "profiles/tc_kernel_fp16_bs_last_1_768_192_4.md",
                                       "choice": ("tensor", 0, False)},
    ("fp16", False, (1, 768, 192, 4)): {"bytes": 136.5e6, "profile": "profiles/tc_bsfirst_d_kernel_fp16_1_768_192_4.md",
                                        "choice": ("tensor", 0, False)},
}


def flops_of(p, batch):
    a, b, c, d = p
    return 2.0 * a * b * c * d * batch


def min_bytes_of(p, batch, es):
    a, b, c, d = p
    return float(es) * (a * c * d * batch + a * b * d * batch + a * b * c * d)


def cases(only=None):
    """Every (dtype, layout, pattern) of the sweep; `only` = "fp16:bs_last:1,768,192,4"
    (any field may be empty) restricts it, e.g. for a profiler capture of one kernel."""
    out = []
    for dt in DTYPES:
        for bs_last in (True, False):
            for p in PATTERNS:
                out.append({"pattern": p, "dtype": dt, "bs_last": bs_last})
    if only:
        f = (only.split(":") + ["", "", ""])[:3]
        pat = tuple(int(v) for v in f[2].split(",")) if f[2] else None
        out = [c for c in out
               if (not f[0] or c["dtype"] == f[0])
               and (not f[1] or ("bs_last" if c["bs_last"] else "bs_first") == f[1])
               and (pat is None or c["pattern"] == pat)]
        if pat is not None and not out:
            for dt in ([f[0]] if f[0] else DTYPES):
                for bl in ([f[1] == "bs_last"] if f[1] else [True, False]):
                    out.append({"pattern": pat, "dtype": dt, "bs_last": bl})
    return out


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            pk = json.load(f)
        return {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops": float(pk["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


# ---------------------------------------------------------------------------
# clocks: sampled through NVML while the timed region runs (read-only)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks_setting"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# the reference's CPU algorithm (torch einsum, all host threads), bounded sample
# ---------------------------------------------------------------------------
def cpu_reference_pass(sample_cols, seed=0, algos=("einsum",), min_run_time=0.05):
    """The fp32 half of the sweep on the host at `sample_cols` batch columns with the reference's
    CPU algorithms (`einsum`, `bmm`), each case timed with torch.utils.benchmark.Timer
    .blocked_autorange as the reference's own timing script does
    (src/ksmm_py/benchmark/ksmm_time.py:168-190).  Returns {algo: (flops, seconds)} where seconds
    is the sum of the per-case medians."""
    from torch.utils import benchmark as tbench

    from oracle import reference_port as rp
    g = torch.Generator().manual_seed(seed)
    out = {al: [0.0, 0.0] for al in algos}
    nthreads = torch.get_num_threads()
    for bs_last in (True, False):
        for p in PATTERNS:
            a, b, c, d = p
            w = (torch.rand((a, b, c, d), generator=g) * 2 - 1) / (c ** 0.5)
            shape = (a * c * d, sample_cols) if bs_last else (sample_cols, a * c * d)
            x = torch.randn(shape, generator=g)
            for al in algos:
                chain = rp.ChainCPU([p], [w], al, bs_last)
                m = tbench.Timer(stmt="chain(x)", globals={"chain": chain, "x": x},
                                 num_threads=nthreads).blocked_autorange(min_run_time=min_run_time)
                out[al][0] += flops_of(p, sample_cols)
                out[al][1] += m.median
    return {al: tuple(v) for al, v in out.items()}


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs use every core the process may run on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))


REF_COLS = 3136   # batch columns of the bounded CPU sample (1/8 of the benchmark batch)


def reference_sample_text(algos):
    return (f"fp32 half of the sweep (16 of the 32 cases), first {REF_COLS} of {BATCH} batch columns, "
            f"reference algo={'/'.join(algos)} restated on torch CPU (oracle/reference_port.py), every "
            "case timed with torch.utils.benchmark blocked_autorange, all host threads")


def run_reference(args, rank, world):
    if rank != 0:
        return
    use_all_host_threads()
    for _ in range(min(args.warmup, 1)):
        cpu_reference_pass(REF_COLS, min_run_time=0.02)
    fl, secs = 0.0, 0.0
    # each step is one pass of the bounded sample; einsum is the reference's fastest CPU algorithm
    # on these patterns and the one the line reports (bmm is timed in the default arm's cpu_baseline)
    budget = 150.0
    t_start = time.perf_counter()
    steps_done = 0
    for _ in range(args.steps):
        f, s_ = cpu_reference_pass(REF_COLS, min_run_time=0.02)["einsum"]
        fl += f
        secs += s_
        steps_done += 1
        if time.perf_counter() - t_start > budget:
            break
    val = fl / secs / 1e12
    cfg = workload_config()
    cfg["sample"] = reference_sample_text(("einsum",)) + f"; {steps_done} passes timed"
    line = {
        "impl": "reference", "metric": "ksmm_sweep_throughput", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs / steps_done, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": cfg["sample"]},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config():
    return {"workload": "single-factor sweep (configs[1] restricted to the 8 benchmark patterns): "
                        "fp32+fp16 x batch-last+batch-first, B=25088 per GPU, 32 cases per step",
            "patterns": [list(p) for p in PATTERNS], "batch_per_gpu": BATCH,
            "l2": "a step touches ~5.4 GB of distinct buffers (> 126 MB L2) before any buffer repeats"}


# ---------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------
def run_profile_case(name, local_rank):
    """A few launches of one workload that `--only` cannot name (chains, backward), for a profiler
    capture: no timing, nothing printed but the launch count."""
    import ksmm_b200 as kb
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(3)
    before = kb.launch_count()
    with torch.no_grad():
        if name == "mlp_pair":
            p1, p2 = [(4, 192, 192, 1), (1, 768, 192, 4)], [(1, 192, 768, 4), (4, 192, 192, 1)]
            fc1 = kb.KSLinear(p1, bias=True, dtype=torch.float16, bs_last=False, device=dev, out_bs_last=True,
                              activation="gelu")
            fc2 = kb.KSLinear(p2, bias=True, dtype=torch.float16, bs_last=True, device=dev, out_bs_last=False)
            x = torch.randn((BATCH, 768), device=dev, dtype=torch.float16, generator=gen)
            for _ in range(3):
                y = fc2(fc1(x))
        elif name == "wgrad":
            a, b, c, d = 1, 768, 192, 4
            x = torch.randn((a * c * d, BATCH), device=dev, dtype=torch.float16, generator=gen)
            g = torch.randn((a * b * d, BATCH), device=dev, dtype=torch.float16, generator=gen)
            for _ in range(3):
                y = kb.backward_weights(x, g, True, a, b, c, d)
        elif name == "qkv":
            layers = [kb.KSLinear([(1, 768, 768, 1)], bias=False, dtype=torch.float16, bs_last=False, device=dev)
                      for _ in range(3)]
            group = kb.KSLinearGroup(layers)
            x = torch.randn((BATCH, 768), device=dev, dtype=torch.float16, generator=gen)
            for _ in range(3):
                y = group(x)
        elif name == "chain_fp32":
            # the fp32 three-factor chain on batch-first rows as the layout planner runs it: the input
            # transposed once, two batch-last factors, the last factor writes batch-first rows
            pats = [(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)]
            layer = kb.KSLinear(pats, bias=False, dtype=torch.float32, bs_last=False, device=dev)
            x = torch.randn((BATCH, 1024), device=dev, generator=gen)
            for _ in range(3):
                y = layer(x)
        else:
            raise SystemExit(f"unknown --profile-case {name}")
    torch.cuda.synchronize()
    kb.check_device()
    print(json.dumps({"profile_case": name, "launches": kb.launch_count() - before}), flush=True)


def run_ours(args, rank, world, local_rank):
    import ksmm_b200 as kb
    from ksmm_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    cs = cases(args.only)
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    for c in cs:
        a, b, cc, d = c["pattern"]
        dt = TORCH_DT[c["dtype"]]
        shape = (a * cc * d, BATCH) if c["bs_last"] else (BATCH, a * cc * d)
        c["x"] = torch.randn(shape, generator=g).to(dt).to(dev)
        w = (torch.rand((a, b, cc, d), generator=g) * 2 - 1) / (cc ** 0.5)
        c["w"] = kb.generate_factor(a, b, cc, d, "kernel", w, dt, dev)
        oshape = (a * b * d, BATCH) if c["bs_last"] else (BATCH, a * b * d)
        c["y"] = torch.empty(oshape, dtype=dt, device=dev)
        c["flops"] = flops_of(c["pattern"], BATCH)
        c["bytes"] = min_bytes_of(c["pattern"], BATCH, ESIZE[c["dtype"]])
    step_flops = sum(c["flops"] for c in cs)

    def one_step():
        for c in cs:
            a, b, cc, d = c["pattern"]
            kb.forward_ex(c["x"], c["w"], c["bs_last"], a, b, cc, d, out=c["y"])

    def barrier():
        if world > 1:
            torch.distributed.barrier()

    # The step is captured once in a CUDA graph and replayed: the launches are
    # short (10-500 us), so without a graph the host's launch path would be timed
    # instead of the kernels.
    for _ in range(2):
        one_step()
    torch.cuda.synchronize()
    kb.check_device()
    step_graph = torch.cuda.CUDAGraph()
    launches_before = kb.launch_count()
    with torch.cuda.graph(step_graph):
        one_step()
    launches_per_step = kb.launch_count() - launches_before  # kernels recorded into the graph
    for _ in range(max(args.warmup, 3)):
        step_graph.replay()
    torch.cuda.synchronize()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for s in range(args.steps):
        step_graph.replay()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop()
    launches = args.steps * launches_per_step
    elapsed_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    kb.check_device()
    value = world * step_flops * args.steps / (elapsed_ms * 1e-3) / 1e12

    # Per-case launch duration: a graph of REP launches of the one kernel over
    # rotating input/output buffers whose combined size exceeds L2, timed with one
    # CUDA-event pair on the launching stream (event overhead amortised over REP).
    REP = 20
    L2_BYTES = 126 * 1024 * 1024

    def case_ms(c, algo=0, config=-1):
        a, b, cc, d = c["pattern"]
        foot = c["x"].numel() * c["x"].element_size() + c["y"].numel() * c["y"].element_size()
        ncopy = min(REP, max(1, -(-2 * L2_BYTES // foot)))
        xs = [c["x"]] + [c["x"].clone() for _ in range(ncopy - 1)]
        ys = [c["y"]] + [torch.empty_like(c["y"]) for _ in range(ncopy - 1)]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for r in range(REP):
                kb.forward_ex(xs[r % ncopy], c["w"], c["bs_last"], a, b, cc, d, out=ys[r % ncopy],
                              algo=algo, config=config)
        g.replay()
        torch.cuda.synchronize()
        best = []
        for _ in range(3):
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            g.replay()
            s1.record()
            torch.cuda.synchronize()
            best.append(s0.elapsed_time(s1) / REP)
        del g, xs, ys
        return statistics.median(best)

    if args.sweep_configs:
        # every tile configuration of both kernel families on every case (tuning aid)
        for c in cs:
            code = _lib.KSMM_F32 if c["dtype"] == "fp32" else _lib.KSMM_F16
            row = []
            for algo in (_lib.KSMM_ALGO_TC, _lib.KSMM_ALGO_SIMT):
                for cfg in range(lib.ksmm_cu_num_configs(algo)):
                    if not lib.ksmm_cu_config_supported(algo, cfg, BATCH, *c["pattern"], code, code,
                                                        int(c["bs_last"])):
                        continue
                    ms = case_ms(c, algo, cfg)
                    row.append(f"{'tc' if algo == _lib.KSMM_ALGO_TC else 'ffma'}{cfg}={ms * 1e3:.1f}us")
            if rank == 0:
                print(c["dtype"], "bs_last" if c["bs_last"] else "bs_first", c["pattern"], " ".join(row),
                      file=sys.stderr, flush=True)

    ffma = ctypes.c_float(0.0)
    _lib.check(lib.ksmm_cu_measure_ffma_peak(ctypes.byref(ffma), None))
    ffma_peak = float(ffma.value)
    # Compute roofs.  fp16: the measured dense bf16 tensor throughput.  fp32: what the library's
    # default runs decides: the FFMA kernels are bound by the fp32 FMA rate (live probe); the
    # tensor-core kernel issues three tf32 MMAs per product, and tf32 runs at half the bf16
    # rate, so its roof for useful flops is the measured bf16 figure / 6.
    tf32x3_peak = peaks["bf16_tflops"] / 6.0
    per = []
    ms_exact = {}
    for idx, c in enumerate(cs):
        ms = case_ms(c)
        tdt = torch.float32 if c["dtype"] == "fp32" else torch.float16
        family, cfg, conv = kb.default_choice(c["pattern"], BATCH, tdt, c["bs_last"])
        t_hbm = c["bytes"] / (peaks["hbm_gbs"] * 1e9)
        if c["dtype"] != "fp32":
            pk, cb = peaks["bf16_tflops"], "tensor"
        elif family == "tensor":
            pk, cb = tf32x3_peak, "tensor_tf32x3"
        else:
            pk, cb = ffma_peak, "ffma"
        t_fl = c["flops"] / (pk * 1e12)
        t_roof = max(t_hbm, t_fl)
        ms_ffma = None
        if c["dtype"] == "fp32" and (family == "tensor") and not args.only and not args.no_ffma_compare:
            # the same case on the exact-fp32 FFMA family, for the comparison line below
            ms_ffma = ms_exact[idx] = case_ms(c, _lib.KSMM_ALGO_SIMT, -1)
        per.append({"pattern": list(c["pattern"]), "dtype": c["dtype"],
                    "layout": "bs_last" if c["bs_last"] else "bs_first", "ms": round(ms, 5),
                    "ms_ffma_family": None if ms_ffma is None else round(ms_ffma, 5),
                    "kernel": family + (" via transposes" if conv else ""),
                    "gbs": round(c["bytes"] / (ms * 1e-3) / 1e9, 1),
                    "tflops": round(c["flops"] / (ms * 1e-3) / 1e12, 2),
                    "bound": "hbm" if t_hbm >= t_fl else cb,
                    "roofline_frac": round(t_roof / (ms * 1e-3), 4)})

    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) at B = 25088, copied from the
    # ncu captures summarised under profiles/ together with the kernel family and configuration
    # the capture ran.  A figure is reported only while the default dispatch still picks that
    # kernel; otherwise `traffic` is null (the summary no longer describes what was timed).
    ncu_traffic = NCU_TRAFFIC

    def roofline_of(entry, c):
        ms = entry["ms"]
        traffic, traffic_src = None, None
        rec = ncu_traffic.get((c["dtype"], bool(c["bs_last"]), tuple(c["pattern"])))
        if rec is not None and BATCH == 25088:
            tdt_ = torch.float32 if c["dtype"] == "fp32" else torch.float16
            fam_, cfg_, conv_ = kb.default_choice(c["pattern"], BATCH, tdt_, c["bs_last"])
            if (fam_, cfg_, conv_) == rec["choice"]:
                traffic, traffic_src = rec["bytes"], rec["profile"]
        if entry["bound"] == "hbm":
            ach, pk, unit = c["bytes"] / (ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
            src = f"MEASURED_PEAKS.json ({peaks['source']})"
        else:
            ach = c["flops"] / (ms * 1e-3) / 1e12
            unit = "TFLOP/s"
            if entry["bound"] == "ffma":
                pk = ffma_peak
                src = "ksmm_cu_measure_ffma_peak (live FFMA probe; no fp32 figure in MEASURED_PEAKS.json)"
            elif entry["bound"] == "tensor_tf32x3":
                pk = tf32x3_peak
                src = (f"MEASURED_PEAKS.json ({peaks['source']}) bf16_tflops / 6: tf32 at half the bf16 "
                       "rate, three MMAs per product")
            else:
                pk = peaks["bf16_tflops"]
                src = f"MEASURED_PEAKS.json ({peaks['source']})"
        return {"bound": "tensor" if entry["bound"] == "tensor_tf32x3" else entry["bound"],
                "achieved": round(ach, 2), "peak": round(pk, 2), "unit": unit,
                "frac": round(ach / pk, 4), "traffic": traffic, "traffic_source": traffic_src,
                "algorithmic_bytes": c["bytes"],
                "kernel": f"{entry['dtype']} {entry['layout']} {tuple(entry['pattern'])} ({entry['kernel']})",
                "peak_source": src,
                "share_of_step": round(ms / (elapsed_ms / args.steps), 4)}

    # the sweep with every fp32 case on the FFMA family (sum of the per-case launch durations)
    fp32_exact = None
    if ms_exact:
        t_all = sum(ms_exact.get(q, per[q]["ms"]) for q in range(len(cs)))
        fp32_exact = {"value": round(world * step_flops / (t_all * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                      "ms_per_step": round(t_all, 4),
                      "note": "same sweep with algo=KSMM_ALGO_SIMT (fp32 FFMA, no tf32 split) for the fp32 "
                              "cases; sum of per-case launch durations"}
    # the roofline object describes one kernel: the longest case that is a single launch
    direct = [q for q in range(len(cs)) if "via transposes" not in per[q]["kernel"]] or list(range(len(cs)))
    dom = max(direct, key=lambda q: per[q]["ms"])
    hbm_idx = [q for q in range(len(cs)) if per[q]["bound"] == "hbm"]
    dom_hbm = max(hbm_idx, key=lambda q: per[q]["ms"]) if hbm_idx else None

    # ---- end to end through the C ABI with pinned HOST buffers ------------------------------
    e2e = None
    if not args.no_e2e:
        host = []
        for c in cs:
            a, b, cc, d = c["pattern"]
            hx = torch.empty(c["x"].shape, dtype=c["x"].dtype, pin_memory=True).copy_(c["x"])
            hw = torch.empty(c["w"].shape, dtype=c["w"].dtype, pin_memory=True).copy_(c["w"])
            hy = torch.empty(c["y"].shape, dtype=c["y"].dtype, pin_memory=True)
            host.append((hx, hw, hy, _lib.int32_array([a, b, cc, d]),
                         (ctypes.c_void_p * 1)(hw.data_ptr())))
        torch.cuda.synchronize()
        h2d = sum(hx.numel() * hx.element_size() + hw.numel() * hw.element_size()
                  for hx, hw, _, _, _ in host)
        d2h = sum(hy.numel() * hy.element_size() for _, _, hy, _, _ in host)

        def e2e_step():
            # every case is enqueued through the asynchronous host-buffer call, then all tickets are
            # waited for: the upload of case k + 1 overlaps the download of case k
            tickets = []
            for c, (hx, hw, hy, pat, vals) in zip(cs, host):
                code = _lib.KSMM_F32 if c["dtype"] == "fp32" else _lib.KSMM_F16
                t = ctypes.c_uint64(0)
                _lib.check(lib.ksmm_cu_chain_forward_host_async(
                    hx.data_ptr(), vals, hy.data_ptr(), None, BATCH, 1, pat, code,
                    int(c["bs_last"]), local_rank, ctypes.byref(t)))
                tickets.append(t.value)
            for t in tickets:
                _lib.check(lib.ksmm_cu_host_wait(t))

        e2e_step()  # warm-up: the library allocates its staging buffers here
        e2e_steps = max(1, min(args.steps, 3))
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_s = time.perf_counter() - t0
        barrier()
        if world > 1:
            t = torch.tensor([e2e_s], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            e2e_s = float(t.item())
        # the result really came back: compare one case with the device-resident run
        chk = cs[0]
        kb.forward_ex(chk["x"], chk["w"], chk["bs_last"], *chk["pattern"], out=chk["y"])
        torch.cuda.synchronize()
        assert torch.equal(host[0][2], chk["y"].cpu()), "host-path result differs from device path"
        e2e = {"value": world * step_flops * e2e_steps / e2e_s / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps,
               "h2d_gbs_per_rank": round(h2d * e2e_steps / e2e_s / 1e9, 1),
               "d2h_gbs_per_rank": round(d2h * e2e_steps / e2e_s / 1e9, 1),
               "api": "ksmm_cu_chain_forward_host_async + ksmm_cu_host_wait (C ABI, pinned host buffers, "
                      "32 calls in flight per step, wall clock)"}

    # ---- KS-ViT-B/16 forward (128 images per GPU, fp16): the second half of the headline metric --
    ksvit = None
    if not args.no_vit and not args.only:
        from ksmm_b200.ksvit import KSViTB
        torch.manual_seed(7 + rank)
        img = torch.randn(128, 3, 224, 224, device=dev, dtype=torch.float16)

        def time_model(dense):
            model = KSViTB(dtype=torch.float16, device=dev, dense_mlp=dense).eval()
            with torch.no_grad():
                for _ in range(2):
                    model(img)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    out = model(img)
                for _ in range(3):
                    g.replay()
                torch.cuda.synchronize()
                barrier()
                v0, v1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 10
                v0.record()
                for _ in range(reps):
                    g.replay()
                v1.record()
                torch.cuda.synchronize()
                barrier()
            ms = v0.elapsed_time(v1) / reps
            if world > 1:
                t = torch.tensor([ms], device=dev)
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
                ms = float(t.item())
            assert torch.isfinite(out.float()).all()
            del g, model
            return ms

        ks_ms = time_model(False)
        dense_ms = time_model(True)
        kb.check_device()
        ksvit = {"imgs_per_s": world * 128 / (ks_ms * 1e-3), "ms_per_forward": ks_ms,
                 "dense_mlp_imgs_per_s": world * 128 / (dense_ms * 1e-3), "dense_mlp_ms_per_forward": dense_ms,
                 "config": "SimpleViT-B/16, 12 layers, 128 images of 224x224 per GPU, fp16, random init, "
                           "fc1=[(4,192,192,1),(1,768,192,4)], fc2=[(1,192,768,4),(4,192,192,1)], batch-first; "
                           "attention / LayerNorm are stock PyTorch; the MLP keeps its 3072-feature activations "
                           "batch-last between fc1 and fc2 and applies the GELU in fc1's epilogue; forward "
                           "captured in a CUDA graph"}

    # ---- fp8-e4m3 and bf16 factors (per-tensor scale, fp32 accumulate) --------------------------
    lowp = None
    if not args.no_vit and not args.only:
        lowp = []
        for pat in ((4, 192, 192, 1), (1, 768, 192, 4), (1, 192, 768, 4)):
            for nb in (BATCH, 4096):
                a_, b_, c_, d_ = pat
                gen = torch.Generator(device=dev).manual_seed(5)
                x32 = torch.randn((a_ * c_ * d_, nb), device=dev, generator=gen)
                w32 = kb.generate_factor(a_, b_, c_, d_, "kernel", None, torch.float32, dev)
                ref = kb.forward_ex(x32, w32, True, a_, b_, c_, d_, algo=_lib.KSMM_ALGO_SIMT).float()
                xq, sx = kb.quantize_e4m3(x32)
                wq, sw = kb.quantize_e4m3(w32)
                xb, wb = x32.bfloat16(), w32.bfloat16()
                yq = torch.empty((a_ * b_ * d_, nb), device=dev, dtype=torch.bfloat16)
                yb = torch.empty_like(yq)

                def t_of(fn):
                    fn()
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        for _ in range(20):
                            fn()
                    g.replay()
                    torch.cuda.synchronize()
                    t0_, t1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0_.record()
                    g.replay()
                    t1_.record()
                    torch.cuda.synchronize()
                    del g
                    return t0_.elapsed_time(t1_) / 20

                ms8 = t_of(lambda: kb.forward_fp8(xq, wq, True, a_, b_, c_, d_, sx, sw, out=yq))
                ms16 = t_of(lambda: kb.forward_ex(xb, wb, True, a_, b_, c_, d_, out=yb))
                e8 = float((yq.float() - ref).norm() / ref.norm())
                e16 = float((yb.float() - ref).norm() / ref.norm())
                lowp.append({"pattern": list(pat), "batch": nb, "layout": "bs_last",
                             "fp8_e4m3_ms": round(ms8, 5), "fp8_rel_err_vs_fp32": round(e8, 5),
                             "bf16_ms": round(ms16, 5), "bf16_rel_err_vs_fp32": round(e16, 5)})
                del x32, w32, ref, xq, wq, xb, wb, yq, yb
        kb.check_device()

    # ---- chains: one chained call (layout-fused intermediates) against per-factor calls ------------
    chains = None
    if not args.no_vit and not args.only:
        import math
        chain_list = [("ks_vit_fc1", [(4, 192, 192, 1), (1, 768, 192, 4)], torch.float16),
                      ("ks_vit_fc2", [(1, 192, 768, 4), (4, 192, 192, 1)], torch.float16),
                      ("three_factor_1024", [(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)], torch.float16),
                      ("ks_vit_fc1", [(4, 192, 192, 1), (1, 768, 192, 4)], torch.float32),
                      ("three_factor_1024", [(1, 64, 64, 16), (4, 64, 64, 4), (16, 64, 64, 1)], torch.float32)]
        chains = []
        for name, pats, cdt in chain_list:
            gen = torch.Generator(device=dev).manual_seed(11)
            n_in = pats[0][0] * pats[0][2] * pats[0][3]
            xs = [torch.randn((BATCH, n_in), device=dev, dtype=cdt, generator=gen) for _ in range(4)]
            layer = kb.KSLinear(pats, weights=None, bias=False, algo="kernel", dtype=cdt,
                                bs_last=False, device=dev)

            def run_chained(x):
                return layer(x)

            def run_per_factor(x):
                for p_, w_ in zip(pats, layer.factors):
                    x = kb.forward_ex(x, w_, False, *p_)
                return x

            res = {}
            with torch.no_grad():
                for label, fn in (("chained", run_chained), ("per_factor", run_per_factor)):
                    for x in xs[:2]:
                        fn(x)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        for r in range(8):
                            fn(xs[r % 4])
                    g.replay()
                    torch.cuda.synchronize()
                    t0_, t1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0_.record()
                    g.replay()
                    t1_.record()
                    torch.cuda.synchronize()
                    res[label] = t0_.elapsed_time(t1_) / 8
                    del g
                ya, yb = run_chained(xs[0]).float(), run_per_factor(xs[0]).float()
                rel = float((ya - yb).norm() / yb.norm())
            chains.append({"chain": name, "patterns": [list(p_) for p_ in pats],
                           "dtype": "fp16" if cdt == torch.float16 else "fp32",
                           "layout": "bs_first", "ms_chained": round(res["chained"], 5),
                           "ms_per_factor": round(res["per_factor"], 5),
                           "speedup": round(res["per_factor"] / res["chained"], 3),
                           "rel_diff_between_the_two": rel})
            del layer, xs
        # the KS-ViT-B MLP pair: fc1 -> GELU -> fc2 on batch-first tokens.  Chained: two library calls,
        # the 3072-feature activations kept batch-last between them (layout-changing d = 1 factors), GELU
        # in fc1's epilogue.  Per factor: four batch-first factor calls and a separate GELU kernel.
        with torch.no_grad():
            gen = torch.Generator(device=dev).manual_seed(12)
            xs = [torch.randn((BATCH, 768), device=dev, dtype=torch.float16, generator=gen) for _ in range(4)]
            p1, p2 = chain_list[0][1], chain_list[1][1]
            fc1 = kb.KSLinear(p1, bias=True, algo="kernel", dtype=torch.float16, bs_last=False, device=dev,
                              out_bs_last=True, activation="gelu")
            fc2 = kb.KSLinear(p2, bias=True, algo="kernel", dtype=torch.float16, bs_last=True, device=dev,
                              out_bs_last=False)
            b1, b2 = fc1.bias.reshape(-1), fc2.bias.reshape(-1)

            def mlp_chained(x):
                return fc2(fc1(x))

            def mlp_per_factor(x):
                h = kb.forward_ex(x, fc1.factors[0], False, *p1[0])
                h = kb.forward_ex(h, fc1.factors[1], False, *p1[1], bias=b1)
                h = torch.nn.functional.gelu(h)
                h = kb.forward_ex(h, fc2.factors[0], False, *p2[0])
                return kb.forward_ex(h, fc2.factors[1], False, *p2[1], bias=b2)

            res = {}
            for label, fn in (("chained", mlp_chained), ("per_factor", mlp_per_factor)):
                for x in xs[:2]:
                    fn(x)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for r in range(8):
                        fn(xs[r % 4])
                g.replay()
                torch.cuda.synchronize()
                t0_, t1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0_.record()
                g.replay()
                t1_.record()
                torch.cuda.synchronize()
                res[label] = t0_.elapsed_time(t1_) / 8
                del g
            ya, yb = mlp_chained(xs[0]).float(), mlp_per_factor(xs[0]).float()
            chains.append({"chain": "ks_vit_mlp_pair (fc1, GELU, fc2)", "patterns": [list(p_) for p_ in p1 + p2],
                           "dtype": "fp16", "layout": "bs_first tokens in and out",
                           "ms_chained": round(res["chained"], 5), "ms_per_factor": round(res["per_factor"], 5),
                           "speedup": round(res["per_factor"] / res["chained"], 3),
                           "rel_diff_between_the_two": float((ya - yb).norm() / yb.norm())})
            del fc1, fc2, xs
        kb.check_device()

    if rank != 0:
        return

    # ---- CPU baseline: bounded sample on the host cores (rank 0, N = 1 only) -----------------
    cpu = None
    if world == 1 and not args.no_cpu:
        use_all_host_threads()
        algos = ("einsum", "bmm")
        acc = {al: [0.0, 0.0] for al in algos}
        passes, t_start = 0, time.perf_counter()
        while time.perf_counter() - t_start < 20.0 and passes < 10:
            for al, (f, s_) in cpu_reference_pass(REF_COLS, seed=passes, algos=algos).items():
                acc[al][0] += f
                acc[al][1] += s_
            passes += 1
        rates = {al: acc[al][0] / acc[al][1] / 1e12 for al in algos}
        cpu = {"value": rates["einsum"], "unit": "TFLOP/s", "cores": torch.get_num_threads(),
               "kind": "port", "einsum_tflops": round(rates["einsum"], 4), "bmm_tflops": round(rates["bmm"], 4),
               "sample": f"{passes} passes; " + reference_sample_text(algos)}

    # The line ends with what a reader who keeps only its tail needs: the compact per-case table
    # comes first, the summary objects after it.
    per_compact = [[q["dtype"], "L" if q["layout"] == "bs_last" else "F", q["pattern"], q["ms"],
                    q["roofline_frac"], q["bound"], q["kernel"]] for q in per]
    line = {
        "metric": "ksmm_sweep_throughput", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (three tf32 tensor-core products per term where the default dispatch picks that "
                 "kernel, else fp32 FFMA) + f16; fp32 accumulate",
        "data": "synthetic",
        "config": workload_config(),
        "per_pattern_columns": ["dtype", "layout (L = batch-last, F = batch-first)", "pattern", "ms",
                                "fraction of roofline", "bound", "kernel"],
        "per_pattern": per_compact,
        "per_pattern_ms_ffma_family": {f"{q['dtype']}:{q['layout']}:{','.join(map(str, q['pattern']))}": q["ms_ffma_family"]
                                       for q in per if q["ms_ffma_family"] is not None},
        "ffma_peak_tflops": round(ffma_peak, 2), "fp32_ffma_only": fp32_exact,
        "fp8_bf16": lowp, "chains": chains, "ksvit_b": ksvit,
        "roofline_hbm": roofline_of(per[dom_hbm], cs[dom_hbm]) if dom_hbm is not None else None,
        "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e,
        "roofline": roofline_of(per[dom], cs[dom]),
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-vit", action="store_true", help="skip the KS-ViT-B/16 forward timing")
    ap.add_argument("--no-ffma-compare", action="store_true",
                    help="skip re-timing the fp32 cases on the FFMA family (the fp32_ffma_only line)")
    ap.add_argument("--sweep-configs", action="store_true",
                    help="also time every tile configuration of every case (printed to stderr)")
    ap.add_argument("--profile-case", default=None, choices=["mlp_pair", "wgrad", "qkv", "chain_fp32"],
                    help="run a few launches of a chain / backward / grouped workload and exit (profiler captures)")
    ap.add_argument("--only", default=None,
                    help='restrict the sweep: "dtype:layout:a,b,c,d", e.g. "fp16:bs_last:1,768,192,4"')
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.profile_case:
        run_profile_case(args.profile_case, local_rank)
        return
    if world > 1:
        torch.cuda.set_device(local_rank)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
