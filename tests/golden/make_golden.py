"""Generate tests/golden/ksmm_golden.npz from the UNMODIFIED reference.

Run once in a container where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <checkout>/src

The reference has no golden vectors of its own, so the pin is its own
``KSLinear`` run on the CPU with ``algo`` = dense, einsum and bmm
(src/ksmm_py/layer/kronecker_sparse/interface.py:116-478).  Inputs are NOT
stored: they are regenerated from ``numpy.random.RandomState(seed)`` (a frozen
stream) by ``tests/golden_cases.py``, which this script shares with the
tests.  Only the reference's outputs are stored.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from golden_cases import CASES, make_inputs  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to the reference's src/ directory")
    ap.add_argument("--out", default=os.path.join(HERE, "ksmm_golden.npz"))
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from ksmm_py.layer.kronecker_sparse.interface import (  # type: ignore
        KSLinear, from_kernel_format_to_dense, generate_factor)

    torch.set_num_threads(4)
    out = {}
    meta = {}
    for case in CASES:
        name = case["name"]
        x, ws, bias = make_inputs(case)
        tdt = {"float32": torch.float32, "float16": torch.float16}[case["dtype"]]
        xt = torch.from_numpy(x).to(tdt)
        wts = [torch.from_numpy(w).to(tdt) for w in ws]
        per_algo = {}
        for algo in case["algos"]:
            wl = wts
            if algo == "bmm":
                # the reference's bmm format conversion calls .view on a permuted
                # tensor (interface.py:35-36); hand it weights whose permutation
                # is already contiguous so that the view is legal for a>1 and d>1
                wl = [w.permute(0, 3, 1, 2).contiguous().permute(0, 2, 3, 1) for w in wts]
            layer = KSLinear(case["patterns"], weights=wl, bias=bias is not None, algo=algo,
                             dtype=tdt, bs_last=case["bs_last"], device="cpu")
            if bias is not None:
                with torch.no_grad():
                    layer.bias.copy_(torch.from_numpy(bias).to(tdt).reshape(layer.bias.shape))
            with torch.no_grad():
                y = layer(xt)
            per_algo[algo] = y.float().numpy()
        # kernel-format round trip pins the (a*d*c, b) weight layout
        for fi, (p, w) in enumerate(zip(case["patterns"], wts)):
            wk = generate_factor(*p, "kernel", w, tdt, "cpu")
            dense_from_kernel = from_kernel_format_to_dense(wk, p)
            if fi == 0 and case.get("store_kernel_format", False):
                out[f"{name}/kernel_format0"] = wk.float().numpy()
                out[f"{name}/dense_from_kernel0"] = dense_from_kernel.float().numpy()
        first = case["algos"][0]
        out[f"{name}/y"] = per_algo[first]
        spread = {}
        for algo, y in per_algo.items():
            ref = per_algo[first].astype(np.float64)
            spread[algo] = float(np.linalg.norm(y.astype(np.float64) - ref) / np.linalg.norm(ref))
        meta[name] = {"algo": first, "spread_vs_first": spread, "shape": list(per_algo[first].shape)}
        print(name, meta[name])
    out["__meta__"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
