"""Child process of tests/test_zz_no_alloc.py.

Runs ksmm_cu_chain_forward_static as the FIRST library call of a fresh process
(no ordinary chain call has grown any library-owned buffer yet), twice in a row
per case, and reports for every case: how many device allocations the library
made during the two calls (its own counter), how much free device memory moved
(cudaMemGetInfo through torch), and the error against the ordinary entry point
(called afterwards) and against the CPU oracle.  Prints one JSON line.
"""
import ctypes
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import ksmm_b200 as kb  # noqa: E402
from golden_cases import make_weights  # noqa: E402
from ksmm_b200 import _lib  # noqa: E402
from oracle import ksmm_oracle as ko  # noqa: E402

DEV = "cuda:0"

# (patterns, dtype, bs_last, batches of the two calls)
CASES = [
    ([(4, 192, 192, 1), (1, 768, 192, 4)], torch.float32, True, (1024, 1536)),
    ([(4, 192, 192, 1), (1, 768, 192, 4)], torch.float32, False, (1024, 1536)),   # fp32 batch-first d = 4: layout conversion
    ([(4, 192, 192, 1), (1, 768, 192, 4)], torch.float16, True, (1024, 1536)),
    ([(4, 192, 192, 1), (1, 768, 192, 4)], torch.float16, False, (1024, 1536)),
    ([(1, 64, 64, 16), (16, 64, 64, 1)], torch.float16, False, (2048, 1024)),     # fp16 batch-first d = 16
    ([(4, 64, 64, 4), (16, 64, 64, 1)], torch.float32, False, (2048, 2048)),      # fp32 batch-first d = 4, small blocks
    ([(1, 96, 48, 8)], torch.float16, False, (1024, 1024)),                       # one factor, d = 8: scratch, no intermediate
]


def main():
    lib = _lib.load()
    torch.zeros(1, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    results = []
    prepared = []
    for ci, (pats, dtype, bs_last, batches) in enumerate(CASES):
        for call, batch in enumerate(batches):
            rng = np.random.RandomState(50 + 10 * ci + call)
            ws = make_weights(pats, rng)
            n_in = pats[0][0] * pats[0][2] * pats[0][3]
            n_out = pats[-1][0] * pats[-1][1] * pats[-1][3]
            x = torch.from_numpy(rng.standard_normal((n_in, batch) if bs_last else (batch, n_in)).astype(np.float32))
            xg = x.to(dtype).to(DEV)
            wk = [kb.generate_factor(*p, "kernel", torch.from_numpy(w), dtype, DEV) for p, w in zip(pats, ws)]
            bias = torch.from_numpy(rng.standard_normal(n_out).astype(np.float32)).to(dtype).to(DEV)
            out = torch.full((n_out, batch) if bs_last else (batch, n_out), float("nan"), dtype=dtype, device=DEV)
            prepared.append((ci, call, pats, dtype, bs_last, batch, xg, wk, bias, out, ws))
    torch.cuda.synchronize()
    # ---- the static calls come first: nothing has grown a library-owned buffer yet ----
    for (ci, call, pats, dtype, bs_last, batch, xg, wk, bias, out, ws) in prepared:
        flat = _lib.int32_array([v for p in pats for v in p])
        vals = (ctypes.c_void_p * len(wk))(*[w.data_ptr() for w in wk])
        code = kb.kernel.dtype_code(dtype)
        torch.cuda.synchronize()
        allocs0 = lib.ksmm_cu_alloc_count()
        free0 = torch.cuda.mem_get_info()[0]
        st = lib.ksmm_cu_chain_forward_static(xg.data_ptr(), vals, out.data_ptr(), bias.data_ptr(), batch,
                                              len(pats), flat, code, int(bs_last), stream)
        msg = lib.ksmm_cu_last_error().decode() if st else ""
        torch.cuda.synchronize()
        results.append(dict(case=ci, call=call, status=int(st), message=msg,
                            allocs=int(lib.ksmm_cu_alloc_count() - allocs0),
                            free_delta=int(free0 - torch.cuda.mem_get_info()[0])))
    # ---- then the ordinary entry point and the oracle ----
    for res, (ci, call, pats, dtype, bs_last, batch, xg, wk, bias, out, ws) in zip(results, prepared):
        ref = kb.chain_forward(xg, wk, pats, bs_last, bias=bias)
        half = dtype == torch.float16
        w_seen = [w.astype(np.float16).astype(np.float32) if half else w for w in ws]
        oracle = ko.chain_apply(xg.float().cpu().numpy(), w_seen, bs_last, bias=bias.float().cpu().numpy(),
                                round_to=np.float16 if half else None)
        o = out.float().cpu().numpy()
        res["nan"] = bool(np.isnan(o).any())
        res["err_vs_ordinary"] = float(ko.rel_fro_error(o, ref.float().cpu().numpy()))
        res["err_vs_oracle"] = float(ko.rel_fro_error(o, oracle))
        res["half"] = half
    kb.check_device()
    print("NO_ALLOC_RESULT " + json.dumps(results))


if __name__ == "__main__":
    main()
