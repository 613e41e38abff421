"""Host-side logic of the Python layer that needs no GPU."""
import os

import numpy as np
import pytest
import torch

from golden_cases import CASES, make_inputs
from ksmm_b200 import interface as itf
from ksmm_b200 import kernel as kmod
from oracle import ksmm_oracle as ko

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "ksmm_golden.npz"))


def test_kernel_algo_refuses_cpu_like_the_reference():
    # interface.py:163-164 of the reference raises Exception("kernel expects device='cuda'.")
    with pytest.raises(Exception, match="kernel expects device='cuda'"):
        itf.KSLinear([(1, 4, 4, 1)], algo="kernel", device="cpu")


def test_other_algorithms_are_not_silently_emulated():
    with pytest.raises(NotImplementedError):
        itf.KSLinear([(1, 4, 4, 1)], algo="dense", device="cuda")


def test_mismatched_chain_is_rejected():
    with pytest.raises(ValueError):
        itf.KSLinear([(6, 64, 64, 1), (1, 768, 100, 2)], algo="kernel", device="cuda")


@pytest.mark.parametrize("name", ["f_1_16_16_1_last", "f_2_3_5_4_last"])
def test_generate_factor_layout_matches_reference(name):
    case = next(c for c in CASES if c["name"] == name)
    _, ws, _ = make_inputs(case)
    p = case["patterns"][0]
    wk = itf.generate_factor(*p, "kernel", torch.from_numpy(ws[0]), torch.float32, "cpu")
    assert np.array_equal(wk.numpy(), GOLDEN[name + "/kernel_format0"])
    dense = itf.from_kernel_format_to_dense(wk, p)
    assert np.array_equal(dense.numpy(), GOLDEN[name + "/dense_from_kernel0"])
    assert np.array_equal(itf.from_kernel_format_to_abcd(wk, p).numpy(), ws[0])


def test_default_init_range():
    wk = itf.generate_factor(2, 8, 16, 3, "kernel", None, torch.float32, "cpu")
    assert tuple(wk.shape) == (2 * 3 * 16, 8)
    assert float(wk.abs().max()) <= 0.25 + 1e-6


def test_dtype_codes_and_strings():
    assert kmod.dtype_code(torch.float32) == 0 and kmod.dtype_code("torch.float") == 0
    assert kmod.dtype_code(torch.float16) == 1 and kmod.dtype_code("torch.half") == 1
    assert kmod.dtype_code(torch.bfloat16) == 2
    assert kmod.dtype_code("torch.float8_e4m3fn") == 3
    with pytest.raises(TypeError):
        kmod.dtype_code(torch.float64)


def test_operator_rejects_cpu_tensors_and_bad_shapes():
    x = torch.zeros(8, 4)
    w = torch.zeros(8, 2)
    with pytest.raises(ValueError, match="CUDA"):
        kmod.Kernel.forward(x, w, True, 1, 2, 8, 1, torch.float32)


def test_quantize_e4m3_matches_oracle():
    rng = np.random.RandomState(2)
    x = rng.standard_normal((64, 32)).astype(np.float32)
    q, s = kmod.quantize_e4m3(torch.from_numpy(x))
    s_ref = ko.e4m3_scale(x)
    assert abs(s - s_ref) < 1e-7 * s_ref + 1e-12
    ref = ko.quantize_e4m3(x.astype(np.float32) / np.float32(s))
    assert np.array_equal(q.float().numpy(), ref.astype(np.float32))


def test_tuner_table_round_trip(tmp_path):
    """A saved tuner table is pushed back into the library without timing anything."""
    import json
    from ksmm_b200 import _lib, tuner
    table = {"format": "ksmm_b200.tuner/1", "entries": [
        {"sm": 100, "dtype": "f16", "out_dtype": "f16", "bs_last": True, "pattern": [1, 768, 192, 4],
         "batch": 25088, "family": "tensor", "config": 0, "ms": 0.047},
        {"sm": 100, "dtype": "f32", "out_dtype": "f32", "bs_last": True, "pattern": [1, 768, 192, 4],
         "batch": 25088, "family": "ffma", "config": 7, "ms": 0.57},
        # an entry the build cannot run (the fp32 tensor kernel has configurations 0..3) is skipped
        {"sm": 100, "dtype": "f32", "out_dtype": "f32", "bs_last": True, "pattern": [1, 64, 64, 1],
         "batch": 64, "family": "tensor", "config": 4, "ms": 1.0},
        {"sm": 90, "dtype": "f16", "out_dtype": "f16", "bs_last": True, "pattern": [1, 64, 64, 1],
         "batch": 64, "family": "tensor", "config": 1, "ms": 1.0}]}
    path = tmp_path / "tuned.json"
    path.write_text(json.dumps(table))
    assert tuner.load(str(path), sm=100) == 2
    lib = _lib.load()
    import ctypes
    algo, cfg = ctypes.c_int(), ctypes.c_int()
    assert lib.ksmm_cu_get_choice(25088, 1, 768, 192, 4, _lib.KSMM_F32, _lib.KSMM_F32, 1,
                                  ctypes.byref(algo), ctypes.byref(cfg)) == 0
    assert (algo.value, cfg.value) == (_lib.KSMM_ALGO_SIMT, 7)
    out = tmp_path / "again.json"
    tuner.save(str(out))
    assert len(json.loads(out.read_text())["entries"]) >= 2
    best = tmp_path / "kernel.best"
    tuner.export_best_rows(str(best))
    rows = best.read_text().splitlines()
    assert rows[0] == tuner.BEST_HEADER
    assert any(r.split()[:5] == ["25088", "1", "768", "192", "4"] for r in rows[1:])
    assert len(tuner.read_best_rows(str(best))) == len(rows) - 1      # its own export parses back
    with pytest.raises(ValueError):
        bad = tmp_path / "bad.json"
        bad.write_text("{}")
        tuner.load(str(bad))


def test_reference_best_table_as_priors(tmp_path):
    """A table in the reference's `.best` format (batch a b c d TILEX TILEK TILEY TX TY VSIZE ms std
    mse, one header line) names the problems to tune and seeds the FFMA family's configuration for
    the problems that only that family can run; tensor-core problems are left to the heuristic."""
    import ctypes

    import torch

    from ksmm_b200 import _lib, tuner
    path = tmp_path / "kernel_bs_last_float.best"
    path.write_text(tuner.BEST_HEADER + "\n"
                    "25088 1 16 16 6 16 16 64 4 4 4 0.0301 0.0002 1.1e-08\n"      # tiny block: FFMA only
                    "25088 2 8 8 3 8 8 128 2 8 4 0.0202 0.0002 1.0e-08\n"
                    "12544 1 768 192 2 64 16 64 8 4 4 0.9000 0.0010 2.0e-08\n")   # tensor-core kernel exists
    rows = tuner.read_best_rows(str(path))
    assert [r["pattern"] for r in rows] == [[1, 16, 16, 6], [2, 8, 8, 3], [1, 768, 192, 2]]
    assert rows[0]["tile"] == (16, 16, 64, 4, 4, 4) and rows[2]["ms"] == 0.9
    known, seeded = tuner.import_best_rows(str(path), torch.float32, True)
    assert known == [((1, 16, 16, 6), 25088), ((2, 8, 8, 3), 25088), ((1, 768, 192, 2), 12544)]
    assert seeded == 2
    lib = _lib.load()
    algo, cfg = ctypes.c_int(), ctypes.c_int()
    assert lib.ksmm_cu_get_choice(25088, 1, 16, 16, 6, 0, 0, 1, ctypes.byref(algo), ctypes.byref(cfg)) == 0
    assert (algo.value, cfg.value) == (_lib.KSMM_ALGO_SIMT, 3)            # 16 rows x 128 batch entries
    assert lib.ksmm_cu_get_choice(25088, 2, 8, 8, 3, 0, 0, 1, ctypes.byref(algo), ctypes.byref(cfg)) == 0
    assert (algo.value, cfg.value) == (_lib.KSMM_ALGO_SIMT, 5)            # 8 rows
    assert lib.ksmm_cu_get_choice(12544, 1, 768, 192, 2, 0, 0, 1, ctypes.byref(algo), ctypes.byref(cfg)) != 0
    assert tuner.ffma_config_from_tile(64, 256) == 4 and tuner.ffma_config_from_tile(128, 128) == 0
    with pytest.raises(ValueError):
        (tmp_path / "x.best").write_text("1 2 3\n")
        tuner.read_best_rows(str(tmp_path / "x.best"))
