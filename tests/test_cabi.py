"""The C-ABI library loads and exports everything include/ksmm_cu.h declares;
argument validation runs without a GPU (no compute call is made here)."""
import ctypes
import os
import re

import pytest

from ksmm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ksmm_cu.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ksmm_cu_\w+)\s*\(", text)))


def test_header_and_binding_list_agree():
    assert declared_symbols() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.ksmm_cu_version() >= 100
    assert lib.ksmm_cu_status_string(0) == b"ok"
    assert b"timed out" in lib.ksmm_cu_status_string(_lib.KSMM_ERR_DEVICE_TIMEOUT)
    assert lib.ksmm_cu_status_string(12345) == b"unknown status"


def test_null_pointers_are_rejected_not_dereferenced():
    lib = _lib.load()
    st = lib.ksmm_cu_forward(None, None, None, 8, 1, 2, 3, 4, _lib.KSMM_F32, 1, None)
    assert st == _lib.KSMM_ERR_BAD_ARGUMENT
    assert b"null pointer" in lib.ksmm_cu_last_error()
    with pytest.raises(_lib.KsmmError):
        _lib.check(st)


def test_bad_pattern_dtype_layout():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.ksmm_cu_forward(p, p, p, 8, 0, 2, 3, 4, _lib.KSMM_F32, 1, None) == _lib.KSMM_ERR_BAD_ARGUMENT
    assert lib.ksmm_cu_forward(p, p, p, -1, 1, 2, 3, 4, _lib.KSMM_F32, 1, None) == _lib.KSMM_ERR_BAD_ARGUMENT
    assert lib.ksmm_cu_forward(p, p, p, 8, 1, 2, 3, 4, 9, 1, None) == _lib.KSMM_ERR_BAD_ARGUMENT
    assert lib.ksmm_cu_forward(p, p, p, 8, 1, 2, 3, 4, _lib.KSMM_F32, 2, None) == _lib.KSMM_ERR_BAD_ARGUMENT
    # fp8 through the plain call has no output type / scale: explicit refusal
    assert lib.ksmm_cu_forward(p, p, p, 8, 1, 2, 3, 4, _lib.KSMM_F8E4M3, 1, None) == _lib.KSMM_ERR_UNSUPPORTED
    # empty batch is legal and launches nothing
    before = lib.ksmm_cu_launch_count()
    assert lib.ksmm_cu_forward(p, p, p, 0, 1, 2, 3, 4, _lib.KSMM_F32, 1, None) == _lib.KSMM_OK
    assert lib.ksmm_cu_launch_count() == before


def test_chain_validation_and_workspace():
    lib = _lib.load()
    pats = _lib.int32_array([6, 64, 64, 1, 1, 768, 192, 2])
    # intermediate is 6*64*1 = 384 features of fp32
    assert lib.ksmm_cu_chain_workspace_bytes(2, pats, 25088, _lib.KSMM_F32) == 384 * 25088 * 4
    assert lib.ksmm_cu_chain_workspace_bytes(1, pats, 25088, _lib.KSMM_F32) == 0
    three = _lib.int32_array([1, 64, 64, 16, 4, 64, 64, 4, 16, 64, 64, 1])
    assert lib.ksmm_cu_chain_workspace_bytes(3, three, 128, _lib.KSMM_F16) == 2 * 1024 * 128 * 2
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    vals = (ctypes.c_void_p * 2)(p, p)
    # mismatched chain
    bad = _lib.int32_array([6, 64, 64, 1, 1, 768, 100, 2])
    st = lib.ksmm_cu_chain_forward(p, vals, p, None, None, 0, 16, 2, bad, _lib.KSMM_F32, 1, None)
    assert st == _lib.KSMM_ERR_BAD_ARGUMENT and b"expects" in lib.ksmm_cu_last_error()
    # missing workspace
    st = lib.ksmm_cu_chain_forward(p, vals, p, None, None, 0, 16, 2, pats, _lib.KSMM_F32, 1, None)
    assert st == _lib.KSMM_ERR_WORKSPACE


def test_config_tables():
    lib = _lib.load()
    assert lib.ksmm_cu_num_configs(_lib.KSMM_ALGO_SIMT) == 9
    assert lib.ksmm_cu_num_configs(_lib.KSMM_ALGO_TC) >= 2
    assert lib.ksmm_cu_num_configs(99) == 0
    sup = lib.ksmm_cu_config_supported
    F16, F32, F8, BF16 = _lib.KSMM_F16, _lib.KSMM_F32, _lib.KSMM_F8E4M3, _lib.KSMM_BF16
    # the fp32 FFMA family takes anything
    assert sup(_lib.KSMM_ALGO_SIMT, 0, 25088, 1, 449, 514, 3, F32, F32, 0) == 1
    # tensor-core family: TMA stride rules; fp32 (three tf32 products) covers batch-last and
    # batch-first d = 1; configuration 0 picks the j tile, 1..3 force 128, 96, 64 columns
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 1, 768, 192, 4, F16, F16, 1) == 1
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 1, 768, 192, 4, F32, F32, 1) == 1
    assert sup(_lib.KSMM_ALGO_TC, 3, 25088, 1, 768, 192, 4, F32, F32, 1) == 1
    assert sup(_lib.KSMM_ALGO_TC, 4, 25088, 1, 768, 192, 4, F32, F32, 1) == 0
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 1, 768, 192, 4, F32, F32, 0) == 0
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 4, 192, 192, 1, F32, F32, 0) == 1
    assert sup(_lib.KSMM_ALGO_TC, 0, 25080, 4, 192, 192, 1, F32, F32, 1) == 0   # batch % 32 != 0
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 4, 200, 192, 1, F32, F32, 1) == 0   # b % 32 != 0
    assert sup(_lib.KSMM_ALGO_TC, 0, 25087, 1, 768, 192, 4, F16, F16, 1) == 0   # batch*2 % 16 != 0
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 1, 449, 192, 4, F16, F16, 1) == 0   # b*2 % 16 != 0
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 4, 192, 192, 1, BF16, BF16, 0) == 1
    assert sup(_lib.KSMM_ALGO_TC, 0, 25088, 1, 768, 192, 4, F8, BF16, 1) == 1
    assert sup(_lib.KSMM_ALGO_TC, 4, 25088, 1, 768, 192, 4, F8, BF16, 1) == 0   # N tile 64 < one fp8 box row


def test_choice_cache_round_trip():
    lib = _lib.load()
    algo, cfg = ctypes.c_int(-1), ctypes.c_int(-1)
    assert lib.ksmm_cu_get_choice(77, 1, 64, 64, 1, 0, 0, 1, ctypes.byref(algo), ctypes.byref(cfg)) != 0
    assert lib.ksmm_cu_set_choice(77, 1, 64, 64, 1, 0, 0, 1, _lib.KSMM_ALGO_SIMT, 1) == 0
    assert lib.ksmm_cu_get_choice(77, 1, 64, 64, 1, 0, 0, 1, ctypes.byref(algo), ctypes.byref(cfg)) == 0
    assert (algo.value, cfg.value) == (_lib.KSMM_ALGO_SIMT, 1)
    # a configuration that cannot run the problem is refused
    assert lib.ksmm_cu_set_choice(77, 1, 64, 64, 1, 0, 0, 1, _lib.KSMM_ALGO_TC, 0) == _lib.KSMM_ERR_UNSUPPORTED


def test_default_choice_reports_family_and_conversion_path():
    """What the automatic dispatch would run (no launch is made): fp32 and fp16 benchmark factors go
    to the tensor-core family; 16-bit batch-first factors have direct kernels for d = 2, 4 and
    multiples of 8, other d and fp32 with d > 1 go through the layout conversion; a block too
    small for the tensor cores stays on the FFMA family."""
    import torch
    import ksmm_b200 as kb
    assert kb.default_choice((1, 768, 192, 4), 4096, torch.float32, True)[::2] == ("tensor", False)
    assert kb.default_choice((1, 768, 192, 4), 4096, torch.float16, False)[::2] == ("tensor", False)
    assert kb.default_choice((1, 64, 64, 16), 4096, torch.float16, False)[::2] == ("tensor", False)
    assert kb.default_choice((1, 64, 64, 12), 4096, torch.float16, False)[::2] == ("tensor", True)
    assert kb.default_choice((1, 64, 64, 16), 4096, torch.float32, False)[::2] == ("tensor", True)
    assert kb.default_choice((4, 64, 64, 4), 4096, torch.float32, False)[::2] == ("ffma", False)
    assert kb.default_choice((1, 8, 8, 1), 4096, torch.float32, True)[::2] == ("ffma", False)
    assert kb.default_choice((1, 64, 2048, 1), 4096, torch.float32, True)[0] == "ffma"  # c > 1024


def test_layout_scratch_planning():
    """Which calls need memory beside their operands, and how much: only batch-first factors with
    d > 1 that run through the layout conversion (two transposed copies).  A chain workspace of the
    `_ex` size holds that as well, so a chain call given that much never allocates."""
    lib = _lib.load()
    F16, F32 = _lib.KSMM_F16, _lib.KSMM_F32
    batch = 4096

    def desc(pattern, dtype, bs_last, algo=0, config=-1):
        a, b, c, d = pattern
        return _lib.ForwardDesc(input=256, values=256, output=256, bias=None, batch=batch, a=a, b=b, c=c, d=d,
                                in_dtype=dtype, out_dtype=dtype, bs_last=bs_last, algo=algo, config=config,
                                alpha=1.0, activation=0)

    need = lib.ksmm_cu_layout_scratch_bytes
    assert need(ctypes.byref(desc((1, 64, 64, 16), F16, 1))) == 0
    assert need(ctypes.byref(desc((4, 192, 192, 1), F16, 0))) == 0
    assert need(ctypes.byref(desc((1, 64, 64, 3), F16, 0))) == 2 * 192 * batch * 2
    assert need(ctypes.byref(desc((1, 768, 192, 4), F32, 0))) == (768 + 3072) * batch * 4
    # forced families: the conversion path by name; a direct kernel needs nothing
    assert need(ctypes.byref(desc((1, 64, 64, 4), F16, 0, _lib.KSMM_ALGO_CONVERT, 0))) == 2 * 256 * batch * 2
    assert need(ctypes.byref(desc((1, 64, 64, 4), F16, 0, _lib.KSMM_ALGO_SIMT, 0))) == 0
    # chains: intermediates, plus the largest layout scratch of any factor in that layout
    pats = _lib.int32_array([4, 192, 192, 1, 1, 768, 192, 4])
    inter = lib.ksmm_cu_chain_workspace_bytes(2, pats, batch, F32)
    assert inter == 768 * batch * 4
    assert lib.ksmm_cu_chain_workspace_bytes_ex(2, pats, batch, F32, 1) == inter
    assert lib.ksmm_cu_chain_workspace_bytes_ex(2, pats, batch, F32, 0) == inter + (768 + 3072) * batch * 4
    assert lib.ksmm_cu_chain_workspace_bytes_ex(2, pats, batch, F16, 0) == 768 * batch * 2  # direct kernels
    one = _lib.int32_array([1, 64, 64, 3])
    assert lib.ksmm_cu_chain_workspace_bytes_ex(1, one, batch, F16, 0) == 2 * 192 * batch * 2
    assert lib.ksmm_cu_alloc_count() == 0          # planning never allocates (and there is no device here)


def test_conversion_family_in_the_choice_cache():
    lib = _lib.load()
    assert lib.ksmm_cu_num_configs(_lib.KSMM_ALGO_CONVERT) == 1
    sup = lib.ksmm_cu_config_supported
    assert sup(_lib.KSMM_ALGO_CONVERT, 0, 512, 1, 64, 64, 16, _lib.KSMM_F16, _lib.KSMM_F16, 0) == 1
    assert sup(_lib.KSMM_ALGO_CONVERT, 0, 512, 1, 64, 64, 16, _lib.KSMM_F16, _lib.KSMM_F16, 1) == 0  # batch-last
    assert sup(_lib.KSMM_ALGO_CONVERT, 0, 512, 16, 64, 64, 1, _lib.KSMM_F16, _lib.KSMM_F16, 0) == 0  # d = 1
    assert lib.ksmm_cu_set_choice(78, 1, 64, 64, 4, 1, 1, 0, _lib.KSMM_ALGO_CONVERT, 0) == 0
    algo, cfg = ctypes.c_int(-1), ctypes.c_int(-1)
    assert lib.ksmm_cu_get_choice(78, 1, 64, 64, 4, 1, 1, 0, ctypes.byref(algo), ctypes.byref(cfg)) == 0
    assert (algo.value, cfg.value) == (_lib.KSMM_ALGO_CONVERT, 0)
    assert lib.ksmm_cu_set_choice(78, 1, 64, 64, 4, 1, 1, 1, _lib.KSMM_ALGO_CONVERT, 0) == _lib.KSMM_ERR_UNSUPPORTED
