"""Per-factor and chained operators on top of the C ABI.

Mirrors ``Kernel.forward(input, factor, bs_last, a, b, c, d, dtype, vsize)`` of
the reference (src/ksmm_py/layer/kronecker_sparse/kernel.py:63-73) and the
pybind signature below it (kernel.cpp:25-50): same argument order and meaning,
same ownership (inputs borrowed, output freshly allocated on the input's
device, kernel.cu:50-52).  Differences, all on purpose:

* nothing is generated or compiled at call time (the reference rewrites its
  own .cuh/.cpp files and runs nvcc per new pattern, kernel.py:92-298);
* launches go to torch's *current* stream, not the legacy default stream;
* failures raise (the reference asserts or silently returns garbage for fp8,
  kernel.cu:66-82, 123-125);
* ``vsize`` is accepted and ignored: vector widths are chosen by the library.

torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import ForwardDesc, KsmmError  # noqa: F401

_DTYPE_CODE = {
    torch.float32: _lib.KSMM_F32,
    torch.float16: _lib.KSMM_F16,
    torch.bfloat16: _lib.KSMM_BF16,
    torch.float8_e4m3fn: _lib.KSMM_F8E4M3,
}
# dtype strings that the reference's extension receives (kernel.cu:66,83-84,103-104)
_DTYPE_FROM_STR = {
    "torch.float32": torch.float32, "torch.float": torch.float32,
    "torch.float16": torch.float16, "torch.half": torch.float16,
    "torch.bfloat16": torch.bfloat16,
    "torch.float8_e4m3fn": torch.float8_e4m3fn,
}


def dtype_code(dtype):
    if isinstance(dtype, str):
        dtype = _DTYPE_FROM_STR.get(dtype)
    if dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {dtype}: expected float32, float16, bfloat16 or float8_e4m3fn")
    return _DTYPE_CODE[dtype]


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check_inputs(input, factor, bs_last, a, b, c, d):
    if not input.is_cuda:
        raise ValueError("input must be a CUDA tensor")
    if not factor.is_cuda:
        raise ValueError("factor must be a CUDA tensor")
    if not input.is_contiguous():
        raise ValueError("input must be contiguous")
    if not factor.is_contiguous():
        raise ValueError("factor must be contiguous")
    if input.dim() != 2:
        raise ValueError(f"input must be 2-D, got shape {tuple(input.shape)}")
    feat = input.shape[0] if bs_last else input.shape[1]
    if feat != a * c * d:
        raise ValueError(f"input has {feat} features, pattern ({a},{b},{c},{d}) expects {a * c * d}")
    if tuple(factor.shape) != (a * d * c, b):
        raise ValueError(f"factor must have shape ({a * d * c}, {b}) = (a*d*c, b), got {tuple(factor.shape)}")
    if factor.dtype != input.dtype:
        raise TypeError(f"factor dtype {factor.dtype} differs from input dtype {input.dtype}")
    if factor.device != input.device:
        raise ValueError("input and factor live on different devices")


def forward_ex(input, factor, bs_last, a, b, c, d, *, out_dtype=None, alpha=1.0, bias=None,
               algo=_lib.KSMM_ALGO_AUTO, config=-1, out=None, activation=None, residual=None):
    """One factor with every option of ``ksmm_cu_forward_ex``."""
    lib = _lib.load()
    bs_last = int(bool(bs_last))
    _check_inputs(input, factor, bs_last, a, b, c, d)
    out_dtype = input.dtype if out_dtype is None else out_dtype
    if input.dtype == torch.float8_e4m3fn and out_dtype == torch.float8_e4m3fn:
        raise TypeError("fp8 inputs need a bfloat16, float16 or float32 output")
    batch = input.shape[1] if bs_last else input.shape[0]
    shape = (a * b * d, batch) if bs_last else (batch, a * b * d)
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=input.device)
    elif tuple(out.shape) != shape or out.dtype != out_dtype or not out.is_contiguous():
        raise ValueError("out has the wrong shape, dtype or strides")
    if bias is not None:
        if bias.numel() != a * b * d or bias.dtype != out_dtype or not bias.is_contiguous():
            raise ValueError("bias must hold a*b*d contiguous elements of the output dtype")
    if residual is not None and (tuple(residual.shape) != shape or residual.dtype != out_dtype
                                 or not residual.is_contiguous() or residual.device != input.device):
        raise ValueError("residual must be a contiguous tensor shaped and typed like the output")
    desc = ForwardDesc(
        input=input.data_ptr(), values=factor.data_ptr(), output=out.data_ptr(),
        residual=residual.data_ptr() if residual is not None else None,
        bias=bias.data_ptr() if bias is not None else None, batch=batch, a=a, b=b, c=c, d=d,
        in_dtype=dtype_code(input.dtype), out_dtype=dtype_code(out_dtype), bs_last=bs_last,
        algo=algo, config=config, alpha=float(alpha), activation=_lib.ACTIVATIONS[activation])
    # A factor that runs through a layout conversion needs room for its transposed copies.  It comes
    # from torch's allocator (stream-ordered, and legal inside a CUDA-graph capture), so that the
    # library never has to grow a buffer of its own on behalf of a Python caller.
    need = lib.ksmm_cu_layout_scratch_bytes(ctypes.byref(desc))
    if need:
        scratch = torch.empty(need, dtype=torch.uint8, device=input.device)
        desc.scratch, desc.scratch_bytes = scratch.data_ptr(), need
    with torch.cuda.device(input.device):
        _lib.check(lib.ksmm_cu_forward_ex(ctypes.byref(desc), _stream_ptr(input.device)))
    return out


def default_choice(pattern, batch, dtype, bs_last, out_dtype=None):
    """What the automatic dispatch runs for one factor: ``(family, config, via_transpose)`` with
    family ``"ffma"`` or ``"tensor"``; ``via_transpose`` is true when the call goes through the
    layout-conversion path (transpose, batch-last kernel, transpose)."""
    lib = _lib.load()
    a, b, c, d = (int(v) for v in pattern)
    out_dtype = dtype if out_dtype is None else out_dtype
    desc = ForwardDesc(input=256, values=256, output=256, bias=None, batch=int(batch), a=a, b=b, c=c,
                       d=d, in_dtype=dtype_code(dtype), out_dtype=dtype_code(out_dtype),
                       bs_last=int(bool(bs_last)), algo=0, config=-1, alpha=1.0, activation=0)
    algo, cfg, conv = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    _lib.check(lib.ksmm_cu_default_choice(ctypes.byref(desc), ctypes.byref(algo), ctypes.byref(cfg),
                                          ctypes.byref(conv)))
    return ("tensor" if algo.value == _lib.KSMM_ALGO_TC else "ffma"), cfg.value, bool(conv.value)


def alloc_count():
    """Device allocations made by the library itself since it was loaded."""
    return int(_lib.load().ksmm_cu_alloc_count())


class Kernel:
    """Drop-in for the reference's ``Kernel`` (kernel.py:62-329).  Inference
    only, like the reference (its ``backward`` is a stub, kernel.py:323-329)."""

    @staticmethod
    def forward(input, factor, bs_last, a, b, c, d, dtype=None, vsize=4):
        if dtype is not None:
            code = dtype_code(dtype)
            if code != dtype_code(input.dtype):
                raise TypeError(f"dtype argument {dtype} does not match the input's {input.dtype}")
        return forward_ex(input, factor, bs_last, a, b, c, d)


def forward(input, factor, bs_last, a, b, c, d, dtype, vsize=4):
    """Same signature as the reference extension's ``forward`` (kernel.cpp:25-45)."""
    return Kernel.forward(input, factor, bool(bs_last), a, b, c, d, dtype, vsize)


def chain_forward(input, factors, patterns, bs_last, bias=None, workspace=None, out=None,
                  activation=None, out_bs_last=None, residual=None):
    """All factors of one KSLinear in one library call (``ksmm_cu_chain_forward_layouts``).

    ``factors[f]`` is the kernel-format (a*d*c, b) weight of ``patterns[f]``;
    ``patterns[0]`` is applied first.  ``bias`` (out features, output dtype)
    and ``activation`` (None, "gelu" or "relu") are fused into the last factor.
    ``out_bs_last`` (default: same as ``bs_last``) asks for the output in the other
    layout: (out, batch) when true, (batch, out) when false.  ``residual`` (shaped like the
    output) is added last: ``act(chain(x) + bias) + residual``.
    """
    lib = _lib.load()
    bs_last = int(bool(bs_last))
    out_last = bs_last if out_bs_last is None else int(bool(out_bs_last))
    nf = len(patterns)
    if nf == 0 or len(factors) != nf:
        raise ValueError("need one factor per pattern")
    for f, (p, w) in enumerate(zip(patterns, factors)):
        a, b, c, d = p
        if f == 0:
            _check_inputs(input, w, bs_last, a, b, c, d)
        elif tuple(w.shape) != (a * d * c, b) or w.dtype != input.dtype or not w.is_contiguous() \
                or w.device != input.device:
            raise ValueError(f"factor {f} must be a contiguous ({a * d * c}, {b}) tensor of {input.dtype}")
    batch = input.shape[1] if bs_last else input.shape[0]
    la, lb, lc, ld = patterns[-1]
    n_out = la * lb * ld
    shape = (n_out, batch) if out_last else (batch, n_out)
    if out is None:
        out = torch.empty(shape, dtype=input.dtype, device=input.device)
    elif tuple(out.shape) != shape or out.dtype != input.dtype or not out.is_contiguous():
        raise ValueError("out has the wrong shape, dtype or strides")
    flat = [int(v) for p in patterns for v in p]
    pat = _lib.int32_array(flat)
    code = dtype_code(input.dtype)
    need = lib.ksmm_cu_chain_workspace_bytes_layouts(nf, pat, batch, code, bs_last, out_last)
    if need > 0 and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=input.device)
    if bias is not None and (bias.numel() != n_out or bias.dtype != input.dtype):
        raise ValueError("bias must hold out_size elements of the input dtype")
    if residual is not None and (tuple(residual.shape) != shape or residual.dtype != input.dtype
                                 or not residual.is_contiguous() or residual.device != input.device):
        raise ValueError("residual must be a contiguous tensor shaped and typed like the output")
    vals = (ctypes.c_void_p * nf)(*[w.data_ptr() for w in factors])
    desc = _lib.ChainDesc(
        input=input.data_ptr(), values=vals, output=out.data_ptr(),
        bias=bias.data_ptr() if bias is not None else None,
        residual=residual.data_ptr() if residual is not None else None,
        workspace=workspace.data_ptr() if workspace is not None else None,
        workspace_bytes=workspace.numel() * workspace.element_size() if workspace is not None else 0,
        batch=batch, nfactors=nf, patterns=pat, dtype=code, bs_last=bs_last, out_layout=2 if out_last else 1,
        activation=_lib.ACTIVATIONS[activation])
    with torch.cuda.device(input.device):
        _lib.check(lib.ksmm_cu_chain_forward_desc(ctypes.byref(desc), _stream_ptr(input.device)))
    return out


def grouped_chain_forward(input, stacked_factors, patterns, bs_last, groups, bias=None):
    """``groups`` chains with the same ``patterns`` on one shared input (``ksmm_cu_grouped_chain_forward``):
    ``stacked_factors[f]`` is the (groups * a*d*c, b) concatenation of the groups' kernel-format
    factors f.  Returns the stacked output (groups, out, batch) / (groups, batch, out); ``out[g]`` is
    group g's result, a contiguous tensor."""
    lib = _lib.load()
    bs_last = int(bool(bs_last))
    nf = len(patterns)
    if nf == 0 or len(stacked_factors) != nf or groups < 1:
        raise ValueError("need one stacked factor per pattern and at least one group")
    a0, b0, c0, d0 = patterns[0]
    if input.dim() != 2 or not input.is_cuda or not input.is_contiguous():
        raise ValueError("input must be a contiguous 2-D CUDA tensor")
    if (input.shape[0] if bs_last else input.shape[1]) != a0 * c0 * d0:
        raise ValueError(f"input has the wrong number of features for pattern {tuple(patterns[0])}")
    feats = a0 * c0 * d0
    for f, (p, w) in enumerate(zip(patterns, stacked_factors)):
        a, b, c, d = p
        if a * c * d != feats:
            raise ValueError(f"factor {f} expects {a * c * d} features but receives {feats}")
        if tuple(w.shape) != (groups * a * d * c, b) or w.dtype != input.dtype or not w.is_contiguous() \
                or w.device != input.device:
            raise ValueError(f"stacked factor {f} must be a contiguous ({groups * a * d * c}, {b}) tensor of {input.dtype}")
        feats = a * b * d
    batch = input.shape[1] if bs_last else input.shape[0]
    out = torch.empty((groups, feats, batch) if bs_last else (groups, batch, feats), dtype=input.dtype,
                      device=input.device)
    if bias is not None and (bias.numel() != groups * feats or bias.dtype != input.dtype or not bias.is_contiguous()):
        raise ValueError("bias must hold groups * out_size contiguous elements of the input dtype")
    flat = [int(v) for p in patterns for v in p]
    pat = _lib.int32_array(flat)
    code = dtype_code(input.dtype)
    need = groups * lib.ksmm_cu_chain_workspace_bytes_ex(nf, pat, batch, code, bs_last)
    workspace = torch.empty(need, dtype=torch.uint8, device=input.device) if need else None
    vals = (ctypes.c_void_p * nf)(*[w.data_ptr() for w in stacked_factors])
    with torch.cuda.device(input.device):
        _lib.check(lib.ksmm_cu_grouped_chain_forward(
            input.data_ptr(), vals, out.data_ptr(), bias.data_ptr() if bias is not None else None,
            workspace.data_ptr() if workspace is not None else None, need, batch, nf, pat, code, bs_last,
            int(groups), _stream_ptr(input.device)))
    return out


def _check_grad_output(grad_output, input_like_shape, bs_last, a, b, d):
    if not grad_output.is_cuda or grad_output.dim() != 2:
        raise ValueError("grad_output must be a 2-D CUDA tensor")
    batch = input_like_shape[1] if bs_last else input_like_shape[0]
    want = (a * b * d, batch) if bs_last else (batch, a * b * d)
    if tuple(grad_output.shape) != want:
        raise ValueError(f"grad_output must have the forward output's shape {want}, got {tuple(grad_output.shape)}")


def backward_input(grad_output, factor, bs_last, a, b, c, d):
    """Gradient of one factor with respect to its input (``ksmm_cu_backward_input``): the
    multiplication with pattern (a, c, b, d) and transposed blocks."""
    lib = _lib.load()
    bs_last = int(bool(bs_last))
    grad_output = grad_output.contiguous()
    batch = grad_output.shape[1] if bs_last else grad_output.shape[0]
    _check_grad_output(grad_output, (a * c * d, batch) if bs_last else (batch, a * c * d), bs_last, a, b, d)
    if tuple(factor.shape) != (a * d * c, b) or factor.dtype != grad_output.dtype or not factor.is_contiguous() \
            or factor.device != grad_output.device:
        raise ValueError(f"factor must be a contiguous ({a * d * c}, {b}) tensor of {grad_output.dtype}")
    code = dtype_code(grad_output.dtype)
    out = torch.empty((a * c * d, batch) if bs_last else (batch, a * c * d), dtype=grad_output.dtype,
                      device=grad_output.device)
    need = lib.ksmm_cu_backward_input_workspace_bytes(batch, a, b, c, d, code, bs_last)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=grad_output.device)
    with torch.cuda.device(grad_output.device):
        _lib.check(lib.ksmm_cu_backward_input(grad_output.data_ptr(), factor.data_ptr(), out.data_ptr(),
                                              ws.data_ptr(), need, batch, a, b, c, d, code, bs_last,
                                              _stream_ptr(grad_output.device)))
    return out


def backward_weights(input, grad_output, bs_last, a, b, c, d):
    """Gradient of one factor with respect to its kernel-format weights
    (``ksmm_cu_backward_weights``): (a*d*c, b), the input's dtype, fp32 accumulation."""
    lib = _lib.load()
    bs_last = int(bool(bs_last))
    input, grad_output = input.contiguous(), grad_output.contiguous()
    if not input.is_cuda or input.dim() != 2 or (input.shape[0] if bs_last else input.shape[1]) != a * c * d:
        raise ValueError(f"input must be a 2-D CUDA tensor with {a * c * d} features")
    _check_grad_output(grad_output, input.shape, bs_last, a, b, d)
    if grad_output.dtype != input.dtype or grad_output.device != input.device:
        raise ValueError("input and grad_output share dtype and device")
    batch = input.shape[1] if bs_last else input.shape[0]
    code = dtype_code(input.dtype)
    out = torch.empty((a * d * c, b), dtype=input.dtype, device=input.device)
    need = lib.ksmm_cu_backward_weights_workspace_bytes(batch, a, b, c, d, code, bs_last)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=input.device)
    with torch.cuda.device(input.device):
        _lib.check(lib.ksmm_cu_backward_weights(input.data_ptr(), grad_output.data_ptr(), out.data_ptr(),
                                                ws.data_ptr(), need, batch, a, b, c, d, code, bs_last,
                                                _stream_ptr(input.device)))
    return out


class FactorFunction(torch.autograd.Function):
    """One factor as a differentiable operation.  The reference wires its kernel into autograd the
    same way but leaves ``backward`` a stub (kernel.py:62-73, 323-329)."""

    @staticmethod
    def forward(ctx, input, factor, bs_last, a, b, c, d):
        ctx.save_for_backward(input, factor)
        ctx.pattern = (bool(bs_last), a, b, c, d)
        return forward_ex(input, factor.detach(), bs_last, a, b, c, d)

    @staticmethod
    def backward(ctx, grad_output):
        input, factor = ctx.saved_tensors
        bs_last, a, b, c, d = ctx.pattern
        grad_input = grad_factor = None
        if ctx.needs_input_grad[0]:
            grad_input = backward_input(grad_output, factor.detach(), bs_last, a, b, c, d)
        if ctx.needs_input_grad[1]:
            grad_factor = backward_weights(input.detach(), grad_output, bs_last, a, b, c, d)
        return grad_input, grad_factor, None, None, None, None, None


def quantize_e4m3(t):
    """Per-tensor e4m3 quantisation: returns (t / s cast to float8_e4m3fn, s) with
    s = amax(|t|) / 448 (the largest finite e4m3 value)."""
    amax = t.detach().abs().amax().float()
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (t.float() / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, float(scale)


def forward_fp8(input_q, factor_q, bs_last, a, b, c, d, scale_x, scale_w,
                out_dtype=torch.bfloat16, **kw):
    """fp8-e4m3 factor: y = scale_x * scale_w * (W_q x_q), fp32 accumulation."""
    return forward_ex(input_q, factor_q, bs_last, a, b, c, d, out_dtype=out_dtype,
                      alpha=float(scale_x) * float(scale_w), **kw)


def check_device(device=None):
    """Synchronise the current stream and raise if a kernel recorded a device-side timeout."""
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _lib.check(lib.ksmm_cu_check_device(_stream_ptr(dev)))


def launch_count():
    return int(_lib.load().ksmm_cu_launch_count())
