"""``KSLinear`` with ``algo='kernel'`` backed by libksmm_cu.

Drop-in for the reference layer
(src/ksmm_py/layer/kronecker_sparse/interface.py:116-478) on its ``kernel``
path: same constructor signature and attribute names, the same ``(a*d*c, b)``
Parameter layout for every factor (so ``state_dict`` keys ``factors.{i}`` and
``bias`` are interchangeable with the reference's), the same treatment of extra
batch dimensions (``pre_process`` / ``post_process``, interface.py:439-467) and
the same error when asked for the kernel on the CPU (interface.py:163-164).

Only ``algo='kernel'`` exists here: the other five algorithms of the reference
are PyTorch compositions that this library does not re-implement, and there is
deliberately no fallback to them.  Beyond the reference, ``dtype`` may also be
``torch.bfloat16`` or ``torch.float8_e4m3fn`` (per-tensor scales, fp32
accumulation, bf16 activations between factors).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from . import kernel as _k


def generate_factor(a, b, c, d, algo="kernel", weights=None, dtype=torch.float16, device="cuda"):
    """Kernel-format factor: ``weights.permute(0, 3, 2, 1).reshape(a*d*c, b)`` or a
    fresh U(-1/sqrt(c), 1/sqrt(c)) draw (interface.py:30, 65-69)."""
    if algo != "kernel":
        raise NotImplementedError("this library implements algo='kernel' only")
    scaling = 1.0 / math.sqrt(c)
    if weights is None:
        factor = torch.empty(a * d * c, b).uniform_(-scaling, scaling)
    else:
        if tuple(weights.shape) != (a, b, c, d):
            raise ValueError(f"weights must have shape ({a},{b},{c},{d}), got {tuple(weights.shape)}")
        factor = weights.permute(0, 3, 2, 1).reshape(a * d * c, b)
    return factor.to(dtype).to(device).contiguous()


def from_kernel_format_to_abcd(factor, pattern):
    a, b, c, d = pattern
    return factor.reshape(a, d, c, b).permute(0, 3, 2, 1)


def from_kernel_format_to_dense(factor, pattern):
    """Dense (a*b*d, a*c*d) matrix of one kernel-format factor
    (same result as interface.py:75-86)."""
    a, b, c, d = pattern
    w = from_kernel_format_to_abcd(factor, pattern)                       # (a,b,c,d)
    blocks = torch.diag_embed(w).permute(0, 1, 3, 2, 4).reshape(a, b * d, c * d)
    return torch.block_diag(*torch.unbind(blocks, dim=0))


class KSLinear(nn.Module):
    r"""Kronecker-sparse linear layer: the weight is a product of factors with
    patterns ``(a,b,c,d)`` (support :math:`I_a \otimes 1_{b\times c} \otimes I_d`),
    ``patterns[0]`` applied first.  Optional weights are 4-D ``(a,b,c,d)`` tensors."""

    def __init__(self, patterns, weights=None, bias=True, algo="kernel",
                 dtype: torch.dtype = torch.float16, bs_last: bool = False, vsize: int = 4,
                 device: str = "cuda", fuse_chain: bool = True, activation=None,
                 requires_grad: bool = False, out_bs_last=None):
        super().__init__()
        # `requires_grad` is an addition as well: the reference's kernel path is inference-only (its
        # backward is a stub).  With trainable factors the forward runs factor by factor through
        # autograd (FactorFunction: dX and dW kernels of the library)
        # `activation` (None, "gelu", "relu") is an addition to the reference's signature: it is applied
        # after the bias inside the last factor's epilogue instead of as a separate kernel
        if activation not in (None, "gelu", "relu"):
            raise ValueError(f"activation={activation!r}: expected None, 'gelu' or 'relu'")
        self.activation = activation
        if algo != "kernel":
            raise NotImplementedError(
                f"algo={algo!r}: this library implements the reference's algo='kernel' only")
        for pattern in patterns:
            assert len(pattern) == 4
        for p, q in zip(patterns[:-1], patterns[1:]):
            if p[0] * p[1] * p[3] != q[0] * q[2] * q[3]:
                raise ValueError(f"pattern {tuple(p)} feeds {p[0] * p[1] * p[3]} features into {tuple(q)}")
        self.in_size = patterns[0][0] * patterns[0][2] * patterns[0][3]
        self.out_size = patterns[-1][0] * patterns[-1][1] * patterns[-1][3]
        self.algo = algo
        self.num_mat = len(patterns)
        self.patterns = [tuple(int(v) for v in p) for p in patterns]
        self.dtype = dtype
        self.bs_last = bs_last
        self.vsize = vsize
        self.weights = weights
        self.device = device
        self.fuse_chain = fuse_chain
        # `out_bs_last` (an addition; default: the input's layout) makes the layer return the other
        # layout, as a 2-D tensor: (out_size, batch) or (batch, out_size).  Two layers of an MLP can
        # then keep the activations between them batch-last inside a batch-first network, which is
        # the fast form for factors with d > 1.
        self.out_bs_last = bs_last if out_bs_last is None else bool(out_bs_last)
        if self.out_bs_last != bool(bs_last) and dtype == torch.float8_e4m3fn:
            raise ValueError("fp8 layers keep one layout")
        if str(self.device) == "cpu":
            raise Exception("kernel expects device='cuda'.")
        _k.dtype_code(dtype)  # validates
        if self.weights is None:
            self.weights = [None] * len(self.patterns)
        assert len(self.weights) == len(self.patterns)

        self.is_fp8 = dtype == torch.float8_e4m3fn
        store_dtype = torch.float32 if self.is_fp8 else dtype
        parameters = []
        for p, w in zip(self.patterns, self.weights):
            factor = generate_factor(*p, "kernel", w, store_dtype, device)
            parameters.append(nn.Parameter(factor, requires_grad=bool(requires_grad) and not self.is_fp8))
        self.factors = nn.ParameterList(parameters)
        self._fp8_cache = None

        bias_dtype = torch.bfloat16 if self.is_fp8 else dtype
        if bias:
            bound = 1 / math.sqrt(self.in_size)
            shape = (self.out_size, 1) if self.bs_last else (self.out_size,)
            self.bias = nn.Parameter(
                torch.empty(*shape, device=device).uniform_(-bound, bound).to(bias_dtype),
                requires_grad=bool(requires_grad) and not self.is_fp8)
        else:
            self.register_parameter("bias", None)
        self._workspace = None

    # -- fp8: weights are quantised once, lazily (per-tensor scale amax/448) -------------
    def _fp8_factors(self):
        if self._fp8_cache is None:
            self._fp8_cache = [_k.quantize_e4m3(f.data) for f in self.factors]
        return self._fp8_cache

    def _forward_2d(self, x, residual=None):
        bias = None if self.bias is None else self.bias.reshape(-1)
        if self.is_fp8:
            y = x
            for idx, (p, (wq, sw)) in enumerate(zip(self.patterns, self._fp8_factors())):
                xq, sx = _k.quantize_e4m3(y)
                last = idx + 1 == self.num_mat
                y = _k.forward_fp8(xq, wq, self.bs_last, *p, sx, sw, out_dtype=torch.bfloat16,
                                   bias=bias if last else None)
            if self.activation == "gelu":
                y = torch.nn.functional.gelu(y)
            elif self.activation == "relu":
                y = torch.relu(y)
            return y
        if residual is None and torch.is_grad_enabled() and (
                x.requires_grad or any(f.requires_grad for f in self.factors)
                or (self.bias is not None and self.bias.requires_grad)):
            # differentiable path: one autograd node per factor; bias and activation are torch ops
            y = x
            for p, f in zip(self.patterns, self.factors):
                y = _k.FactorFunction.apply(y, f, self.bs_last, *p)
            if self.bias is not None:
                y = y + (self.bias.reshape(-1, 1) if self.bs_last else self.bias.reshape(1, -1))
            if self.out_bs_last != bool(self.bs_last):
                y = y.t().contiguous()
            if self.activation == "gelu":
                y = torch.nn.functional.gelu(y)
            elif self.activation == "relu":
                y = torch.relu(y)
            return y
        if self.fuse_chain or self.num_mat == 1:
            ws = self._ensure_workspace(x)
            return _k.chain_forward(x, list(self.factors), self.patterns, self.bs_last, bias=bias,
                                    workspace=ws, activation=self.activation, out_bs_last=self.out_bs_last,
                                    residual=residual)
        if self.out_bs_last != bool(self.bs_last):
            raise ValueError("a layer that changes the layout runs as one chain call (fuse_chain=True)")
        y = x
        for idx, (p, f) in enumerate(zip(self.patterns, self.factors)):
            last = idx + 1 == self.num_mat
            y = _k.forward_ex(y, f, self.bs_last, *p, bias=bias if last else None,
                              activation=self.activation if last else None)
        return y

    def _ensure_workspace(self, x):
        from . import _lib
        lib = _lib.load()
        batch = x.shape[1] if self.bs_last else x.shape[0]
        flat = [v for p in self.patterns for v in p]
        need = lib.ksmm_cu_chain_workspace_bytes_layouts(self.num_mat, _lib.int32_array(flat), batch,
                                                         _k.dtype_code(x.dtype), int(bool(self.bs_last)),
                                                         int(bool(self.out_bs_last)))
        if need == 0:
            return None
        ws = self._workspace
        if ws is None or ws.device != x.device or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=x.device)
            self._workspace = ws
        return ws

    def forward(self, tensor, residual=None):
        """tensor: (..., in_size) for batch-first, (in_size, ...) for batch-last.  ``residual`` (an
        addition to the reference's signature; inference path only): a tensor with the shape of the
        result that is added to it inside the last factor's kernel."""
        output = self.pre_process(tensor)
        if not self.is_fp8 and output.dtype != self.dtype:
            raise TypeError(f"input dtype {output.dtype} differs from the layer's {self.dtype}")
        res2d = None
        if residual is not None:
            if self.is_fp8 or not (self.fuse_chain or self.num_mat == 1):
                raise ValueError("a residual needs the chained 16/32-bit path")
            res2d = (residual.reshape(self.out_size, -1) if self.out_bs_last
                     else residual.reshape(-1, self.out_size)).contiguous()
        output = self._forward_2d(output, res2d)
        return self.post_process(tensor, output)

    def pre_process(self, tensor):
        if self.bs_last:
            output = tensor.reshape(tensor.size(0), -1)
        else:
            output = tensor.reshape(-1, tensor.size(-1))
        return output.contiguous()

    def post_process(self, tensor, output):
        # the bias has already been added by the last factor's epilogue
        if self.out_bs_last != bool(self.bs_last):
            return output              # 2-D, in the requested layout
        if self.bs_last:
            return output.view(self.out_size, *tensor.shape[1:])
        return output.view(*tensor.shape[:-1], self.out_size)

    def get_dense_product(self):
        """Dense (out_size, in_size) matrix of the whole chain (interface.py:363-437)."""
        dense = None
        for factor, pattern in zip(self.factors, self.patterns):
            m = from_kernel_format_to_dense(factor.data.float(), pattern)
            dense = m if dense is None else torch.matmul(m, dense)
        return dense

    def extra_repr(self):
        return "in_size={}, out_size={}, num_mat={}, patterns={}, algo={}, bias={}".format(
            self.in_size, self.out_size, self.num_mat, self.patterns, self.algo,
            self.bias is not None)


class KSLinearGroup(nn.Module):
    """Several ``KSLinear`` layers with the same patterns applied to the same input in one library
    call: the q, k and v projections of an attention layer, which the reference builds from one
    pattern list and calls one after the other on the same tensor
    (src/ksmm_py/model/get_vit.py:164-215, src/ksmm_py/model/vit.py:477-478).  ``forward`` returns
    one output per layer.  The layers stay ordinary ``KSLinear`` modules (their parameters are the
    source of truth); the stacked copy of their factors that the grouped kernel reads is rebuilt
    whenever a factor changes."""

    def __init__(self, layers):
        super().__init__()
        layers = list(layers)
        if not layers:
            raise ValueError("need at least one layer")
        first = layers[0]
        for l in layers:
            if not isinstance(l, KSLinear):
                raise TypeError("KSLinearGroup holds KSLinear layers")
            if l.patterns != first.patterns or l.dtype != first.dtype or l.bs_last != first.bs_last \
                    or l.is_fp8 or l.activation is not None or (l.bias is None) != (first.bias is None):
                raise ValueError("the layers of a group share patterns, dtype, layout and bias setting "
                                 "(fp8 layers and fused activations are not grouped)")
        self.layers = nn.ModuleList(layers)
        self._stacked = None
        self._versions = None

    def _stack(self):
        versions = [(f._version, f.data_ptr()) for l in self.layers for f in l.factors]
        if self.layers[0].bias is not None:
            versions += [(l.bias._version, l.bias.data_ptr()) for l in self.layers]
        if self._stacked is None or versions != self._versions:
            nf = self.layers[0].num_mat
            factors = [torch.cat([l.factors[f].data for l in self.layers], dim=0).contiguous() for f in range(nf)]
            bias = None
            if self.layers[0].bias is not None:
                bias = torch.cat([l.bias.data.reshape(-1) for l in self.layers]).contiguous()
            self._stacked, self._versions = (factors, bias), versions
        return self._stacked

    def forward(self, tensor):
        first = self.layers[0]
        x = first.pre_process(tensor)
        if x.dtype != first.dtype:
            raise TypeError(f"input dtype {x.dtype} differs from the layers' {first.dtype}")
        factors, bias = self._stack()
        out = _k.grouped_chain_forward(x, factors, first.patterns, first.bs_last, len(self.layers), bias=bias)
        return tuple(first.post_process(tensor, out[g]) for g in range(len(self.layers)))
