"""CPU oracle for Kronecker-sparse matrix multiplication (KSMM).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module: it is the checker used by the tests, by ``__graft_entry__.smoke()``
and by the CPU-baseline / reference legs of ``bench.py``.

It restates, in plain numpy (float64 by default), the algorithm that the
reference project implements with torch on the CPU:

* one factor with pattern ``(a, b, c, d)`` and 4-D weights ``W[a, b, c, d]``
  has support ``I_a (x) 1_{b x c} (x) I_d``
  (src/ksmm_py/layer/kronecker_sparse/interface.py:116-123);
* batch-first ``einsum("... a c d, a b c d -> ... a b d")``
  (interface.py:254-264), batch-last ``einsum("a c d ..., a b c d -> a b d ...")``
  (interface.py:332-342);
* a chain applies ``patterns[0]`` first and ``patterns[-1]`` last
  (interface.py:137, 193-211, 269-291); the bias is added once after the
  whole chain (interface.py:451-467);
* the ``kernel`` weight storage is ``W.permute(0, 3, 2, 1).reshape(a*d*c, b)``
  (interface.py:65-69), inverted by ``from_kernel_format_to_dense``
  (interface.py:75-86);
* the dense equivalent is block-diagonal over ``a`` with ``diag_embed`` over
  ``d`` (interface.py:108-113).

Parity pin: ``tests/golden/*.npz`` holds outputs of the reference's own
``dense``, ``einsum`` and ``bmm`` algorithms (imported unchanged in the build
container by ``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks
this module against every one of them.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "in_size", "out_size", "abcd_to_kernel_format", "kernel_format_to_abcd",
    "abcd_to_dense", "factor_apply", "factor_apply_einsum", "factor_grad_input",
    "factor_grad_weights", "chain_apply", "chain_dense",
    "rel_fro_error", "quantize_e4m3", "e4m3_scale", "flops", "min_bytes",
]


def in_size(pattern):
    """a*c*d: number of input features of one factor (interface.py:151)."""
    a, b, c, d = pattern
    return a * c * d


def out_size(pattern):
    """a*b*d: number of output features of one factor (interface.py:152-154)."""
    a, b, c, d = pattern
    return a * b * d


def abcd_to_kernel_format(w):
    """(a,b,c,d) -> (a*d*c, b), element [((i*d+l)*c+k), j] = W[i,j,k,l].

    Follows generate_factor(..., 'kernel') (interface.py:65-69).
    """
    a, b, c, d = w.shape
    return np.ascontiguousarray(np.transpose(w, (0, 3, 2, 1)).reshape(a * d * c, b))


def kernel_format_to_abcd(wk, pattern):
    """Inverse of :func:`abcd_to_kernel_format` (interface.py:75-78)."""
    a, b, c, d = pattern
    return np.ascontiguousarray(np.transpose(wk.reshape(a, d, c, b), (0, 3, 2, 1)))


def abcd_to_dense(w):
    """Dense (a*b*d, a*c*d) matrix K with K[i*b*d + j*d + l, i*c*d + k*d + l] = W[i,j,k,l].

    Follows from_abcd_to_dense (interface.py:108-113).
    """
    a, b, c, d = w.shape
    dense = np.zeros((a * b * d, a * c * d), dtype=w.dtype)
    for i in range(a):
        for l in range(d):
            rows = i * b * d + np.arange(b) * d + l
            cols = i * c * d + np.arange(c) * d + l
            dense[np.ix_(rows, cols)] = w[i, :, :, l]
    return dense


def factor_apply(x, w, bs_last, acc_dtype=np.float64):
    """Apply one factor.  ``x`` is (a*c*d, B) if ``bs_last`` else (B, a*c*d).

    ``w`` is the 4-D (a,b,c,d) weight.  Accumulates in ``acc_dtype`` and
    returns an array of that dtype, shaped (a*b*d, B) or (B, a*b*d).
    """
    a, b, c, d = w.shape
    x = np.asarray(x, dtype=acc_dtype)
    # Both einsums are one (b x c) @ (c x B) product per block (i, l); written as a batched matmul
    # over (a, d) so that numpy hands the inner products to BLAS (same sums, same accumulation
    # type; the literal einsum forms take minutes on the largest patterns of patterns.in).
    wt = np.ascontiguousarray(np.transpose(np.asarray(w), (0, 3, 1, 2)), dtype=acc_dtype)  # (a, d, b, c)
    if bs_last:
        assert x.shape[0] == a * c * d, (x.shape, w.shape)
        nb = x.shape[1]
        xt = np.transpose(x.reshape(a, c, d, nb), (0, 2, 1, 3))          # (a, d, c, B)
        y = np.matmul(wt, xt)                                            # (a, d, b, B)
        return np.ascontiguousarray(np.transpose(y, (0, 2, 1, 3))).reshape(a * b * d, nb)
    assert x.shape[1] == a * c * d, (x.shape, w.shape)
    nb = x.shape[0]
    xt = np.transpose(x.reshape(nb, a, c, d), (1, 3, 2, 0))              # (a, d, c, B)
    y = np.matmul(wt, xt)                                                # (a, d, b, B)
    return np.ascontiguousarray(np.transpose(y, (3, 0, 2, 1))).reshape(nb, a * b * d)


def factor_apply_einsum(x, w, bs_last, acc_dtype=np.float64):
    """The same factor written literally as the reference's einsum strings
    (interface.py:254-264, 332-342); kept to pin :func:`factor_apply` in the tests."""
    a, b, c, d = w.shape
    x = np.asarray(x, dtype=acc_dtype)
    w = np.asarray(w, dtype=acc_dtype)
    if bs_last:
        nb = x.shape[1]
        return np.einsum("acdn,abcd->abdn", x.reshape(a, c, d, nb), w, optimize=True).reshape(a * b * d, nb)
    nb = x.shape[0]
    return np.einsum("nacd,abcd->nabd", x.reshape(nb, a, c, d), w, optimize=True).reshape(nb, a * b * d)


def factor_grad_input(grad_out, w, bs_last, acc_dtype=np.float64):
    """dL/dx of one factor: the transposed operator K^T applied to dL/dy, i.e. the factor with
    pattern (a, c, b, d) and weights W^T[i,k,j,l] = W[i,j,k,l] (the dense K of interface.py:108-113
    transposed).  The reference's kernel path has no backward (kernel.py:323-329); this is what
    autograd yields for its ``einsum`` and ``dense`` algorithms."""
    return factor_apply(grad_out, np.transpose(np.asarray(w), (0, 2, 1, 3)), bs_last, acc_dtype)


def factor_grad_weights(x, grad_out, pattern, bs_last, acc_dtype=np.float64):
    """dL/dW[i,j,k,l] = sum_n dL/dy[(i,j,l), n] * x[(i,k,l), n], as a 4-D (a,b,c,d) array."""
    a, b, c, d = pattern
    x = np.asarray(x, dtype=acc_dtype)
    g = np.asarray(grad_out, dtype=acc_dtype)
    if not bs_last:
        x, g = x.T, g.T
    nb = x.shape[1]
    x4 = np.transpose(x.reshape(a, c, d, nb), (0, 2, 1, 3))      # (a, d, c, B)
    g4 = np.transpose(g.reshape(a, b, d, nb), (0, 2, 1, 3))      # (a, d, b, B)
    dw = np.matmul(g4, np.transpose(x4, (0, 1, 3, 2)))           # (a, d, b, c)
    return np.ascontiguousarray(np.transpose(dw, (0, 2, 3, 1)))  # (a, b, c, d)


def chain_apply(x, weights, bs_last, bias=None, acc_dtype=np.float64, round_to=None):
    """Apply a chain of factors, ``weights[0]`` first (interface.py:193-211, 269-291).

    ``round_to``: optional numpy dtype (e.g. ``np.float16``) to which every
    intermediate is rounded, mimicking a per-factor execution that stores
    activations in that type.  The bias (shape (out,) or (out,1)) is added
    once at the end (interface.py:451-467).
    """
    y = np.asarray(x, dtype=acc_dtype)
    for w in weights:
        y = factor_apply(y, w, bs_last, acc_dtype)
        if round_to is not None:
            y = y.astype(round_to).astype(acc_dtype)
    if bias is not None:
        bias = np.asarray(bias, dtype=acc_dtype).reshape(-1)
        y = y + (bias[:, None] if bs_last else bias[None, :])
    return y


def chain_dense(weights):
    """Dense product K_last ... K_first (interface.py:434-437)."""
    dense = abcd_to_dense(np.asarray(weights[0], dtype=np.float64))
    for w in weights[1:]:
        dense = abcd_to_dense(np.asarray(w, dtype=np.float64)) @ dense
    return dense


def rel_fro_error(out, ref):
    """|| out - ref ||_F / || ref ||_F, the error the reference prints with
    ``--correctness`` (src/ksmm_py/benchmark/ksmm_time.py:148-164)."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    num = np.linalg.norm(out - ref)
    return float(num / den) if den > 0 else float(num)


# --------------------------------------------------------------------------
# fp8-e4m3 helpers (no reference implementation exists: the torch fp8 branch
# of the reference is an empty stub, kernel.cu:66-82).  Semantics used by the
# library: x_q = round_e4m3(x / s), s = amax(|x|) / 448, fp32 accumulate,
# y = s_x * s_w * sum(w_q * x_q).
# --------------------------------------------------------------------------

def e4m3_scale(x):
    amax = float(np.max(np.abs(x))) if x.size else 0.0
    return amax / 448.0 if amax > 0 else 1.0


def quantize_e4m3(x):
    """Round-to-nearest-even onto the e4m3fn grid (max 448, no inf); returns
    float64 values that are exactly representable in e4m3."""
    x = np.asarray(x, dtype=np.float64)
    ax = np.minimum(np.abs(x), 448.0)
    # exponent of the binade; subnormals share the exponent of 2^-6
    e = np.floor(np.log2(np.maximum(ax, 2.0 ** -20)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)            # 3 mantissa bits
    q = np.round(ax / step) * step   # np.round is half-to-even
    q = np.minimum(q, 448.0)
    return np.sign(x) * q


# --------------------------------------------------------------------------
# Algorithmic work of one factor (used for roofline arithmetic in the bench)
# --------------------------------------------------------------------------

def flops(pattern, batch):
    a, b, c, d = pattern
    return 2.0 * a * b * c * d * batch


def min_bytes(pattern, batch, s_in, s_out=None, s_w=None):
    a, b, c, d = pattern
    s_out = s_in if s_out is None else s_out
    s_w = s_in if s_w is None else s_w
    return float(s_in * a * c * d * batch + s_out * a * b * d * batch + s_w * a * b * c * d)
