"""Torch-on-CPU port of the reference's three CPU-capable algorithms.

TEST / BASELINE INFRASTRUCTURE ONLY.  The shipped package never imports this
module.  It exists because the reference project itself (a Python package)
is not present on the GPU machine: ``bench.py``'s ``cpu_baseline`` leg and its
``--impl reference`` arm time these functions on the host cores instead.

Each function restates one ``algo`` of the reference's ``KSLinear`` with the
same torch operator underneath, so that its speed on a given host is the
reference's speed:

* ``einsum``: rearrange -> torch.einsum -> rearrange
  (src/ksmm_py/layer/kronecker_sparse/interface.py:254-264 and 332-342);
* ``bmm``: permute + contiguous copy -> torch.bmm -> permute back
  (src/ksmm_py/layer/bmm/forward_bmm.py:38-52 and 55-69), weights stored as
  (a*d, b, c) (interface.py:31-36);
* ``dense``: F.linear / matmul with the densified factor
  (interface.py:252-253, 330-331, 108-113).

``tests/test_oracle.py`` checks them against the golden outputs of the real
reference.
"""
from __future__ import annotations

import torch


def weights_to_bmm_format(w):
    """(a,b,c,d) -> (a*d, b, c) as generate_factor(..., 'bmm') stores it
    (interface.py:31-36)."""
    a, b, c, d = w.shape
    return w.permute(0, 3, 1, 2).reshape(a * d, b, c).contiguous()


def weights_to_dense(w):
    """(a,b,c,d) -> dense (a*b*d, a*c*d) (interface.py:108-113)."""
    a, b, c, d = w.shape
    blocks = torch.diag_embed(w).permute(0, 1, 3, 2, 4).reshape(a, b * d, c * d)
    return torch.block_diag(*torch.unbind(blocks, dim=0))


def einsum_factor(x, w, bs_last):
    a, b, c, d = w.shape
    if bs_last:
        nb = x.shape[1:]
        y = torch.einsum("acdn,abcd->abdn", x.reshape(a, c, d, -1), w)
        return y.reshape(a * b * d, *nb)
    lead = x.shape[:-1]
    y = torch.einsum("nacd,abcd->nabd", x.reshape(-1, a, c, d), w)
    return y.reshape(*lead, a * b * d)


def bmm_factor(x, w_bmm, pattern, bs_last):
    a, b, c, d = pattern
    if bs_last:
        n = x.shape[1]
        xs = x.reshape(a, c, d, n).transpose(1, 2).reshape(a * d, c, n).contiguous()
        out = torch.bmm(w_bmm, xs)                                   # (a*d, b, n)
        return out.reshape(a, d, b, n).transpose(1, 2).reshape(a * b * d, n)
    n = x.shape[0]
    xs = x.reshape(n, a, c, d).transpose(-1, -2).reshape(n, a * d, c).contiguous().transpose(0, 1)
    out = torch.bmm(xs, w_bmm.transpose(-1, -2))                     # (a*d, n, b)
    return out.transpose(0, 1).reshape(n, a, d, b).transpose(-1, -2).reshape(n, a * b * d)


def dense_factor(x, w_dense, bs_last):
    if bs_last:
        return torch.matmul(w_dense, x)
    return torch.nn.functional.linear(x, w_dense)


class ChainCPU:
    """A chain of factors prepared once for one algorithm, then applied to
    inputs: the CPU counterpart of ``KSLinear(..., algo=algo, device='cpu')``
    without bias."""

    def __init__(self, patterns, weights, algo, bs_last):
        assert algo in ("einsum", "bmm", "dense")
        self.patterns = [tuple(p) for p in patterns]
        self.algo = algo
        self.bs_last = bs_last
        if algo == "einsum":
            self.factors = [w.contiguous() for w in weights]
        elif algo == "bmm":
            self.factors = [weights_to_bmm_format(w) for w in weights]
        else:
            self.factors = [weights_to_dense(w).contiguous() for w in weights]

    @torch.no_grad()
    def __call__(self, x):
        y = x
        for p, f in zip(self.patterns, self.factors):
            if self.algo == "einsum":
                y = einsum_factor(y, f, self.bs_last)
            elif self.algo == "bmm":
                y = bmm_factor(y, f, p, self.bs_last)
            else:
                y = dense_factor(y, f, self.bs_last)
        return y
