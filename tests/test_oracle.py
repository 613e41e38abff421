"""The CPU oracle against the reference's own outputs (tests/golden) and
against itself through independent formulations.  No GPU needed."""
import json
import os

import numpy as np
import pytest
import torch

from golden_cases import CASES, make_inputs
from oracle import ksmm_oracle as ko
from oracle import reference_port as rp

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "ksmm_golden.npz"))
META = json.loads(bytes(GOLDEN["__meta__"]).decode())

# relative Frobenius tolerances of the benchmark specification
TOL = {"float32": 1e-5, "float16": 1e-2}


def _flatten(case, x):
    """(in, *lead) / (*lead, in) -> 2-D as KSLinear.pre_process does (interface.py:439-449)."""
    return x.reshape(x.shape[0], -1) if case["bs_last"] else x.reshape(-1, x.shape[-1])


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_outputs(case):
    x, ws, bias = make_inputs(case)
    ref = GOLDEN[case["name"] + "/y"]
    y = ko.chain_apply(_flatten(case, x), ws, case["bs_last"], bias=bias)
    assert y.size == ref.size
    err = ko.rel_fro_error(y.reshape(ref.shape), ref)
    assert err < TOL[case["dtype"]], (case["name"], err)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_reference_algorithms_agree_with_each_other(case):
    """dense, einsum and bmm of the reference agree far inside the tolerance."""
    tol = TOL[case["dtype"]]
    for algo, spread in META[case["name"]]["spread_vs_first"].items():
        assert spread < tol, (case["name"], algo, spread)


@pytest.mark.parametrize("algo", ["einsum", "bmm", "dense"])
@pytest.mark.parametrize("case", [c for c in CASES if c["dtype"] == "float32" and not c["bias"]],
                         ids=lambda c: c["name"])
def test_torch_port_matches_reference_outputs(case, algo):
    x, ws, _ = make_inputs(case)
    chain = rp.ChainCPU(case["patterns"], [torch.from_numpy(w) for w in ws], algo, case["bs_last"])
    y = chain(torch.from_numpy(_flatten(case, x))).numpy()
    ref = GOLDEN[case["name"] + "/y"]
    assert ko.rel_fro_error(y.reshape(ref.shape), ref) < 1e-5


@pytest.mark.parametrize("name", ["f_1_16_16_1_last", "f_2_3_5_4_last"])
def test_kernel_weight_format_matches_reference(name):
    case = next(c for c in CASES if c["name"] == name)
    _, ws, _ = make_inputs(case)
    wk = ko.abcd_to_kernel_format(ws[0])
    assert np.array_equal(wk, GOLDEN[name + "/kernel_format0"])
    assert np.array_equal(ko.kernel_format_to_abcd(wk, case["patterns"][0]), ws[0])
    # the reference's own kernel-format -> dense conversion equals the oracle's dense matrix
    assert np.array_equal(ko.abcd_to_dense(ws[0]), GOLDEN[name + "/dense_from_kernel0"])


@pytest.mark.parametrize("pattern", [(2, 3, 5, 4), (1, 8, 4, 1), (3, 2, 2, 3), (1, 1, 1, 5)])
@pytest.mark.parametrize("bs_last", [True, False])
def test_einsum_equals_dense_matrix(pattern, bs_last):
    rng = np.random.RandomState(7)
    a, b, c, d = pattern
    w = rng.standard_normal((a, b, c, d))
    x = rng.standard_normal((a * c * d, 9) if bs_last else (9, a * c * d))
    dense = ko.abcd_to_dense(w)
    ref = dense @ x if bs_last else x @ dense.T
    assert np.allclose(ko.factor_apply(x, w, bs_last), ref, atol=1e-12)


def test_chain_dense_product_and_order():
    rng = np.random.RandomState(3)
    pats = [(2, 8, 4, 2), (4, 6, 4, 2)]
    ws = [rng.standard_normal(p) for p in pats]
    x = rng.standard_normal((pats[0][0] * pats[0][2] * pats[0][3], 5))
    assert np.allclose(ko.chain_apply(x, ws, True), ko.chain_dense(ws) @ x, atol=1e-12)
    assert np.allclose(ko.chain_apply(x.T, ws, False), x.T @ ko.chain_dense(ws).T, atol=1e-12)


def test_empty_batch():
    w = np.ones((2, 3, 4, 2))
    assert ko.factor_apply(np.zeros((16, 0)), w, True).shape == (12, 0)
    assert ko.factor_apply(np.zeros((0, 16)), w, False).shape == (0, 12)


def test_e4m3_quantiser_matches_torch_cast():
    rng = np.random.RandomState(11)
    x = np.concatenate([rng.standard_normal(4096) * 50, [0.0, 448.0, -448.0, 1e-4, 2.0 ** -9,
                                                         2.0 ** -10, 0.0009765625 * 3, 500.0]])
    x = np.clip(x, -448, 448).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(ko.quantize_e4m3(x).astype(np.float32), ref)


def test_work_formulas():
    # figures quoted for the (1,768,192,4) pattern at batch 25088
    assert abs(ko.flops((1, 768, 192, 4), 25088) - 29.60e9) < 0.01e9
    assert abs(ko.min_bytes((1, 768, 192, 4), 25088, 2) - 193.9e6) < 0.1e6
    assert abs(ko.min_bytes((1, 768, 192, 4), 25088, 4) - 387.7e6) < 0.1e6


def test_matmul_form_equals_the_literal_einsum_form():
    """factor_apply hands the block products to BLAS; it must give the sums of the reference's
    einsum strings."""
    rng = np.random.RandomState(5)
    for pattern in [(2, 3, 5, 4), (1, 48, 24, 3), (3, 7, 9, 2), (4, 8, 8, 1), (1, 1, 1, 8)]:
        a, b, c, d = pattern
        w = rng.standard_normal(pattern)
        for bs_last in (True, False):
            x = rng.standard_normal((a * c * d, 7) if bs_last else (7, a * c * d))
            assert np.allclose(ko.factor_apply(x, w, bs_last), ko.factor_apply_einsum(x, w, bs_last),
                               rtol=1e-12, atol=1e-12)


def test_gradients_against_autograd_of_the_dense_operator():
    """The oracle's input and weight gradients of one factor equal what torch autograd gives for
    y = K x with the dense K of the reference (interface.py:108-113)."""
    import torch
    rng = np.random.RandomState(6)
    for pattern in [(2, 3, 5, 4), (1, 6, 4, 3), (3, 4, 4, 1)]:
        a, b, c, d = pattern
        w = torch.tensor(rng.standard_normal(pattern), requires_grad=True)
        x = torch.tensor(rng.standard_normal((a * c * d, 5)), requires_grad=True)
        g = torch.tensor(rng.standard_normal((a * b * d, 5)))
        blocks = torch.diag_embed(w).permute(0, 1, 3, 2, 4).reshape(a, b * d, c * d)
        dense = torch.block_diag(*torch.unbind(blocks, dim=0))
        (dense @ x * g).sum().backward()
        assert np.allclose(ko.factor_grad_input(g.numpy(), w.detach().numpy(), True), x.grad.numpy())
        assert np.allclose(ko.factor_grad_weights(x.detach().numpy(), g.numpy(), pattern, True), w.grad.numpy())
        assert np.allclose(ko.factor_grad_input(g.numpy().T, w.detach().numpy(), False), x.grad.numpy().T)
        assert np.allclose(ko.factor_grad_weights(x.detach().numpy().T, g.numpy().T, pattern, False),
                           w.grad.numpy())
