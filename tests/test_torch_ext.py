"""The PyTorch C++ extension: the module surface of the reference's kernel.cpp
(src/ksmm_py/layer/kronecker_sparse/kernel.cpp:25-50) over the C ABI."""
import math

import numpy as np
import pytest
import torch

from golden_cases import make_weights
from ksmm_b200.build import load_torch_extension
from oracle import ksmm_oracle as ko


@pytest.fixture(scope="module")
def ext():
    return load_torch_extension()


def test_module_surface_and_argument_checks(ext):
    assert callable(ext.forward) and callable(ext.chain_forward)
    x = torch.zeros(8, 4)
    w = torch.zeros(8, 4)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ext.forward(x, w, 1, 1, 4, 8, 1, "float", 4)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ext.chain_forward(x, [w], [[1, 4, 8, 1]], 1)


@pytest.mark.gpu
@pytest.mark.parametrize("bs_last", [1, 0])
@pytest.mark.parametrize("dtype,name,tol", [(torch.float32, "float", 1e-5), (torch.float16, "half", 1e-2)])
def test_forward_matches_the_oracle(ext, dtype, name, tol, bs_last):
    import ksmm_b200 as kb
    for pi, pattern in enumerate([(2, 96, 48, 2), (1, 128, 64, 4), (3, 40, 24, 1)]):
        a, b, c, d = pattern
        rng = np.random.RandomState(900 + pi)
        batch = 136
        shape = (a * c * d, batch) if bs_last else (batch, a * c * d)
        x = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dtype)
        w = torch.from_numpy(make_weights([pattern], rng)[0]).to(dtype)
        wk = kb.generate_factor(a, b, c, d, "kernel", w, dtype, "cuda:0")
        y = ext.forward(x.cuda(), wk, bs_last, a, b, c, d, name, 4)
        assert y.shape == ((a * b * d, batch) if bs_last else (batch, a * b * d)) and y.dtype == dtype
        ref = ko.factor_apply(x.float().numpy(), w.float().numpy(), bool(bs_last))
        assert ko.rel_fro_error(y.float().cpu().numpy(), ref) < tol, (pattern, dtype, bs_last)
    with pytest.raises(RuntimeError, match="features"):
        ext.forward(x.cuda(), wk, bs_last, a, b, c + 1, d, name, 4)


@pytest.mark.gpu
def test_chain_forward_with_bias_and_activation(ext):
    import ksmm_b200 as kb
    pats = [(4, 192, 192, 1), (1, 768, 192, 4)]
    rng = np.random.RandomState(910)
    ws = [torch.from_numpy(v).half() for v in make_weights(pats, rng)]
    x = torch.from_numpy(rng.standard_normal((136, 768)).astype(np.float32)).half()
    bias = torch.from_numpy(rng.standard_normal(3072).astype(np.float32)).half()
    wk = [kb.generate_factor(*p, "kernel", w, torch.float16, "cuda:0") for p, w in zip(pats, ws)]
    y = ext.chain_forward(x.cuda(), wk, [list(p) for p in pats], 0, bias.cuda(), 1)
    ref = ko.chain_apply(x.float().numpy(), [w.float().numpy() for w in ws], False) + bias.float().numpy()[None, :]
    ref = 0.5 * ref * (1.0 + np.vectorize(math.erf)(ref / math.sqrt(2.0)))
    assert ko.rel_fro_error(y.float().cpu().numpy(), ref) < 1e-2
    # runs on the caller's current stream
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        y2 = ext.chain_forward(x.cuda(), wk, [list(p) for p in pats], 0, bias.cuda(), 1)
    s.synchronize()
    assert torch.equal(y, y2)


@pytest.mark.gpu
def test_chain_forward_validates_shapes_before_anything_runs(ext):
    """A factor, pattern or input that does not fit is refused by the binding: nothing may reach
    the kernels with sizes that would make them read or write out of bounds."""
    x = torch.zeros(16, 768, dtype=torch.float16, device="cuda:0")
    w0 = torch.zeros(768, 192, dtype=torch.float16, device="cuda:0")
    w1 = torch.zeros(768, 768, dtype=torch.float16, device="cuda:0")
    pats = [[4, 192, 192, 1], [1, 768, 192, 4]]
    ext.chain_forward(x, [w0, w1], pats, 0)
    with pytest.raises(RuntimeError, match="receives"):
        ext.chain_forward(x[:, :760].contiguous(), [w0, w1], pats, 0)
    with pytest.raises(RuntimeError, match="must have shape"):
        ext.chain_forward(x, [w0, w1[:700].contiguous()], pats, 0)
    with pytest.raises(RuntimeError, match="receives"):
        ext.chain_forward(x, [w0, w1], [[4, 192, 192, 1], [1, 768, 96, 4]], 0)
    with pytest.raises(RuntimeError, match="positive"):
        ext.chain_forward(x, [w0, w1], [[4, 192, 192, 1], [1, 768, 192, 0]], 0)
    with pytest.raises(RuntimeError, match="2-D"):
        ext.chain_forward(x.view(4, 4, 768), [w0, w1], pats, 0)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.chain_forward(x, [w0, w1.cpu()], pats, 0)
