"""The library's dense BF16 GEMV against exact arithmetic, with the reference's own test shapes (needs a B200).

Contract (the reference's tests/test_miv_gemv.py:32-71): rows of y bitwise independent of M for M = 1..8; every output
within one BF16 unit in the last place of the float64 product; the bias is added in FP32 before the one rounding.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

SHAPES = [(48, 5120), (96, 5120), (1024, 5120), (5120, 6144), (777, 1032), (64, 17408), (8, 8), (300, 200)]


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from georefine_b200 import _native

    _native.lib()
    return torch.device("cuda:0")


@pytest.mark.parametrize("n,k", SHAPES)
def test_dense_gemv_is_m_invariant_and_within_one_ulp(dev, n, k):
    from georefine_b200.dense import DenseLinear, dense_gemv

    g = torch.Generator().manual_seed(n * 31 + k)
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    x = torch.randn(8, k, generator=g).to(torch.bfloat16).to(dev)
    bias = torch.randn(n, generator=g).to(torch.bfloat16).to(dev)
    exact = x.cpu().double() @ w.cpu().double().T
    full = None
    for m in range(8, 0, -1):
        y = torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16)
        dense_gemv(w, x[:m], y)
        got = y.view(torch.int16).cpu().numpy()
        if full is None:
            full = got
        assert np.array_equal(got, full[:m]), f"rows differ between M={m} and M=8"
        ulp = exact[:m].abs().clamp_min(1e-30).log2().floor().sub(7).exp2()
        assert ((y.cpu().double() - exact[:m]).abs() <= 1.01 * ulp + 2e-3 * exact[:m].abs().max()).all()
    yb = torch.empty(3, n, device=dev, dtype=torch.bfloat16)
    dense_gemv(w, x[:3], yb, bias)
    want = (exact[:3] + bias.cpu().double())
    ulp = want.abs().clamp_min(1e-30).log2().floor().sub(7).exp2()
    assert ((yb.cpu().double() - want).abs() <= 1.01 * ulp + 2e-3 * want.abs().max()).all()
    lin = DenseLinear(w)
    assert (lin.kind, lin.N, lin.K, lin.bytes) == ("dense", n, k, 2 * n * k)
    y20 = lin.linear(torch.cat([x, x, x[:4]]))
    assert np.array_equal(y20[8:16].view(torch.int16).cpu().numpy(), full)


def test_dense_gemv_strided_operands_and_refusals(dev):
    from georefine_b200.dense import dense_gemv

    w = torch.randn(64, 512, device=dev).to(torch.bfloat16)[:, :256]          # row stride 512, 256 columns
    x = torch.randn(4, 264, device=dev).to(torch.bfloat16)[:, :256]           # row stride 264 (a multiple of 8, not of 16)
    y = torch.empty(4, 64, device=dev, dtype=torch.bfloat16)
    dense_gemv(w, x, y)
    ref = x.float() @ w.float().T
    assert ((y.float() - ref).abs().max() / ref.abs().max()).item() <= 1e-2
    with pytest.raises(RuntimeError):
        dense_gemv(w, torch.zeros(9, 256, device=dev, dtype=torch.bfloat16), torch.empty(9, 64, device=dev, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):                                         # 260 columns: not a multiple of 8
        dense_gemv(torch.zeros(8, 260, device=dev, dtype=torch.bfloat16), torch.zeros(1, 260, device=dev, dtype=torch.bfloat16),
                   torch.empty(1, 8, device=dev, dtype=torch.bfloat16))


def test_linear_and_install_dense_route_small_batches_to_the_gemv(dev):
    """``dense.linear`` (F.linear semantics) and ``install_dense``: 1 to 8 rows go to the GEMV - bitwise the rows a larger
    eligible batch gives -, more rows to ``F.linear``; the counters say which (glc_serve/miv_gemv.py:916-969)."""
    from torch import nn

    from georefine_b200 import dense

    dense.STATS.reset()
    g = torch.Generator().manual_seed(77)
    model = nn.Sequential(nn.Linear(256, 512), nn.Linear(512, 64, bias=False)).to(torch.bfloat16).to(dev)
    x = torch.randn(2, 4, 256, generator=g).to(torch.bfloat16).to(dev)
    want = model(x)                                                  # cuBLAS
    assert dense.install_dense(model) == 2
    got = model(x)
    assert got.shape == (2, 4, 64) and dense.STATS.gemv_by_m == {8: 2} and not dense.STATS.fallback_by_reason
    assert ((got.float() - want.float()).abs().max() / want.float().abs().max()).item() <= 2e-2
    one = model(x[:1, :1])
    assert torch.equal(one.reshape(-1), got[0, 0])                   # a row does not depend on the batch it is in
    big = model(torch.cat([x.reshape(8, 256)] * 2))                  # 16 rows: F.linear
    assert big.shape == (16, 64) and dense.STATS.fallback_by_reason == {"m_gt8": 2}
    y = dense.linear(x[0], model[0].weight, model[0].bias.float())   # a bias of another dtype is converted
    assert torch.equal(y, model[0](x[0]))
