"""The benchmark configuration as it is written down, checked against the CPU oracle (needs a B200).

Hybrid-decoder linear shapes at hidden 5120, seed 1: QKV 7168 x 5120, O 5120 x 5120, gate|up 34816 x 5120, down
5120 x 17408, weights N(0, 0.02) x LogNormal(0, 0.25) per row.  Each weight takes the whole path: host encode into a
BCTX frame, host index, resident image, fused decode-GEMM at M = 1, 64 and 128 (and 768, the speculative-verify batch, on
gate|up).  The reference for y is the FP32 product with the words the ORACLE decodes from the same frame; the bar is
1e-2 relative to the call's largest magnitude (BF16 output, FP32 accumulation) and rows that are bitwise the same at
every batch size.  The reference's own tests for this contract: tests/test_miv_gemv.py:42-71 (M-invariance, tolerance)
and tests/test_georefine_verify.py:273-280 (exact decode).
"""
import hashlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-2
SHAPES = [("qkv", 7168, 5120, (1, 64, 128)), ("o", 5120, 5120, (1, 64, 128)),
          ("gate_up", 34816, 5120, (1, 64, 128, 768)), ("down", 5120, 17408, (1, 64, 128))]


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from georefine_b200 import _native

    _native.lib()
    return torch.device("cuda:0")


def _u16(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("name,n,k,batches", SHAPES)
def test_frame_to_fused_product_against_the_oracle(orc, oracle_coder, dev, name, n, k, batches):
    from georefine_b200 import codec
    from georefine_b200.gpu import CudaContextTensor

    words = orc.synthetic_weight_words(n, k, 1)
    frame = codec.encode(words)
    decoded = oracle_coder.decode(frame)                      # the oracle's words, not the generator's
    assert hashlib.sha256(decoded.tobytes()).digest() == hashlib.sha256(words.tobytes()).digest()
    t = CudaContextTensor(frame, device=dev, max_m=max(batches))
    assert t.resident.mode == 3                               # the default layout, not a demoted one
    assert np.array_equal(_u16(t.resident.decode()), decoded)
    w = torch.from_numpy(decoded.view(np.int16)).view(torch.bfloat16).to(dev)
    g = torch.Generator().manual_seed(1000 + n)
    xfull = torch.randn(max(batches), k, generator=g).to(torch.bfloat16).to(dev)
    rows = {}
    for m in batches:
        x = xfull[:m].contiguous()
        y = torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16)
        t(x, y)
        assert t.resident.check_status() == 0
        worst, scale = 0.0, 0.0
        for lo in range(0, m, 128):                           # FP32 reference in slabs: 768 x 34816 floats at a time is plenty
            ref = x[lo:lo + 128].float() @ w.float().T
            worst = max(worst, float((y[lo:lo + 128].float() - ref).abs().max()))
            scale = max(scale, float(ref.abs().max()))
        assert not torch.isnan(y.float()).any()
        assert worst <= REL_TOL * scale, f"{name} M={m}: {worst / scale:.3e}"
        rows[m] = _u16(y)
    top = max(batches)
    for m in batches:
        assert np.array_equal(rows[m], rows[top][:m]), f"{name}: rows differ between M={m} and M={top}"


@pytest.mark.parametrize("layout", ["window", "rans"])
def test_other_layouts_on_the_smallest_benchmark_shape(orc, dev, layout):
    """5120 x 5120 through the 3-bit and the entropy-coded images: tolerance, and rows independent of the batch size."""
    from georefine_b200.resident import ResidentWeight

    words = orc.synthetic_weight_words(5120, 5120, 1)
    r = ResidentWeight.from_words(words, dev, verify=False, layout=layout, max_m=128)
    w = torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(dev).float()
    xfull = torch.randn(128, 5120, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).to(dev)
    rows = {}
    for m in (1, 64, 128):
        y = torch.empty(m, 5120, device=dev, dtype=torch.bfloat16)
        r.gemm(xfull[:m].contiguous(), y)
        ref = xfull[:m].float() @ w.T
        assert r.check_status() == 0 and float((y.float() - ref).abs().max()) <= REL_TOL * float(ref.abs().max())
        rows[m] = _u16(y)
    assert np.array_equal(rows[1], rows[128][:1]) and np.array_equal(rows[64], rows[128][:64])
