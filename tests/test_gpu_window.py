"""GPU parity of the window resident layouts: fixed 3-bit exponent codes (csrc/bxw_kernels.cuh, operand tile in shared
memory) and fixed 4-bit codes (csrc/bxq_kernels.cuh, operand in tensor memory).

The decode twin must return the source words bit for bit; the fused product must agree with the FP32 reference
within the stated tolerance and give rows that do not depend on the batch size.
"""
import hashlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-2  # BF16 output, FP32 accumulation: relative to the largest reference magnitude of the call
LAYOUTS = [("window", 2), ("window4", 3)]   # layout name, header mode


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from georefine_b200 import _native

    _native.lib()
    return torch.device("cuda:0")


def _u16(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _reference_product(words, x):
    w = torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(x.device)
    return x.float() @ w.float().T


def _sprinkle(words, rate, seed):
    """Zeros, denormals, infinities, NaNs and far-off exponents at the given rate."""
    special = np.array([0, 0x8000, 0x7F80, 0xFF80, 0x7FC1, 0xFFE5, 1, 0x8001, 0x0080, 0x7F00, 0x4F80, 0x1000], dtype=np.uint16)
    rng = np.random.default_rng(seed)
    out = words.copy()
    at = rng.random(out.shape) < rate
    out[at] = rng.choice(special, size=int(at.sum()))
    return out


@pytest.mark.parametrize("shape,seed", [((128, 128), 0), ((256, 512), 1), ((300, 200), 2), ((64, 67), 3), ((1000, 1536), 4),
                                        ((777, 1032), 5), ((64, 17408), 6), ((4096, 4096), 0)])
@pytest.mark.parametrize("layout,mode", LAYOUTS)
def test_window_decode_is_bit_exact(orc, dev, shape, seed, layout, mode):
    from georefine_b200.resident import ResidentWeight, build_image, decode_image_host

    words = orc.synthetic_weight_words(*shape, seed)
    image, h = build_image(words, 148, layout=layout)
    assert h.mode == mode
    assert np.array_equal(decode_image_host(image), words)
    r = ResidentWeight(image, dev)
    assert np.array_equal(_u16(r.decode()), words)
    assert r.check_status() == 0


@pytest.mark.parametrize("layout,mode", LAYOUTS)
def test_window_decode_special_words_and_far_exponents(orc, dev, layout, mode):
    from georefine_b200.resident import ResidentWeight

    words = _sprinkle(orc.synthetic_weight_words(384, 640, 11), 5e-4, 11)
    r = ResidentWeight.from_words(words, dev, layout=layout)
    assert r.mode == mode and np.array_equal(_u16(r.decode()), words)
    # rows of very different scale, one constant row, one row of zeros
    words = orc.synthetic_weight_words(256, 384, 12)
    words[7] = 0x3F80
    words[9] = 0
    words[100] = (words[100] & 0x807F) | (np.uint16(3) << 7)
    words[101] = (words[101] & 0x807F) | (np.uint16(250) << 7)
    r = ResidentWeight.from_words(words, dev, layout=layout)
    assert np.array_equal(_u16(r.decode()), words)
    # a tensor whose exceptions do not fit falls back to another layout and still decodes exactly
    noisy = _sprinkle(orc.synthetic_weight_words(200, 300, 17), 0.2, 17)
    r = ResidentWeight.from_words(noisy, dev, layout=layout)
    assert r.mode in (0, 1) and np.array_equal(_u16(r.decode()), noisy)


SHAPES = [((128, 128), 0), ((256, 512), 1), ((300, 200), 2), ((1024, 4096), 3), ((4096, 4096), 0), ((2048, 5120), 1),
          ((777, 1032), 5), ((64, 17408), 6)]


@pytest.mark.parametrize("layout,mode", LAYOUTS)
@pytest.mark.parametrize("shape,seed", SHAPES)
def test_window_gemm_matches_reference_and_rows_do_not_depend_on_batch(orc, dev, shape, seed, layout, mode):
    from georefine_b200.resident import ResidentWeight

    words = orc.synthetic_weight_words(*shape, seed)
    r = ResidentWeight.from_words(words, dev, max_m=256, layout=layout)
    coded = ResidentWeight.from_words(words, dev, max_m=256, layout="rans")
    assert r.mode == mode and coded.mode == 0
    n, k = shape
    g = torch.Generator(device="cpu").manual_seed(300 + seed)
    xfull = torch.randn(200, k, generator=g).to(torch.bfloat16).to(dev)
    rows = {}
    for m in (1, 5, 16, 17, 64, 128, 200):
        x = xfull[:m].contiguous()
        y = torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16)
        r.gemm(x, y)
        assert r.check_status() == 0
        ref = _reference_product(words, x)
        assert not torch.isnan(y.float()).any()
        assert ((y.float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL
        rows[m] = _u16(y)
    for m, got in rows.items():                                    # bitwise identical rows across M
        assert np.array_equal(got, rows[200][:m]), f"rows differ between M={m} and M=200"
    # the entropy-coded layout rebuilds the same tiles; its kernel keeps one accumulator per item where this one keeps
    # two, so the two products agree to rounding, not to the bit
    yc = torch.empty((200, n), device=dev, dtype=torch.bfloat16)
    coded.gemm(xfull, yc)
    ref = _reference_product(words, xfull)
    assert ((yc.float() - torch.from_numpy(rows[200].view(np.int16)).view(torch.bfloat16).to(dev).float()).abs().max()
            / ref.abs().max()).item() <= REL_TOL
    # the small-batch entry point serves window images through the same path
    y3 = torch.empty((3, n), device=dev, dtype=torch.bfloat16)
    r.gemv(xfull[:3].contiguous(), y3)
    assert r.check_status() == 0 and np.array_equal(_u16(y3), rows[200][:3])


@pytest.mark.parametrize("layout,mode", LAYOUTS)
def test_window_linear_with_bias_exceptions_and_module(orc, oracle_coder, dev, layout, mode):
    from georefine_b200.resident import ResidentWeight

    words = _sprinkle(orc.synthetic_weight_words(384, 520, 31), 5e-4, 31)
    words[(words & 0x7F80) >= 0x6000] = 0x3C00                      # keep zeros, denormals and far small exponents; drop huge, inf, NaN
    r = ResidentWeight.from_words(words, dev, layout=layout)
    assert r.mode == mode
    bias = torch.randn(384, device=dev).to(torch.bfloat16)
    x = torch.randn(4, 9, 1040, device=dev).to(torch.bfloat16)[..., ::2]      # strided batched input
    y = r.linear(x, bias=bias)
    ref = _reference_product(words, x.reshape(-1, 520)) + bias.float()
    assert r.check_status() == 0
    assert ((y.reshape(-1, 384).float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL


@pytest.mark.parametrize("layout,mode", LAYOUTS)
@pytest.mark.parametrize("shape", [(34816, 5120), (5120, 17408)])
def test_window_full_size_images_reproduce_their_source_digest(orc, dev, shape, layout, mode):
    from georefine_b200.resident import ResidentWeight

    words = orc.synthetic_weight_words(*shape, 1)
    r = ResidentWeight.from_words(words, dev, verify=False, layout=layout)
    assert r.mode == mode
    got = _u16(r.decode())
    assert r.check_status() == 0
    assert hashlib.sha256(got.tobytes()).digest() == hashlib.sha256(words.tobytes()).digest()
    assert (1.35 if layout == "window" else 1.30) < 2 * words.size / r.coded_bytes < 1.50
    x = torch.randn(2, shape[1], device=dev).to(torch.bfloat16)
    y = torch.empty(2, shape[0], device=dev, dtype=torch.bfloat16)
    r.gemm(x, y)
    ref = _reference_product(words, x)
    assert r.check_status() == 0 and ((y.float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL


def _uneven_exceptions(orc):
    """A 256 x 512 weight whose first chunk has ~150 weights outside every row window and whose other chunks have
    none: the blobs of its wide-window image differ by more than the builder pads away."""
    words = orc.synthetic_weight_words(256, 512, 11)
    rng = np.random.default_rng(11)
    rows, cols = rng.integers(0, 128, 150), rng.integers(0, 128, 150)
    words[rows, cols] = 0x0100 | (words[rows, cols] & 0x807F)   # exponent 2: some 120 binades below the row's window
    return words


def test_wide_window_images_with_blobs_of_different_sizes(orc, dev):
    """Blobs are padded to one size only when they differ little; otherwise the kernel's loader follows the offset
    table.  Both paths must decode bit-exactly and multiply alike."""
    from georefine_b200.resident import ResidentWeight

    words = _uneven_exceptions(orc)
    uneven = ResidentWeight.from_words(words, dev, max_m=64, workers=7, layout="window4")
    even = ResidentWeight.from_words(orc.synthetic_weight_words(256, 512, 11), dev, max_m=64, workers=7, layout="window4")
    assert uneven.header.mode == 3 and uneven.header.blob_stride16 == 0
    assert even.header.mode == 3 and even.header.blob_stride16 * 16 >= 24640
    assert np.array_equal(_u16(uneven.decode()), words)
    g = torch.Generator().manual_seed(5)
    x64 = (torch.randn(64, 512, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    y64 = uneven.linear(x64)
    ref = _reference_product(words, x64)
    assert float((y64.float() - ref).abs().max()) <= REL_TOL * float(ref.abs().max())
    y1 = uneven.linear(x64[:1])
    assert torch.equal(y1.view(torch.int16), y64[:1].view(torch.int16))   # rows do not depend on the batch size
    assert uneven.check_status() == 0


def test_next_weight_hint_changes_nothing_but_the_timing(orc, dev):
    """`then()` tells a weight which image the stream reads next; the kernel uses it for an L2 prefetch only."""
    from georefine_b200.resident import ResidentWeight

    a = ResidentWeight.from_words(orc.synthetic_weight_words(512, 1024, 51), dev, layout="window4")
    b = ResidentWeight.from_words(orc.synthetic_weight_words(640, 512, 52), dev, layout="window4")
    c = ResidentWeight.from_words(orc.synthetic_weight_words(256, 640, 53), dev, layout="window")     # other layout: hint ignored
    x = torch.randn(64, 1024, device=dev).to(torch.bfloat16)
    plain = [torch.empty(64, 512, device=dev, dtype=torch.bfloat16), torch.empty(64, 640, device=dev, dtype=torch.bfloat16),
             torch.empty(64, 256, device=dev, dtype=torch.bfloat16)]
    a(x, plain[0]); b(plain[0], plain[1]); c(plain[1], plain[2])
    assert a.then(b) is b and b.then(c) is c and c.then(a) is a
    hinted = [torch.empty_like(t) for t in plain]
    for _ in range(3):
        a(x, hinted[0]); b(hinted[0], hinted[1]); c(hinted[1], hinted[2])
    torch.cuda.synchronize()
    assert all(torch.equal(p.view(torch.int16), h.view(torch.int16)) for p, h in zip(plain, hinted))
    assert a.check_status() == 0 and b.check_status() == 0 and c.check_status() == 0
    a.then(None)
    a(x, hinted[0])
    assert torch.equal(plain[0].view(torch.int16), hinted[0].view(torch.int16))
