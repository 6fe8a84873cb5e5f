"""Parity of the CUDA path with the CPU oracle, through the C ABI (needs a B200)."""
import hashlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FRAME_TAGS = ["special", "uniform13x17", "constant", "synthetic64x512", "synthetic48x320.r4c1", "conditional96x160"]
REL_TOL = 1e-2  # BF16 output, FP32 accumulation: relative to the largest reference magnitude of the call


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from georefine_b200 import _native

    _native.lib()  # the extension must load; nothing below has another path
    return torch.device("cuda:0")


def _u16(t):
    return t.contiguous().view(torch.uint16).cpu().numpy()


def _reference_product(words, x):
    w = torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(x.device).float()
    return x.float() @ w.T


# ---------------------------------------------------------------- unchanged BCTX streams
@pytest.mark.parametrize("tag", FRAME_TAGS)
@pytest.mark.parametrize("stride", [1, 7, 128, 1024])
def test_indexed_decode_is_bit_exact(golden, oracle_coder, dev, tag, stride):
    from georefine_b200.gpu import CudaContextTensor

    frame = golden[tag + ".frame"].tobytes()
    t = CudaContextTensor(frame, stride=stride, device=dev, fused=False)
    expect = oracle_coder.decode(frame)
    assert t.shape == expect.shape and t.source_sha256 == hashlib.sha256(expect.tobytes()).hexdigest()
    assert np.array_equal(_u16(t.decode()), expect)
    assert t.stride == stride and t.walk_stride == (128 if stride == 1024 else stride)      # the device index may be finer than asked
    if t.mode != 1:
        assert t.buffers["main_states"].numel() == (expect.size + t.walk_stride - 1) // t.walk_stride
        assert t.resident_bytes >= sum(v.numel() * v.element_size() for v in t.buffers.values())
    if stride == 1024:                                       # the reference's geometry: one lane per block of the caller's stride
        coarse = CudaContextTensor(frame, stride=stride, walk_stride=stride, device=dev, fused=False)
        assert np.array_equal(_u16(coarse.decode()), expect)
        if coarse.mode != 1:
            assert coarse.buffers["main_states"].numel() == (expect.size + stride - 1) // stride
        with pytest.raises(ValueError):
            CudaContextTensor(frame, stride=stride, walk_stride=100, device=dev, fused=False)


@pytest.mark.parametrize("nr,nc", [(1, 1), (16, 4), (64, 16)])
def test_indexed_decode_class_configurations_and_gather(orc, oracle_coder, dev, nr, nc):
    from georefine_b200.gpu import CudaContextTensor

    words = orc.synthetic_weight_words(96, 2048, 11)
    frame = oracle_coder.encode(words, row_classes=nr, col_classes=nc)
    t = CudaContextTensor(frame, stride=1024, device=dev, fused=False)
    assert np.array_equal(_u16(t.decode()), words)
    ids = torch.tensor([[5, 95, 0], [5, 17, 64]])
    assert np.array_equal(_u16(t.gather_rows(ids)), words[ids.numpy()])
    assert t.gather_rows(torch.empty(0, dtype=torch.int64)).shape == (0, 2048)
    with pytest.raises(IndexError):
        t.gather_rows(torch.tensor([96]))
    coarse = CudaContextTensor(frame, stride=1024, walk_stride=1024, device=dev, fused=False)
    assert np.array_equal(_u16(coarse.gather_rows(ids)), words[ids.numpy()])
    # a stride that does not divide the row length falls back to a full decode + index
    t2 = CudaContextTensor(frame, stride=1000, device=dev, fused=False)
    assert t2.walk_stride == 1000 and np.array_equal(_u16(t2.gather_rows(ids)), words[ids.numpy()])


def test_indexed_decode_reports_corruption_without_faulting(orc, oracle_coder, dev):
    from georefine_b200 import codec
    from georefine_b200.gpu import CudaContextTensor

    words = orc.synthetic_weight_words(64, 1024, 12)
    t = CudaContextTensor(oracle_coder.encode(words), stride=256, device=dev, fused=False)
    good = t.buffers["main_states"].clone()
    t.buffers["main_states"].view(torch.int32)[3] += 0x55   # host-injected: a wrong restart state
    with pytest.raises(codec.CodecError):
        t.decode()
    assert int(t.error.item()) != 0
    t.buffers["main_states"].copy_(good)
    t.buffers["main_stream"][100:140] = 255      # host-injected: damaged bytes in the middle of the stream
    with pytest.raises(codec.CodecError):
        t.decode()
    t.decode(check=False)                        # still returns, status says discard
    assert int(t.error.item()) != 0


# ---------------------------------------------------------------- resident image: decode twin
@pytest.mark.parametrize("shape,seed", [((128, 128), 0), ((256, 512), 1), ((300, 200), 2), ((64, 67), 3),
                                        ((1000, 1536), 4), ((4096, 4096), 0)])
def test_resident_decode_is_bit_exact(orc, oracle_coder, dev, shape, seed):
    from georefine_b200.gpu import CudaContextTensor

    words = orc.synthetic_weight_words(*shape, seed)
    frame = oracle_coder.encode(words)
    t = CudaContextTensor(frame, device=dev, layout="rans")
    assert np.array_equal(oracle_coder.decode(frame), words)
    assert np.array_equal(_u16(t.resident.decode()), words)      # image walked by the fused kernels' decoder
    assert np.array_equal(_u16(t.decode()), words)               # unchanged streams
    assert t.resident.check_status() == 0


def test_resident_decode_special_words(dev):
    from georefine_b200.resident import ResidentWeight

    special = np.resize(np.array([0, 0x8000, 0x7F80, 0xFF80, 0x7FC1, 0xFFE5, 1, 0x8001], dtype=np.uint16), (64, 67))
    r = ResidentWeight.from_words(special, dev, layout="rans")
    assert np.array_equal(_u16(r.decode()), special)
    # ordinary weights with 2 % zeros, denormals, infinities and NaNs: the exception lists of a coded image
    from oracle import bcx_oracle as orc_mod
    sprinkled = orc_mod.synthetic_weight_words(200, 300, 17)
    rng = np.random.default_rng(17)
    at = rng.random(sprinkled.shape) < 0.02
    sprinkled[at] = rng.choice(special.ravel()[:8], size=int(at.sum()))
    r = ResidentWeight.from_words(sprinkled, dev, layout="rans")
    assert r.mode == 0 and np.array_equal(_u16(r.decode()), sprinkled)
    finite = sprinkled.copy()
    finite[(finite & 0x7F80) == 0x7F80] = 0x3C00                      # keep zeros and denormals, drop inf/NaN
    r = ResidentWeight.from_words(finite, dev, layout="rans")
    x = torch.randn(8, 300, device=dev).to(torch.bfloat16)
    ref = _reference_product(finite, x)
    y, yv = r.linear(x), torch.empty(8, 200, device=dev, dtype=torch.bfloat16)
    r.gemv(x.contiguous() if x.stride(0) % 8 == 0 else torch.nn.functional.pad(x, (0, 4))[:, :300], yv)
    assert r.check_status() == 0
    assert ((y.float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL
    assert ((yv.float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL
    every = np.arange(65536, dtype=np.uint16).reshape(256, 256)   # every BF16 pattern once
    r = ResidentWeight.from_words(every, dev, layout="rans")
    if r.mode == 0:
        assert np.array_equal(_u16(r.decode()), every)


def test_resident_decode_flags_a_corrupt_image(orc, dev):
    from georefine_b200.resident import ResidentWeight, build_image

    words = orc.synthetic_weight_words(256, 512, 21)
    image, h = build_image(words, 148, layout="rans")
    image[h.states_at + 8] ^= 0x40                                # host-injected: one stream starts from a wrong state
    r = ResidentWeight(image, dev, verify=False)
    with pytest.raises(ValueError):
        r.decode()
    assert r.check_status() & 8


# ---------------------------------------------------------------- fused linears
# includes the reference's own MIV test shapes with a ragged K (777 x 1032) and a long K (64 x 17408)
SHAPES = [((128, 128), 0), ((256, 512), 1), ((300, 200), 2), ((1024, 4096), 3), ((4096, 4096), 0), ((2048, 5120), 1),
          ((777, 1032), 5), ((64, 17408), 6)]


@pytest.mark.parametrize("shape,seed", SHAPES)
def test_gemm_matches_reference_and_rows_do_not_depend_on_batch(orc, dev, shape, seed):
    from georefine_b200.resident import ResidentWeight

    words = orc.synthetic_weight_words(*shape, seed)
    r = ResidentWeight.from_words(words, dev, max_m=256, layout="rans")
    n, k = shape
    g = torch.Generator(device="cpu").manual_seed(100 + seed)
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


@pytest.mark.parametrize("shape,seed", SHAPES)
def test_gemv_matches_reference_and_is_m_invariant(orc, dev, shape, seed):
    from georefine_b200.resident import ResidentWeight

    words = orc.synthetic_weight_words(*shape, seed)
    r = ResidentWeight.from_words(words, dev, layout="rans")
    n, k = shape
    g = torch.Generator(device="cpu").manual_seed(200 + seed)
    xfull = torch.randn(8, k, generator=g).to(torch.bfloat16).to(dev)
    w64 = torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).double()
    exact = (xfull.cpu().double() @ w64.T)
    y8 = None
    for m in range(8, 0, -1):
        y = torch.empty((m, n), device=dev, dtype=torch.bfloat16)
        r.gemv(xfull[:m].contiguous(), y)
        assert r.check_status() == 0
        if y8 is None:
            y8 = _u16(y)
        assert np.array_equal(_u16(y), y8[:m])
        # at most one BF16 ulp away from the correctly rounded float64 result (relative to the call's scale)
        got = y.cpu().double()
        ulp = exact[:m].abs().clamp_min(1e-30).log2().floor().sub(7).exp2()
        assert ((got - exact[:m]).abs() <= 1.01 * ulp + 2e-3 * exact[:m].abs().max()).all()
    with pytest.raises(RuntimeError):
        r.gemv(torch.zeros(9, k, device=dev, dtype=torch.bfloat16), torch.empty(9, n, device=dev, dtype=torch.bfloat16))


def test_bias_strided_input_and_module_contract(orc, oracle_coder, dev):
    from georefine_b200.gpu import CudaContextTensor
    from georefine_b200.serving import BctxLinear

    words = orc.synthetic_weight_words(384, 256, 31)
    t = CudaContextTensor(oracle_coder.encode(words), device=dev, layout="rans")
    bias = torch.nn.Parameter(torch.randn(384, device=dev).to(torch.bfloat16), requires_grad=False)
    layer = BctxLinear(t, bias)
    assert (layer.out_features, layer.in_features) == (384, 256) and "weight" not in layer.state_dict()
    x = torch.randn(4, 9, 512, device=dev).to(torch.bfloat16)[..., ::2]      # strided batched input
    y = layer(x)
    assert y.shape == (4, 9, 384) and layer.forward_calls == 1 and layer.weight_materializations == 0
    ref = _reference_product(words, x.reshape(-1, 256)) + bias.float()
    assert ((y.reshape(-1, 384).float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL
    assert np.array_equal(_u16(layer.weight), words) and layer.weight_materializations == 1
    yv = torch.empty(3, 384, device=dev, dtype=torch.bfloat16)
    t.resident.gemv(x.reshape(-1, 256)[:3].contiguous(), yv, bias)
    assert ((yv.float() - ref[:3]).abs().max() / ref.abs().max()).item() <= REL_TOL
    # descriptor protocol: preallocated output, nothing returned
    out = torch.empty(36, 384, device=dev, dtype=torch.bfloat16)
    assert t(x.reshape(-1, 256).contiguous(), out) is None
    assert t.resident.kind == "bctx" and t.resident.coded_bytes < 2 * words.size + 40000


@pytest.mark.parametrize("shape", [(34816, 5120), (5120, 17408)])
def test_full_size_images_reproduce_their_source_digest(orc, dev, shape):
    """Benchmark-size weights: the GPU decode of the resident image hashes to the digest of the source words."""
    from georefine_b200.resident import ResidentWeight

    words = orc.synthetic_weight_words(*shape, 1)
    r = ResidentWeight.from_words(words, dev, verify=False, layout="rans")
    got = _u16(r.decode())
    assert r.check_status() == 0
    assert hashlib.sha256(got.tobytes()).digest() == hashlib.sha256(words.tobytes()).digest()
    assert 1.40 < 2 * words.size / r.coded_bytes < 1.55


def test_linearity_round_trip_at_full_size(orc, dev):
    """Size-independent property at a benchmark shape: W(x1 + x2) == W x1 + W x2 within rounding, and the
    decode twin reproduces the source digest."""
    from georefine_b200.resident import ResidentWeight

    words = orc.synthetic_weight_words(7168, 5120, 1)
    r = ResidentWeight.from_words(words, dev, verify=False, layout="rans")
    assert hashlib.sha256(_u16(r.decode()).tobytes()).digest() == bytes(r.header.source_sha256)
    x = torch.randn(2, 5120, device=dev).to(torch.bfloat16)
    xs = (x[0].float() + x[1].float()).to(torch.bfloat16)[None]
    y = torch.empty(2, 7168, device=dev, dtype=torch.bfloat16)
    ys = torch.empty(1, 7168, device=dev, dtype=torch.bfloat16)
    r.gemm(x, y)
    r.gemm(xs, ys)
    ref = _reference_product(words, xs)
    assert ((ys.float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL
    assert ((y[0].float() + y[1].float() - ys[0].float()).abs().max() / ref.abs().max()).item() <= 3 * REL_TOL


def test_raw_mode_images_decode_and_multiply(orc, oracle_coder, golden, dev):
    """Incompressible weights are kept as plain tiles; the tensor-core path multiplies them without decoders."""
    from georefine_b200.gpu import CudaContextTensor
    from georefine_b200.resident import ResidentWeight

    noise = np.random.default_rng(3).integers(0, 65536, (300, 256), dtype=np.uint16)
    noise = (noise & 0xBFFF).astype(np.uint16)                    # keep the exponents finite
    r = ResidentWeight.from_words(noise, dev, max_m=256, layout="rans")
    assert r.mode == 1
    assert np.array_equal(_u16(r.decode()), noise)
    forced = ResidentWeight.from_words(orc.synthetic_weight_words(256, 384, 8), dev, force_raw=True, max_m=256)
    coded = ResidentWeight.from_words(orc.synthetic_weight_words(256, 384, 8), dev, max_m=256, layout="rans")
    assert forced.mode == 1 and coded.mode == 0
    x = torch.randn(200, 384, device=dev).to(torch.bfloat16)
    ya, yb = torch.empty(200, 256, device=dev, dtype=torch.bfloat16), torch.empty(200, 256, device=dev, dtype=torch.bfloat16)
    forced.gemm(x, ya)
    coded.gemm(x, yb)
    assert forced.check_status() == 0 and np.array_equal(_u16(ya), _u16(yb))   # same tiles, same arithmetic
    rows = {}
    for m in (1, 3, 64, 200):
        xm = torch.randn(200, 256, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(dev)[:m].contiguous()
        y = torch.empty(m, 300, device=dev, dtype=torch.bfloat16)
        (r.gemv if m == 3 else r.gemm)(xm, y)
        assert r.check_status() == 0
        ref = _reference_product(noise, xm)
        assert ((y.float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL
        rows[m] = _u16(y)
    assert all(np.array_equal(v, rows[200][:m]) for m, v in rows.items())
    # a raw BCTX frame (mode 1) with an odd column count: the resident image still reproduces it, and the
    # linear pads the activation rows to the 16-byte stride the kernels want
    t = CudaContextTensor(golden["uniform13x17.frame"].tobytes(), device=dev)
    words = (golden["uniform13x17.words"] & 0xBFFF).astype(np.uint16)
    assert t.mode == 1 and np.array_equal(_u16(t.resident.decode()), golden["uniform13x17.words"])
    r17 = ResidentWeight.from_words(words, dev, layout="rans")
    x17 = torch.randn(5, 17, device=dev).to(torch.bfloat16)
    y17 = r17.linear(x17)
    ref = _reference_product(words, x17)
    assert r17.check_status() == 0 and ((y17.float() - ref).abs().max() / ref.abs().max()).item() <= REL_TOL
