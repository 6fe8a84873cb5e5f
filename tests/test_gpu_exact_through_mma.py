"""Bit-exact check of the decode that feeds the tensor cores (needs a B200).

The decode twin (``grb_bxr_decode``) stores its words to global memory; the fused kernels put the same words into
tensor memory (4-bit window layout) or into a swizzled shared-memory operand tile (3-bit window, entropy-coded and raw
layouts) and never show them to anybody.  A one-hot activation makes them visible: with x[m, c0 + m] = 1 and zeros
elsewhere, ``grb_bxr_gemm`` must return y[m, n] = W[n, c0 + m] bit for bit (1 x w is exact in FP32, every other product
is a zero, and a BF16 value survives the final rounding), whatever the tile width, through partial tiles and the
closing reduction.  A wrong exception patch, a swapped column pair or a misplaced operand column shows as a wrong word.

Two notes on what "bit for bit" means here: a zero weight may come back with the other sign (a sum of signed zeros is
+0 unless every term is -0), so zeros are compared as zeros; and the matrices hold finite words only, because
0 x infinity would poison its whole output row (the decode twin covers infinities and NaNs).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

LAYOUTS = ["window4", "window", "rans", "raw"]
TILES = [16, 64, 128]   # batch sizes that select the 16-, 64- and 128-column accumulator tiles


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from georefine_b200 import _native

    _native.lib()
    return torch.device("cuda:0")


def _resident(words, dev, layout, workers=None):
    from georefine_b200.resident import ResidentWeight

    if layout == "raw":
        return ResidentWeight.from_words(words, dev, force_raw=True, max_m=128, workers=workers)
    return ResidentWeight.from_words(words, dev, layout=layout, max_m=128, workers=workers)


def _columns_through_the_product(r, words, m, dev):
    """W rebuilt column by column from products with shifted identity rows, m columns per call."""
    n, k = words.shape
    kpad = (k + 7) // 8 * 8                       # the kernels want a row stride that is a multiple of 16 bytes
    got = np.empty((n, k), dtype=np.uint16)
    y = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    for c0 in range(0, k, m):
        x = torch.zeros(m, kpad, device=dev, dtype=torch.bfloat16)
        width = min(m, k - c0)
        x[torch.arange(width), c0 + torch.arange(width)] = 1.0
        y.fill_(float("nan"))
        r.gemm(x[:, :k], y)
        got[:, c0:c0 + width] = y[:width].view(torch.int16).cpu().numpy().view(np.uint16).T
    assert r.check_status() == 0
    return got


def _assert_same_words(got, want):
    zero = (want & 0x7FFF) == 0
    assert np.array_equal(got[~zero], want[~zero]), f"{int((got[~zero] != want[~zero]).sum())} nonzero words differ"
    assert not (got[zero] & 0x7FFF).any(), "a zero weight came back nonzero"


def every_finite_pattern():
    """255 x 256: row = exponent 0..254 (denormals included), column = sign and mantissa: each finite BF16 word once."""
    e = np.arange(255, dtype=np.uint16)[:, None]
    sm = np.arange(256, dtype=np.uint16)[None, :]
    return ((sm >> 7) << 15 | e << 7 | (sm & 0x7F)).astype(np.uint16)


def exponents_walking_through_the_window():
    """255 x 256: the exponent climbs by one every 16 columns from the row's own start, so every code of a 16-binade
    row window is used, next to every mantissa."""
    r = np.arange(255, dtype=np.uint32)[:, None]
    c = np.arange(256, dtype=np.uint32)[None, :]
    e = np.minimum(r + (c >> 4), 254)
    return (((c * 7 + r) & 1) << 15 | e << 7 | ((c * 37 + r * 11) & 0x7F)).astype(np.uint16)


def exceptions_in_every_decoder_warp(orc, rows, cols, seed):
    """Gaussian weights with one far-off exponent planted in each (32-row group, 32-column phase) of every 128 x 128
    chunk: each of the sixteen decoder warps of each chunk has at least one entry of the exception list to apply."""
    words = orc.synthetic_weight_words(rows, cols, seed)
    for rb in range(-(-rows // 128)):
        for c in range(-(-cols // 128)):
            for q in range(4):
                for rg in range(4):
                    row = rb * 128 + rg * 32 + (7 * q + 3 * rg + c) % 32
                    col = c * 128 + q * 32 + (5 * rg + 11 * q + rb) % 32
                    if row < rows - 1 and col < cols:   # (padded rows repeat the last row: keep that one plain)
                        words[row, col] = (words[row, col] & 0x807F) | np.uint16((2 + (q + rg) % 3) << 7)
    return words


@pytest.mark.parametrize("m", TILES)
@pytest.mark.parametrize("layout", LAYOUTS)
def test_every_finite_word_survives_the_tensor_core_path(dev, layout, m):
    words = every_finite_pattern()
    r = _resident(words, dev, layout)
    if layout != "raw":
        assert r.mode == {"window4": 3, "window": 2, "rans": 0}[layout], "the builder demoted the image"
    _assert_same_words(_columns_through_the_product(r, words, m, dev), words)
    # sixteen binades per row: made for the 4-bit window; the narrower layouts are allowed to demote it
    words = exponents_walking_through_the_window()
    r = _resident(words, dev, layout)
    assert layout != "window4" or r.mode == 3
    _assert_same_words(_columns_through_the_product(r, words, m, dev), words)


@pytest.mark.parametrize("m", TILES)
@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("shape,seed", [((300, 200), 2), ((777, 1032), 5), ((256, 512), 1)])
def test_ragged_shapes_with_exceptions_in_every_decoder_warp(orc, dev, layout, m, shape, seed):
    words = exceptions_in_every_decoder_warp(orc, *shape, seed)
    r = _resident(words, dev, layout)
    if layout != "raw":
        assert r.mode == {"window4": 3, "window": 2, "rans": 0}[layout], "the builder demoted the image"
    _assert_same_words(_columns_through_the_product(r, words, m, dev), words)


@pytest.mark.parametrize("layout", LAYOUTS)
def test_split_row_blocks_and_uneven_blobs_stay_exact(orc, dev, layout):
    """Few workers (whole row blocks per CTA), many workers (every row block cut into several partial tiles) and, for the
    4-bit layout, an image whose blobs are too uneven to be padded to one size."""
    words = exceptions_in_every_decoder_warp(orc, 384, 1536, 9)
    for workers in (2, 148):
        r = _resident(words, dev, layout, workers=workers)
        _assert_same_words(_columns_through_the_product(r, words, 128, dev), words)
    if layout == "window4":
        rng = np.random.default_rng(11)
        rows, cols = rng.integers(0, 128, 150), rng.integers(0, 128, 150)
        words[rows, cols] = 0x0100 | (words[rows, cols] & 0x807F)
        r = _resident(words, dev, layout, workers=7)
        assert r.header.mode == 3 and r.header.blob_stride16 == 0
        _assert_same_words(_columns_through_the_product(r, words, 64, dev), words)


@pytest.mark.parametrize("parts", [2, 3, 4, 5, 8])
def test_row_blocks_reduced_inside_a_thread_block_cluster(orc, dev, parts):
    """An aligned partition (workers = row blocks x P, 2 <= P <= 8) runs the 4-bit window kernel as one cluster of P CTAs
    per row block, whose partial tiles are added over distributed shared memory instead of through global memory.  The
    words must come through exactly, the order of additions must be the K order of the other path (same bits as an
    image cut for one CTA per row block would give only up to rounding, so the comparison is with FP32 arithmetic), and
    rows must not depend on the batch size."""
    from georefine_b200.resident import ResidentWeight

    words = exceptions_in_every_decoder_warp(orc, 300, 2048, 21)       # 3 row blocks (the last one ragged), 16 chunks
    r = ResidentWeight.from_words(words, dev, layout="window4", workers=3 * parts, max_m=256)
    assert r.mode == 3 and r.header.workers == 3 * parts and r.header.partial_slots == 3 * parts
    for m in TILES:
        _assert_same_words(_columns_through_the_product(r, words, m, dev), words)
    g = torch.Generator().manual_seed(parts)
    x = torch.randn(200, 2048, generator=g).to(torch.bfloat16).to(dev)
    bias = torch.randn(300, generator=g).to(torch.bfloat16).to(dev)
    w = torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(dev).float()
    ref = x.float() @ w.T + bias.float()
    rows = {}
    for m in (1, 5, 16, 64, 128, 200):
        y = torch.full((m, 300), float("nan"), device=dev, dtype=torch.bfloat16)
        r.gemm(x[:m].contiguous(), y, bias)
        assert r.check_status() == 0
        assert float((y.float() - ref[:m]).abs().max()) <= 1e-2 * float(ref.abs().max())
        rows[m] = y.view(torch.int16).cpu().numpy()
    assert all(np.array_equal(v, rows[200][:m]) for m, v in rows.items())
    # the same weight cut for a worker count that is no multiple of the row blocks takes the other path (partial tiles in
    # global memory): same K order inside a row block only when the cuts coincide, so compare to rounding
    other = ResidentWeight.from_words(words, dev, layout="window4", workers=3 * parts + 1, max_m=256)
    y2 = torch.empty(200, 300, device=dev, dtype=torch.bfloat16)
    other.gemm(x, y2, bias)
    assert float((y2.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
