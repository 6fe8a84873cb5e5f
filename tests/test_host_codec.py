"""Host side of the product library against the oracle and the golden vectors (no GPU needed)."""
import ctypes
import hashlib
import re
from pathlib import Path

import numpy as np
import pytest

from georefine_b200 import _native, codec, resident
from georefine_b200.gpu import checkpoints, index_frame

ROOT = Path(__file__).resolve().parents[1]
FRAME_TAGS = ["special", "uniform13x17", "constant", "synthetic64x512", "synthetic48x320.r4c1", "conditional96x160"]


def test_library_exports_every_declared_symbol():
    text = (ROOT / "include" / "georefine_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b((?:bcx|bxr|grb)_[a-z0-9_]+)\s*\(", text))
    assert {"bcx_encode", "bcx_checkpoint", "grb_bctx_decode_words", "grb_bxr_gemm", "grb_bxr_gemv", "bxr_build"} <= declared
    lib = ctypes.CDLL(str(_native.library_path()))
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing
    assert declared == set(_native.EXPORTS)


@pytest.mark.parametrize("tag", FRAME_TAGS)
def test_frames_are_byte_identical_to_the_reference(golden, tag):
    nr, nc = map(int, golden[tag + ".classes"])
    words = golden[tag + ".words"]
    frame = golden[tag + ".frame"].tobytes()
    assert codec.encode(words, row_classes=nr, col_classes=nc) == frame
    assert np.array_equal(codec.decode(frame), words)


@pytest.mark.parametrize("tag,strides", [("special", (1, 7, 128, 1024)), ("constant", (128, 1024)),
                                         ("synthetic64x512", (128, 1024)), ("conditional96x160", (1, 100, 1024))])
def test_index_frame_matches_reference_restart_points(golden, tag, strides):
    frame = golden[tag + ".frame"].tobytes()
    words = golden[tag + ".words"]
    for stride in strides:
        idx = index_frame(frame, stride, keep_words=True)
        assert idx["source_sha256"] == hashlib.sha256(words.tobytes()).hexdigest()
        assert idx["frame_sha256"] == hashlib.sha256(frame).hexdigest()
        assert idx["shape"] == words.shape and np.array_equal(idx["words"], words)
        assert len(idx["main_states"]) == (words.size + stride - 1) // stride
        assert np.array_equal(idx["main_states"], golden[f"{tag}.s{stride}.main_states"])
        assert np.array_equal(idx["main_offsets"], golden[f"{tag}.s{stride}.main_offsets"])
        if idx["mode"] == 128:
            assert np.array_equal(idx["residual_states"], golden[f"{tag}.s{stride}.residual_states"])
            assert np.array_equal(idx["residual_offsets"], golden[f"{tag}.s{stride}.residual_offsets"])


def test_index_frame_raw_and_rejections(golden):
    frame = golden["uniform13x17.frame"].tobytes()
    idx = index_frame(frame)
    assert idx["mode"] == 1 and np.array_equal(idx["raw"].reshape(13, 17), golden["uniform13x17.words"])
    with pytest.raises(codec.CodecError, match="checksum"):
        index_frame(frame[:-1] + bytes([frame[-1] ^ 1]))
    with pytest.raises(codec.CodecError, match="stride"):
        index_frame(frame, 0)
    with pytest.raises(codec.CodecError):
        codec.decode(frame + b"\0")
    with pytest.raises(codec.CodecError):
        codec.encode(np.zeros((4, 4), dtype=np.uint16), row_classes=3)
    with pytest.raises(codec.CodecError):
        codec.encode(np.zeros((0, 4), dtype=np.uint16))


@pytest.mark.parametrize("kind", [0, 1])
def test_abi_case_matches_reference_and_rejects_faults(golden, orc, kind):
    tag = f"abi9x17.k{kind}"
    vals, freq, stream = golden[tag + ".vals"], golden[tag + ".freq"], golden[tag + ".stream"].tobytes()
    rows_n, cols_n, nr, nc = 9, 17, 4, 3
    rc = (np.arange(rows_n, dtype=np.uint8) % nr).copy()
    cc = (np.arange(cols_n, dtype=np.uint8) % nc).copy()
    lib = _native.lib()
    f2, s2 = codec._encode_kind(lib, np.ascontiguousarray(vals), rc, cc, nr, nc, kind)
    assert s2 == stream and np.array_equal(np.frombuffer(f2, dtype="<u4").reshape(freq.shape), freq)
    assert codec._frequencies_kind(lib, np.ascontiguousarray(vals), rc, cc, nr, nc, kind) == f2
    main, resid = orc.split_words(vals)
    resctx = main.ravel() if kind else None
    for stride in (1, 7, 19, 128):
        st, of, sym = checkpoints(stream, freq, rc, cc, (rows_n, cols_n), nr, nc, stride, resctx)
        assert np.array_equal(st, golden[f"{tag}.s{stride}.states"]) and np.array_equal(of, golden[f"{tag}.s{stride}.offsets"])
        assert np.array_equal(sym, (resid if kind else main).ravel())
    bad = freq.copy()
    used_ctx = int(resctx[0]) if kind else int(rc[0]) * nc + int(cc[0])
    bad[used_ctx, int((resid if kind else main).ravel()[0])] += 1
    for s, f in ((stream[:-1], freq), (stream + b"\0", freq), (stream, bad), (b"\0\0\0\0" + stream[4:], freq)):
        with pytest.raises(codec.CodecError):
            checkpoints(s, f, rc, cc, (rows_n, cols_n), nr, nc, 19, resctx)
        with pytest.raises(codec.CodecError):
            codec._decode_kind(lib, s, np.ascontiguousarray(f, dtype="<u4").tobytes(), rc, cc, rows_n, cols_n, nr, nc, kind, resctx)


def test_checkpoint_leaves_outputs_untouched_on_failure(golden):
    tag = "abi9x17.k0"
    vals, freq, stream = golden[tag + ".vals"], golden[tag + ".freq"], golden[tag + ".stream"].tobytes()
    rc = (np.arange(9, dtype=np.uint8) % 4).copy()
    cc = (np.arange(17, dtype=np.uint8) % 3).copy()
    lib = _native.lib()
    p = lambda a, t: a.ctypes.data_as(ctypes.POINTER(t))
    out = np.full(vals.size, 0xFFFF, dtype=np.uint16)
    states = np.full(9, 7, dtype=np.uint32)
    offsets = np.full(9, 7, dtype=np.uint32)
    f = np.ascontiguousarray(freq, dtype="<u4")

    def call(data, n=vals.size, rcv=rc, stream_ptr=True):
        d = np.frombuffer(data, dtype=np.uint8).copy()
        return lib.bcx_checkpoint(p(d, ctypes.c_uint8) if stream_ptr else None, d.size, n, 9, 17, p(rcv, ctypes.c_uint8),
                                  p(cc, ctypes.c_uint8), 4, 3, 0, None, p(f, ctypes.c_uint32), 19, p(states, ctypes.c_uint32),
                                  p(offsets, ctypes.c_uint32), p(out, ctypes.c_uint16))

    bad_rc = rc.copy()
    bad_rc[0] = 4
    assert call(stream[:-1]) == 3 and call(stream + b"\0") == 3
    assert call(stream, n=vals.size - 1) == 1 and call(stream, rcv=bad_rc) == 1 and call(stream, stream_ptr=False) == 1
    assert np.all(out == 0xFFFF) and np.all(states == 7) and np.all(offsets == 7)
    assert call(stream) == 0 and np.any(out != 0xFFFF) and offsets[0] == 4


def test_lookup_tables_invert_every_slot(golden):
    freq = golden["abi9x17.k0.freq"]
    nctx, vocab = freq.shape
    cum = np.empty((nctx, vocab + 1), dtype=np.uint32)
    bucket = np.empty((nctx, 4096), dtype=np.uint16)
    f = np.ascontiguousarray(freq, dtype="<u4")
    assert _native.lib().grb_bctx_build_lookup(f.ctypes.data_as(_native.U32P), nctx, vocab, cum.ctypes.data_as(_native.U32P),
                                               bucket.ctypes.data_as(_native.U16P)) == 0
    for cx in range(nctx):
        if freq[cx].sum() == 0:
            continue
        expect = np.repeat(np.arange(vocab), freq[cx])
        s = bucket[cx][np.arange(65536) >> 4].astype(np.int64)
        for _ in range(vocab):
            advance = cum[cx][s + 1] <= np.arange(65536)
            if not advance.any():
                break
            s = s + advance
        assert np.array_equal(s, expect)


@pytest.mark.parametrize("shape,seed,workers", [((128, 128), 0, 148), ((300, 200), 2, 148), ((64, 67), 3, 5),
                                                ((1, 1), 4, 148), ((513, 1024), 5, 37), ((256, 4096), 6, 148)])
def test_resident_image_round_trips_and_plan_is_balanced(orc, shape, seed, workers):
    words = orc.synthetic_weight_words(*shape, seed)
    image, h = resident.build_image(words, workers, layout="rans")
    assert h.mode == 0 and h.rows == shape[0] and h.cols == shape[1] and h.total_bytes == image.size
    assert bytes(h.source_sha256) == hashlib.sha256(words.tobytes()).digest()
    assert np.array_equal(resident.decode_image_host(image), words)
    items = (_native.BxrItem * h.items).from_buffer_copy(image[h.items_at:h.items_at + 32 * h.items].tobytes())
    wi = np.frombuffer(image[h.worker_items_at:h.worker_items_at + 4 * (workers + 1)].tobytes(), dtype=np.uint32)
    loads = [sum(items[i].chunk_end - items[i].chunk_begin for i in range(wi[w], wi[w + 1])) for w in range(workers)]
    assert sum(loads) == h.row_blocks * h.chunks and max(loads) - min(loads) <= 1
    covered = np.zeros((h.row_blocks, h.chunks), dtype=np.int32)
    for it in items:
        covered[it.row_block, it.chunk_begin:it.chunk_end] += 1
        assert it.part < it.parts and (it.parts == 1 or it.slot < h.partial_slots)
    assert np.all(covered == 1)


def test_resident_image_special_values_and_raw_fallback(orc):
    special = np.resize(np.array([0, 0x8000, 0x7F80, 0xFF80, 0x7FC1, 0xFFE5, 1, 0x8001], dtype=np.uint16), (64, 67))
    image, h = resident.build_image(special, 9, layout="rans")          # half of these words lie outside any 15-binade window
    assert h.mode == 1 and np.array_equal(resident.decode_image_host(image), special)
    sprinkled = orc.synthetic_weight_words(200, 300, 17)    # ordinary weights with 2 % special values: exception lists
    rng = np.random.default_rng(17)
    at = rng.random(sprinkled.shape) < 0.02
    sprinkled[at] = rng.choice(special.ravel()[:8], size=int(at.sum()))
    image, h = resident.build_image(sprinkled, 9, layout="rans")
    assert h.mode == 0 and np.array_equal(resident.decode_image_host(image), sprinkled)
    noise = np.random.default_rng(0).integers(0, 65536, (256, 256), dtype=np.uint16)
    image, h = resident.build_image(noise, 148, layout="rans")
    assert h.mode == 1 and np.array_equal(resident.decode_image_host(image), noise)
    image, h = resident.build_image(orc.synthetic_weight_words(128, 256, 1), 4, force_raw=True)
    assert h.mode == 1


def test_corrupt_resident_image_is_rejected_on_the_host(orc):
    words = orc.synthetic_weight_words(128, 256, 9)
    image, h = resident.build_image(words, 3, layout="rans")
    bad = image.copy()
    bad[h.states_at] ^= 1
    status = _native.lib().bxr_decode_host(bad.ctypes.data_as(_native.U8P), bad.size, np.empty_like(words).ctypes.data_as(_native.U16P))
    assert status == 2
    bad = image.copy()
    bad[0] ^= 1
    with pytest.raises(ValueError):
        resident.decode_image_host(bad)


@pytest.mark.parametrize("shape,seed,workers", [((128, 128), 0, 148), ((300, 200), 2, 148), ((64, 67), 3, 5),
                                                ((1, 1), 4, 148), ((513, 1024), 5, 37), ((256, 4096), 6, 148)])
@pytest.mark.parametrize("layout,mode", [("window", 2), ("window4", 3)])
def test_window_image_round_trips_on_the_host(orc, shape, seed, workers, layout, mode):
    """Window layouts (fixed 3-bit / 4-bit exponent codes): the host twin returns the source words; the plan is the coded one."""
    words = orc.synthetic_weight_words(*shape, seed)
    image, h = resident.build_image(words, workers, layout=layout)
    coded, hc = resident.build_image(words, workers, layout="rans")
    assert h.mode == mode and (h.rows, h.cols, h.items, h.partial_slots) == (hc.rows, hc.cols, hc.items, hc.partial_slots)
    assert bytes(h.source_sha256) == hashlib.sha256(words.tobytes()).digest()
    assert np.array_equal(resident.decode_image_host(image), words)
    assert np.array_equal(image[h.items_at:h.items_at + 32 * h.items], coded[hc.items_at:hc.items_at + 32 * hc.items])


def test_window_image_entries_far_list_and_fallbacks(orc):
    special = np.array([0, 0x8000, 0x7F80, 0xFF80, 0x7FC1, 0xFFE5, 1, 0x8001, 0x0080, 0x7F00, 0x4F80, 0x1000], dtype=np.uint16)
    words = orc.synthetic_weight_words(384, 640, 11)
    rng = np.random.default_rng(11)
    at = rng.random(words.shape) < 5e-4
    words[at] = rng.choice(special, size=int(at.sum()))
    words[9] = 0                                                # a row of zeros: every weight is an entry
    words[100] = (words[100] & 0x807F) | (np.uint16(250) << 7)   # a row at the top of the exponent range
    image, h = resident.build_image(words, 148, layout="window")
    assert h.mode == 2 and np.array_equal(resident.decode_image_host(image), words)
    blob0 = image[h.blobs_at:h.blobs_at + 64]
    assert int(np.frombuffer(blob0[32:34].tobytes(), dtype=np.uint16)[0]) > 0        # entries exist in the first chunk
    # corrupt entry bounds or a missing far record are refused by the host twin
    bad = image.copy()
    bad[h.blobs_at + 32:h.blobs_at + 34] = 0xFF
    with pytest.raises(ValueError):
        resident.decode_image_host(bad)
    # too many exceptions for the slot: the builder demotes the image (entropy-coded, then raw)
    noisy = words.copy()
    at = rng.random(noisy.shape) < 0.2
    noisy[at] = rng.choice(special, size=int(at.sum()))
    image, h = resident.build_image(noisy, 148, layout="window")
    assert h.mode in (0, 1) and np.array_equal(resident.decode_image_host(image), noisy)
    # the 4-bit layout keeps exceptions in its own list (full exponents, no far list)
    image, h = resident.build_image(words, 148, layout="window4")
    assert h.mode == 3 and np.array_equal(resident.decode_image_host(image), words)
    bad = image.copy()
    bad[h.blobs_at + 32:h.blobs_at + 34] = 0xFF
    with pytest.raises(ValueError):
        resident.decode_image_host(bad)
    image, h = resident.build_image(noisy, 148, layout="window4")
    assert h.mode in (0, 1) and np.array_equal(resident.decode_image_host(image), noisy)


def test_wide_window_blobs_share_one_size_unless_they_differ_much(orc):
    """The builder pads the blobs of a wide-window image to one size (header blob_stride16) so that a kernel can
    address blob b as b x size; an image whose blobs differ by more than 512 bytes keeps its offset table only."""
    import numpy as np

    from georefine_b200 import resident

    words = orc.synthetic_weight_words(256, 512, 11)
    image, header = resident.build_image(words, 7, layout="window4")
    assert header.mode == 3 and header.blob_stride16 * 16 >= 24640
    assert np.array_equal(resident.decode_image_host(image), words)
    rng = np.random.default_rng(11)
    rows, cols = rng.integers(0, 128, 150), rng.integers(0, 128, 150)
    words[rows, cols] = 0x0100 | (words[rows, cols] & 0x807F)   # ~150 weights far below their row windows, all in one chunk
    image, header = resident.build_image(words, 7, layout="window4")
    assert header.mode == 3 and header.blob_stride16 == 0
    assert np.array_equal(resident.decode_image_host(image), words)
