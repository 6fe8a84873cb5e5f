"""Pins the CPU oracle: golden vectors made by the reference codec, and the reference library itself."""
import hashlib

import numpy as np
import pytest

FRAME_TAGS = ["special", "uniform13x17", "constant", "synthetic64x512", "synthetic48x320.r4c1", "conditional96x160"]


@pytest.mark.parametrize("tag", FRAME_TAGS)
def test_oracle_decodes_reference_frames(golden, oracle_coder, tag):
    frame = golden[tag + ".frame"].tobytes()
    assert np.array_equal(oracle_coder.decode(frame), golden[tag + ".words"])


@pytest.mark.parametrize("tag", FRAME_TAGS)
def test_oracle_encoder_reproduces_reference_frames_byte_for_byte(golden, oracle_coder, tag):
    nr, nc = map(int, golden[tag + ".classes"])
    assert oracle_coder.encode(golden[tag + ".words"], row_classes=nr, col_classes=nc) == golden[tag + ".frame"].tobytes()


def test_modes_seen_in_golden_set(golden):
    modes = {tag: int(golden[tag + ".frame"][5]) for tag in FRAME_TAGS}
    assert modes["uniform13x17"] == 1 and modes["conditional96x160"] == 128 and modes["synthetic64x512"] == 0


@pytest.mark.parametrize("name", ["all_words", "constant", "sparse"])
@pytest.mark.parametrize("nr,nc", [(1, 1), (4, 4), (16, 4), (64, 16)])
def test_distribution_frames_match_reference_digest(golden, oracle_coder, name, nr, nc):
    words = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    if name == "constant":
        words = np.full((64, 128), 0x3F80, dtype=np.uint16)
    elif name == "sparse":
        words = words.copy()
        words[:240] = 0x3F80
    frame = oracle_coder.encode(words, row_classes=nr, col_classes=nc)
    mode, length = map(int, golden[f"dist.{name}.{nr}x{nc}.mode_len"])
    assert (frame[5], len(frame)) == (mode, length)
    assert hashlib.sha256(frame).digest() == golden[f"dist.{name}.{nr}x{nc}.frame_sha256"].tobytes()
    assert np.array_equal(oracle_coder.decode(frame), words)


@pytest.mark.parametrize("tag,strides", [("special", (1, 7, 128, 1024)), ("constant", (128, 1024)),
                                         ("synthetic64x512", (128, 1024)), ("conditional96x160", (1, 100, 1024))])
def test_index_matches_reference_restart_points(golden, oracle_coder, tag, strides):
    frame = golden[tag + ".frame"].tobytes()
    for stride in strides:
        idx = oracle_coder.index_frame(frame, stride)
        assert idx["source_sha256"] == hashlib.sha256(golden[tag + ".words"].tobytes()).hexdigest()
        n = golden[tag + ".words"].size
        assert len(idx["main_states"]) == (n + stride - 1) // stride
        assert np.array_equal(idx["main_states"], golden[f"{tag}.s{stride}.main_states"])
        assert np.array_equal(idx["main_offsets"], golden[f"{tag}.s{stride}.main_offsets"])
        assert idx["main_states"][0] >= 1 << 23 and idx["main_offsets"][0] == 4
        if idx["mode"] == 128:
            assert np.array_equal(idx["residual_states"], golden[f"{tag}.s{stride}.residual_states"])
            assert np.array_equal(idx["residual_offsets"], golden[f"{tag}.s{stride}.residual_offsets"])


def _python_chunk_decode(stream, state, offset, start, end, freq, ctx_of):
    """Independent pure-Python rANS walk used to cross-check every restart point."""
    out = []
    for i in range(start, end):
        row = freq[ctx_of(i)]
        slot = state & 65535
        acc = 0
        for s, f in enumerate(row):
            f = int(f)
            if acc <= slot < acc + f:
                break
            acc += f
        else:
            raise AssertionError("slot not covered")
        out.append(s)
        state = f * (state >> 16) + slot - acc
        while state < (1 << 23):
            state = (state << 8) | stream[offset]
            offset += 1
    return out, state, offset


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("stride", [1, 7, 19, 128])
def test_abi_case_every_restart_point_resumes(golden, orc, oracle_coder, kind, stride):
    tag = f"abi9x17.k{kind}"
    vals = golden[tag + ".vals"]
    rows_n, cols_n, nr, nc = 9, 17, 4, 3
    rc = (np.arange(rows_n, dtype=np.uint8) % nr).copy()
    cc = (np.arange(cols_n, dtype=np.uint8) % nc).copy()
    freq, stream = oracle_coder.encode_stream(vals, rc, cc, nr, nc, kind)
    assert np.array_equal(freq, golden[tag + ".freq"])
    assert stream == golden[tag + ".stream"].tobytes()
    main, resid = orc.split_words(vals)
    resctx = main.ravel() if kind else None
    states, offsets, sym = oracle_coder.checkpoint(stream, freq, rc, cc, rows_n, cols_n, nr, nc, kind, stride, resctx)
    assert np.array_equal(states, golden[f"{tag}.s{stride}.states"])
    assert np.array_equal(offsets, golden[f"{tag}.s{stride}.offsets"])
    expected = (resid if kind else main).ravel()
    assert np.array_equal(sym, expected) and np.array_equal(sym, golden[tag + ".symbols"])
    ctx_of = (lambda i: int(resctx[i])) if kind else (lambda i: int(rc[i // cols_n]) * nc + int(cc[i % cols_n]))
    n = vals.size
    for cp, start in enumerate(range(0, n, stride)):
        end = min(start + stride, n)
        chunk, state, offset = _python_chunk_decode(stream, int(states[cp]), int(offsets[cp]), start, end, freq, ctx_of)
        assert chunk == expected[start:end].tolist()
        if cp + 1 < len(states):
            assert (state, offset) == (int(states[cp + 1]), int(offsets[cp + 1]))
        else:
            assert state == 1 << 23 and offset == len(stream)


@pytest.mark.parametrize("kind", [0, 1])
def test_malformed_inputs_rejected_and_output_untouched(golden, orc, oracle_coder, kind):
    tag = f"abi9x17.k{kind}"
    vals = golden[tag + ".vals"]
    freq = golden[tag + ".freq"]
    stream = golden[tag + ".stream"].tobytes()
    rows_n, cols_n, nr, nc = 9, 17, 4, 3
    rc = (np.arange(rows_n, dtype=np.uint8) % nr).copy()
    cc = (np.arange(cols_n, dtype=np.uint8) % nc).copy()
    main, resid = orc.split_words(vals)
    resctx = main.ravel() if kind else None

    def run(stream=stream, freq=freq, rc=rc, n=None):
        out = np.full(vals.size, 0xFFFF, dtype=np.uint16)
        st, _, _, out = oracle_coder.checkpoint_status(stream, freq, rc, cc, rows_n, cols_n, nr, nc, kind, 19, resctx,
                                                      n=n, out=out)
        return st, out

    st, out = run()
    assert st == 0 and np.array_equal(out, (resid if kind else main).ravel())
    bad = freq.copy()
    used_ctx = int(resctx[0]) if kind else int(rc[0]) * nc + int(cc[0])
    bad[used_ctx, int((resid if kind else main).ravel()[0])] += 1
    for kwargs in (dict(stream=stream[:-1]), dict(stream=stream + b"\0"), dict(freq=bad), dict(n=vals.size - 1)):
        st, out = run(**kwargs)
        assert st != 0 and np.all(out == 0xFFFF), kwargs
    if kind == 0:
        bad_rc = rc.copy()
        bad_rc[0] = nr
        st, out = run(rc=bad_rc)
        assert st != 0 and np.all(out == 0xFFFF)
    # plain decode honours the same stream faults
    for s in (b"\0\0\0\0" + stream[4:], stream[:-1], stream + b"\0"):
        st, _ = oracle_coder.decode_stream_status(s, freq, rc, cc, rows_n, cols_n, nr, nc, kind, resctx)
        assert st == 2
    st, _ = oracle_coder.decode_stream_status(stream, np.zeros_like(freq), rc, cc, rows_n, cols_n, nr, nc, kind, resctx)
    assert st == 2


def test_pack6_msb_first_and_tail_rule(oracle_coder):
    words = np.array([0x801F, 0x0001, 0x8000, 0x001F, 0x0015], dtype=np.uint16)  # residuals 63,1,32,31,21
    packed = oracle_coder.pack6(words)
    bits = "".join(f"{v:06b}" for v in (63, 1, 32, 31, 21))
    bits += "0" * (-len(bits) % 8)
    assert packed == int(bits, 2).to_bytes(len(bits) // 8, "big")
    assert oracle_coder.unpack6(packed, 5).tolist() == [63, 1, 32, 31, 21]
    with pytest.raises(ValueError):
        oracle_coder.unpack6(packed[:-1] + bytes([packed[-1] | 1]), 5)
    with pytest.raises(ValueError):
        oracle_coder.unpack6(packed + b"\0", 5)


def test_oracle_agrees_with_reference_library_on_random_cases(orc, oracle_coder):
    if not orc.ref_available():
        pytest.skip("oracle/_ref/libbcx_ref.so not built in this checkout")
    ref = orc.Coder("ref")
    rng = np.random.default_rng(5)
    for trial in range(12):
        rows_n, cols_n = int(rng.integers(1, 40)), int(rng.integers(1, 90))
        nr, nc = int(rng.choice([1, 4, 16, 64])), int(rng.choice([1, 4, 16]))
        if trial % 3 == 0:
            words = rng.integers(0, 65536, (rows_n, cols_n), dtype=np.uint16)
        else:
            words = orc.synthetic_weight_words(rows_n, cols_n, 100 + trial)
        rc, cc = orc.labels(words, nr, nc)
        main = orc.split_words(words)[0].ravel()
        for kind in (0, 1):
            fa, sa = oracle_coder.encode_stream(words, rc, cc, nr, nc, kind)
            fb, sb = ref.encode_stream(words, rc, cc, nr, nc, kind)
            assert np.array_equal(fa, fb) and sa == sb
            assert np.array_equal(oracle_coder.frequencies(words, rc, cc, nr, nc, kind), fb)
            resctx = main if kind else None
            stride = int(rng.integers(1, 300))
            a = oracle_coder.checkpoint(sb, fb, rc, cc, rows_n, cols_n, nr, nc, kind, stride, resctx)
            b = ref.checkpoint(sb, fb, rc, cc, rows_n, cols_n, nr, nc, kind, stride, resctx)
            assert all(np.array_equal(x, y) for x, y in zip(a, b))
            assert np.array_equal(oracle_coder.decode_stream(sb, fb, rc, cc, rows_n, cols_n, nr, nc, kind, resctx), b[2])
        assert oracle_coder.pack6(words) == ref.pack6(words)
        assert oracle_coder.encode(words, row_classes=nr, col_classes=nc) == ref.encode(words, row_classes=nr, col_classes=nc)
