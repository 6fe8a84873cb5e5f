"""The drop-in claim, exercised: the REFERENCE's own Python modules bound to this library.

When a checkout of the reference project is reachable ($REFERENCE_ROOT, or a directory ``reference`` beside this
repository) its ``bitexact_context_codec`` and ``bitexact_context_gpu`` modules are imported unmodified and their
native-library loaders (``_lib`` / ``_index_lib``, which normally compile and load the reference's C++ coder) are
pointed at libgeorefine_b200.so instead.  Every frame the reference's container code then builds on top of OUR
``bcx_encode`` / ``bcx_pack6`` must equal, byte for byte, the golden frame the reference made with its own coder;
decode, the compact decoder, the restart index and the error behaviour must hold as well.  Skipped where no checkout is
reachable (the golden vectors under tests/golden/ pin the same facts there).
"""
import importlib
import sys

import numpy as np
import pytest

from georefine_b200 import _native
from oracle import bcx_oracle as orc

TAGS = ["special", "uniform13x17", "constant", "synthetic64x512", "synthetic48x320.r4c1", "conditional96x160"]


@pytest.fixture(scope="module")
def reference():
    root = orc.reference_root()
    if root is None or not (root / "context-runtime" / "georefine_context_runtime").is_dir():
        pytest.skip("no reference checkout reachable")
    sys.path.insert(0, str(root / "context-runtime"))
    try:
        codec = importlib.import_module("georefine_context_runtime.bitexact_context_codec")
        index = importlib.import_module("georefine_context_runtime.bitexact_context_gpu")
    finally:
        sys.path.pop(0)
    saved = codec._lib, index._index_lib
    codec._lib = _native.lib             # the reference's modules now call into this repository's library
    index._index_lib = _native.lib
    yield codec, index
    codec._lib, index._index_lib = saved


@pytest.mark.parametrize("tag", TAGS)
def test_reference_container_over_this_library_reproduces_the_golden_frames(reference, golden, tag):
    codec, index = reference
    words = golden[tag + ".words"]
    nr, nc = (int(v) for v in golden[tag + ".classes"])
    frame = codec.encode(words, row_classes=nr, col_classes=nc)
    assert frame == golden[tag + ".frame"].tobytes()
    assert np.array_equal(codec.decode(frame), words)


def test_reference_index_over_this_library_matches_its_own_restart_points(reference, golden):
    codec, index = reference
    frame = golden["synthetic64x512.frame"].tobytes()
    for stride in (1, 7, 128, 1024):
        got = index.index_frame(frame, stride)
        key = f"synthetic64x512.s{stride}"
        if key + ".main_states" in golden:
            assert np.array_equal(got["main_states"], golden[key + ".main_states"])
            assert np.array_equal(got["main_offsets"], golden[key + ".main_offsets"])
        assert got["main_states"].size == -(-64 * 512 // stride) and int(got["main_offsets"][0]) == 4
    ours = importlib.import_module("georefine_b200.gpu").index_frame(frame, 128)
    theirs = index.index_frame(frame, 128)
    for name in ("main_states", "main_offsets", "rows", "columns", "main_freq", "main_stream", "residual_stream"):
        assert np.array_equal(ours[name], theirs[name]), name
    assert ours["source_sha256"] == theirs["source_sha256"] and ours["frame_sha256"] == theirs["frame_sha256"]


def test_reference_error_behaviour_over_this_library(reference, golden, monkeypatch):
    codec, index = reference
    frame = bytearray(golden["synthetic64x512.frame"].tobytes())
    frame[200] ^= 0x10
    with pytest.raises(codec.CodecError):
        codec.decode(bytes(frame))
    with pytest.raises(codec.CodecError, match="checksum"):
        index.index_frame(bytes(frame), 128)
    with pytest.raises(codec.CodecError, match="stride"):
        index.index_frame(golden["synthetic64x512.frame"].tobytes(), 0)
    monkeypatch.setenv("GEOREFINE_CONTEXT_COMPACT_RANS", "1")   # the reference then calls bcx_decode_compact
    good = golden["conditional96x160.frame"].tobytes()
    assert np.array_equal(codec.decode(good), golden["conditional96x160.words"])


def test_frames_cross_between_the_two_python_codecs(reference, golden):
    """Frames made here decode there and the other way round (with the reference's container over this library)."""
    from georefine_b200 import codec as ours

    codec, _ = reference
    words = orc.synthetic_weight_words(40, 300, 5)
    assert ours.encode(words) == codec.encode(words)
    assert np.array_equal(codec.decode(ours.encode(words, row_classes=4, col_classes=1)), words)
    assert np.array_equal(ours.decode(codec.encode(words, row_classes=64, col_classes=16)), words)
