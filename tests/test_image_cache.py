"""The verified cache of resident images and the parallel load-time builder (host only).

Follows the behaviour the reference tests for its transcode cache: a hit returns the stored bytes, a request that
differs in any key field misses, a damaged entry is moved aside and reported as a miss, nothing here is ever fatal.
"""
import hashlib
import json

import numpy as np
import pytest

from georefine_b200 import codec, image_cache, resident


@pytest.fixture()
def frame_and_words(orc):
    words = orc.synthetic_weight_words(160, 384, 77)
    return codec.encode(words), words


def test_frame_identity_needs_no_decoding(frame_and_words):
    frame, words = frame_and_words
    source, shape = image_cache.frame_identity(frame)
    assert shape == words.shape and source == hashlib.sha256(words.tobytes()).hexdigest()
    with pytest.raises(codec.CodecError):
        image_cache.frame_identity(frame[:-1] + bytes([frame[-1] ^ 1]))


@pytest.mark.parametrize("layout", ["window", "rans"])
def test_miss_then_hit_returns_the_same_image(tmp_path, frame_and_words, layout):
    frame, words = frame_and_words
    cache = image_cache.ImageCache(tmp_path, verify="full")
    image, header, hit = image_cache.image_for_frame(frame, 148, layout=layout, cache=cache)
    assert not hit and cache.stats["writes"] == 1 and np.array_equal(resident.decode_image_host(image), words)
    again, header2, hit2 = image_cache.image_for_frame(frame, 148, layout=layout, cache=cache)
    assert hit2 and np.array_equal(again, image) and header2.mode == header.mode
    # any field of the key changes the entry
    assert cache.get(bytes(header.source_sha256).hex(), words.shape, layout, 147) is None
    assert cache.get(bytes(header.source_sha256).hex(), words.shape, "raw", 148) is None
    assert cache.get("00" * 32, words.shape, layout, 148) is None


def test_damaged_entries_are_moved_aside_and_rebuilt(tmp_path, frame_and_words):
    frame, words = frame_and_words
    cache = image_cache.ImageCache(tmp_path)
    image, header, _ = image_cache.image_for_frame(frame, 9, cache=cache)
    source = bytes(header.source_sha256).hex()
    key = image_cache.cache_key(source, words.shape, resident.DEFAULT_LAYOUT, 9)
    image_path, meta_path = cache._paths(key)
    # a flipped payload byte: the recorded SHA-256 no longer matches
    data = bytearray(image_path.read_bytes())
    data[len(data) // 2] ^= 0x10
    image_path.write_bytes(bytes(data))
    assert cache.get(source, words.shape, resident.DEFAULT_LAYOUT, 9) is None
    assert cache.stats["quarantined"] == 1 and not image_path.exists() and not meta_path.exists()
    assert any(".bad-" in p.name for p in image_path.parent.iterdir())
    # the next load rebuilds and stores a good entry
    rebuilt, _, hit = image_cache.image_for_frame(frame, 9, cache=cache)
    assert not hit and np.array_equal(rebuilt, image)
    assert cache.get(source, words.shape, resident.DEFAULT_LAYOUT, 9) is not None
    # an image that hashes right but belongs to other words is refused by the header check / the full check
    other = resident.build_image(np.ascontiguousarray(words[::-1]), 9)[0]
    image_path.write_bytes(other.tobytes())
    meta = json.loads(meta_path.read_text())
    meta["image_sha256"], meta["image_bytes"] = hashlib.sha256(other.tobytes()).hexdigest(), int(other.size)
    meta_path.write_text(json.dumps(meta))
    assert cache.get(source, words.shape, resident.DEFAULT_LAYOUT, 9) is None and cache.stats["quarantined"] == 2
    # an entry without its description (an interrupted write) is simply not there
    image_cache.image_for_frame(frame, 9, cache=cache)
    meta_path.unlink()
    assert cache.get(source, words.shape, resident.DEFAULT_LAYOUT, 9) is None and cache.stats["quarantined"] == 2


def test_full_verification_catches_a_consistent_forgery(tmp_path, frame_and_words):
    frame, words = frame_and_words
    cache = image_cache.ImageCache(tmp_path, verify="full")
    image, header, _ = image_cache.image_for_frame(frame, 5, cache=cache)
    source = bytes(header.source_sha256).hex()
    forged_words = words.copy()
    forged_words[3, 7] ^= 0x0100
    forged = resident.build_image(forged_words, 5, source_sha256=bytes.fromhex(source))[0]   # claims the original digest
    image_path, meta_path = cache._paths(image_cache.cache_key(source, words.shape, resident.DEFAULT_LAYOUT, 5))
    image_path.write_bytes(forged.tobytes())
    meta = json.loads(meta_path.read_text())
    meta["image_sha256"], meta["image_bytes"] = hashlib.sha256(forged.tobytes()).hexdigest(), int(forged.size)
    meta_path.write_text(json.dumps(meta))
    assert image_cache.ImageCache(tmp_path, verify="hash").get(source, words.shape, resident.DEFAULT_LAYOUT, 5) is not None
    assert cache.get(source, words.shape, resident.DEFAULT_LAYOUT, 5) is None


def test_unwritable_root_is_not_fatal(tmp_path, frame_and_words):
    frame, words = frame_and_words
    blocker = tmp_path / "file"
    blocker.write_text("not a directory")
    messages = []
    cache = image_cache.ImageCache(blocker / "below", log=messages.append)
    image, _, hit = image_cache.image_for_frame(frame, 4, cache=cache)
    assert not hit and np.array_equal(resident.decode_image_host(image), words)
    assert cache.stats["writes"] == 0 and any("cannot write" in m for m in messages)


def test_many_tensors_in_parallel(tmp_path, orc):
    frames, expect = {}, {}
    for i, shape in enumerate([(128, 256), (96, 640), (257, 130), (64, 1024)]):
        words = orc.synthetic_weight_words(*shape, 90 + i)
        frames[f"layer{i}.weight"], expect[f"layer{i}.weight"] = codec.encode(words), words
    cache = image_cache.ImageCache(tmp_path)
    first = image_cache.images_for_frames(frames, 148, cache=cache, pool_threads=4)
    assert all(not hit for _, _, hit in first.values()) and cache.stats["writes"] == 4
    for name, (image, header, _) in first.items():
        assert (header.rows, header.cols) == expect[name].shape and np.array_equal(resident.decode_image_host(image), expect[name])
    second = image_cache.images_for_frames(frames, 148, cache=cache, pool_threads=4)
    assert all(hit for _, _, hit in second.values())
    assert all(np.array_equal(second[n][0], first[n][0]) for n in frames)
