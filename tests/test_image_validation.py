"""Structural validation of resident images on the host: a malformed, stale or foreign image must be refused before any
offset inside it is followed (by the host twin here; the kernels follow the same offsets unchecked on the GPU)."""
import ctypes

import numpy as np
import pytest

from georefine_b200 import _native, image_cache, resident

HEADER_OFFSETS = ["lut_at", "base_at", "items_at", "worker_items_at", "states_at", "blob_index_at", "blobs_at"]


@pytest.fixture(scope="module")
def images(orc):
    words = orc.synthetic_weight_words(300, 520, 3)
    return {layout: resident.build_image(words, 12, layout=layout)[0] for layout in ("window4", "window", "rans")} | {
        "raw": resident.build_image(words, 12, force_raw=True)[0]}, words


def _validate(image):
    return _native.lib().bxr_validate(image.ctypes.data_as(_native.U8P), image.size)


def _with_header(image, **fields):
    bad = image.copy()
    h = resident.header_of(bad)
    for name, value in fields.items():
        setattr(h, name, value)
    bad[:ctypes.sizeof(h)] = np.frombuffer(bytes(h), dtype=np.uint8)
    return bad


def test_built_images_validate_and_carry_the_layout_version(images):
    imgs, words = images
    for layout, image in imgs.items():
        assert _validate(image) == 0
        assert resident.header_of(image).layout_version == _native.lib().bxr_layout_version()
        assert np.array_equal(resident.decode_image_host(image), words)


@pytest.mark.parametrize("layout", ["window4", "window", "rans", "raw"])
def test_every_corrupt_header_offset_is_refused(images, layout):
    image = images[0][layout]
    h = resident.header_of(image)
    for name in HEADER_OFFSETS:
        if name in ("lut_at", "states_at") and layout != "rans":
            continue                       # arrays a fixed-code or raw image does not have
        for value in (int(h.total_bytes) + 4096, 2**63, 8, getattr(h, name) + 1):
            bad = _with_header(image, **{name: value})
            assert _validate(bad) == 1, f"{layout}: {name} = {value} accepted"
            out = np.zeros((h.rows, h.cols), dtype=np.uint16)
            assert _native.lib().bxr_decode_host(bad.ctypes.data_as(_native.U8P), bad.size, out.ctypes.data_as(_native.U16P)) == 1
            assert not out.any(), "a refused image must not be decoded"
            with pytest.raises(ValueError):
                resident.validate_image(bad)
    for fields in ({"row_blocks": h.row_blocks + 1}, {"chunks": 10**6}, {"items": h.items + 1}, {"workers": h.workers + 1},
                   {"partial_slots": h.partial_slots + 3}, {"layout_version": h.layout_version + 1}, {"mode": 9},
                   {"total_bytes": h.total_bytes - 16}, {"rows": 0}, {"blob_stride16": 7}):
        assert _validate(_with_header(image, **fields)) == 1, f"{layout}: {fields} accepted"
    assert _validate(image[:-16].copy()) == 1 and _validate(image[:64].copy()) == 1


@pytest.mark.parametrize("layout", ["window4", "window", "rans"])
def test_corrupt_blob_index_and_partition_are_refused(images, layout):
    image = images[0][layout]
    h = resident.header_of(image)
    index_at = int(h.blob_index_at)
    for entry, value in ((3, 0xFFFFFFF0), (3, 0), (int(h.row_blocks * h.chunks), 1), (0, 1)):
        bad = image.copy()
        bad[index_at + 4 * entry:index_at + 4 * entry + 4] = np.frombuffer(np.uint32(value).tobytes(), dtype=np.uint8)
        assert _validate(bad) == 1
    bad = image.copy()
    bad[int(h.items_at) + 4] ^= 1        # an item that starts at another chunk than the partition says
    assert _validate(bad) == 1
    bad = image.copy()
    bad[int(h.worker_items_at) + 4] ^= 1
    assert _validate(bad) == 1
    bad = image.copy()
    bad[int(h.base_at)] = 255            # a row window that would run past exponent 255
    assert _validate(bad) == 1


def test_a_stale_cache_entry_is_quarantined_not_served(images, tmp_path):
    """An entry whose file and description agree with each other but whose image belongs to another layout version (or is
    damaged inside its arrays) is moved aside and reported as a miss."""
    import hashlib
    import json

    image = images[0]["window4"]
    h = resident.header_of(image)
    cache = image_cache.ImageCache(tmp_path)
    assert cache.put(image, "window4")
    source, shape = bytes(h.source_sha256).hex(), (int(h.rows), int(h.cols))
    assert cache.get(source, shape, "window4", int(h.workers)) is not None
    image_path, meta_path = cache._paths(image_cache.cache_key(source, shape, "window4", int(h.workers)))
    stale = _with_header(image, layout_version=h.layout_version - 1)
    stale.tofile(image_path)
    meta = json.loads(meta_path.read_text())
    meta["image_sha256"] = hashlib.sha256(stale.tobytes()).hexdigest()
    meta_path.write_text(json.dumps(meta))
    assert cache.get(source, shape, "window4", int(h.workers)) is None
    assert cache.stats["quarantined"] == 1 and not image_path.exists()
    # and the key itself depends on the layout version
    assert image_cache.cache_key(source, shape, "window4", 12) != hashlib.sha256(json.dumps(
        {"schema": image_cache.SCHEMA, "cache_format": image_cache.CACHE_FORMAT, "source_sha256": source, "shape": list(shape),
         "layout": "window4", "workers": 12}, sort_keys=True, separators=(",", ":")).encode()).hexdigest()
