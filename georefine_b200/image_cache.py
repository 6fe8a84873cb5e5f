"""Verified on-disk cache of resident images, and parallel building of many tensors at load time.

The serial part of loading a BCTX tensor is the host walk that decodes its single rANS stream (seconds per large
tensor) before the resident image can be built.  The reference removes that cost from restarts with a verified
cache of its load-time transcode (``glc_serve/transcode_cache.py``: a key over the source identity and every flag
that changes the content, writes renamed into place last, a completion marker, per-row source digests, "hash" and
"full" verification, a failed entry moved aside and never fatal) and spreads first-time conversion over CPU workers
(``glc_serve/context_parallel_startup.py``).  This module does the same for resident images.

Layout under the cache root, one entry per (source digest, shape, layout, workers, layout version of the library)::

    <root>/<key[:2]>/<key>.bxr        the image, written to <key>.bxr.partial-<host>-<pid>-<nonce> and renamed
    <root>/<key[:2]>/<key>.json       the entry's description, written last: its presence marks the entry complete

An entry is served only if its description matches the request, the file has the recorded size and SHA-256, the
image passes the library's structural check (``bxr_validate``: layout version, every offset and extent, the work
partition, the blob index), its header agrees (shape, workers, source digest) and - with ``verify="full"`` - the host twin of the GPU
decoder reproduces the source digest from it.  Anything else moves the entry aside and reports a miss.
"""
from __future__ import annotations

import hashlib
import json
import os
import socket
import uuid
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

from . import codec, resident

CACHE_FORMAT = 1
SCHEMA = "georefine_b200.resident_image_cache.v1"
VERIFY_MODES = ("hash", "full")
ENV_CACHE_DIR = "GEOREFINE_B200_IMAGE_CACHE"


class ImageCacheError(RuntimeError):
    pass


def default_cache_root() -> Path:
    """``$GEOREFINE_B200_IMAGE_CACHE``, else ``$XDG_CACHE_HOME/georefine-b200/images``, else ``~/.cache/...``."""
    env = os.environ.get(ENV_CACHE_DIR)
    if env:
        return Path(env).expanduser()
    xdg = os.environ.get("XDG_CACHE_HOME")
    return (Path(xdg).expanduser() if xdg else Path.home() / ".cache") / "georefine-b200" / "images"


def layout_version() -> int:
    """The resident layout version of the loaded library: part of every key, so entries written by a build with
    another blob layout or work partition are never looked at."""
    from . import _native

    return int(_native.lib().bxr_layout_version())


def cache_key(source_sha256: str, shape, layout: str, workers: int) -> str:
    material = {"schema": SCHEMA, "cache_format": CACHE_FORMAT, "layout_version": layout_version(),
                "source_sha256": source_sha256, "shape": [int(shape[0]), int(shape[1])], "layout": layout,
                "workers": int(workers)}
    return hashlib.sha256(json.dumps(material, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def frame_identity(frame: bytes):
    """(source_sha256 hex, (rows, cols)) from the frame header and its checksum alone: no entropy decoding."""
    if len(frame) < codec.HEADER.size + 32 or hashlib.sha256(frame[:-32]).digest() != bytes(frame[-32:]):
        raise codec.CodecError("frame checksum mismatch")
    magic, ver, _mode, _nr, _nc, r, c, *_rest, dig = codec.HEADER.unpack_from(frame)
    if magic != codec.MAGIC or ver != codec.VERSION or not r or not c:
        raise codec.CodecError("unsupported frame header")
    return dig.hex(), (r, c)


class ImageCache:
    def __init__(self, root=None, *, verify: str = "hash", log=None):
        if verify not in VERIFY_MODES:
            raise ImageCacheError(f"verify must be one of {VERIFY_MODES}")
        self.root = Path(root).expanduser() if root is not None else default_cache_root()
        self.verify = verify
        self.log = log or (lambda message: None)
        self.stats = {"hits": 0, "misses": 0, "writes": 0, "quarantined": 0, "bytes_read": 0, "bytes_written": 0}

    def _paths(self, key: str):
        d = self.root / key[:2]
        return d / f"{key}.bxr", d / f"{key}.json"

    def _quarantine(self, key: str, reason: str) -> None:
        tag = uuid.uuid4().hex[:8]
        for path in self._paths(key):
            try:
                if path.exists():
                    path.rename(path.with_name(path.name + f".bad-{tag}"))
            except OSError:
                pass
        self.stats["quarantined"] += 1
        self.log(f"[image-cache] entry {key[:12]} failed verification ({reason}); moved aside")

    def get(self, source_sha256: str, shape, layout: str, workers: int):
        """The cached image as a uint8 array, or None.  Never raises for a bad or unreadable entry."""
        key = cache_key(source_sha256, shape, layout, workers)
        image_path, meta_path = self._paths(key)
        try:
            if not meta_path.is_file() or not image_path.is_file():
                self.stats["misses"] += 1
                return None
            meta = json.loads(meta_path.read_text(encoding="utf-8"))
            want = {"schema": SCHEMA, "cache_format": CACHE_FORMAT, "layout_version": layout_version(),
                    "source_sha256": source_sha256, "shape": [int(shape[0]), int(shape[1])], "layout": layout,
                    "workers": int(workers)}
            for name, value in want.items():
                if meta.get(name) != value:
                    raise ImageCacheError(f"description field {name} differs")
            if image_path.stat().st_size != meta.get("image_bytes"):
                raise ImageCacheError("image size differs from its description")
            image = np.fromfile(image_path, dtype=np.uint8)
            if hashlib.sha256(image.tobytes()).hexdigest() != meta.get("image_sha256"):
                raise ImageCacheError("image SHA-256 differs from its description")
            resident.validate_image(image)   # raises ValueError: offsets, partition, blob index, layout version
            h = resident.header_of(image)
            if (h.total_bytes != image.size or (h.rows, h.cols) != tuple(shape) or h.workers != workers
                    or bytes(h.source_sha256).hex() != source_sha256):
                raise ImageCacheError("image header does not match the request")
            if self.verify == "full":
                words = resident.decode_image_host(image)
                if hashlib.sha256(words.astype("<u2").tobytes()).hexdigest() != source_sha256:
                    raise ImageCacheError("image does not reproduce the source digest")
        except (ImageCacheError, ValueError) as exc:
            self._quarantine(key, str(exc))
            self.stats["misses"] += 1
            return None
        except OSError as exc:   # e.g. a cache directory owned by someone else: serve uncached
            self.log(f"[image-cache] cannot read {image_path} ({type(exc).__name__}: {exc})")
            self.stats["misses"] += 1
            return None
        self.stats["hits"] += 1
        self.stats["bytes_read"] += int(image.size)
        return image

    def put(self, image: np.ndarray, layout: str) -> bool:
        """Stores an image under the key its own header implies; False (and a log line) if that is not possible."""
        h = resident.header_of(image)
        source, shape, workers = bytes(h.source_sha256).hex(), (int(h.rows), int(h.cols)), int(h.workers)
        key = cache_key(source, shape, layout, workers)
        image_path, meta_path = self._paths(key)
        partial = image_path.with_name(f"{image_path.name}.partial-{socket.gethostname()}-{os.getpid()}-{uuid.uuid4().hex[:8]}")
        try:
            image_path.parent.mkdir(parents=True, exist_ok=True)
            data = np.ascontiguousarray(image, dtype=np.uint8).tobytes()
            with open(partial, "wb") as f:
                f.write(data)
                f.flush()
                os.fsync(f.fileno())
            os.replace(partial, image_path)
            meta = {"schema": SCHEMA, "cache_format": CACHE_FORMAT, "layout_version": int(h.layout_version),
                    "source_sha256": source, "shape": list(shape),
                    "layout": layout, "workers": workers, "mode": int(h.mode), "image_bytes": len(data),
                    "image_sha256": hashlib.sha256(data).hexdigest(), "coded_bytes": int(h.coded_bytes)}
            tmp = meta_path.with_name(meta_path.name + f".partial-{uuid.uuid4().hex[:8]}")
            tmp.write_text(json.dumps(meta, sort_keys=True), encoding="utf-8")
            os.replace(tmp, meta_path)   # last: an entry without its description is ignored
        except OSError as exc:
            self.log(f"[image-cache] cannot write {image_path} ({type(exc).__name__}: {exc}); serving uncached")
            try:
                if partial.exists():
                    partial.unlink()
            except OSError:
                pass
            return False
        self.stats["writes"] += 1
        self.stats["bytes_written"] += len(data)
        return True


def image_for_frame(frame: bytes, workers: int, *, layout: str = resident.DEFAULT_LAYOUT, cache: ImageCache | None = None,
                    threads: int = 0):
    """(image, header, hit) for a BCTX frame: from the cache when it holds a verified entry, else decoded on the
    host, built and stored.  On a hit the frame's entropy streams are never walked."""
    source, shape = frame_identity(frame)
    if cache is not None:
        image = cache.get(source, shape, layout, workers)
        if image is not None:
            return image, resident.header_of(image), True
    words = codec.decode(frame)   # verifies the source digest
    image, header = resident.build_image(words, workers, threads=threads, layout=layout, source_sha256=bytes.fromhex(source))
    if cache is not None:
        cache.put(image, layout)
    return image, header, False


def images_for_frames(frames: dict, workers: int, *, layout: str = resident.DEFAULT_LAYOUT, cache: ImageCache | None = None,
                      pool_threads: int | None = None):
    """Builds (or fetches) the images of many tensors at once: one host thread per tensor (the native calls release
    the interpreter lock), each tensor's builder single-threaded.  Returns {name: (image, header, hit)}."""
    names = list(frames)
    pool_threads = pool_threads or max(1, min(len(names), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=pool_threads, thread_name_prefix="grb-image") as pool:
        results = list(pool.map(lambda name: image_for_frame(frames[name], workers, layout=layout, cache=cache, threads=1), names))
    return dict(zip(names, results))


class CachedLinear:
    """A BCTX weight served by its resident image alone, for linears that are never gathered row by row: the tensor
    contract the reference's loader checks (``shape``, ``source_sha256``, ``frame_sha256``, ``resident_bytes``,
    ``decode``; ``bitexact_context_serving.py:560-569``) without the unchanged streams and their restart index, so a
    cache hit costs a file read, a hash and one host-to-device copy."""

    def __init__(self, frame: bytes, *, device="cuda:0", cache: ImageCache | None = None, layout: str = resident.DEFAULT_LAYOUT,
                 max_m: int = 128, workers: int | None = None, stride: int = 1024):
        import torch

        self.device = torch.device(device)
        if workers is None:
            _, (rows, cols) = frame_identity(frame)
            workers = resident.default_workers(rows, cols, resident.sm_count(self.device))
        image, header, self.cache_hit = image_for_frame(frame, workers, layout=layout, cache=cache)
        self.resident = resident.ResidentWeight(image, self.device, max_m=max_m, verify=False)
        self.shape = (int(header.rows), int(header.cols))
        self.n = self.shape[0] * self.shape[1]
        self.stride = stride
        self.source_sha256 = bytes(header.source_sha256).hex()
        self.frame_sha256 = hashlib.sha256(frame).hexdigest()
        self.frame_bytes = len(frame)
        self.mode = int(header.mode)
        self.resident_bytes = self.resident.resident_bytes

    def decode(self, *, check=True):
        return self.resident.decode(check=check)

    def gather_rows(self, ids, *, check=True):
        return self.decode(check=check)[ids.to(self.device)]

    def linear(self, x, out=None, bias=None):
        return self.resident.linear(x, out=out, bias=bias)

    def __call__(self, x, y):
        self.resident(x, y)
