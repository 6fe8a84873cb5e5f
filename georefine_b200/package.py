"""BCTX packages: a safetensors checkpoint turned into one verified frame per BF16 tensor, and back, byte for byte.

Counterpart of the reference's package tool (``georefine_context_runtime/bitexact_context_package.py:298-763``:
``build``, ``verify``, ``restore``, the decode check, manifest and per-tensor receipts).  The reference's tool is pinned
to one checkpoint (shard names, digests and tensor counts are constants in its source); this one keeps the on-disk
layout and the receipt fields a loader reads, for any safetensors checkpoint::

    <package>/manifest.json                 schema, completeness flag, source shards, one receipt per tensor
    <package>/frames/<sha256(name)>.bctx    the frame of a BF16 tensor (rank-N tensors are coded as rows x rest)
    <package>/raw/<sha256(name)>.bin        the verbatim bytes of a tensor of any other dtype
    <package>/headers/<shard>.header        the verbatim safetensors header of every source shard
    <package>/sidecars/...                  config.json, tokenizer files and the like, copied verbatim and pinned

A receipt: ``name, shard, begin, end, shape, dtype, source_bytes, source_sha256, frame, frame_bytes, frame_sha256,
mode, complete``.  ``build`` is resumable (a receipt file per finished tensor is written last, atomically) and spreads
the encoding over threads (the native coder releases the interpreter lock); ``verify`` checks the inventory (nothing
missing, nothing extra, no symlinks, no path leaving the package), every digest and - unless told otherwise - decodes
every frame; ``restore`` rebuilds the shards and compares their digests with the manifest.

    python -m georefine_b200.package build  <model dir> <package dir> [--jobs N] [--row-classes 16 --col-classes 4]
    python -m georefine_b200.package verify <package dir> [--no-decode]
    python -m georefine_b200.package restore <package dir> <destination dir>
    python -m georefine_b200.package decode-check <package dir> <tensor name or frames/<key>.bctx> ...
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import struct
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path, PurePosixPath

import numpy as np

from . import codec

SCHEMA = "bitexact-context-package-v1"
SIDECAR_SUFFIXES = (".json", ".txt", ".model", ".jinja", ".md")


def sha(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def sha_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(8 << 20), b""):
            h.update(block)
    return h.hexdigest()


def atomic_write(path: Path, data: bytes) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + ".partial")
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _dump(value) -> bytes:
    return json.dumps(value, sort_keys=True, separators=(",", ":")).encode() + b"\n"


def _no_duplicate_keys(pairs):
    out = {}
    for key, value in pairs:
        if key in out:
            raise ValueError(f"duplicate JSON key: {key}")
        out[key] = value
    return out


def key_for(name: str) -> str:
    return sha(name.encode())


def frame_shape(shape):
    """How a tensor is laid out as a 2-D word array: first dimension x the rest (a vector is one row)."""
    if len(shape) == 1:
        return 1, int(shape[0])
    return int(shape[0]), int(math.prod(shape[1:]))


# ---------------------------------------------------------------------------------------------- safetensors
def read_shard_header(path: Path):
    """(raw header bytes including the 8-byte length, parsed header, offset of the data section)."""
    with open(path, "rb") as f:
        size = struct.unpack("<Q", f.read(8))[0]
        if size > 100 << 20:
            raise ValueError(f"{path.name}: implausible safetensors header")
        text = f.read(size)
    if len(text) != size:
        raise ValueError(f"{path.name}: truncated safetensors header")
    return struct.pack("<Q", size) + text, json.loads(text, object_pairs_hook=_no_duplicate_keys), 8 + size


def tensor_descriptors(model_dir: Path):
    """Every tensor of every ``*.safetensors`` shard of a directory: name -> {shard, begin, end, shape, dtype}; plus the
    raw headers.  Offsets are absolute file offsets."""
    out, headers = {}, {}
    shards = sorted(p for p in model_dir.iterdir() if p.suffix == ".safetensors" and p.is_file() and not p.is_symlink())
    if not shards:
        raise ValueError("no safetensors shards found")
    for path in shards:
        raw, header, base = read_shard_header(path)
        headers[path.name] = raw
        for name, entry in header.items():
            if name == "__metadata__":
                continue
            if name in out:
                raise ValueError(f"tensor {name} appears in two shards")
            begin, end = entry["data_offsets"]
            out[name] = {"name": name, "shard": path.name, "begin": base + begin, "end": base + end, "shape": [int(d) for d in entry["shape"]],
                         "dtype": entry["dtype"]}
    return out, headers


def _read_range(path: Path, begin: int, end: int) -> bytes:
    with open(path, "rb") as f:
        f.seek(begin)
        data = f.read(end - begin)
    if len(data) != end - begin:
        raise ValueError(f"{path.name}: short read")
    return data


# ---------------------------------------------------------------------------------------------- build
def build(model_dir, output, *, jobs: int = 2, row_classes: int = 16, col_classes: int = 4, log=lambda message: None):
    """Encodes every tensor of the checkpoint in ``model_dir`` into ``output``.  Returns the manifest."""
    model_dir, output = Path(model_dir), Path(output)
    if jobs < 1:
        raise ValueError("jobs must be positive")
    if output.exists() and not output.is_dir():
        raise ValueError("output must be a directory")
    if (output / "manifest.json").exists():
        return verify(output, jobs=jobs)
    output.mkdir(parents=True, exist_ok=True)
    descriptors, headers = tensor_descriptors(model_dir)
    pin = {"schema": SCHEMA, "row_classes": row_classes, "col_classes": col_classes,
           "tensors": sha(_dump(sorted((d["name"], d["shard"], d["begin"], d["end"]) for d in descriptors.values())))}
    pin_path = output / "build_inputs.json"
    if pin_path.exists() and json.loads(pin_path.read_text()) != pin:
        raise ValueError("partial package inputs differ from the requested build")
    atomic_write(pin_path, _dump(pin))
    for shard, raw in headers.items():
        atomic_write(output / "headers" / (shard + ".header"), raw)
    sidecars = {}
    for path in sorted(model_dir.iterdir()):
        if path.is_file() and not path.is_symlink() and path.suffix in SIDECAR_SUFFIXES:
            data = path.read_bytes()
            atomic_write(output / "sidecars" / path.name, data)
            sidecars["sidecars/" + path.name] = {"bytes": len(data), "sha256": sha(data)}

    def process(d):
        receipt_path = output / "receipts" / (key_for(d["name"]) + ".json")
        if receipt_path.exists():
            row = json.loads(receipt_path.read_text())
            if row.get("complete") is True and row.get("name") == d["name"] and (output / row["frame"]).is_file():
                return row
        raw = _read_range(model_dir / d["shard"], d["begin"], d["end"])
        row = dict(d, source_bytes=len(raw), source_sha256=sha(raw))
        if d["dtype"] == "BF16" and len(raw) and len(raw) == 2 * math.prod(d["shape"]):
            words = np.frombuffer(raw, dtype="<u2").reshape(frame_shape(d["shape"]))
            frame = codec.encode(words, row_classes=row_classes, col_classes=col_classes)
            if codec.decode(frame).tobytes() != raw:                       # the decode check, before anything is recorded
                raise ValueError(f"frame of {d['name']} does not decode to its source")
            rel = "frames/" + key_for(d["name"]) + ".bctx"
            row.update(mode=frame[5], codec="bctx")
        else:
            frame, rel = raw, "raw/" + key_for(d["name"]) + ".bin"
            row.update(mode=None, codec="raw")
        atomic_write(output / rel, frame)
        row.update(frame=rel, frame_bytes=len(frame), frame_sha256=sha(frame), complete=True)
        atomic_write(receipt_path, _dump(row))                               # last: marks the tensor done
        log(f"[package] {d['name']}: {len(raw)} -> {len(frame)} bytes")
        return row

    with ThreadPoolExecutor(jobs) as pool:
        rows = list(pool.map(process, sorted(descriptors.values(), key=lambda d: (d["shard"], d["begin"]))))
    shards = {}
    for shard in headers:
        path = model_dir / shard
        shards[shard] = {"bytes": path.stat().st_size, "sha256": sha_file(path)}
    manifest = {"schema": SCHEMA, "complete": True, "row_classes": row_classes, "col_classes": col_classes, "shards": shards,
                "metadata_assets": sidecars, "tensors": rows,
                "source_bytes": sum(r["source_bytes"] for r in rows), "frame_bytes": sum(r["frame_bytes"] for r in rows)}
    atomic_write(output / "manifest.json", _dump(manifest))
    return manifest


# ---------------------------------------------------------------------------------------------- verify
def read_manifest(package: Path):
    try:
        manifest = json.loads((Path(package) / "manifest.json").read_text(encoding="utf-8"), object_pairs_hook=_no_duplicate_keys)
    except (OSError, json.JSONDecodeError) as exc:
        raise ValueError(f"cannot read package manifest: {exc}") from exc
    if manifest.get("schema") != SCHEMA or manifest.get("complete") is not True or not isinstance(manifest.get("tensors"), list):
        raise ValueError("unsupported, corrupt or incomplete package manifest")
    return manifest


def safe_member(package: Path, relative) -> Path:
    """A path named by the manifest, refused if it could leave the package or is a symlink."""
    if not isinstance(relative, str) or not relative:
        raise ValueError("unsafe package path")
    rel = PurePosixPath(relative)
    if rel.is_absolute() or ".." in rel.parts or rel.parts[0] not in ("frames", "raw", "sidecars", "headers"):
        raise ValueError(f"unsafe package path: {relative}")
    path = Path(package).joinpath(*rel.parts)
    if path.is_symlink():
        raise ValueError(f"symlink in package: {relative}")
    if Path(package).resolve() not in path.resolve().parents:
        raise ValueError(f"path outside the package: {relative}")
    return path


def inventory(package: Path):
    out = set()
    for root, dirs, files in os.walk(package):
        for name in dirs + files:
            if (Path(root) / name).is_symlink():
                raise ValueError(f"symlink in package: {name}")
        for name in files:
            out.add((Path(root) / name).relative_to(package).as_posix())
    return out


def verify(package, *, jobs: int = 8, decode_frames: bool = True):
    """Checks a package against its manifest; raises ValueError on the first problem, returns the manifest."""
    package = Path(package)
    manifest = read_manifest(package)
    rows, names = manifest["tensors"], set()
    expected = {"manifest.json", "build_inputs.json"}
    for row in rows:
        if not isinstance(row, dict) or row.get("complete") is not True or not isinstance(row.get("name"), str) or row["name"] in names:
            raise ValueError("corrupt or incomplete tensor receipt")
        names.add(row["name"])
        expected.add(row["frame"])
        expected.add("receipts/" + key_for(row["name"]) + ".json")
    expected |= {"headers/" + s + ".header" for s in manifest["shards"]} | set(manifest["metadata_assets"])
    found = inventory(package)
    if found - expected:
        raise ValueError(f"package inventory has files the manifest does not name: {sorted(found - expected)[:5]}")
    if expected - found:
        raise ValueError(f"package inventory omits files the manifest names: {sorted(expected - found)[:5]}")
    for rel, pin in manifest["metadata_assets"].items():
        data = safe_member(package, rel).read_bytes()
        if len(data) != pin["bytes"] or sha(data) != pin["sha256"]:
            raise ValueError(f"sidecar differs from its pin: {rel}")

    def check(row):
        frame = safe_member(package, row["frame"]).read_bytes()
        if len(frame) != row["frame_bytes"] or sha(frame) != row["frame_sha256"]:
            raise ValueError(f"frame identity mismatch: {row['name']}")
        if row["end"] - row["begin"] != row["source_bytes"]:
            raise ValueError(f"receipt geometry mismatch: {row['name']}")
        if decode_frames:
            raw = codec.decode(frame).tobytes() if row.get("codec") == "bctx" else frame
            if len(raw) != row["source_bytes"] or sha(raw) != row["source_sha256"]:
                raise ValueError(f"decoded-source identity mismatch: {row['name']}")
        return True

    with ThreadPoolExecutor(jobs) as pool:
        list(pool.map(check, rows))
    return manifest


def decode_check(package, name: str) -> bool:
    """Decodes one tensor's frame from a package and compares it with its receipt."""
    package = Path(package)
    row = next((r for r in read_manifest(package)["tensors"] if r["name"] == name), None)
    if row is None:
        raise KeyError(name)
    frame = safe_member(package, row["frame"]).read_bytes()
    raw = codec.decode(frame).tobytes() if row.get("codec") == "bctx" else frame
    return sha(frame) == row["frame_sha256"] and sha(raw) == row["source_sha256"]


# ---------------------------------------------------------------------------------------------- restore
def restore(package, destination, *, jobs: int = 8):
    """Rebuilds the source shards (and sidecars) byte for byte; every shard's digest is compared with the manifest."""
    package, destination = Path(package), Path(destination)
    manifest = verify(package, jobs=jobs, decode_frames=False)
    destination.mkdir(parents=True, exist_ok=True)
    by_shard = {}
    for row in manifest["tensors"]:
        by_shard.setdefault(row["shard"], []).append(row)

    def restore_shard(item):
        shard, rows = item
        header = (package / "headers" / (shard + ".header")).read_bytes()
        tmp = destination / (shard + ".partial")
        with open(tmp, "wb") as f:
            f.write(header)
            for row in sorted(rows, key=lambda r: r["begin"]):
                frame = safe_member(package, row["frame"]).read_bytes()
                raw = codec.decode(frame).tobytes() if row.get("codec") == "bctx" else frame
                if f.tell() > row["begin"]:
                    raise ValueError(f"overlapping tensors in {shard}")
                f.write(b"\0" * (row["begin"] - f.tell()))               # (safetensors has no gaps; kept for safety)
                f.write(raw)
            size = manifest["shards"][shard]["bytes"]
            if f.tell() > size:
                raise ValueError(f"restored shard larger than its source: {shard}")
            f.write(b" " * 0)
            f.flush()
            os.fsync(f.fileno())
        if tmp.stat().st_size != manifest["shards"][shard]["bytes"] or sha_file(tmp) != manifest["shards"][shard]["sha256"]:
            tmp.unlink()
            raise ValueError(f"restored shard differs from its source: {shard}")
        os.replace(tmp, destination / shard)
        return shard

    with ThreadPoolExecutor(jobs) as pool:
        done = list(pool.map(restore_shard, sorted(by_shard.items())))
    for rel in manifest["metadata_assets"]:
        atomic_write(destination / PurePosixPath(rel).name, safe_member(package, rel).read_bytes())
    return done


def main(argv=None):
    ap = argparse.ArgumentParser(description="build, verify and restore BCTX packages of safetensors checkpoints")
    sub = ap.add_subparsers(dest="command", required=True)
    b = sub.add_parser("build")
    b.add_argument("model_dir")
    b.add_argument("package")
    b.add_argument("--jobs", type=int, default=2)
    b.add_argument("--row-classes", type=int, default=16)
    b.add_argument("--col-classes", type=int, default=4)
    v = sub.add_parser("verify")
    v.add_argument("package")
    v.add_argument("--jobs", type=int, default=8)
    v.add_argument("--no-decode", action="store_true")
    r = sub.add_parser("restore")
    r.add_argument("package")
    r.add_argument("destination")
    r.add_argument("--jobs", type=int, default=8)
    c = sub.add_parser("decode-check", help="decode tensors of a package afresh and compare them with their receipts")
    c.add_argument("package")
    c.add_argument("tensors", nargs="+", help="tensor names, or frame paths as the manifest names them (frames/<key>.bctx)")
    args = ap.parse_args(argv)
    if args.command == "decode-check":
        rows = read_manifest(Path(args.package))["tensors"]
        by_frame = {r["frame"]: r["name"] for r in rows}
        results = {}
        for item in args.tensors:
            relative = item[len(str(args.package)):].lstrip("/") if item.startswith(str(args.package)) else item
            name = by_frame.get(relative, item)
            try:
                results[name] = bool(decode_check(args.package, name))
            except (KeyError, OSError, ValueError):
                results[name] = False
        print(json.dumps({"decode_check": results, "ok": all(results.values())}))
        if not all(results.values()):
            raise SystemExit(1)
        return
    if args.command == "build":
        m = build(args.model_dir, args.package, jobs=args.jobs, row_classes=args.row_classes, col_classes=args.col_classes, log=print)
    elif args.command == "verify":
        m = verify(args.package, jobs=args.jobs, decode_frames=not args.no_decode)
    else:
        print(json.dumps({"restored": restore(args.package, args.destination, jobs=args.jobs)}))
        return
    print(json.dumps({"tensors": len(m["tensors"]), "source_bytes": m["source_bytes"], "frame_bytes": m["frame_bytes"],
                      "ratio": round(m["source_bytes"] / max(m["frame_bytes"], 1), 6)}))


if __name__ == "__main__":
    main()
