"""Packages (build / verify / restore, byte for byte) and the loader that fills a model from frames alone (CPU).

The loader is exercised the way the reference's own tests exercise theirs (tests/test_bitexact_context_serving.py:14-49):
a tiny model, and a stand-in tensor factory that records what it is given - here over REAL frames of a package built
from a hand-written safetensors checkpoint.  The package cases follow tests/test_bitexact_context_package.py:27-241
(round trip, resumed build, inventory additions and omissions, corruption, unsafe paths, symlinks).
"""
import hashlib
import json
import os
import struct

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from torch import nn  # noqa: E402

from georefine_b200 import codec, package, serving  # noqa: E402


def _write_safetensors(path, tensors):
    header, blob = {}, b""
    for name, (dtype, shape, raw) in tensors.items():
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    path.write_bytes(struct.pack("<Q", len(text)) + text + blob)


def _bf16(t):
    return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()


@pytest.fixture()
def checkpoint(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {
        "emb.weight": torch.randn(8, 4, generator=g), "lin.weight": torch.randn(3, 4, generator=g),
        "lin.bias": torch.tensor([0.25, -0.5, 1.0]), "norm.weight": torch.tensor([1.0, 0.75, 1.25, 0.5]),
        "norm.bias": torch.zeros(4), "cube": torch.arange(24.0).reshape(2, 3, 4),
    }
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    items = list(tensors.items())
    _write_safetensors(model_dir / "model-00001-of-00002.safetensors",
                       {n: ("BF16", t.shape, _bf16(t)) for n, t in items[:3]} | {"step": ("F32", (2,), np.array([2.0, -3.0], dtype="<f4").tobytes())})
    _write_safetensors(model_dir / "model-00002-of-00002.safetensors", {n: ("BF16", t.shape, _bf16(t)) for n, t in items[3:]})
    (model_dir / "config.json").write_text('{"hidden": 4}')
    return model_dir, {n: t.to(torch.bfloat16) for n, t in tensors.items()}


def test_build_verify_restore_round_trip(checkpoint, tmp_path):
    model_dir, tensors = checkpoint
    out = tmp_path / "package"
    manifest = package.build(model_dir, out, jobs=2)
    assert manifest["complete"] and len(manifest["tensors"]) == 7 and manifest["schema"] == "bitexact-context-package-v1"
    assert package.build(model_dir, out)["tensors"] == manifest["tensors"]          # a finished package is verified, not rebuilt
    assert package.verify(out)["source_bytes"] == sum(r["source_bytes"] for r in manifest["tensors"])
    assert package.decode_check(out, "cube")
    row = next(r for r in manifest["tensors"] if r["name"] == "cube")
    assert codec.decode((out / row["frame"]).read_bytes()).shape == (2, 12)          # rank 3: rows x the rest
    dest = tmp_path / "restored"
    assert sorted(package.restore(out, dest)) == sorted(p.name for p in model_dir.glob("*.safetensors"))
    for p in model_dir.glob("*.safetensors"):
        assert (dest / p.name).read_bytes() == p.read_bytes()
    assert (dest / "config.json").read_bytes() == (model_dir / "config.json").read_bytes()


def test_resumed_build_and_changed_inputs(checkpoint, tmp_path):
    model_dir, _ = checkpoint
    out = tmp_path / "package"
    package.build(model_dir, out)
    (out / "manifest.json").unlink()                                                  # as if the build had died before the end
    victim = sorted((out / "frames").iterdir())[0]
    victim.unlink()
    manifest = package.build(model_dir, out)
    assert victim.exists() and package.verify(out) == manifest
    (out / "manifest.json").unlink()
    with pytest.raises(ValueError, match="differ"):
        package.build(model_dir, out, row_classes=4)


def test_verify_refuses_additions_omissions_corruption_and_unsafe_paths(checkpoint, tmp_path):
    model_dir, _ = checkpoint
    out = tmp_path / "package"
    manifest = package.build(model_dir, out)
    (out / "frames" / "extra.bctx").write_bytes(b"x")
    with pytest.raises(ValueError, match="inventory"):
        package.verify(out)
    (out / "frames" / "extra.bctx").unlink()
    frame = out / manifest["tensors"][0]["frame"]
    good = frame.read_bytes()
    frame.unlink()
    with pytest.raises(ValueError, match="omit"):
        package.verify(out)
    frame.write_bytes(good[:-1] + bytes([good[-1] ^ 1]))
    with pytest.raises(ValueError, match="identity"):
        package.verify(out)
    frame.write_bytes(good)
    doc = json.loads((out / "manifest.json").read_text())
    doc["tensors"][0]["frame"] = "../outside.bctx"
    (out / "manifest.json").write_text(json.dumps(doc))
    with pytest.raises(ValueError, match="inventory|unsafe"):
        package.verify(out)
    doc["tensors"][0]["frame"] = manifest["tensors"][0]["frame"]
    doc["complete"] = False
    (out / "manifest.json").write_text(json.dumps(doc))
    with pytest.raises(ValueError, match="corrupt|incomplete"):
        package.verify(out)
    doc["complete"] = True
    (out / "manifest.json").write_text(json.dumps(doc))
    frame.unlink()
    os.symlink(tmp_path / "elsewhere", frame)
    with pytest.raises(ValueError, match="symlink"):
        package.verify(out)


class TinyModel(nn.Module):
    def __init__(self, config=None):
        super().__init__()
        self.emb = nn.Embedding(8, 4)
        self.lin = nn.Linear(4, 3)
        self.norm = nn.LayerNorm(4)
        self.step = nn.Parameter(torch.empty(2, dtype=torch.float32))
        self.config = config

    def forward(self, ids):
        return self.lin(self.norm(self.emb(ids)))


class RecordingContext:
    """A stand-in for the CUDA tensor: decodes on the host, remembers how it was made."""

    made = []

    def __init__(self, frame, *, stride, device):
        words = codec.decode(frame)
        self.values = torch.from_numpy(words.view(np.int16).copy()).view(torch.bfloat16)
        self.shape = tuple(words.shape)
        self.source_sha256 = hashlib.sha256(words.tobytes()).hexdigest()
        self.frame_sha256 = hashlib.sha256(frame).hexdigest()
        self.resident_bytes = 37
        self.device = torch.device(device)
        RecordingContext.made.append((self.shape, stride))

    def decode(self):
        return self.values.clone()

    def gather_rows(self, ids):
        return self.values[ids]

    def linear(self, x, out=None, bias=None):
        y = x.float() @ self.values.float().T
        return (y + bias.float() if bias is not None else y).to(torch.bfloat16)


def test_loader_fills_a_model_from_frames_only(checkpoint, tmp_path):
    model_dir, tensors = checkpoint
    out = tmp_path / "package"
    package.build(model_dir, out)
    RecordingContext.made = []
    model, receipt = serving.load_bctx_model(out, model_factory=TinyModel, device="cpu", tensor_factory=RecordingContext, stride=128,
                                             log=lambda m: None)
    assert model.config == {"hidden": 4}
    assert isinstance(model.lin, serving.BctxLinear) and isinstance(model.emb, serving.BctxEmbedding)
    assert sorted(RecordingContext.made) == [((3, 4), 128), ((8, 4), 128)]
    assert receipt["compressed_tensors"] == 2 and receipt["resident_context_bytes"] == 74 and receipt["unused_receipts"] == ["cube"]
    assert "lin.weight" not in model.state_dict() and torch.equal(model.lin.bias, tensors["lin.bias"])
    assert model.step.dtype == torch.bfloat16 and torch.equal(model.norm.weight, tensors["norm.weight"])
    ids = torch.tensor([[1, 5, 7]])
    dense = TinyModel()
    with torch.no_grad():
        dense.emb.weight.copy_(tensors["emb.weight"].float()); dense.lin.weight.copy_(tensors["lin.weight"].float())
        dense.lin.bias.copy_(tensors["lin.bias"].float()); dense.norm.weight.copy_(tensors["norm.weight"].float()); dense.norm.bias.zero_()
    assert torch.allclose(model(ids).float(), dense(ids), atol=3e-2, rtol=3e-2)
    assert model.lin.forward_calls == 1 and model.lin.weight_materializations == 0


def test_loader_refusals(checkpoint, tmp_path):
    model_dir, _ = checkpoint
    out = tmp_path / "package"
    manifest = package.build(model_dir, out)
    load = lambda **kw: serving.load_bctx_model(out, model_factory=TinyModel, device="cpu", tensor_factory=RecordingContext, log=lambda m: None, **kw)

    class Bigger(TinyModel):
        def __init__(self, config=None):
            super().__init__(config)
            self.extra = nn.Linear(2, 2)

    with pytest.raises(serving.ContextServingError, match="missing required model parameters"):
        serving.load_bctx_model(out, model_factory=Bigger, device="cpu", tensor_factory=RecordingContext, log=lambda m: None)
    row = next(r for r in manifest["tensors"] if r["name"] == "lin.weight")
    frame = out / row["frame"]
    good = frame.read_bytes()
    frame.write_bytes(good[:-1] + bytes([good[-1] ^ 1]))
    with pytest.raises(serving.ContextServingError, match="frame identity mismatch"):
        load()
    frame.write_bytes(good)

    class LyingContext(RecordingContext):
        def __init__(self, frame, *, stride, device):
            super().__init__(frame, stride=stride, device=device)
            self.source_sha256 = "0" * 64

    with pytest.raises(serving.ContextServingError, match="identity mismatch"):
        serving.load_bctx_model(out, model_factory=TinyModel, device="cpu", tensor_factory=LyingContext, log=lambda m: None)
    doc = json.loads((out / "manifest.json").read_text())
    for r in doc["tensors"]:
        if r["name"] == "norm.weight":
            r["source_sha256"] = "0" * 64
    (out / "manifest.json").write_text(json.dumps(doc))
    with pytest.raises(serving.ContextServingError, match="decoded-source identity mismatch: norm.weight"):
        load()

    class Stuck(TinyModel):
        def __init__(self, config=None):
            super().__init__(config)
            self.register_buffer("stuck", torch.empty(1), persistent=False)

    (out / "manifest.json").write_text(json.dumps(json.loads((out / "manifest.json").read_text()) | {"tensors": manifest["tensors"]}))
    with pytest.raises(serving.ContextServingError, match="unfilled meta tensors"):
        serving.load_bctx_model(out, model_factory=Stuck, device="cpu", tensor_factory=RecordingContext, log=lambda m: None)


def test_speculation_head_linear_counts_calls_and_checks_shapes():
    """``BCTXLinear`` (the module the reference's speculation-head loader puts in place of a dense linear): the product
    goes to the tensor's fused ``linear``, calls are counted, a tensor that answers with another shape is refused."""
    import torch

    from georefine_b200 import serving

    class Stand:
        shape = (6, 4)

        def __init__(self, out_features=6):
            self.out_features = out_features

        def linear(self, x, bias=None):
            return torch.ones(*x.shape[:-1], self.out_features, dtype=torch.float32)

    layer = serving.BCTXLinear(Stand(), "mtp.fc")
    y = layer(torch.zeros(3, 4, dtype=torch.bfloat16))
    assert y.shape == (3, 6) and y.dtype == torch.bfloat16 and layer.calls == 1 and layer.name == "mtp.fc"
    assert not list(layer.state_dict())
    with pytest.raises(ValueError):
        serving.BCTXLinear(Stand(out_features=5), "mtp.fc")(torch.zeros(3, 4, dtype=torch.bfloat16))
    with pytest.raises(serving.ContextServingError):
        bad = Stand()
        bad.shape = (6,)
        serving.BCTXLinear(bad, "v")


def test_command_line_build_verify_decode_check_restore(checkpoint, tmp_path, capsys):
    """The tool's four commands (the reference's: build / verify / restore / decode-check,
    bitexact_context_package.py:766-830)."""
    model_dir, _ = checkpoint
    out = tmp_path / "package"
    package.main(["build", str(model_dir), str(out), "--jobs", "2"])
    built = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert built["tensors"] == 7 and built["frame_bytes"] > 0
    package.main(["verify", str(out)])
    assert json.loads(capsys.readouterr().out)["tensors"] == 7
    row = next(r for r in package.read_manifest(out)["tensors"] if r["name"] == "lin.weight")
    package.main(["decode-check", str(out), "cube", row["frame"], str(out / row["frame"])])
    assert json.loads(capsys.readouterr().out) == {"decode_check": {"cube": True, "lin.weight": True}, "ok": True}
    frame = out / row["frame"]
    data = bytearray(frame.read_bytes())
    data[-40] ^= 1
    frame.write_bytes(bytes(data))
    with pytest.raises(SystemExit):
        package.main(["decode-check", str(out), "lin.weight", "cube", "no.such.tensor"])
    assert json.loads(capsys.readouterr().out) == {"decode_check": {"lin.weight": False, "cube": True, "no.such.tensor": False}, "ok": False}
    frame.write_bytes(bytes(data[:-40]) + bytes([data[-40] ^ 1]) + bytes(data[-39:]))
    package.main(["restore", str(out), str(tmp_path / "restored")])
    assert sorted(json.loads(capsys.readouterr().out)["restored"]) == sorted(p.name for p in model_dir.glob("*.safetensors"))
