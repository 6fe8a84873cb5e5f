"""nn.Module adapters over a compressed weight.

Mirrors ``BctxLinear`` / ``BctxEmbedding`` of
``context-runtime/georefine_context_runtime/bitexact_context_serving.py:346-400``: same constructor, counters
and attributes, not part of ``state_dict``.  ``forward`` calls the fused kernel instead of decoding the whole
weight and running a dense matmul; ``.weight`` still decodes transiently for helpers that want a dense tensor.
"""
from __future__ import annotations

import torch
from torch import nn


class ContextServingError(RuntimeError):
    pass


class BctxLinear(nn.Module):
    """Linear whose weight stays compressed; the product never materialises a dense copy."""

    def __init__(self, tensor, bias=None):
        super().__init__()
        if len(tensor.shape) != 2:
            raise ContextServingError("linear BCTX weight must be rank two")
        self.context_weight = tensor
        self.out_features, self.in_features = map(int, tensor.shape)
        self.forward_calls = 0
        self.weight_materializations = 0
        self.register_parameter("bias", bias)

    @property
    def weight(self):
        self.weight_materializations += 1
        return self.context_weight.decode()

    def forward(self, x):
        self.forward_calls += 1
        bias = None if self.bias is None else self.bias.to(torch.bfloat16)
        return self.context_weight.linear(x, bias=bias)


class BCTXLinear(nn.Module):
    """The linear of the speculation head (``BCTXLinear`` of
    ``context-runtime/georefine_context_runtime/bitexact_context_mtp.py:279-297``): ``tensor``, ``name`` and a ``calls``
    counter, no bias.  The reference decodes the weight for every call and runs a dense product; here the product
    reads the compressed image, and a tensor whose decoded shape no longer matches its descriptor is refused as there."""

    def __init__(self, tensor, name: str):
        super().__init__()
        if len(tensor.shape) != 2:
            raise ContextServingError("linear BCTX weight must be rank two")
        self.tensor = tensor
        self.name = str(name)
        self.calls = 0

    def forward(self, x):
        self.calls += 1
        y = self.tensor.linear(x)
        if y.shape[-1] != int(self.tensor.shape[0]) or x.shape[-1] != int(self.tensor.shape[1]):
            raise ValueError(f"decoded shape changed for {self.name}")
        return y if y.dtype == x.dtype else y.to(dtype=x.dtype)


class BctxEmbedding(nn.Module):
    """Embedding table that stays compressed; rows are decoded by indexed gather."""

    def __init__(self, tensor, *, padding_idx=None):
        super().__init__()
        if len(tensor.shape) != 2:
            raise ContextServingError("embedding BCTX weight must be rank two")
        self.context_weight = tensor
        self.num_embeddings, self.embedding_dim = map(int, tensor.shape)
        self.padding_idx = padding_idx
        self.forward_calls = 0
        self.weight_materializations = 0

    @property
    def weight(self):
        self.weight_materializations += 1
        return self.context_weight.decode()

    def forward(self, input):
        self.forward_calls += 1
        return self.context_weight.gather_rows(input)


# ---------------------------------------------------------------------------------------------- loader
def _module_and_leaf(model, dotted: str):
    parent = model
    *path, leaf = dotted.split(".")
    for part in path:
        parent = getattr(parent, part)
    return parent, leaf


def load_bctx_model(package, *, model=None, model_factory=None, config_loader=None, device="cuda:0", dtype=None, stride: int = 1024,
                    tensor_factory=None, host_decoder=None, log=print, progress_callback=None):
    """Fills a model from the frames of a BCTX package alone and returns ``(model, receipt)``.

    Counterpart of the reference's loader (``bitexact_context_serving.py:409-712``).  The model comes from ``model`` (an
    ``nn.Module`` whose parameters may live on the meta device) or from ``model_factory(config)`` with
    ``config = config_loader(<package>/sidecars/config.json)`` (default: the parsed JSON).  Every named parameter must
    have a receipt of the same shape.  The weight of every ``nn.Linear`` and ``nn.Embedding`` stays compressed: its frame
    goes to ``tensor_factory(frame, stride=..., device=...)`` (default: ``CudaContextTensor``, whose ``linear`` is the
    fused decode-GEMM), the module is replaced by ``BctxLinear`` / ``BctxEmbedding``, and what the factory returns is
    checked against the receipt - ``shape``, ``source_sha256``, ``frame_sha256``, a positive integer ``resident_bytes``.
    Every other parameter is decoded on the host (``host_decoder(frame)``, default ``codec.decode``), checked against
    its source digest and materialised on ``device``.  There is no dense-checkpoint fallback: anything that does not
    check out raises ``ContextServingError``."""
    import hashlib
    import json
    import math
    from pathlib import Path

    import numpy as np

    from . import codec, package as pkg

    package = Path(package)
    try:
        manifest = pkg.read_manifest(package)
    except ValueError as exc:
        raise ContextServingError(f"unsupported or incomplete BCTX package manifest: {exc}") from exc
    entries = {}
    for row in manifest["tensors"]:
        name = row.get("name") if isinstance(row, dict) else None
        if not isinstance(name, str) or name in entries:
            raise ContextServingError("malformed or duplicate tensor receipt")
        shape = row.get("shape")
        if row.get("complete") is not True or not isinstance(shape, list) or any(type(d) is not int or d <= 0 for d in shape):
            raise ContextServingError(f"incomplete or malformed tensor receipt: {name}")
        for key in ("source_sha256", "frame_sha256"):
            value = row.get(key)
            if not (isinstance(value, str) and len(value) == 64 and all(c in "0123456789abcdef" for c in value)):
                raise ContextServingError(f"invalid source/frame SHA: {name}")
        entries[name] = row
    if model is None:
        if model_factory is None:
            raise ContextServingError("either model= or model_factory= is required")
        config_path = package / "sidecars" / "config.json"
        if not config_path.is_file():
            raise ContextServingError(f"model config missing: {config_path}")
        config = (config_loader or (lambda path: json.loads(path.read_text())))(config_path)
        with torch.device("meta"):
            model = model_factory(config)
    dtype = torch.bfloat16 if dtype is None else (getattr(torch, dtype) if isinstance(dtype, str) else dtype)
    params = dict(model.named_parameters())
    if not params:
        raise ContextServingError("model has no named parameters")
    missing = sorted(set(params) - set(entries))
    if missing:
        raise ContextServingError(f"package missing required model parameters: {missing[:12]}")
    wrong = [(n, tuple(entries[n]["shape"]), tuple(p.shape)) for n, p in params.items() if tuple(entries[n]["shape"]) != tuple(p.shape)]
    if wrong:
        raise ContextServingError(f"manifest/model shape mismatch: {wrong[:8]}")
    if tensor_factory is None:
        from .gpu import CudaContextTensor

        tensor_factory = CudaContextTensor
    host_decoder = host_decoder or codec.decode
    compressed = {}
    for mod_name, module in list(model.named_modules()):
        if isinstance(module, (nn.Linear, nn.Embedding)) and (mod_name + ".weight" if mod_name else "weight") in params:
            compressed[mod_name + ".weight" if mod_name else "weight"] = (mod_name, module)

    def read_frame(name):
        row = entries[name]
        try:
            frame = pkg.safe_member(package, row.get("frame")).read_bytes()
        except (OSError, ValueError) as exc:
            raise ContextServingError(f"cannot read BCTX frame for {name}: {exc}") from exc
        if len(frame) != row.get("frame_bytes") or hashlib.sha256(frame).hexdigest() != row["frame_sha256"]:
            raise ContextServingError(f"BCTX frame identity mismatch: {name}")
        return frame

    def host_tensor(name, target_dtype):
        row = entries[name]
        frame = read_frame(name)
        if row.get("codec", "bctx") == "raw":
            if row.get("dtype") not in ("F32", "F16", "BF16"):
                raise ContextServingError(f"unsupported raw tensor dtype: {name}")
            np_dtype = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16}[row["dtype"]]
            raw = np.frombuffer(frame, dtype=np_dtype)
            if hashlib.sha256(frame).hexdigest() != row["source_sha256"]:
                raise ContextServingError(f"decoded-source identity mismatch: {name}")
            t = torch.from_numpy(raw.copy())
            t = t.view(torch.bfloat16) if row["dtype"] == "BF16" else t
        else:
            try:
                words = np.ascontiguousarray(host_decoder(frame), dtype="<u2")
            except ValueError as exc:
                raise ContextServingError(f"cannot decode BCTX frame for {name}: {exc}") from exc
            if words.size != math.prod(row["shape"]) or hashlib.sha256(words.tobytes()).hexdigest() != row["source_sha256"]:
                raise ContextServingError(f"decoded-source identity mismatch: {name}")
            t = torch.from_numpy(words.view(np.int16).copy()).view(torch.bfloat16)
        return t.reshape(row["shape"]).to(device=device, dtype=target_dtype)

    resident, done, total = 0, 0, len(params)
    for name, (mod_name, module) in compressed.items():
        row = entries[name]
        context = tensor_factory(read_frame(name), stride=stride, device=device)
        expect = pkg.frame_shape(row["shape"])
        problems = {"shape": tuple(getattr(context, "shape", ())) != tuple(expect),
                    "source_sha256": getattr(context, "source_sha256", None) != row["source_sha256"],
                    "frame_sha256": getattr(context, "frame_sha256", None) != row["frame_sha256"],
                    "resident_bytes": type(getattr(context, "resident_bytes", None)) is not int or context.resident_bytes <= 0}
        bad = [k for k, v in problems.items() if v]
        if bad:
            raise ContextServingError(f"context tensor identity mismatch ({', '.join(bad)}): {name}")
        resident += context.resident_bytes
        parent, leaf = _module_and_leaf(model, mod_name) if mod_name else (None, None)
        if isinstance(module, nn.Linear):
            bias = None
            if module.bias is not None:
                bias = nn.Parameter(host_tensor(mod_name + ".bias" if mod_name else "bias", dtype), requires_grad=False)
                done += 1
            new = BctxLinear(context, bias)
        else:
            new = BctxEmbedding(context, padding_idx=module.padding_idx)
        if parent is None:
            raise ContextServingError("the model itself cannot be a compressed module")
        setattr(parent, leaf, new)
        done += 1
        if progress_callback:
            progress_callback(done, total, name)
    for name, p in params.items():
        mod_name = name.rsplit(".", 1)[0] if "." in name else ""
        if name in compressed or (name.endswith(".bias") and mod_name + ".weight" in compressed):
            continue
        target = torch.float32 if p.dtype == torch.float32 and getattr(model, "_keep_in_fp32_modules_strict", None) and name in model._keep_in_fp32_modules_strict else dtype
        parent, leaf = _module_and_leaf(model, name)
        setattr(parent, leaf, nn.Parameter(host_tensor(name, target), requires_grad=False))
        done += 1
        if progress_callback:
            progress_callback(done, total, name)
    for name, buffer in model.named_buffers():
        if buffer.is_meta:
            raise ContextServingError(f"unfilled meta tensors after load: {name}")
    left = [n for n, p in model.named_parameters() if p.is_meta]
    if left:
        raise ContextServingError(f"unfilled meta tensors after load: {left[:8]}")
    receipt = {"schema": "georefine_b200.load_receipt.v1", "package": str(package), "compressed_tensors": len(compressed),
               "materialized_parameters": total - len(compressed), "resident_context_bytes": resident,
               "unused_receipts": sorted(set(entries) - set(params))}
    log(f"[load] {len(compressed)} compressed tensors resident in {resident} bytes, {receipt['materialized_parameters']} parameters materialised")
    return model, receipt
