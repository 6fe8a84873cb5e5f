"""From a BCTX package of a decoder checkpoint to the decode engine's weights - frames alone, no dense checkpoint.

What the reference does in ``FastSession.load(bundle=...)`` (``glc_serve/fastserve.py:114-178``: a session from a
directory on disk) and ``load_bctx_mtp`` (``georefine_context_runtime/bitexact_context_mtp.py:327-400``: the draft head's
tensors from the package's frames only, every frame checked against its receipt, a receipt of what was loaded).  The
engine here is a plain grouped-query decoder (RMSNorm, rotary attention without per-head norms, gates or biases, SwiGLU),
so the tensor names are those of that family's checkpoints::

    model.embed_tokens.weight                        -> embed
    model.layers.<i>.input_layernorm.weight          -> layers.<i>.norm1
    model.layers.<i>.self_attn.{q,k,v}_proj.weight   -> layers.<i>.qkv      (rows concatenated q | k | v)
    model.layers.<i>.self_attn.o_proj.weight         -> layers.<i>.o
    model.layers.<i>.post_attention_layernorm.weight -> layers.<i>.norm2
    model.layers.<i>.mlp.{gate,up}_proj.weight       -> layers.<i>.gate_up  (rows concatenated gate | up)
    model.layers.<i>.mlp.down_proj.weight            -> layers.<i>.down
    model.norm.weight                                -> final_norm
    lm_head.weight (or the embedding, when tied)     -> lm_head
    mtp.fc.weight, mtp.pre_fc_norm_embedding.weight, mtp.pre_fc_norm_hidden.weight, mtp.norm.weight,
    mtp.layers.0.<the same per-layer names>          -> the draft head

A tensor of the package that belongs to a layer and is not in this list (a bias, a per-head norm) means the checkpoint
is not of this family: loading refuses it instead of dropping it.
"""
from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path

import numpy as np

from . import codec, package as pkg
from .serving import ContextServingError

_LAYER = {
    "norm1": ("input_layernorm.weight",),
    "qkv": ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight"),
    "o": ("self_attn.o_proj.weight",),
    "norm2": ("post_attention_layernorm.weight",),
    "gate_up": ("mlp.gate_proj.weight", "mlp.up_proj.weight"),
    "down": ("mlp.down_proj.weight",),
}
_LAYER_TENSORS = {t for parts in _LAYER.values() for t in parts}
_MTP_TOP = {"fc": "mtp.fc.weight", "norm_e": "mtp.pre_fc_norm_embedding.weight", "norm_h": "mtp.pre_fc_norm_hidden.weight",
            "final_norm": "mtp.norm.weight"}


def decoder_config(config, **overrides):
    """``serve.DecoderConfig`` from a checkpoint's ``config.json`` (a dict, or a path to the file; a nested ``text_config``
    is followed).  ``overrides``: ``tp_world`` / ``tp_rank`` and the like."""
    from .serve import DecoderConfig

    if not isinstance(config, dict):
        config = json.loads(Path(config).read_text())
    config = config.get("text_config", config)
    try:
        heads, hidden = int(config["num_attention_heads"]), int(config["hidden_size"])
        fields = dict(hidden=hidden, layers=int(config["num_hidden_layers"]), heads=heads,
                      kv_heads=int(config.get("num_key_value_heads", heads)), head_dim=int(config.get("head_dim") or hidden // heads),
                      ffn=int(config["intermediate_size"]), vocab=int(config["vocab_size"]),
                      rope_theta=float(config.get("rope_theta", 10000.0)), eps=float(config.get("rms_norm_eps", 1e-6)))
    except (KeyError, TypeError, ValueError) as exc:
        raise ContextServingError(f"model config lacks a decoder field: {exc}") from exc
    for flag in ("attention_bias", "mlp_bias"):
        if config.get(flag):
            raise ContextServingError(f"unsupported decoder family: {flag} is set")
    fields.update(overrides)
    return DecoderConfig(**fields)


def mtp_shapes(cfg):
    """Names and shapes of the draft head's tensors for a decoder of configuration ``cfg`` (the plain-decoder form of the
    reference's ``MTP_SHAPES``, ``bitexact_context_mtp.py:244-260``)."""
    h, d = cfg.hidden, cfg.head_dim
    layer = {"input_layernorm.weight": (h,), "post_attention_layernorm.weight": (h,),
             "self_attn.q_proj.weight": (cfg.heads * d, h), "self_attn.k_proj.weight": (cfg.kv_heads * d, h),
             "self_attn.v_proj.weight": (cfg.kv_heads * d, h), "self_attn.o_proj.weight": (h, cfg.heads * d),
             "mlp.gate_proj.weight": (cfg.ffn, h), "mlp.up_proj.weight": (cfg.ffn, h), "mlp.down_proj.weight": (h, cfg.ffn)}
    out = {"mtp.fc.weight": (h, 2 * h), "mtp.pre_fc_norm_embedding.weight": (h,), "mtp.pre_fc_norm_hidden.weight": (h,),
           "mtp.norm.weight": (h,)}
    out.update({"mtp.layers.0." + k: v for k, v in layer.items()})
    return out


class PackageWords:
    """``words_of(name)`` over a package: the BF16 bit patterns of an engine tensor (module docstring), decoded from the
    package's frames on the host.  Every frame is checked against its receipt before it is decoded (length, SHA-256) and
    the decoded words against the source digest; a tensor that is missing, of another dtype or of another shape than the
    configuration implies raises ``ContextServingError``.  ``consumed`` lists the package tensors read so far."""

    def __init__(self, package, config=None, *, host_decoder=None):
        self.package = Path(package)
        try:
            manifest = pkg.read_manifest(self.package)
        except ValueError as exc:
            raise ContextServingError(f"unsupported or incomplete BCTX package manifest: {exc}") from exc
        self.rows = {}
        for row in manifest["tensors"]:
            name = row.get("name") if isinstance(row, dict) else None
            if not isinstance(name, str) or name in self.rows or row.get("complete") is not True:
                raise ContextServingError("malformed, duplicate or incomplete tensor receipt")
            self.rows[name] = row
        if config is None:
            path = self.package / "sidecars" / "config.json"
            if not path.is_file():
                raise ContextServingError(f"model config missing: {path}")
            config = decoder_config(path)
        self.config = config
        self.decode = host_decoder or codec.decode
        self.consumed = {}
        self.tied = "lm_head.weight" not in self.rows
        self._check_family()

    def _check_family(self):
        cfg = self.config
        for name in self.rows:
            parts = name.split(".")
            if name.startswith("model.layers.") and len(parts) > 3:
                if not parts[2].isdigit() or int(parts[2]) >= cfg.layers or ".".join(parts[3:]) not in _LAYER_TENSORS:
                    raise ContextServingError(f"tensor outside the plain grouped-query decoder family: {name}")
            elif name.startswith("mtp.") and name not in mtp_shapes(cfg):
                raise ContextServingError(f"tensor outside the plain draft-head family: {name}")

    @property
    def has_mtp(self) -> bool:
        return any(name.startswith("mtp.") for name in self.rows)

    def tensor(self, name: str, shape):
        """One package tensor as uint16 words of ``pkg.frame_shape(shape)``, all checks applied."""
        row = self.rows.get(name)
        if row is None:
            raise ContextServingError(f"package lacks a tensor the decoder needs: {name}")
        if row.get("dtype") != "BF16" or row.get("codec", "bctx") != "bctx" or tuple(row.get("shape", ())) != tuple(shape):
            raise ContextServingError(f"manifest shape/dtype mismatch for {name}: {row.get('dtype')} {row.get('shape')}, wanted BF16 {list(shape)}")
        try:
            frame = pkg.safe_member(self.package, row.get("frame")).read_bytes()
        except (OSError, ValueError) as exc:
            raise ContextServingError(f"cannot read BCTX frame for {name}: {exc}") from exc
        if len(frame) != row.get("frame_bytes") or hashlib.sha256(frame).hexdigest() != row.get("frame_sha256"):
            raise ContextServingError(f"BCTX frame identity mismatch: {name}")
        try:
            words = np.ascontiguousarray(self.decode(frame), dtype="<u2")
        except ValueError as exc:
            raise ContextServingError(f"cannot decode BCTX frame for {name}: {exc}") from exc
        if words.size != math.prod(shape) or hashlib.sha256(words.tobytes()).hexdigest() != row.get("source_sha256"):
            raise ContextServingError(f"decoded-source identity mismatch: {name}")
        self.consumed[name] = {"frame_sha256": row["frame_sha256"], "source_sha256": row["source_sha256"], "frame_bytes": len(frame)}
        return words.reshape(pkg.frame_shape(shape))

    def members(self, name: str):
        """The package tensors an engine tensor is made of, in row order: [(package name, shape), ...]."""
        cfg = self.config
        layer_shapes = {k.removeprefix("mtp.layers.0."): v for k, v in mtp_shapes(cfg).items() if k.startswith("mtp.layers.0.")}

        def layer(prefix, leaf):
            if leaf not in _LAYER:
                raise KeyError(name)
            return [(prefix + t, layer_shapes[t]) for t in _LAYER[leaf]]

        if name == "embed" or (name == "lm_head" and self.tied):
            return [("model.embed_tokens.weight", (cfg.vocab, cfg.hidden))]
        if name == "lm_head":
            return [("lm_head.weight", (cfg.vocab, cfg.hidden))]
        if name == "final_norm":
            return [("model.norm.weight", (cfg.hidden,))]
        parts = name.split(".")
        if len(parts) == 3 and parts[0] == "layers" and parts[1].isdigit() and int(parts[1]) < cfg.layers:
            return layer(f"model.layers.{int(parts[1])}.", parts[2])
        if len(parts) == 2 and parts[0] == "mtp":
            if parts[1] in _MTP_TOP:
                return [(_MTP_TOP[parts[1]], mtp_shapes(cfg)[_MTP_TOP[parts[1]]])]
            return layer("mtp.layers.0.", parts[1])
        raise KeyError(name)

    def __call__(self, name: str):
        parts = [self.tensor(tensor, shape) for tensor, shape in self.members(name)]
        return parts[0] if len(parts) == 1 else np.concatenate(parts, axis=0)

    def identity(self, name: str, plan: str) -> str:
        """A digest that names the resident image of an engine linear without decoding anything: the source and frame
        digests of its member tensors as the manifest records them, the way they are joined and sharded, and ``plan`` -
        whatever else decides how the image is built (layout, tune record)."""
        cfg = self.config
        members = []
        for tensor, shape in self.members(name):
            row = self.rows.get(tensor)
            if row is None:
                raise ContextServingError(f"package lacks a tensor the decoder needs: {tensor}")
            members.append([tensor, row.get("source_sha256"), row.get("frame_sha256"), list(shape)])
        text = json.dumps({"members": members, "leaf": name.split(".")[-1], "tp": [cfg.tp_world, cfg.tp_rank],
                           "heads": [cfg.heads, cfg.kv_heads, cfg.head_dim], "ffn": cfg.ffn, "plan": plan}, sort_keys=True)
        return hashlib.sha256(text.encode()).hexdigest()

    def receipt(self) -> dict:
        """What has been loaded so far (the fields of the reference's MTP receipt, ``bitexact_context_mtp.py:379-393``)."""
        return {"format": "BCTX", "package": str(self.package), "tensor_count": len(self.consumed), "tensor_names": sorted(self.consumed),
                "frame_sha256": {n: r["frame_sha256"] for n, r in self.consumed.items()},
                "source_sha256": {n: r["source_sha256"] for n, r in self.consumed.items()},
                "frame_bytes": sum(r["frame_bytes"] for r in self.consumed.values()), "loaded_from_bctx_only": True}


def linear_names(cfg, *, mtp: bool = False):
    """The engine's compressed linears in the order a step runs them."""
    names = [f"layers.{i}.{leaf}" for i in range(cfg.layers) for leaf in ("qkv", "o", "gate_up", "down")] + ["lm_head"]
    return names + (["mtp.qkv", "mtp.o", "mtp.gate_up", "mtp.down", "mtp.fc"] if mtp else [])


def _group_path(cache, identity: str) -> Path:
    return Path(cache.root) / "groups" / identity[:2] / (identity + ".json")


def resident_images(source: PackageWords, names, *, sm_count: int, layout=None, cache=None, tune=None, pool_threads=None, log=None):
    """Resident images of the engine linears ``names``, built on host threads in parallel and - with an
    ``image_cache.ImageCache`` - kept on disk, so that a restart reads images instead of decoding frames.  Returns
    {name: (image, header, hit)}.

    A linear of the engine is a join of package tensors (q | k | v, gate | up), possibly a tensor-parallel shard of it,
    so its words have no digest in the manifest.  The cache entry itself is keyed and verified by the digest of the words
    it was built from, like every entry (``ImageCache.get``); a small record ``groups/<identity>.json`` under the cache
    root maps ``PackageWords.identity`` - known without decoding - to that digest, shape and worker count.  A record
    that points to a missing or refused entry is a miss: the frames are decoded (each checked against its receipt), the
    image is rebuilt and both are written again.  The reference's counterpart is its load-time transcode with a verified
    cache and parallel workers (``glc_serve/bctx_v21_transcode.py``, ``transcode_cache.py``,
    ``context_parallel_startup.py``)."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    from . import resident
    from .package import atomic_write

    cfg = source.config
    log = log or (lambda message: None)

    def plan(rows, cols):
        chosen_layout, workers = layout, None
        if tune and (rows, cols) in tune:
            chosen_layout = tune[(rows, cols)][0] if chosen_layout is None else chosen_layout
            workers = tune[(rows, cols)][1]
        return chosen_layout or resident.DEFAULT_LAYOUT, workers or resident.default_workers(rows, cols, sm_count)

    tuned = hashlib.sha256(repr(sorted((tuple(k), tuple(v)) for k, v in (tune or {}).items())).encode()).hexdigest()[:16]
    build_plan = f"layout={layout},tune={tuned},sms={sm_count}"

    def one(name):
        identity = source.identity(name, build_plan)
        if cache is not None:
            try:
                record = json.loads(_group_path(cache, identity).read_text())
                image = cache.get(record["words_sha256"], tuple(record["shape"]), record["layout"], int(record["workers"]))
                if image is not None:
                    return image, resident.header_of(image), True
            except (OSError, ValueError, KeyError, TypeError):
                pass
        words = np.ascontiguousarray(cfg.shard(name.split(".")[-1], source(name)))
        chosen_layout, workers = plan(int(words.shape[0]), int(words.shape[1]))
        digest = hashlib.sha256(words.astype("<u2").tobytes())
        image, header = resident.build_image(words, workers, threads=1, layout=chosen_layout, source_sha256=digest.digest())
        if cache is not None and cache.put(image, chosen_layout):
            try:
                atomic_write(_group_path(cache, identity), json.dumps({"words_sha256": digest.hexdigest(), "shape": list(words.shape),
                                                                       "layout": chosen_layout, "workers": int(workers)}).encode())
            except OSError as exc:
                log(f"[checkpoint] cannot record {name} in the image cache: {exc}")
        return image, header, False

    names = list(names)
    threads = pool_threads or max(1, min(len(names), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=threads, thread_name_prefix="grb-checkpoint") as pool:
        return dict(zip(names, pool.map(one, names)))


def load_decoder_weights(package, device="cuda:0", *, config=None, tp_world=1, tp_rank=0, host_decoder=None, cache=None,
                         pool_threads=None, lin_factory=None, max_m=128, tune=None, layout=None, log=None):
    """``serve.DecoderWeights`` of the decoder in ``package``.  The linears are resident images built on host threads in
    parallel (``resident_images``; ``cache``: an ``image_cache.ImageCache`` that keeps them across restarts), or whatever
    ``lin_factory(name, words)`` returns.  The receipt of what was read from the package is in
    ``weights.notes['receipt']``, the cache hits in ``weights.notes['image_cache_hits']``, and the ``PackageWords``
    itself, for a later ``load_mtp_head``, in ``weights.notes['source']``."""
    import torch

    from . import resident
    from .serve import DecoderWeights, LayerWeights

    if config is None:
        config = decoder_config(Path(package) / "sidecars" / "config.json", tp_world=tp_world, tp_rank=tp_rank)
    source = PackageWords(package, config, host_decoder=host_decoder)
    if lin_factory is not None:
        weights = DecoderWeights.from_words(config, source, device, lin_factory=lin_factory, max_m=max_m, tune=tune, layout=layout)
        weights.notes.update(receipt=source.receipt(), source=source, image_cache_hits=0)
        return weights
    dev = torch.device(device)
    sms, hits = resident.sm_count(dev), 0

    def dense(name):
        return torch.from_numpy(source(name).view(np.int16).copy()).view(torch.bfloat16).to(dev)

    def linears(names):
        """Built a batch at a time, so that the host holds the images of a few layers, not of the model."""
        nonlocal hits
        images = resident_images(source, names, sm_count=sms, layout=layout, cache=cache, tune=tune, pool_threads=pool_threads, log=log)
        hits += sum(1 for _, _, hit in images.values() if hit)
        return {name: resident.ResidentWeight(images.pop(name)[0], dev, max_m=max_m, verify=False) for name in names}

    layers, per_batch = [], 4
    for lo in range(0, config.layers, per_batch):
        ids = range(lo, min(lo + per_batch, config.layers))
        built = linears([f"layers.{i}.{leaf}" for i in ids for leaf in ("qkv", "o", "gate_up", "down")])
        for i in ids:
            p = f"layers.{i}."
            layers.append(LayerWeights(dense(p + "norm1").reshape(-1), built[p + "qkv"], built[p + "o"], dense(p + "norm2").reshape(-1),
                                       built[p + "gate_up"], built[p + "down"]))
    lm_head = linears(["lm_head"])["lm_head"]
    weights = DecoderWeights(config, dense("embed"), layers, dense("final_norm").reshape(-1), lm_head,
                             {"distinct_layers": config.layers, "layers": config.layers})
    weights.chain()
    weights.notes.update(receipt=source.receipt(), source=source, image_cache_hits=hits)
    return weights


def load_mtp_head(package, decoder, *, lin_factory=None, host_decoder=None, cache=None, pool_threads=None):
    """The draft head (``serve.MTPHead``) over ``decoder`` from the package's ``mtp.*`` frames: all thirteen tensors or an
    error, each checked against its receipt.  ``head.receipt`` says what was loaded (with a warm ``cache`` the matrices
    come from their cached images, and the receipt lists only what was read from the package)."""
    import torch

    from . import resident
    from .serve import LayerWeights, MTPHead

    cfg, dev = decoder.cfg, decoder.dev
    source = package if isinstance(package, PackageWords) else PackageWords(package, cfg, host_decoder=host_decoder)
    missing = sorted(set(mtp_shapes(cfg)) - set(source.rows))
    if missing:
        raise ContextServingError(f"MTP manifest keys differ: missing={missing}")
    matrices = ["mtp.qkv", "mtp.o", "mtp.gate_up", "mtp.down", "mtp.fc"]
    images = {} if lin_factory is not None else resident_images(source, matrices, sm_count=resident.sm_count(dev), cache=cache,
                                                                pool_threads=pool_threads)

    def norm(name):
        return torch.from_numpy(source("mtp." + name).view(np.int16).copy()).view(torch.bfloat16).reshape(-1).to(dev)

    def linear(name):
        if lin_factory is not None:
            return lin_factory("mtp." + name, np.ascontiguousarray(source("mtp." + name)))
        return resident.ResidentWeight(images.pop("mtp." + name)[0], dev, max_m=min(decoder.max_rows, 128), verify=False)

    layer = LayerWeights(norm("norm1"), linear("qkv"), linear("o"), norm("norm2"), linear("gate_up"), linear("down"))
    head = MTPHead(decoder, fc=linear("fc"), norm_e=norm("norm_e"), norm_h=norm("norm_h"), layer=layer, final_norm=norm("final_norm"))
    names = [n for n in sorted(source.consumed) if n.startswith("mtp.")]
    whole = source.receipt()
    head.receipt = dict(whole, tensor_names=names, tensor_count=len(names), frame_sha256={n: whole["frame_sha256"][n] for n in names},
                        source_sha256={n: whole["source_sha256"][n] for n in names},
                        frame_bytes=sum(source.consumed[n]["frame_bytes"] for n in names))
    return head
