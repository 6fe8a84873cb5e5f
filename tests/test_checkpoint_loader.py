"""The decode engine's weights from a BCTX package (georefine_b200/checkpoint.py), on the CPU: the tensor-name mapping, the
concatenated groups, the checks of every frame against its receipt, and the draft head's all-or-nothing load - with
stand-in linears that record what they are given, the way the reference tests its loaders
(tests/test_bitexact_context_serving.py:33-49; the MTP loader's checks: bitexact_context_mtp.py:344-360).
"""
import json
import types

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from georefine_b200 import checkpoint, package, serve  # noqa: E402
from georefine_b200.serving import ContextServingError  # noqa: E402

FIELDS = dict(hidden=128, layers=2, heads=2, kv_heads=1, ffn=256, vocab=96)


class FakeLinear:
    def __init__(self, name, words):
        self.name, self.words = name, np.array(words)
        self.N, self.K = words.shape
        self.coded_bytes = words.size

    def __call__(self, x, y):
        raise AssertionError("not called on the CPU")


@pytest.fixture(scope="module")
def packaged(tmp_path_factory, write_decoder_checkpoint):
    root = tmp_path_factory.mktemp("ckpt")
    tensors = write_decoder_checkpoint(root / "model", seed=3, **FIELDS)
    package.build(root / "model", root / "package", jobs=4)
    return root / "package", tensors


def test_config_mapping(packaged):
    pkg_dir, _ = packaged
    cfg = checkpoint.decoder_config(pkg_dir / "sidecars" / "config.json")
    assert (cfg.hidden, cfg.layers, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab) == (128, 2, 2, 1, 128, 256, 96)
    assert cfg.rope_theta == 10000.0 and cfg.eps == 1e-6 and cfg.tp_world == 1
    nested = {"text_config": json.loads((pkg_dir / "sidecars" / "config.json").read_text())}
    assert checkpoint.decoder_config(nested, tp_world=1) == cfg
    plain = dict(nested["text_config"])
    del plain["head_dim"], plain["num_key_value_heads"]
    derived = checkpoint.decoder_config(plain)
    assert derived.head_dim == 64 and derived.kv_heads == 2
    with pytest.raises(ContextServingError):
        checkpoint.decoder_config({"hidden_size": 128})
    with pytest.raises(ContextServingError):
        checkpoint.decoder_config(dict(nested["text_config"], attention_bias=True))


def test_engine_names_map_to_package_tensors(packaged):
    pkg_dir, t = packaged
    src = checkpoint.PackageWords(pkg_dir)
    assert src.has_mtp and not src.tied
    assert np.array_equal(src("embed"), t["model.embed_tokens.weight"]) and np.array_equal(src("lm_head"), t["lm_head.weight"])
    assert np.array_equal(src("final_norm"), t["model.norm.weight"][None])
    p = "model.layers.1."
    assert np.array_equal(src("layers.1.qkv"), np.concatenate([t[p + f"self_attn.{x}_proj.weight"] for x in "qkv"]))
    assert np.array_equal(src("layers.1.gate_up"), np.concatenate([t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"]]))
    assert np.array_equal(src("layers.0.o"), t["model.layers.0.self_attn.o_proj.weight"])
    assert np.array_equal(src("layers.0.down"), t["model.layers.0.mlp.down_proj.weight"])
    assert np.array_equal(src("layers.0.norm2"), t["model.layers.0.post_attention_layernorm.weight"][None])
    assert np.array_equal(src("mtp.fc"), t["mtp.fc.weight"]) and np.array_equal(src("mtp.norm_h"), t["mtp.pre_fc_norm_hidden.weight"][None])
    assert np.array_equal(src("mtp.qkv"), np.concatenate([t[f"mtp.layers.0.self_attn.{x}_proj.weight"] for x in "qkv"]))
    for bad in ("layers.2.qkv", "layers.0.bias", "mtp.nothing", "elsewhere"):
        with pytest.raises(KeyError):
            src(bad)
    receipt = src.receipt()
    assert receipt["loaded_from_bctx_only"] and receipt["tensor_count"] == len(receipt["tensor_names"]) == len(src.consumed)
    rows = {r["name"]: r for r in package.read_manifest(pkg_dir)["tensors"]}
    assert all(receipt["frame_sha256"][n] == rows[n]["frame_sha256"] and receipt["source_sha256"][n] == rows[n]["source_sha256"] for n in src.consumed)


def test_decoder_weights_and_draft_head_from_frames_alone(packaged):
    pkg_dir, t = packaged
    made = []

    def factory(name, words):
        made.append(name)
        return FakeLinear(name, words)

    w = checkpoint.load_decoder_weights(pkg_dir, "cpu", lin_factory=factory)
    assert len(w.layers) == 2 and w.config.hidden == 128
    assert made == ["layers.0.qkv", "layers.0.o", "layers.0.gate_up", "layers.0.down", "layers.1.qkv", "layers.1.o", "layers.1.gate_up",
                    "layers.1.down", "lm_head"]
    assert w.layers[1].down.words.shape == (128, 256) and w.layers[0].qkv.N == (2 + 2 * 1) * 128
    assert w.embed.dtype == torch.bfloat16 and w.embed.shape == (96, 128)
    assert np.array_equal(w.final_norm.view(torch.int16).numpy().view(np.uint16), t["model.norm.weight"])
    every_trunk_tensor = {n for n in t if not n.startswith("mtp.")}
    assert set(w.notes["receipt"]["tensor_names"]) == every_trunk_tensor
    assert w.streamed_bytes() == sum(x.coded_bytes for x in w.linears()) and w.descriptor_kinds() == {"FakeLinear": 9}
    # tensor parallelism: rank 1 of 2 gets its head's rows of q, and the second half of the FFN columns of down
    # (one KV head cannot be split: the configuration refuses)
    with pytest.raises(ValueError):
        checkpoint.load_decoder_weights(pkg_dir, "cpu", lin_factory=factory, tp_world=2, tp_rank=1)
    # the draft head over a stand-in decoder (what MTPHead reads of it: configuration, device, rows, the KV pool's pages)
    decoder = types.SimpleNamespace(cfg=w.config, dev=torch.device("cpu"), max_rows=4, kv=torch.zeros(1, 2, 3, 1, 1, 1))
    made.clear()
    head = checkpoint.load_mtp_head(w.notes["source"], decoder, lin_factory=factory)
    assert made == ["mtp.qkv", "mtp.o", "mtp.gate_up", "mtp.down", "mtp.fc"]
    assert head.fc.words.shape == (128, 256) and head.norm_e.shape == (128,)
    assert np.array_equal(head.final_norm.view(torch.int16).numpy().view(np.uint16), t["mtp.norm.weight"])
    assert head.receipt["tensor_count"] == 13 == len(checkpoint.mtp_shapes(w.config)) and head.receipt["loaded_from_bctx_only"]
    assert set(head.receipt["tensor_names"]) == set(checkpoint.mtp_shapes(w.config))
    assert set(head.receipt["frame_sha256"]) == set(head.receipt["tensor_names"])


def test_tied_output_head_and_missing_draft_head(tmp_path, write_decoder_checkpoint):
    t = write_decoder_checkpoint(tmp_path / "model", seed=4, mtp=False, tied=True, **dict(FIELDS, layers=1))
    package.build(tmp_path / "model", tmp_path / "package")
    src = checkpoint.PackageWords(tmp_path / "package")
    assert src.tied and not src.has_mtp and np.array_equal(src("lm_head"), t["model.embed_tokens.weight"])
    decoder = types.SimpleNamespace(cfg=src.config, dev=torch.device("cpu"), max_rows=4, kv=torch.zeros(1, 2, 3, 1, 1, 1))
    with pytest.raises(ContextServingError, match="MTP manifest keys differ"):
        checkpoint.load_mtp_head(src, decoder, lin_factory=FakeLinear)


def test_foreign_or_damaged_packages_are_refused(tmp_path, write_decoder_checkpoint):
    small = dict(FIELDS, layers=1)
    bias = np.zeros(256, dtype=np.uint16)
    write_decoder_checkpoint(tmp_path / "m1", mtp=False, extra={"model.layers.0.self_attn.q_proj.bias": bias}, **small)
    package.build(tmp_path / "m1", tmp_path / "p1")
    with pytest.raises(ContextServingError, match="outside the plain"):
        checkpoint.PackageWords(tmp_path / "p1")
    write_decoder_checkpoint(tmp_path / "m2", mtp=False, extra={"mtp.layers.0.self_attn.q_norm.weight": bias[:128]}, **small)
    package.build(tmp_path / "m2", tmp_path / "p2")
    with pytest.raises(ContextServingError, match="draft-head family"):
        checkpoint.PackageWords(tmp_path / "p2")
    # a good package: wrong configuration, a missing tensor, a damaged frame
    write_decoder_checkpoint(tmp_path / "m3", mtp=False, **small)
    package.build(tmp_path / "m3", tmp_path / "p3")
    wrong = checkpoint.decoder_config(tmp_path / "p3" / "sidecars" / "config.json")
    wrong = serve.DecoderConfig(**{**wrong.__dict__, "ffn": 512})
    with pytest.raises(ContextServingError, match="shape/dtype mismatch"):
        checkpoint.PackageWords(tmp_path / "p3", wrong)("layers.0.down")
    src = checkpoint.PackageWords(tmp_path / "p3")
    del src.rows["model.norm.weight"]
    with pytest.raises(ContextServingError, match="lacks a tensor"):
        src("final_norm")
    row = src.rows["model.layers.0.mlp.down_proj.weight"]
    frame = tmp_path / "p3" / row["frame"]
    data = bytearray(frame.read_bytes())
    data[len(data) // 2] ^= 1
    frame.write_bytes(bytes(data))
    with pytest.raises(ContextServingError, match="frame identity mismatch"):
        src("layers.0.down")
    with pytest.raises(ContextServingError):
        checkpoint.PackageWords(tmp_path / "nowhere")


def test_resident_images_are_built_once_and_served_from_the_cache(packaged, tmp_path):
    """The engine's linears as resident images: built from verified frames on the first start, read back from the image
    cache - without touching a frame - on the next, and rebuilt when a record or an entry does not check out."""
    from georefine_b200 import resident
    from georefine_b200.image_cache import ImageCache

    pkg_dir, t = packaged
    cache = ImageCache(tmp_path / "cache")
    cfg = checkpoint.decoder_config(pkg_dir / "sidecars" / "config.json")
    names = checkpoint.linear_names(cfg, mtp=True)
    assert names[:4] == ["layers.0.qkv", "layers.0.o", "layers.0.gate_up", "layers.0.down"] and names[-1] == "mtp.fc" and len(names) == 14
    cold_source = checkpoint.PackageWords(pkg_dir)
    cold = checkpoint.resident_images(cold_source, names, sm_count=148, cache=cache, pool_threads=4)
    assert not any(hit for _, _, hit in cold.values()) and cache.stats["writes"] == len(names)
    matrices = {n for n, w in t.items() if w.ndim == 2} - {"model.embed_tokens.weight"}
    assert set(cold_source.consumed) == matrices                         # every matrix was read; the norms and the embedding were not
    image, header, _ = cold["layers.1.qkv"]
    want = np.concatenate([t[f"model.layers.1.self_attn.{x}_proj.weight"] for x in "qkv"])
    assert (header.rows, header.cols) == want.shape and np.array_equal(resident.decode_image_host(image), want)
    warm_source = checkpoint.PackageWords(pkg_dir)
    warm = checkpoint.resident_images(warm_source, names, sm_count=148, cache=cache, pool_threads=4)
    assert all(hit for _, _, hit in warm.values()) and not warm_source.consumed
    assert all(np.array_equal(warm[n][0], cold[n][0]) for n in names)
    # another build plan (layout, SM count) is another identity: nothing is served across plans
    other = checkpoint.resident_images(checkpoint.PackageWords(pkg_dir), names[:2], sm_count=148, layout="rans", cache=cache)
    assert not any(hit for _, _, hit in other.values()) and other["layers.0.qkv"][1].mode == resident.LAYOUTS["rans"]
    assert warm_source.identity("layers.0.qkv", "a") != warm_source.identity("layers.0.qkv", "b") != warm_source.identity("layers.0.o", "b")
    # a damaged record, and a record whose entry has been damaged, are misses that heal
    records = sorted((tmp_path / "cache" / "groups").rglob("*.json"))
    assert len(records) == len(names) + 2
    records[0].write_text("{not json")
    entry = next(p for p in (tmp_path / "cache").rglob("*.bxr"))
    data = bytearray(entry.read_bytes())
    data[-1] ^= 0xFF
    entry.write_bytes(bytes(data))
    again = checkpoint.resident_images(checkpoint.PackageWords(pkg_dir), names, sm_count=148, cache=cache)
    assert 1 <= sum(1 for _, _, hit in again.values() if not hit) <= 2
    assert all(np.array_equal(resident.decode_image_host(again[n][0]), resident.decode_image_host(cold[n][0])) for n in names)
    assert all(hit for _, _, hit in checkpoint.resident_images(checkpoint.PackageWords(pkg_dir), names, sm_count=148, cache=cache).values())
    # without a cache every call builds
    assert not any(hit for _, _, hit in checkpoint.resident_images(checkpoint.PackageWords(pkg_dir), names[:3], sm_count=148).values())


def test_shards_of_different_ranks_have_different_identities(tmp_path, write_decoder_checkpoint):
    fields = dict(hidden=128, layers=1, heads=4, kv_heads=2, ffn=512, vocab=64)
    t = write_decoder_checkpoint(tmp_path / "model", seed=9, mtp=False, **fields)
    package.build(tmp_path / "model", tmp_path / "package")
    from georefine_b200 import resident

    got = {}
    for rank in (0, 1):
        cfg = checkpoint.decoder_config(tmp_path / "package" / "sidecars" / "config.json", tp_world=2, tp_rank=rank)
        src = checkpoint.PackageWords(tmp_path / "package", cfg)
        got[rank] = (src.identity("layers.0.down", "p"), checkpoint.resident_images(src, ["layers.0.down", "layers.0.qkv"], sm_count=148))
    assert got[0][0] != got[1][0]
    down = t["model.layers.0.mlp.down_proj.weight"]
    for rank in (0, 1):
        image, header, _ = got[rank][1]["layers.0.down"]
        assert (header.rows, header.cols) == (128, 256)
        assert np.array_equal(resident.decode_image_host(image), down[:, rank * 256:(rank + 1) * 256])
        q, k, v = (t[f"model.layers.0.self_attn.{x}_proj.weight"] for x in "qkv")
        want = np.concatenate([q[rank * 256:(rank + 1) * 256], k[rank * 128:(rank + 1) * 128], v[rank * 128:(rank + 1) * 128]])
        assert np.array_equal(resident.decode_image_host(got[rank][1]["layers.0.qkv"][0]), want)
