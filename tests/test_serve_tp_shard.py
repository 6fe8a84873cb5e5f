"""How a decoder's weights are cut for tensor parallelism (``DecoderConfig.shard``), on the CPU: the ranks' query, key
and value heads partition the whole QKV weight; the ranks' partial O and down products add up to the whole product; the
gate|up shards feed exactly the FFN columns that the rank's down shard multiplies."""
import numpy as np
import pytest

from georefine_b200.serve import DecoderConfig


def test_shards_partition_the_layer_and_partial_products_add_up():
    shape = dict(hidden=256, layers=1, heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=64)
    whole = DecoderConfig(**shape)
    rng = np.random.default_rng(0)
    w = {name: rng.standard_normal((n, k)).astype(np.float32) for name, n, k in whole.linear_shapes()}
    x = rng.standard_normal((3, shape["hidden"])).astype(np.float32)
    qkv = x @ w["qkv"].T
    q_heads, k_heads, v_heads = [], [], []
    o_sum = np.zeros((3, shape["hidden"]), dtype=np.float32)
    down_sum = np.zeros_like(o_sum)
    ctx_full = rng.standard_normal((3, shape["heads"] * 128)).astype(np.float32)
    gu = x @ w["gate_up"].T
    act_full = gu[:, :512] * gu[:, 512:]                         # any column-wise function of (gate, up) will do here
    for r in range(2):
        cfg = DecoderConfig(tp_world=2, tp_rank=r, **shape)
        assert (cfg.local_heads, cfg.local_kv_heads, cfg.local_ffn, cfg.local_qkv_rows) == (2, 1, 256, 512)
        part = x @ cfg.shard("qkv", w["qkv"]).T                  # [q heads of the rank | its k head | its v head]
        q_heads.append(part[:, :256]); k_heads.append(part[:, 256:384]); v_heads.append(part[:, 384:])
        o_sum += ctx_full[:, r * 256:(r + 1) * 256] @ cfg.shard("o", w["o"]).T
        local = x @ cfg.shard("gate_up", w["gate_up"]).T
        act = local[:, :256] * local[:, 256:]
        assert np.allclose(act, act_full[:, r * 256:(r + 1) * 256], rtol=1e-5, atol=1e-5)
        down_sum += act @ cfg.shard("down", w["down"]).T
        assert cfg.shard("norm1", w["o"]) is w["o"]               # everything else is replicated
    assert np.allclose(np.concatenate(q_heads + k_heads + v_heads, axis=1), qkv, rtol=1e-5, atol=1e-5)
    assert np.allclose(o_sum, ctx_full @ w["o"].T, rtol=1e-4, atol=1e-4)
    assert np.allclose(down_sum, act_full @ w["down"].T, rtol=1e-4, atol=1e-3)
    assert whole.shard("qkv", w["qkv"]) is w["qkv"]


def test_uneven_splits_are_refused():
    for bad in (dict(tp_world=3), dict(tp_world=2, tp_rank=2), dict(tp_world=2, ffn=17408 + 128), dict(tp_world=16)):
        with pytest.raises(ValueError):
            DecoderConfig(**bad)
    assert DecoderConfig(tp_world=8, tp_rank=7).local_kv_heads == 1
