"""The decoder stack served from compressed weights (needs a B200): the whole-step engine, continuous batching, the
session API and exact speculation, on a small random-init model.

Oracle: a plain torch restatement of the same decoder with the same rounding points (BF16 activations, FP32
accumulation), fed with the weights the engine's resident images decode to.  On top of the tolerance against it, the
engine must keep the invariants that make serving exact: a sequence yields the same tokens alone, inside a batch, from a
CUDA graph or eagerly, after a rollback, and under speculation whatever the drafter proposes (the reference's
"exact speculation" gate, glc_serve/bidec_spec.py:9-22).
"""
import math

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from georefine_b200 import _native

    _native.lib()
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def small(dev):
    from georefine_b200 import serve

    cfg = serve.DecoderConfig(hidden=512, layers=2, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=1000)
    weights = serve.DecoderWeights.synthetic(cfg, dev, seed=3, max_m=64)
    return cfg, weights


def _reference_logits(cfg, w, ids, dev):
    """Logits of every position of one sequence, full causal forward in torch."""
    def lin(x, res):
        return (x.float() @ res.decode().float().T).to(torch.bfloat16)

    def norm(h, weight):
        f = h.float()
        return (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + cfg.eps) * weight.float()).to(torch.bfloat16)

    from georefine_b200 import ops

    n, d = len(ids), cfg.head_dim
    cos, sin = ops.rope_tables(n, cfg.rope_theta, dev)
    h = w.embed[torch.tensor(ids, device=dev)]

    def rope(x):
        c, s = cos[:, None, :].float(), sin[:, None, :].float()
        rot = torch.cat([-x[..., d // 2:], x[..., :d // 2]], dim=-1)
        return ((x * c).to(torch.bfloat16).float() + (rot * s).to(torch.bfloat16).float()).to(torch.bfloat16).float()

    mask = torch.full((n, n), float("-inf"), device=dev).triu(1)
    delta = None
    for layer in w.layers:
        if delta is not None:
            h = (h.float() + delta.float()).to(torch.bfloat16)
        qkv = lin(norm(h, layer.norm1), layer.qkv).float()
        q = rope(qkv[:, :cfg.heads * d].reshape(n, cfg.heads, d))
        k = rope(qkv[:, cfg.heads * d:(cfg.heads + cfg.kv_heads) * d].reshape(n, cfg.kv_heads, d))
        v = qkv[:, (cfg.heads + cfg.kv_heads) * d:].reshape(n, cfg.kv_heads, d)
        g = cfg.heads // cfg.kv_heads
        score = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(g, dim=1)) / math.sqrt(d) + mask
        ctx = torch.einsum("hqk,khd->qhd", torch.softmax(score, dim=-1), v.repeat_interleave(g, dim=1)).reshape(n, -1).to(torch.bfloat16)
        h = (h.float() + lin(ctx, layer.o).float()).to(torch.bfloat16)
        gu = lin(norm(h, layer.norm2), layer.gate_up).float()
        gate, up = gu[:, :cfg.ffn], gu[:, cfg.ffn:]
        act = ((gate / (1 + torch.exp(-gate))).to(torch.bfloat16).float() * up).to(torch.bfloat16)
        delta = lin(act, layer.down)
    h = (h.float() + delta.float()).to(torch.bfloat16)
    return lin(norm(h, w.final_norm), w.lm_head)


def _greedy(decoder, prompt, n):
    from georefine_b200 import serve

    b = serve.Batcher(decoder)
    slot = b.admit(prompt)
    out = list(b.active[slot]["tokens"])
    while len(out) < n:
        out.append(b.step()[slot])
    b.retire(slot)
    return out


def test_prefill_logits_against_the_torch_restatement(dev, small):
    from georefine_b200 import serve

    cfg, w = small
    d = serve.BatchDecoder(w, max_rows=64, max_slots=8, max_context=1024, device=dev)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (50,), generator=g).tolist()
    slot = d.open_slot()
    d.ensure_pages(slot, len(ids))
    d.set_rows([slot] * len(ids), range(len(ids)), ids)
    d.run("verify", len(ids), graph=False)
    got = d.logits[:len(ids)].float()
    want = _reference_logits(cfg, w, ids, dev).float()
    assert (got - want).abs().max().item() <= 4e-2 * want.abs().max().item()
    # the engine's arg-max is (next to) the restatement's maximum in every row
    top = want.max(dim=1).values
    picked = want.gather(1, d.next_token[:len(ids)].long()[:, None])[:, 0]
    assert ((top - picked) <= 4e-2 * want.abs().max()).all()


def test_tokens_do_not_depend_on_batch_graph_or_bucket(dev, small):
    from georefine_b200 import serve

    cfg, w = small
    d = serve.BatchDecoder(w, max_rows=64, max_slots=16, max_context=1024, device=dev)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (5, 70, 256, 257, 31, 9, 300, 2, 64)]
    alone = [_greedy(d, p, 14) for p in prompts]
    b = serve.Batcher(d)
    slots = [b.admit(p) for p in prompts[:5]]
    for _ in range(4):
        b.step()
    slots += [b.admit(p) for p in prompts[5:]]            # the bucket grows from 8 to 16 rows mid-way
    for _ in range(5):
        b.step()
    b.retire(slots[1])                                       # and a sequence leaves
    for _ in range(20):
        b.step(fetch=False)                                  # tokens stay on the device between steps ...
    for i, s in enumerate(slots):
        if i == 1:
            continue
        known = [t for t in b.active[s]["tokens"] if t is not None][:14]
        assert known == alone[i][:len(known)] and len(known) >= 6
    # eager steps give the same tokens as replayed graphs
    s = d.open_slot()
    d.ensure_pages(s, len(prompts[0]) + 14)
    d.set_rows([s] * 5, range(5), prompts[0])
    d.run("verify", 5, graph=False)
    tok, out = int(d.next_token[4]), []
    for j in range(13):
        out.append(tok)
        d.set_rows([s], [5 + j], [tok])
        d.run("ar", 1, graph=False)
        tok = int(d.next_token[0])
    assert out == alone[0][:13]


def test_session_rollback_extend_and_speculation_are_exact(dev, small):
    from georefine_b200 import serve

    cfg, w = small
    d = serve.BatchDecoder(w, max_rows=64, max_slots=8, max_context=1024, device=dev)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    plain = _greedy(d, prompt, 30)
    sess = serve.FastSession(d)
    st = sess.prefill(token_ids=prompt)
    assert list(sess.generate(st, max_tokens=10)) == plain[:10]
    sess.rollback(st, 4)
    assert list(sess.generate(st, max_tokens=6)) == plain[6:12]
    sess.close(st)
    # extend: prompt + first token + more tokens == one longer prompt
    more = torch.randint(0, cfg.vocab, (70,), generator=g).tolist()
    st = sess.prefill(token_ids=prompt)
    sess.extend(st, more)
    got = list(sess.generate(st, max_tokens=5))
    sess.close(st)
    want = _greedy(d, prompt + [plain[0]] + more, 5)
    assert got[-4:] == want[1:5] or got == want[:5]
    # speculation: random drafts (nothing accepted), perfect drafts (everything accepted), mixed - always the greedy tokens
    rng = np.random.default_rng(0)
    for name, drafter in [("random", lambda st, k: rng.integers(0, cfg.vocab, k).tolist()),
                          ("perfect", lambda st, k: plain[len(st.tokens):len(st.tokens) + k] + [0] * max(0, len(st.tokens) + k - len(plain))),
                          ("half", lambda st, k: plain[len(st.tokens):len(st.tokens) + 2] + [1] * (k - 2))]:
        st = sess.prefill(token_ids=prompt)
        got = list(sess.generate(st, max_tokens=24, spec_k=5, drafter=drafter))
        assert got == plain[:24], name
        sess.close(st)


def test_mtp_head_speculation_in_a_batch_is_exact(dev, small):
    from georefine_b200 import serve

    cfg, w = small
    d = serve.BatchDecoder(w, max_rows=64, max_slots=8, max_context=1024, device=dev)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (12, 100, 33)]
    alone = [_greedy(d, p, 20) for p in prompts]
    b = serve.Batcher(d)
    spec = serve.MTPSpeculator(b, serve.MTPHead.synthetic(d), k=5)
    slots = [spec.admit(p) for p in prompts]
    for _ in range(12):
        out = spec.cycle()
        assert all(1 <= len(v) <= 6 for v in out.values())
    assert spec.stats["cycles"] == 36 and spec.stats["emitted"] == sum(len(b.active[s]["tokens"]) - 1 for s in slots)
    assert spec.stats["drafts_accepted"] == spec.stats["emitted"] - 36 and 1 <= spec.mean_tokens_per_cycle <= 6
    for s, want in zip(slots, alone):
        got = b.active[s]["tokens"]
        assert got[:20] == want[:len(got[:20])] and len(got) >= 13
    assert d.w.streamed_bytes() > 0 and d.streamed_bytes([100, 200])["kv"] == 300 * cfg.kv_heads * 128 * 4 * cfg.layers


def test_session_sampling_is_seeded_and_keeps_the_engine_in_step(dev, small):
    """Temperature / top-p sampling through the session (the reference's ``generate(temperature=, top_p=, seed=)``,
    glc_serve/fastserve.py:250-306): reproducible from the seed, arg-max in the limit of an empty nucleus, and the KV
    cache and positions stay those of the tokens that were actually emitted - with and without speculation."""
    from georefine_b200 import sampling, serve

    cfg, w = small
    d = serve.BatchDecoder(w, max_rows=64, max_slots=8, max_context=1024, device=dev)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab, (50,), generator=g).tolist()
    plain = _greedy(d, prompt, 24)
    sess = serve.FastSession(d)
    rng = np.random.default_rng(1)
    drafters = {"none": None, "random": lambda st, k: rng.integers(0, cfg.vocab, k).tolist(),
                "greedy-path": lambda st, k: (plain[len(st.tokens):len(st.tokens) + k] + [0] * k)[:k]}

    def run(seed, drafter, n=16, **kw):
        st = sess.prefill(token_ids=prompt)
        out = list(sess.generate(st, max_tokens=n, seed=seed, spec_k=5 if drafter else 0, drafter=drafter, **kw))
        seq = sess.batcher.active[st.slot]
        assert out == st.tokens and len(out) == n and seq["pos"] == len(prompt) + n - 1
        assert all(0 <= t < cfg.vocab for t in out)
        following = next(iter(sess.generate(st, max_tokens=1)))          # greedy continuation from the sampled state
        sess.close(st)
        return out, following

    for name, drafter in drafters.items():
        # an empty nucleus is arg-max decoding, whatever the drafter proposes
        got, _ = run(0, drafter, n=24, temperature=1.0, top_p=1e-9)
        assert got == plain, name
        rng = np.random.default_rng(1)
        a, after_a = run(7, drafter, temperature=0.8, top_p=0.95)
        rng = np.random.default_rng(1)
        b, after_b = run(7, drafter, temperature=0.8, top_p=0.95)
        assert a == b and after_a == after_b, name
        # the cache behind the sampled tokens is what a fresh pass over prompt + tokens builds
        assert after_a == _greedy(d, prompt + a, 1)[0], name
        others = [run(s, drafter, temperature=0.8, top_p=0.95)[0] for s in (8, 9, 10)]
        assert any(o != a for o in others), name
    # the batched speculator with the draft head, sampling: bookkeeping stays consistent and the run is reproducible
    results = []
    for _ in range(2):
        b = serve.Batcher(d)
        spec = serve.MTPSpeculator(b, serve.MTPHead.synthetic(d), k=3)
        sampler = sampling.Sampler(0.7, 0.9, device=dev, seed=5)
        slots = [spec.admit(prompt[:n], sampler=sampler) for n in (20, 50)]
        for _ in range(5):
            out = spec.cycle(sampler=sampler)
            assert all(1 <= len(v) <= 4 for v in out.values())
        for s, n in zip(slots, (20, 50)):
            assert b.active[s]["pos"] == n + len(b.active[s]["tokens"]) - 1
        results.append([list(b.active[s]["tokens"]) for s in slots])
        for s in reversed(slots):          # slots are handed out from a stack: the second round gets the same ones, and with
            spec.retire(s)                 # them the same order of sequences inside a cycle, which is the order of the draws
    assert results[0] == results[1]


def test_session_from_a_package_serves_the_checkpoint_it_was_built_from(dev, tmp_path, write_decoder_checkpoint):
    """``FastSession.load(package=...)``: decoder and draft head filled from the frames of a BCTX package alone
    (georefine_b200/checkpoint.py) give, token for token, what the same tensors give when handed over in memory."""
    from georefine_b200 import package, serve
    from georefine_b200.resident import ResidentWeight

    fields = dict(hidden=512, layers=2, heads=4, kv_heads=2, ffn=1024, vocab=1000)
    t = write_decoder_checkpoint(tmp_path / "model", seed=5, **fields)
    package.build(tmp_path / "model", tmp_path / "package", jobs=8)
    from georefine_b200.image_cache import ImageCache

    cache = ImageCache(tmp_path / "images")
    sess = serve.FastSession.load(package=tmp_path / "package", device=dev, max_len=1024, max_rows=64, max_m=64, cache=cache)
    assert sess.mtp_head is not None and sess.meta["receipt"]["loaded_from_bctx_only"] and sess.d.w.notes["image_cache_hits"] == 0
    assert sess.mtp_head.receipt["tensor_count"] == 13 and sess.d.cfg.ffn == 1024

    def group(prefix, leaf):           # the engine's tensors straight from the checkpoint in memory
        names = {"norm1": ["input_layernorm"], "norm2": ["post_attention_layernorm"], "o": ["self_attn.o_proj"], "down": ["mlp.down_proj"],
                 "qkv": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], "gate_up": ["mlp.gate_proj", "mlp.up_proj"]}[leaf]
        parts = [np.atleast_2d(t[prefix + n + ".weight"]) for n in names]
        return np.concatenate(parts) if len(parts) > 1 else parts[0]

    def words_of(name):
        if name in ("embed", "lm_head", "final_norm"):
            return np.atleast_2d(t[{"embed": "model.embed_tokens.weight", "lm_head": "lm_head.weight", "final_norm": "model.norm.weight"}[name]])
        _, i, leaf = name.split(".")
        return group(f"model.layers.{i}.", leaf)

    direct = serve.DecoderWeights.from_words(sess.d.cfg, words_of, dev, max_m=64)
    d2 = serve.BatchDecoder(direct, max_rows=64, max_slots=4, max_context=1024, device=dev)
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, 1000, (37,), generator=g).tolist()
    want = _greedy(d2, prompt, 20)
    st = sess.prefill(token_ids=prompt)
    assert list(sess.generate(st, max_tokens=20)) == want
    sess.close(st)
    # the draft head: same drafts and same hidden state as a head built from the tensors in memory
    def res(words):
        return ResidentWeight.from_words(np.ascontiguousarray(words), dev, max_m=64, verify=False)

    def vec(name):
        return torch.from_numpy(t[name].view(np.int16).copy()).view(torch.bfloat16).to(dev)

    layer = serve.LayerWeights(vec("mtp.layers.0.input_layernorm.weight"), res(group("mtp.layers.0.", "qkv")), res(group("mtp.layers.0.", "o")),
                               vec("mtp.layers.0.post_attention_layernorm.weight"), res(group("mtp.layers.0.", "gate_up")),
                               res(group("mtp.layers.0.", "down")))
    head2 = serve.MTPHead(sess.d, fc=res(t["mtp.fc.weight"]), norm_e=vec("mtp.pre_fc_norm_embedding.weight"),
                          norm_h=vec("mtp.pre_fc_norm_hidden.weight"), layer=layer, final_norm=vec("mtp.norm.weight"))
    slot = sess.d.open_slot()
    sess.d.ensure_pages(slot, 16)
    hidden = torch.randn(12, 512, generator=g).to(torch.bfloat16).to(dev)
    toks = torch.randint(0, 1000, (12,), generator=g).tolist()
    drafts = [h.absorb([slot] * 12, list(range(1, 13)), toks, hidden) for h in (sess.mtp_head, head2)]
    assert drafts[0] == drafts[1] and torch.equal(sess.mtp_head.z[:12], head2.z[:12])
    sess.d.close_slot(slot)
    # and speculation with the packaged head is exact
    b = serve.Batcher(sess.d)
    spec = serve.MTPSpeculator(b, sess.mtp_head, k=4)
    s = spec.admit(prompt)
    while len(b.active[s]["tokens"]) < 20:
        spec.cycle()
    assert b.active[s]["tokens"][:20] == want
    spec.retire(s)
    # a second start reads every image from the cache (2 layers x 4 + the output head, and the head's 5) and serves the same tokens
    before = cache.stats["hits"]
    again = serve.FastSession.load(package=tmp_path / "package", device=dev, max_len=1024, max_rows=64, max_m=64, cache=cache)
    assert again.d.w.notes["image_cache_hits"] == 9 and cache.stats["hits"] - before == 14
    assert not any(n.endswith("_proj.weight") for n in again.meta["receipt"]["tensor_names"])
    st = again.prefill(token_ids=prompt)
    assert list(again.generate(st, max_tokens=20)) == want
