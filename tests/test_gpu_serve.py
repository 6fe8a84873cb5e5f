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
    for s, want in zip(slots, alone):
        got = b.active[s]["tokens"]
        assert got[:20] == want[:len(got[:20])] and len(got) >= 13
    assert d.w.streamed_bytes() > 0 and d.streamed_bytes([100, 200])["kv"] == 300 * cfg.kv_heads * 128 * 4 * cfg.layers
