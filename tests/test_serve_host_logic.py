"""Host logic of the serving engine on the CPU: admission, row buckets, device-resident token feedback, retirement, the
acceptance rule of speculation, the session API (generate / stop / rollback / extend) and sampling - over a stand-in for
``BatchDecoder`` whose "model" is a hash of the sequence so far.

The stand-in keeps what makes the real engine's bookkeeping matter: per-slot state indexed by absolute position (stale
entries beyond a rewound position stay where they are, as KV entries do), rows of a pass that may belong to any slot,
and an "ar" step that feeds every row its own arg-max and advances its position without the host.  The GPU suite runs
the same scenarios on the real decoder (tests/test_gpu_serve.py); the reference's gate for them is "exact speculation"
(glc_serve/bidec_spec.py:9-22) and the session semantics of glc_serve/fastserve.py:250-439.
"""
import types

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from georefine_b200 import sampling, serve  # noqa: E402

VOCAB = 97


def _next(history):
    h = 7
    for t in history:
        h = (h * 1000003 + int(t) + 1) % (2 ** 61 - 1)
    return h % VOCAB


def greedy(prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(_next(seq))
        seq.append(out[-1])
    return out


class FakeDecoder:
    def __init__(self, max_rows=8, max_slots=6, tp_world=1):
        self.max_rows, self.max_slots, self.pad_slot = max_rows, max_slots, max_slots
        self.cfg = types.SimpleNamespace(tp_world=tp_world)
        self.dev = torch.device("cpu")
        self.w = types.SimpleNamespace(streamed_bytes=lambda: 123)
        self.tokens, self.row_seq, self.row_pos = (torch.zeros(max_rows, dtype=torch.int32) for _ in range(3))
        self.next_token = torch.zeros(max_rows, dtype=torch.int32)
        self.logits = torch.zeros(max_rows, VOCAB)
        self.cache = {s: {} for s in range(max_slots + 1)}
        self.pages = {s: -1 for s in range(max_slots + 1)}
        self._free = list(range(max_slots - 1, -1, -1))
        self.runs = []

    def open_slot(self):
        if not self._free:
            raise RuntimeError("no free sequence slot")
        return self._free.pop()

    def close_slot(self, slot):
        self.pages[slot] = -1
        self._free.append(slot)

    def ensure_pages(self, slot, upto):
        self.pages[slot] = max(self.pages[slot], upto)

    def set_rows(self, slots, positions, tokens):
        n = len(slots)
        self.row_seq[:n] = torch.tensor(list(slots), dtype=torch.int32)
        self.row_pos[:n] = torch.tensor(list(positions), dtype=torch.int32)
        self.tokens[:n] = torch.tensor(list(tokens), dtype=torch.int32)

    def run(self, kind, n, *, graph=True):
        assert kind in ("ar", "verify") and 1 <= n <= self.max_rows
        self.runs.append((kind, n, graph))
        rows = [(int(self.row_seq[i]), int(self.row_pos[i]), int(self.tokens[i])) for i in range(n)]
        for slot, pos, tok in rows:                       # every append of a pass happens before any read
            if slot != self.pad_slot:
                assert pos <= self.pages[slot], "a row was run without pages for its position"
            self.cache[slot][pos] = tok
        for i, (slot, pos, _) in enumerate(rows):
            history = [self.cache[slot][p] for p in range(pos + 1)] if slot != self.pad_slot else [0]
            nxt = _next(history)
            self.next_token[i] = nxt
            self.logits[i] = -(torch.arange(VOCAB) - nxt).abs().float()
        if kind == "ar":
            self.tokens[:n] = self.next_token[:n]
            self.row_pos[:n] += 1


def test_admission_buckets_feedback_and_retirement():
    d = FakeDecoder(max_rows=8)
    b = serve.Batcher(d)
    assert b.buckets == (1, 2, 4, 8) and b.step() == {}
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], [2, 7], [1]]           # the first is longer than a pass of 8 rows
    slots = [b.admit(p) for p in prompts]
    assert [b.active[s]["tokens"] for s in slots] == [greedy(p, 1) for p in prompts]
    assert [r for r in d.runs if r[1] > 1] == [("verify", 8, False), ("verify", 3, False), ("verify", 2, False)]
    for _ in range(3):
        out = b.step()
        assert set(out) == set(slots)
    assert d.runs[-1] == ("ar", 4, True)                                   # three sequences run in the bucket of four
    # steps without a read-back: the tokens stay on the device and are collected later
    for _ in range(4):
        assert b.step(fetch=False) is None
    b.sync_tokens()
    for s, p in zip(slots, prompts):
        got, want = b.active[s]["tokens"], greedy(p, 8)
        assert got[:4] == want[:4] and got[-1] == want[-1] and got[4:7] == [None] * 3 and b.active[s]["pos"] == len(p) + 7
    b.retire(slots[1])
    out = b.step()
    assert set(out) == {slots[0], slots[2]} and d.runs[-1] == ("ar", 2, True)
    assert out[slots[0]] == greedy(prompts[0], 9)[-1]
    late = b.admit([8, 8, 8])                                              # a freed slot is reused; the others carry on
    assert late == slots[1]
    out = b.step()
    assert out[late] == greedy([8, 8, 8], 2)[-1] and out[slots[2]] == greedy(prompts[2], 10)[-1]
    # a step for some of the sequences only: the others stand still, then everything carries on together
    before = {s: list(b.active[s]["tokens"]) for s in b.active}
    out = b.step(only=[late])
    assert set(out) == {late} and d.runs[-1] == ("ar", 1, True) and out[late] == greedy([8, 8, 8], 3)[-1]
    assert all(b.active[s]["tokens"] == before[s] for s in (slots[0], slots[2]))
    assert b.step(only=[late], fetch=False) is None
    out = b.step()
    assert out[slots[0]] == greedy(prompts[0], 11)[-1] and out[late] == greedy([8, 8, 8], 5)[-1]
    assert b.active[late]["tokens"] == greedy([8, 8, 8], 5)
    with pytest.raises(KeyError):
        b.step(only=[5])
    with pytest.raises(ValueError):
        b.admit([])
    with pytest.raises(ValueError):
        serve.bucket_for(9, (1, 2, 4, 8))


def test_verify_accepts_the_longest_agreeing_prefix_and_rewinds_by_position():
    d = FakeDecoder(max_rows=16)
    b = serve.Batcher(d)
    p1, p2 = [5, 6, 7], [9, 9, 9, 9]
    s1, s2 = b.admit(p1), b.admit(p2)
    w1, w2 = greedy(p1, 12), greedy(p2, 12)
    out = b.verify({s1: w1[1:4], s2: [w2[1], (w2[2] + 1) % VOCAB, w2[3]]})     # all three right; the second one wrong
    assert out[s1] == w1[1:5] and out[s2] == w2[1:3]
    assert b.active[s1]["pos"] == len(p1) + 4 and b.active[s2]["pos"] == len(p2) + 2
    # the surplus rows of the refused drafts are still in the slot's state; the next pass overwrites them
    out = b.verify({s1: [0, 0], s2: w2[3:8]})
    assert out[s1] == [w1[5]] and out[s2] == w2[3:9]
    assert b.step() == {s1: w1[6], s2: w2[9]}
    with pytest.raises(ValueError):
        b.verify({s1: list(range(20))})


def test_session_generate_stop_rollback_extend_and_speculation():
    d = FakeDecoder(max_rows=8)
    sess = serve.FastSession(d)
    assert sess.meta["streamed_bytes_per_step"] == 123
    prompt = [4, 8, 15, 16, 23, 42]
    want = greedy(prompt, 30)
    st = sess.prefill(token_ids=prompt)
    assert st.plen == 6 and list(sess.generate(st, max_tokens=5)) == want[:5]
    assert list(sess.generate(st, max_tokens=3)) == want[5:8]              # a second call carries on
    sess.rollback(st, 3)
    assert st.tokens == want[:5] and list(sess.generate(st, max_tokens=4)) == want[5:9]
    with pytest.raises(ValueError):
        sess.rollback(st, 99)
    # a stop token ends the call with the token emitted, and speculation never runs past it
    stop = want[12]
    first_stop = want.index(stop)
    rng = np.random.default_rng(0)
    for drafter in (None, lambda s, k: want[len(s.tokens):len(s.tokens) + k], lambda s, k: rng.integers(0, VOCAB, k).tolist()):
        st2 = sess.prefill(token_ids=prompt)
        got = list(sess.generate(st2, max_tokens=25, stop_ids=[stop], spec_k=4 if drafter else 0, drafter=drafter))
        assert got == want[:first_stop + 1] and st2.tokens == got
        assert sess.batcher.active[st2.slot]["pos"] == len(prompt) + len(got) - 1
        sess.close(st2)
        assert st.tokens == want[:9]                                       # the other open sequence did not move
    # extend: the next turn's tokens go through the engine; the result is what one long prompt gives
    more = [11, 12, 13, 14, 15, 16, 17, 18, 19, 20]
    sess.extend(st, more)
    got = list(sess.generate(st, max_tokens=3))
    assert got == greedy(prompt + want[:9] + more, 3)
    sess.extend(st, [])
    sess.close(st)
    assert sorted(d._free) == list(range(d.max_slots))


def test_session_sampling_on_the_host_side():
    d = FakeDecoder(max_rows=8)
    sess = serve.FastSession(d)
    prompt = [1, 2, 3]
    want = greedy(prompt, 12)
    rng = np.random.default_rng(3)
    for drafter in (None, lambda s, k: rng.integers(0, VOCAB, k).tolist()):
        kw = dict(spec_k=3, drafter=drafter) if drafter else {}
        st = sess.prefill(token_ids=prompt)
        assert list(sess.generate(st, max_tokens=12, temperature=1.0, top_p=1e-9, seed=0, **kw)) == want   # empty nucleus: arg-max
        sess.close(st)
        runs = []
        for seed in (5, 5, 6):
            st = sess.prefill(token_ids=prompt)
            rng = np.random.default_rng(3)
            runs.append(list(sess.generate(st, max_tokens=12, temperature=3.0, seed=seed, **kw)))
            seq = sess.batcher.active[st.slot]
            assert seq["pos"] == len(prompt) + 11 and st.tokens == runs[-1]
            # whatever was drawn, the state behind it is that of the drawn tokens: the greedy continuation agrees
            assert next(iter(sess.generate(st, max_tokens=1))) == _next(prompt + runs[-1])
            sess.close(st)
        assert runs[0] == runs[1] != runs[2] and runs[0] != want
    # a tensor-parallel decoder refuses to sample without a seed the ranks share
    tp = serve.FastSession(FakeDecoder(tp_world=2))
    st = tp.prefill(token_ids=prompt)
    with pytest.raises(ValueError, match="seed"):
        list(tp.generate(st, max_tokens=2, temperature=0.7))
    assert len(list(tp.generate(st, max_tokens=2, temperature=0.7, seed=1))) == 2
    # the batcher draws for every row of a step, and at admission
    b = serve.Batcher(FakeDecoder())
    sampler = sampling.Sampler(2.0, seed=9)
    slots = [b.admit(p, sampler=sampler) for p in ([1, 2], [3, 4, 5])]
    for _ in range(4):
        out = b.step(sampler=sampler)
        assert set(out) == set(slots) and all(0 <= t < VOCAB for t in out.values())
    drawn = {s: list(b.active[s]["tokens"]) for s in slots}
    out = b.step()                                                         # arg-max again: it continues the drawn sequences
    for s, p in zip(slots, ([1, 2], [3, 4, 5])):
        assert len(drawn[s]) == 5 and out[s] == _next(p + drawn[s])
