"""A decoder stack served from compressed weights: the callers of the fused linears.

Counterparts in the reference (``context-runtime/glc_serve``): the whole-step engine ``FastDecoder``
(``fastdec.py:706-956``: ``_trunk``, ``capture``, ``replay``, ``streamed_bytes``, linears injected through
``lin_factory``, :393,417), its batched twin with a page table, row buckets and one CUDA graph per bucket
(``bidec.py:575-619,1103-1264``), the session API ``FastSession`` (``fastserve.py:114-439``: ``load``, ``prefill``,
``generate``, ``extend``, ``rollback``) and exact speculation (``fastserve.py:308-350``, ``bidec_spec.py``: accept the
longest prefix of the drafts that equals the target's own arg-max rows, emit one more, rewind by setting positions).

What is different here: the model is a plain grouped-query decoder (RMSNorm, rotary attention, SwiGLU; the shapes of
the benchmark's stack), weights are given as BF16 bit patterns (synthetic ones when no checkpoint is at hand) and every
linear is a descriptor ``weight(x, y)`` over a compressed resident image; all other kernels of a step are this
library's own (``georefine_b200.ops``).  Every row of a step is computed independently of the other rows - fused
linears with bitwise batch-invariant rows, per-row norm / attention / arg-max kernels - so a sequence produces the same
tokens alone, inside any batch, and as rows of a speculative verify pass.

All per-sequence state is indexed by absolute position (KV pages), so a rewind is "set the position".
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from . import ops
from .resident import ResidentWeight

PAGE = ops.PAGE


@dataclass(frozen=True)
class DecoderConfig:
    hidden: int = 5120
    layers: int = 64
    heads: int = 40
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 17408
    vocab: int = 152064
    rope_theta: float = 1e6
    eps: float = 1e-6
    tp_world: int = 1        # tensor parallelism over the GPUs of one node: this process is rank tp_rank of tp_world
    tp_rank: int = 0

    def __post_init__(self):
        w = self.tp_world
        if w < 1 or not 0 <= self.tp_rank < w or self.heads % w or self.kv_heads % w or self.ffn % w or (self.ffn // w) % 128:
            raise ValueError("tensor parallelism needs the query heads, the KV heads and the FFN width (in 128-column chunks) to divide evenly")

    @property
    def qkv_rows(self) -> int:
        return (self.heads + 2 * self.kv_heads) * self.head_dim

    # what this rank holds: its share of the heads and of the FFN columns
    @property
    def local_heads(self) -> int:
        return self.heads // self.tp_world

    @property
    def local_kv_heads(self) -> int:
        return self.kv_heads // self.tp_world

    @property
    def local_ffn(self) -> int:
        return self.ffn // self.tp_world

    @property
    def local_qkv_rows(self) -> int:
        return (self.local_heads + 2 * self.local_kv_heads) * self.head_dim

    def linear_shapes(self):
        """(name, weight rows, weight columns) of the four linears of a layer (whole, before any sharding), in the order
        a step runs them."""
        return [("qkv", self.qkv_rows, self.hidden), ("o", self.hidden, self.heads * self.head_dim),
                ("gate_up", 2 * self.ffn, self.hidden), ("down", self.hidden, self.ffn)]

    def shard(self, leaf: str, words):
        """This rank's part of a whole weight: QKV and gate|up by weight rows (the rank's query heads, its key heads, its
        value heads; its columns of the gate half and of the up half), O and down by weight columns (the rank's heads'
        outputs; its FFN columns), whose partial products are then summed over the ranks.  Anything else is replicated."""
        if self.tp_world == 1:
            return words
        r, d = self.tp_rank, self.head_dim
        lh, lkv, lf = self.local_heads * d, self.local_kv_heads * d, self.local_ffn
        if leaf == "qkv":
            k_at, v_at = self.heads * d, (self.heads + self.kv_heads) * d
            return np.concatenate([words[r * lh:(r + 1) * lh], words[k_at + r * lkv:k_at + (r + 1) * lkv], words[v_at + r * lkv:v_at + (r + 1) * lkv]])
        if leaf == "gate_up":
            return np.concatenate([words[r * lf:(r + 1) * lf], words[self.ffn + r * lf:self.ffn + (r + 1) * lf]])
        if leaf == "o":
            return np.ascontiguousarray(words[:, r * lh:(r + 1) * lh])
        if leaf == "down":
            return np.ascontiguousarray(words[:, r * lf:(r + 1) * lf])
        return words


def synthetic_words(rows, cols, seed):
    """BF16 bit patterns of N(0, 0.02) weights with a LogNormal(0, 0.25) scale per row (stand-in for a checkpoint)."""
    import torch

    g = torch.Generator().manual_seed(int(seed))
    w = torch.randn(rows, cols, generator=g) * 0.02
    w = w * torch.exp(0.25 * torch.randn(rows, 1, generator=g))
    return w.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


@dataclass
class LayerWeights:
    norm1: object
    qkv: object
    o: object
    norm2: object
    gate_up: object
    down: object

    def linears(self):
        return [self.qkv, self.o, self.gate_up, self.down]


@dataclass
class DecoderWeights:
    """Everything a step reads: a dense BF16 embedding table, per layer two norm vectors and four linear descriptors
    (any object with ``N``, ``K``, ``coded_bytes`` and ``__call__(x, y)``), the final norm and the output head."""

    config: DecoderConfig
    embed: object
    layers: list
    final_norm: object
    lm_head: object
    notes: dict = field(default_factory=dict)

    @classmethod
    def from_words(cls, config, words_of, device, *, lin_factory=None, max_m=128, tune=None, layout=None, distinct_layers=None):
        """``words_of(name)`` returns BF16 bit patterns [rows, cols] for ``embed``, ``lm_head``, ``final_norm``,
        ``layers.<i>.<qkv|o|gate_up|down|norm1|norm2>``.  ``lin_factory(name, words)`` builds a linear descriptor (default:
        a resident image in the default layout).  With ``distinct_layers = d < layers`` only the first d layers are
        built on the host; layer i >= d gets device copies of layer i mod d (same bytes to stream, a fraction of the
        host time: for benchmarks of random-init stacks)."""
        import torch

        dev = torch.device(device)

        def dense(name):
            return torch.from_numpy(np.ascontiguousarray(words_of(name)).view(np.int16)).view(torch.bfloat16).to(dev)

        def linear(name):
            words = np.ascontiguousarray(config.shard(name.split(".")[-1], words_of(name)))
            if lin_factory is not None:
                return lin_factory(name, words)
            return ResidentWeight.from_words(words, dev, max_m=max_m, verify=False, tune=tune, layout=layout)

        d = config.layers if not distinct_layers else min(int(distinct_layers), config.layers)
        built = []
        for i in range(d):
            p = f"layers.{i}."
            built.append(LayerWeights(dense(p + "norm1").reshape(-1), linear(p + "qkv"), linear(p + "o"), dense(p + "norm2").reshape(-1),
                                      linear(p + "gate_up"), linear(p + "down")))
        layers = list(built)
        for i in range(d, config.layers):
            src = built[i % d]
            layers.append(LayerWeights(src.norm1, src.qkv.clone(), src.o.clone(), src.norm2, src.gate_up.clone(), src.down.clone()))
        out = cls(config, dense("embed"), layers, dense("final_norm").reshape(-1), linear("lm_head"),
                  {"distinct_layers": d, "layers": config.layers})
        out.chain()
        return out

    @classmethod
    def synthetic(cls, config, device, *, seed=1, **kw):
        """Random-init weights of the benchmark's distribution; norm vectors near one."""
        import torch

        shapes = {name: (n, k) for name, n, k in config.linear_shapes()}

        def words_of(name):
            key = sum(ord(c) * (i + 1) for i, c in enumerate(name)) + 1000003 * seed
            leaf = name.split(".")[-1]
            if leaf in ("norm1", "norm2", "final_norm"):
                g = torch.Generator().manual_seed(key)
                return (1 + 0.1 * torch.randn(1, config.hidden, generator=g)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
            if leaf in ("embed", "lm_head"):
                return synthetic_words(config.vocab, config.hidden, key)
            return synthetic_words(*shapes[leaf], key)

        return cls.from_words(config, words_of, device, **kw)

    def linears(self):
        for layer in self.layers:
            yield from layer.linears()
        yield self.lm_head

    def chain(self):
        """Tells every compressed linear which one the stream multiplies by next (see ``ResidentWeight.then``)."""
        seq = [w for w in self.linears() if hasattr(w, "then")]
        for a, b in zip(seq, seq[1:] + seq[:1]):
            a.then(b)

    def descriptor_kinds(self) -> dict:
        """How many of the step's linears are of which kind ("bctx", "dense", ...), as ``FastDecoder.descriptor_kinds``
        reports them (``glc_serve/fastdec.py:942-946``)."""
        kinds = {}
        for w in self.linears():
            kind = getattr(w, "kind", type(w).__name__)
            kinds[kind] = kinds.get(kind, 0) + 1
        return kinds

    def streamed_bytes(self) -> int:
        """Weight bytes one step streams from HBM (the reference's ``FastDecoder.streamed_bytes``)."""
        return int(sum(getattr(w, "coded_bytes", 0) for w in self.linears()))


class BatchDecoder:
    """The whole-step engine: static buffers, a paged KV cache, one CUDA graph per (kind, row count).

    Rows of a step: row r is position ``row_pos[r]`` of the sequence in slot ``row_seq[r]`` and carries token
    ``tokens[r]``.  ``kind`` "ar": one row per sequence, and the step ends by feeding every row its own arg-max and
    advancing its position on the device, so consecutive replays need nothing from the host.  ``kind`` "verify": any
    rows (prompt chunks, speculative drafts), no advance."""

    def __init__(self, weights: DecoderWeights, *, max_rows=128, max_slots=128, max_context=2304, device="cuda:0"):
        import torch

        cfg = weights.config
        if cfg.head_dim != ops.HEAD_DIM:
            raise ValueError("the attention kernels are written for head dimension 128")
        self.w, self.cfg, self.dev = weights, cfg, torch.device(device)
        self.max_rows, self.max_slots = int(max_rows), int(max_slots)
        self.pages_per_seq = -(-int(max_context) // PAGE)
        self.max_context = self.pages_per_seq * PAGE
        n_pages = self.max_slots * self.pages_per_seq + 1           # the last page: where padding rows write
        self.scratch_page, self.pad_slot = n_pages - 1, self.max_slots
        bf, i32 = torch.bfloat16, torch.int32
        self.kv = torch.zeros(cfg.layers, 2, n_pages, cfg.local_kv_heads, PAGE, cfg.head_dim, device=self.dev, dtype=bf)
        self.page_table = torch.full((self.max_slots + 1, self.pages_per_seq), self.scratch_page, device=self.dev, dtype=i32)
        self._table_host = np.full((self.max_slots + 1, self.pages_per_seq), -1, dtype=np.int64)
        self._free_pages = list(range(n_pages - 2, -1, -1))
        self._free_slots = list(range(self.max_slots - 1, -1, -1))
        self.cos, self.sin = ops.rope_tables(self.max_context, cfg.rope_theta, self.dev)
        self.attn = ops.PagedAttention(cfg.local_heads, cfg.local_kv_heads, self.max_rows, self.pages_per_seq, self.dev)
        R, H = self.max_rows, cfg.hidden
        z = lambda *shape, dtype=bf: torch.zeros(*shape, device=self.dev, dtype=dtype)
        self.tokens, self.row_seq, self.row_pos = z(R, dtype=i32), torch.full((R,), self.pad_slot, device=self.dev, dtype=i32), z(R, dtype=i32)
        self.h, self.x, self.qkv, self.ctx = z(R, H), z(R, H), z(R, cfg.local_qkv_rows), z(R, cfg.local_heads * cfg.head_dim)
        self.o_out, self.gate_up, self.act, self.down_out = z(R, H), z(R, 2 * cfg.local_ffn), z(R, cfg.local_ffn), z(R, H)
        self.logits, self.next_token = z(R, cfg.vocab), z(R, dtype=i32)
        # Tensor parallelism: O and down are multiplied by this rank's columns only; the partial outputs land in a buffer
        # the peers can reach and are summed over peer memory (georefine_b200.peer), inside the step's CUDA graph.  The sum
        # has the same bits on every rank, so every rank draws the same tokens and the hosts stay in step without
        # talking to each other.  (Constructing the reducer is a collective: every rank builds its decoder.)
        self.peer = None
        if cfg.tp_world > 1:
            from .peer import PeerReducer

            self.peer = PeerReducer({"o": R * H, "down": R * H}, device=self.dev)
        for w in weights.linears():
            if hasattr(w, "reserve"):
                w.reserve(min(self.max_rows, 128))
        self.graphs = {}

    # ---- sequence slots and pages (host bookkeeping; the device sees only the page table) ---------------------
    def open_slot(self) -> int:
        if not self._free_slots:
            raise RuntimeError("no free sequence slot")
        return self._free_slots.pop()

    def close_slot(self, slot: int) -> None:
        for p in range(self.pages_per_seq):
            if self._table_host[slot, p] >= 0:
                self._free_pages.append(int(self._table_host[slot, p]))
                self._table_host[slot, p] = -1
        self.page_table[slot].fill_(self.scratch_page)
        self._free_slots.append(slot)

    def ensure_pages(self, slot: int, upto_position: int) -> None:
        """Gives the slot pages for positions 0..upto_position (host call, before the step that writes them)."""
        if upto_position >= self.max_context:
            raise ValueError(f"position {upto_position} exceeds the context of {self.max_context}")
        for p in range(upto_position // PAGE + 1):
            if self._table_host[slot, p] < 0:
                if not self._free_pages:
                    raise RuntimeError("KV page pool exhausted")
                page = self._free_pages.pop()
                self._table_host[slot, p] = page
                self.page_table[slot, p] = page

    # ---- the step ----------------------------------------------------------------------------------------------
    def _trunk(self, n: int, advance: bool) -> None:
        """One pass of rows 0..n-1 through the stack on the current stream; no allocation, no host synchronisation."""
        import torch

        cfg, w = self.cfg, self.w
        h, x = self.h[:n], self.x[:n]
        torch.index_select(w.embed, 0, self.tokens[:n], out=h)
        delta = None
        for i, layer in enumerate(w.layers):
            ops.rmsnorm(h, layer.norm1, x, delta=delta, eps=cfg.eps)       # (the previous layer's MLP output joins the stream here)
            layer.qkv(x, self.qkv[:n])
            self.attn(self.qkv[:n], self.cos, self.sin, self.row_seq[:n], self.row_pos[:n], self.page_table, self.kv[i, 0], self.kv[i, 1],
                      self.ctx[:n])
            self._row_parallel(layer.o, "o", self.ctx[:n], self.o_out[:n])
            ops.rmsnorm(h, layer.norm2, x, delta=self.o_out[:n], eps=cfg.eps)
            layer.gate_up(x, self.gate_up[:n])
            ops.silu_mul(self.gate_up[:n], self.act[:n])
            self._row_parallel(layer.down, "down", self.act[:n], self.down_out[:n])
            delta = self.down_out[:n]
        ops.rmsnorm(h, w.final_norm, x, delta=delta, eps=cfg.eps)          # h now holds the final residual stream
        w.lm_head(x, self.logits[:n])
        ops.argmax(self.logits[:n], self.next_token[:n])
        if advance:
            self.tokens[:n].copy_(self.next_token[:n])
            self.row_pos[:n].add_(1)

    def _row_parallel(self, linear, slot: str, x, out) -> None:
        """out = linear(x), summed over the ranks when the weight is split by columns."""
        if self.peer is None:
            linear(x, out)
        else:
            linear(x, self.peer.slot(slot, out.shape[0], out.shape[1]))
            self.peer.reduce(slot, out)

    def run(self, kind: str, n: int, *, graph: bool = True) -> None:
        """Runs rows 0..n-1 ("ar" or "verify"); replays the step's CUDA graph, capturing it on first use."""
        import torch

        if kind not in ("ar", "verify") or not 1 <= n <= self.max_rows:
            raise ValueError("kind must be 'ar' or 'verify' and 1 <= n <= max_rows")
        if not graph:
            return self._trunk(n, kind == "ar")
        key = (kind, n)
        if key not in self.graphs:
            saved = self.tokens.clone(), self.row_pos.clone()
            self._trunk(n, kind == "ar")                                   # warm-up outside the capture (lazy initialisation)
            self.tokens.copy_(saved[0]); self.row_pos.copy_(saved[1])
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._trunk(n, kind == "ar")
            self.tokens.copy_(saved[0]); self.row_pos.copy_(saved[1])      # the capture does not run, but keep the state explicit
            self.graphs[key] = g
        self.graphs[key].replay()

    def capture(self, kinds) -> None:
        """Captures the given (kind, rows) steps ahead of time (the reference's ``FastDecoder.capture``)."""
        for kind, n in kinds:
            self.set_rows([self.pad_slot] * n, [0] * n, [0] * n)
            self.run(kind, n)

    def set_rows(self, slots, positions, tokens) -> None:
        """Host -> device: which (slot, position, token) each of the first len(slots) rows carries."""
        import torch

        n = len(slots)
        rows = torch.tensor([list(slots), list(positions), list(tokens)], dtype=torch.int32)
        self.row_seq[:n].copy_(rows[0]); self.row_pos[:n].copy_(rows[1]); self.tokens[:n].copy_(rows[2])

    def streamed_bytes(self, rows_context) -> dict:
        """Bytes one step streams: the compressed weights, and the KV cache of rows whose contexts are given."""
        kv = sum(int(c) for c in rows_context) * self.cfg.local_kv_heads * self.cfg.head_dim * 2 * 2 * self.cfg.layers
        return {"weights": self.w.streamed_bytes(), "kv": kv}


BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128)


def bucket_for(n: int, buckets=BUCKETS) -> int:
    for b in buckets:
        if n <= b:
            return b
    raise ValueError(f"{n} rows exceed the largest bucket")


class Batcher:
    """Continuous batching over a ``BatchDecoder``: sequences are admitted (prompt processed in chunks of rows) and
    retired between steps; a step decodes one token for every active sequence in the smallest row bucket that holds
    them, padding rows parked on a scratch slot (``glc_serve/bidec.py:1103-1264`` is the reference's admission loop)."""

    def __init__(self, decoder: BatchDecoder, *, buckets=BUCKETS):
        self.d, self.buckets = decoder, tuple(b for b in buckets if b <= decoder.max_rows)
        self.active = {}            # slot -> {"pos": position of the next input token, "tokens": generated so far}
        self._order, self._dirty = [], True

    def admit(self, prompt_ids, *, sampler=None) -> int:
        """Processes a prompt and returns the sequence's slot; its first generated token is in ``active[slot]['tokens']``
        (the arg-max of the last position's logits, or a draw from them when a ``sampling.Sampler`` is given)."""
        ids = [int(t) for t in prompt_ids]
        if not ids:
            raise ValueError("empty prompt")
        d = self.d
        self.sync_tokens()                    # the row buffers are about to be reused for the prompt
        slot = d.open_slot()
        d.ensure_pages(slot, len(ids))
        first = None
        for lo in range(0, len(ids), d.max_rows):
            chunk = ids[lo:lo + d.max_rows]
            d.set_rows([slot] * len(chunk), range(lo, lo + len(chunk)), chunk)
            d.run("verify", len(chunk), graph=False)
            first = int(d.next_token[len(chunk) - 1].item())
        if sampler is not None:
            first = int(sampler.draw(d.logits[len(chunk) - 1][None])[0])
        self.active[slot] = {"pos": len(ids), "tokens": [first]}
        self._dirty = True
        return slot

    def retire(self, slot: int) -> None:
        self.sync_tokens()
        self.d.close_slot(slot)
        del self.active[slot]
        self._dirty = True

    def sync_tokens(self) -> None:
        """After steps taken with ``fetch=False``: reads the pending input token of every row back from the device (it is
        the last token the sequence generated) and puts it in the place of the trailing ``None`` of its token list.
        Tokens of earlier unfetched steps stay unknown on the host."""
        rows = [s for s in self._order if s in self.active and self.active[s]["tokens"] and self.active[s]["tokens"][-1] is None]
        if not rows:
            return
        pending = self.d.tokens[:len(self._order)].tolist()
        for i, s in enumerate(self._order):
            if s in self.active and self.active[s]["tokens"][-1] is None:
                self.active[s]["tokens"][-1] = int(pending[i])

    def step(self, *, fetch: bool = True, sampler=None, only=None):
        """One token for every active sequence - or for the sequences in the slots ``only``, the others standing still.
        Returns {slot: token} (``fetch=False``: nothing is read back, the tokens stay on the device and feed the next
        step; ``sync_tokens`` collects them later).  With a ``sampling.Sampler`` the tokens are drawn from the step's
        logits instead of taken as their arg-max.  As long as consecutive steps run the same sequences, nothing but the
        replay of the step's graph happens on the host side."""
        import torch

        d = self.d
        wanted = sorted(self.active) if only is None else sorted({int(s) for s in only})
        if not wanted:
            return {}
        if any(s not in self.active for s in wanted):
            raise KeyError("step asked for a slot that holds no active sequence")
        n = len(wanted)
        b = bucket_for(n, self.buckets)
        for slot in wanted:
            d.ensure_pages(slot, self.active[slot]["pos"])
        if self._dirty or wanted != self._order:
            self.sync_tokens()
            self._order = wanted
            pad = b - n
            d.set_rows(self._order + [d.pad_slot] * pad, [self.active[s]["pos"] for s in self._order] + [0] * pad,
                       [self.active[s]["tokens"][-1] for s in self._order] + [0] * pad)
            self._dirty = False
        d.run("ar", b)
        for s in self._order:
            self.active[s]["pos"] += 1
        if b > n:                                   # padding rows advanced too: park them again
            d.row_pos[n:b].zero_()
        chosen = d.next_token
        if sampler is not None:                     # the step fed every row its arg-max: put the drawn tokens in their place
            chosen = sampler.draw(d.logits[:n]).to(torch.int32)
            d.tokens[:n].copy_(chosen)
        if not fetch:
            for s in self._order:
                self.active[s]["tokens"].append(None)
            return None
        got = chosen[:n].tolist()
        for s, t in zip(self._order, got):
            self.active[s]["tokens"].append(int(t))
        return dict(zip(self._order, got))

    def verify(self, drafts: dict, *, sampler=None):
        """Exact speculation for every sequence in ``drafts`` ({slot: [k draft tokens]}): one pass over k + 1 rows per
        sequence - its pending token, then the drafts - accepts the longest prefix of drafts equal to the target's own
        arg-max rows and emits one more token.  Returns {slot: emitted tokens}; positions are rewound by bookkeeping
        alone (the surplus KV entries are overwritten by the next pass).  With a ``sampling.Sampler`` a draft is kept with
        the probability the target gives it and the first one refused is redrawn (``sampling.accept_drafts``), so the
        emitted tokens are distributed as plain sampling from the target."""
        d = self.d
        self.sync_tokens()
        slots, positions, tokens = [], [], []
        for slot, ds in drafts.items():
            s = self.active[slot]
            d.ensure_pages(slot, s["pos"] + len(ds))
            seq = [s["tokens"][-1]] + [int(t) for t in ds]
            slots += [slot] * len(seq)
            positions += list(range(s["pos"], s["pos"] + len(seq)))
            tokens += seq
        out, at = {}, 0
        if len(slots) > d.max_rows:
            raise ValueError("verify pass larger than the decoder's row buffers")
        d.set_rows(slots, positions, tokens)
        d.run("verify", len(slots))
        argmax_rows = d.next_token[:len(slots)].tolist()
        for slot, ds in drafts.items():
            k = len(ds)
            if sampler is None:
                own = argmax_rows[at:at + k + 1]
                a = 0
                while a < k and int(ds[a]) == own[a]:
                    a += 1
                emitted = [int(t) for t in own[:a + 1]]
            else:
                emitted = sampler.accept(d.logits[at:at + k + 1], [int(t) for t in ds])
            s = self.active[slot]
            s["tokens"] += emitted
            s["pos"] += len(emitted)
            out[slot] = emitted
            at += k + 1
        self._dirty = True
        return out


@dataclass
class State:
    """A live sequence of a ``FastSession``: prompt length, the tokens generated so far, and the logits the prompt's
    last position produced (what a sampled first token is drawn from)."""

    slot: int
    plen: int
    tokens: list
    first_logits: object = None


class FastSession:
    """Sequences driven one at a time through the batched engine (several may be open; a call moves only its own), under
    the reference's session API
    (``glc_serve/fastserve.py``): ``load`` / ``prefill`` / ``generate`` / ``extend`` / ``rollback``.  Greedy decoding at
    temperature 0, else temperature / top-p sampling from a seeded generator.  ``generate(spec_k=k, drafter=...)`` runs
    speculation: ``drafter(state, k)`` proposes k tokens (an MTP head, or any callable); greedy, the verify pass keeps
    what the target itself would have produced, bit for bit the tokens of plain decoding; sampling, it keeps a draft
    with the probability the target gives it, which leaves the distribution of the output that of plain sampling."""

    def __init__(self, decoder: BatchDecoder):
        self.d = decoder
        self.batcher = Batcher(decoder)
        self.mtp_head = None
        self.meta = {"streamed_bytes_per_step": decoder.w.streamed_bytes()}
        if hasattr(decoder.w, "descriptor_kinds"):
            self.meta["descriptors"] = decoder.w.descriptor_kinds()

    @classmethod
    def load(cls, *, package=None, config: DecoderConfig | None = None, weights: DecoderWeights | None = None, device="cuda:0",
             max_len=4096, seed=1, lin_factory=None, tune=None, max_rows=128, **kw) -> "FastSession":
        """A session over ``weights``; or over the decoder of a BCTX ``package`` directory, filled from its frames alone
        (``georefine_b200.checkpoint``; the draft head too, as ``session.mtp_head``, when the package has ``mtp.*``
        tensors; ``cache=image_cache.ImageCache(...)`` keeps the resident images on disk for the next start); or over
        random-init weights of ``config``."""
        source = None
        if weights is None and package is not None:
            from . import checkpoint

            weights = checkpoint.load_decoder_weights(package, device, config=config, lin_factory=lin_factory, tune=tune, **kw)
            source = weights.notes["source"]
        elif weights is None:
            if config is None:
                raise ValueError("package=, weights= or config= required")
            weights = DecoderWeights.synthetic(config, device, seed=seed, lin_factory=lin_factory, tune=tune, **kw)
        session = cls(BatchDecoder(weights, max_rows=max_rows, max_slots=4, max_context=max_len, device=device))
        if source is not None:
            session.meta["receipt"] = weights.notes["receipt"]
            if source.has_mtp and weights.config.tp_world == 1:
                from . import checkpoint

                session.mtp_head = checkpoint.load_mtp_head(source, session.d, lin_factory=lin_factory, cache=kw.get("cache"),
                                                            pool_threads=kw.get("pool_threads"))
        return session

    def prefill(self, *, token_ids) -> State:
        ids = list(token_ids)
        slot = self.batcher.admit(ids)
        last_row = (len(ids) - 1) % self.d.max_rows            # the prompt ran in chunks of max_rows rows
        return State(slot, len(ids), self.batcher.active[slot]["tokens"], self.d.logits[last_row].clone())

    def generate(self, st: State, *, max_tokens: int, stop_ids=(), temperature: float = 0.0, top_p: float = 1.0, seed=None,
                 spec_k: int = 0, drafter=None):
        """Yields up to ``max_tokens`` new tokens (the token the prefill produced counts as the first).  ``temperature``
        > 0 samples (``top_p`` < 1: from the nucleus); ``seed`` makes the draws reproducible, and a tensor-parallel
        decoder needs one, the same on every rank, for the ranks to stay in step."""
        from .sampling import Sampler

        sampler = None
        if temperature > 0:
            if self.d.cfg.tp_world > 1 and seed is None:
                raise ValueError("sampling on a tensor-parallel decoder needs a seed shared by the ranks")
            sampler = Sampler(temperature, top_p, device=self.d.dev, seed=seed)
        stops = {int(t) for t in stop_ids}
        seq = self.batcher.active[st.slot]
        emitted = 0
        if len(seq["tokens"]) == 1 and not getattr(st, "_first_out", False):
            st._first_out = True
            if sampler is not None and st.first_logits is not None:
                seq["tokens"][0] = int(sampler.draw(st.first_logits[None])[0])
                self.batcher._dirty = True
            emitted += 1
            yield seq["tokens"][0]
            if seq["tokens"][0] in stops:
                return
        while emitted < max_tokens:
            if spec_k and drafter is not None:
                new = self.batcher.verify({st.slot: drafter(st, spec_k)}, sampler=sampler)[st.slot]
            else:
                new = [self.batcher.step(sampler=sampler, only=[st.slot])[st.slot]]
            for j, t in enumerate(new):
                emitted += 1
                yield t
                if t in stops or emitted >= max_tokens:
                    surplus = len(new) - j - 1
                    if surplus:
                        self.rollback(st, surplus)
                    return

    def extend(self, st: State, token_ids) -> None:
        """Appends tokens (the next turn): afterwards the engine's next input is the last appended token."""
        ids = [int(t) for t in token_ids]
        if not ids:
            return
        seq, d = self.batcher.active[st.slot], self.d
        feed = [seq["tokens"][-1]] + ids[:-1]
        d.ensure_pages(st.slot, seq["pos"] + len(ids))
        for lo in range(0, len(feed), d.max_rows):
            chunk = feed[lo:lo + d.max_rows]
            d.set_rows([st.slot] * len(chunk), range(seq["pos"] + lo, seq["pos"] + lo + len(chunk)), chunk)
            d.run("verify", len(chunk), graph=False)
        seq["tokens"] += ids
        seq["pos"] += len(ids)
        self.batcher._dirty = True

    def rollback(self, st: State, n: int) -> None:
        """Drops the last n tokens; the state is indexed by position, so nothing else has to be undone."""
        seq = self.batcher.active[st.slot]
        if n <= 0:
            return
        if n >= len(seq["tokens"]):
            raise ValueError("cannot roll back past the prompt")
        del seq["tokens"][-n:]
        seq["pos"] -= n
        self.batcher._dirty = True

    def close(self, st: State) -> None:
        self.batcher.retire(st.slot)


class MTPHead:
    """A multi-token-prediction draft head on top of a ``BatchDecoder``: one extra decoder layer fed by
    ``fc(concat(norm_e(embed(next token)), norm_h(trunk hidden)))``, sharing the trunk's embedding table and output head
    (the wiring of the reference's ``QwenMTP``, ``georefine_context_runtime/bitexact_context_mtp.py:327-400``; shapes in
    ``MTP_SHAPES``: ``fc`` is [hidden, 2 x hidden]).  It keeps a KV cache of its own under the trunk's page table.

    ``absorb`` feeds it (trunk hidden at position p - 1, token at position p) pairs - the prompt, and after every verify
    pass the accepted tokens - and returns its arg-max for the last row of every sequence: the first draft of the next
    cycle.  ``extend_draft`` chains further drafts on the head's own hidden state."""

    def __init__(self, decoder: BatchDecoder, *, fc, norm_e, norm_h, layer: LayerWeights, final_norm):
        import torch

        d, cfg = decoder, decoder.cfg
        if cfg.tp_world != 1:
            raise ValueError("the draft head runs on one GPU: build it over a decoder without tensor parallelism")
        self.d, self.fc, self.norm_e, self.norm_h, self.layer, self.final_norm = d, fc, norm_e, norm_h, layer, final_norm
        bf, R, H = torch.bfloat16, d.max_rows, cfg.hidden
        z = lambda *shape, dtype=bf: torch.zeros(*shape, device=d.dev, dtype=dtype)
        self.kv = torch.zeros(2, d.kv.shape[2], cfg.kv_heads, PAGE, cfg.head_dim, device=d.dev, dtype=bf)
        self.tok, self.hid = z(R, dtype=torch.int32), z(R, H)
        self.e, self.cat, self.z, self.x = z(R, H), z(R, 2 * H), z(R, H), z(R, H)
        self.qkv, self.ctx, self.o_out = z(R, cfg.qkv_rows), z(R, cfg.heads * cfg.head_dim), z(R, H)
        self.gate_up, self.act, self.down_out = z(R, 2 * cfg.ffn), z(R, cfg.ffn), z(R, H)
        self.logits, self.draft = z(R, cfg.vocab), z(R, dtype=torch.int32)
        for w in [fc] + layer.linears():
            if hasattr(w, "reserve"):
                w.reserve(min(R, 128))

    @classmethod
    def synthetic(cls, decoder: BatchDecoder, *, seed=7, lin_factory=None):
        import torch

        cfg, dev = decoder.cfg, decoder.dev
        shapes = dict((n, (r, c)) for n, r, c in cfg.linear_shapes())
        shapes["fc"] = (cfg.hidden, 2 * cfg.hidden)

        def linear(name, i):
            words = synthetic_words(*shapes[name], 7919 * seed + i)
            return lin_factory("mtp." + name, words) if lin_factory else ResidentWeight.from_words(words, dev, max_m=min(decoder.max_rows, 128), verify=False)

        def norm(i):
            g = torch.Generator().manual_seed(104729 * seed + i)
            return (1 + 0.1 * torch.randn(cfg.hidden, generator=g)).to(torch.bfloat16).to(dev)

        layer = LayerWeights(norm(0), linear("qkv", 1), linear("o", 2), norm(1), linear("gate_up", 3), linear("down", 4))
        return cls(decoder, fc=linear("fc", 5), norm_e=norm(2), norm_h=norm(3), layer=layer, final_norm=norm(4))

    def _pass(self, n: int) -> None:
        """Rows 0..n-1: (self.hid, self.tok) at (decoder.row_seq, decoder.row_pos) -> self.z (the head's hidden), self.draft."""
        import torch

        d, cfg, L = self.d, self.d.cfg, self.layer
        H = cfg.hidden
        torch.index_select(d.w.embed, 0, self.tok[:n], out=self.e[:n])
        ops.rmsnorm(self.e[:n], self.norm_e, self.cat[:n, :H], eps=cfg.eps)
        ops.rmsnorm(self.hid[:n], self.norm_h, self.cat[:n, H:], eps=cfg.eps)
        self.fc(self.cat[:n], self.z[:n])
        z, x = self.z[:n], self.x[:n]
        ops.rmsnorm(z, L.norm1, x, eps=cfg.eps)
        L.qkv(x, self.qkv[:n])
        d.attn(self.qkv[:n], d.cos, d.sin, d.row_seq[:n], d.row_pos[:n], d.page_table, self.kv[0], self.kv[1], self.ctx[:n])
        L.o(self.ctx[:n], self.o_out[:n])
        ops.rmsnorm(z, L.norm2, x, delta=self.o_out[:n], eps=cfg.eps)
        L.gate_up(x, self.gate_up[:n])
        ops.silu_mul(self.gate_up[:n], self.act[:n])
        L.down(self.act[:n], self.down_out[:n])
        ops.rmsnorm(z, self.final_norm, x, delta=self.down_out[:n], eps=cfg.eps)
        d.w.lm_head(x, self.logits[:n])
        ops.argmax(self.logits[:n], self.draft[:n])

    def absorb(self, slots, positions, tokens, hidden_rows):
        """``hidden_rows[i]`` = trunk hidden of the position before ``positions[i]``, ``tokens[i]`` = the token at
        ``positions[i]``.  Returns the head's arg-max per row (a prediction of the token at positions[i] + 1)."""
        import torch

        n = len(slots)
        d = self.d
        rows = torch.tensor([list(slots), list(positions), list(tokens)], dtype=torch.int32)
        d.row_seq[:n].copy_(rows[0]); d.row_pos[:n].copy_(rows[1]); self.tok[:n].copy_(rows[2])
        self.hid[:n].copy_(hidden_rows)
        self._pass(n)
        return self.draft[:n].tolist()

    def extend_draft(self, n: int):
        """One more draft per row from the head's own state: hidden = its last output, token = its last draft, one
        position further."""
        d = self.d
        self.hid[:n].copy_(self.z[:n])
        self.tok[:n].copy_(self.draft[:n])
        d.row_pos[:n].add_(1)
        self._pass(n)
        return self.draft[:n].tolist()


class MTPSpeculator:
    """Exact speculation with an ``MTPHead`` as the drafter, for the sequences of a ``Batcher`` (the batched form of the
    reference's ``FastSession._spec_cycle``, ``glc_serve/fastserve.py:308-350``): per cycle k drafts per sequence, one
    verify pass over (k + 1) rows per sequence, the accepted tokens confirmed into the head.  What reaches the output is
    always the target's own arg-max, so the tokens equal plain greedy decoding whatever the head proposes."""

    def __init__(self, batcher: Batcher, head: MTPHead, k: int = 5):
        self.b, self.head, self.k = batcher, head, int(k)
        self.first = {}     # slot -> the head's pending first draft
        self.hidden = {}    # slot -> the head's own hidden state behind that draft (input of the second draft)
        self.stats = {"cycles": 0, "drafts_accepted": 0, "emitted": 0}     # per sequence and cycle (fastdec.py:930-940)

    @property
    def mean_tokens_per_cycle(self):
        """Tokens emitted per sequence and cycle so far (1 = no draft ever accepted, k + 1 = all of them)."""
        return self.stats["emitted"] / self.stats["cycles"] if self.stats["cycles"] else None

    def admit(self, prompt_ids, *, sampler=None) -> int:
        """Admits a sequence and runs the head over its prompt (trunk hidden of position p - 1 with token p).  ``sampler``:
        the first token is drawn from the prompt's last logits instead of being their arg-max."""
        import torch

        ids = [int(t) for t in prompt_ids]
        d = self.b.d
        slot = d.open_slot()
        d.ensure_pages(slot, len(ids) + self.k + 1)
        pending_hidden, first = None, None
        for lo in range(0, len(ids), d.max_rows):
            chunk = ids[lo:lo + d.max_rows]
            d.set_rows([slot] * len(chunk), range(lo, lo + len(chunk)), chunk)
            d.run("verify", len(chunk), graph=False)
            first = int(d.next_token[len(chunk) - 1].item())
            if sampler is not None and lo + len(chunk) == len(ids):
                first = int(sampler.draw(d.logits[len(chunk) - 1][None])[0])
            hidden = d.h[:len(chunk)].clone()
            # pairs (hidden of p - 1, token p): inside the chunk, plus the pair that straddles the chunk boundary
            pos = list(range(lo + 1, lo + len(chunk)))
            toks, hid = chunk[1:], hidden[:-1]
            if pending_hidden is not None:
                pos, toks, hid = [lo] + pos, [chunk[0]] + toks, torch.cat([pending_hidden, hid])
            if pos:
                self.head.absorb([slot] * len(pos), pos, toks, hid)
            pending_hidden = hidden[-1:].clone()
        self.b.active[slot] = {"pos": len(ids), "tokens": [first]}
        self.first[slot] = self.head.absorb([slot], [len(ids)], [first], pending_hidden)[0]
        self.hidden[slot] = self.head.z[:1].clone()
        self.b._dirty = True
        return slot

    def cycle(self, *, sampler=None):
        """One speculation cycle for every active sequence.  Returns {slot: emitted tokens}.  ``sampler``: see
        ``Batcher.verify``."""
        import torch

        b, d, head, k = self.b, self.b.d, self.head, self.k
        order = sorted(b.active)
        n = len(order)
        for s in order:
            d.ensure_pages(s, b.active[s]["pos"] + k + 1)
        # drafts 2..k chained on the head's own state, starting from the rows of the pending first drafts
        drafts = {s: [self.first[s]] for s in order}
        if k > 1:
            rows = torch.tensor([order, [b.active[s]["pos"] + 1 for s in order], [self.first[s] for s in order]], dtype=torch.int32)
            d.row_seq[:n].copy_(rows[0]); d.row_pos[:n].copy_(rows[1]); head.tok[:n].copy_(rows[2])
            head.hid[:n].copy_(torch.cat([self.hidden[s] for s in order]))
            head._pass(n)
            step = head.draft[:n].tolist()
            for j in range(1, k):
                for s, t in zip(order, step):
                    drafts[s].append(int(t))
                if j + 1 < k:
                    step = head.extend_draft(n)
        start = {s: b.active[s]["pos"] for s in order}
        out = b.verify(drafts, sampler=sampler)
        # confirm: the head sees the accepted tokens with the trunk's hidden states of the verify pass
        slots, positions, tokens, picks, at = [], [], [], [], 0
        for s in order:
            a1 = len(out[s])                       # accepted drafts + the bonus token
            for j in range(a1):
                slots.append(s); positions.append(start[s] + 1 + j); tokens.append(out[s][j]); picks.append(at + j)
            at += len(drafts[s]) + 1
        hidden = d.h[torch.tensor(picks, device=d.dev)]
        got = head.absorb(slots, positions, tokens, hidden)
        at = 0
        for s in order:
            at += len(out[s])
            self.first[s] = got[at - 1]
            self.hidden[s] = head.z[at - 1:at].clone()
            self.stats["cycles"] += 1
            self.stats["emitted"] += len(out[s])
            self.stats["drafts_accepted"] += len(out[s]) - 1
        return out

    def retire(self, slot: int) -> None:
        self.b.retire(slot)
        self.first.pop(slot, None)
        self.hidden.pop(slot, None)
