"""The decode-step kernels around the fused linears against plain torch FP32 arithmetic (needs a B200).

RMSNorm with the residual add, SwiGLU, arg-max and paged decode attention (rotary embedding + KV append + 256-position
splits merged in split order).  Each kernel must agree with the FP32 restatement within BF16 rounding, and a row's
result must not depend on which other rows share the call.  The contracts are those of the reference's step kernels
(glc_serve/fastdec_kernels.cu:83-110, 324-488).
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


def _bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy()


@pytest.mark.parametrize("hidden", [5120, 1024, 8, 16384])
@pytest.mark.parametrize("unit_offset", [False, True])
def test_rmsnorm_with_residual(dev, hidden, unit_offset):
    from georefine_b200 import ops

    g = torch.Generator().manual_seed(hidden)
    h = torch.randn(37, hidden, generator=g).to(torch.bfloat16).to(dev)
    delta = torch.randn(37, hidden, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(hidden, generator=g) * 0.2 + (0 if unit_offset else 1)).to(torch.bfloat16).to(dev)
    summed = (h.float() + delta.float()).to(torch.bfloat16)
    scale = (1 + w.float()) if unit_offset else w.float()
    want = (summed.float() * torch.rsqrt(summed.float().pow(2).mean(-1, keepdim=True) + 1e-6) * scale)
    out = torch.empty_like(h)
    h2 = h.clone()
    ops.rmsnorm(h2, w, out, delta=delta, eps=1e-6, unit_offset=unit_offset)
    assert np.array_equal(_bits(h2), _bits(summed))                       # the residual add is exact BF16 arithmetic
    assert (out.float() - want).abs().max().item() <= 2 ** -7 * want.abs().max().item()
    # a row does not depend on its neighbours, and the plain form (no residual) agrees on the same input
    solo = torch.empty(1, hidden, device=dev, dtype=torch.bfloat16)
    h3 = h[5:6].clone()
    ops.rmsnorm(h3, w, solo, delta=delta[5:6], unit_offset=unit_offset)
    assert np.array_equal(_bits(solo), _bits(out[5:6]))
    plain = torch.empty_like(h)
    ops.rmsnorm(summed.clone(), w, plain, unit_offset=unit_offset)
    assert np.array_equal(_bits(plain), _bits(out))


def test_silu_mul_and_argmax(dev):
    from georefine_b200 import ops

    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(19, 2 * 17408, generator=g) * 3).to(torch.bfloat16).to(dev)
    out = torch.empty(19, 17408, device=dev, dtype=torch.bfloat16)
    ops.silu_mul(gu, out)
    gate, up = gu[:, :17408].float(), gu[:, 17408:].float()
    want = ((gate / (1 + torch.exp(-gate))).to(torch.bfloat16).float() * up)
    assert (out.float() - want).abs().max().item() <= 2 ** -7 * want.abs().max().item()
    assert float((out.float() - want.to(torch.bfloat16).float()).ne(0).float().mean()) < 0.02   # a different exp: rare last-bit flips only
    logits = torch.randn(33, 152064, generator=g).to(torch.bfloat16).to(dev)
    logits[4, 777] = logits[4, 150000] = 99.0                             # a tie: the first index wins
    logits[7, 152063] = 98.0                                              # the last column
    best = torch.empty(33, device=dev, dtype=torch.int32)
    ops.argmax(logits, best)
    want_idx = torch.argmax(logits.float(), dim=1)
    want_idx[4] = 777
    assert torch.equal(best.long(), want_idx) and int(best[7]) == 152063
    ragged = logits[:, :1003]                                             # a vocabulary that is no multiple of 8, strided rows
    ops.argmax(ragged, best)
    for r in range(33):
        row = ragged[r].float()
        assert int(best[r]) == int((row == row.max()).nonzero()[0])


def _reference_attention(qkv, cos, sin, row_seq, row_pos, k_cache, v_cache, nq, nkv):
    """FP32 restatement over plain per-sequence caches [slot][position][kv head][128]; appends first, then attends."""
    rows = qkv.shape[0]
    d = 128
    q = qkv[:, :nq * d].reshape(rows, nq, d).float()
    k = qkv[:, nq * d:(nq + nkv) * d].reshape(rows, nkv, d).float()
    v = qkv[:, (nq + nkv) * d:].reshape(rows, nkv, d)

    def rope(x, pos):
        c, s = cos[pos].float()[:, None, :], sin[pos].float()[:, None, :]
        rot = torch.cat([-x[..., d // 2:], x[..., :d // 2]], dim=-1)
        return ((x * c).to(torch.bfloat16).float() + (rot * s).to(torch.bfloat16).float()).to(torch.bfloat16)

    pos = row_pos.long()
    q, k = rope(q, pos), rope(k, pos)
    for r in range(rows):
        k_cache[row_seq[r], pos[r]] = k[r]
        v_cache[row_seq[r], pos[r]] = v[r]
    out = torch.empty(rows, nq * d, dtype=torch.bfloat16, device=qkv.device)
    for r in range(rows):
        n = int(pos[r]) + 1
        kk = k_cache[row_seq[r], :n].float().repeat_interleave(nq // nkv, dim=1)      # [n, nq, d]
        vv = v_cache[row_seq[r], :n].float().repeat_interleave(nq // nkv, dim=1)
        score = torch.einsum("hd,nhd->hn", q[r].float(), kk) / math.sqrt(d)
        out[r] = torch.einsum("hn,nhd->hd", torch.softmax(score, dim=-1), vv).reshape(-1).to(torch.bfloat16)
    return out


@pytest.mark.parametrize("nq,nkv", [(40, 8), (4, 2), (8, 8), (8, 1)])
def test_paged_attention_step(dev, nq, nkv):
    from georefine_b200 import ops

    g = torch.Generator().manual_seed(nq * 10 + nkv)
    slots, max_pages = 5, 4
    lengths = [0, 255, 256, 700, 513]                     # tokens already cached per sequence slot
    cos, sin = ops.rope_tables(max_pages * ops.PAGE, device=dev)
    pages = torch.randperm(slots * max_pages, generator=g).reshape(slots, max_pages).to(torch.int32).to(dev)   # scattered pages
    k_pages = torch.zeros(slots * max_pages, nkv, ops.PAGE, 128, device=dev, dtype=torch.bfloat16)
    v_pages = torch.zeros_like(k_pages)
    k_ref = torch.zeros(slots, max_pages * ops.PAGE, nkv, 128, device=dev, dtype=torch.bfloat16)
    v_ref = torch.zeros_like(k_ref)
    attn = ops.PagedAttention(nq, nkv, max_rows=64, max_pages=max_pages, device=dev)
    width = (nq + 2 * nkv) * 128

    def run(row_seq, row_pos):
        rows = len(row_seq)
        qkv = torch.randn(rows, width, generator=g).to(torch.bfloat16).to(dev)
        rs, rp = torch.tensor(row_seq, dtype=torch.int32, device=dev), torch.tensor(row_pos, dtype=torch.int32, device=dev)
        out = torch.full((rows, nq * 128), float("nan"), device=dev, dtype=torch.bfloat16)
        attn(qkv, cos, sin, rs, rp, pages, k_pages, v_pages, out)
        want = _reference_attention(qkv, cos, sin, rs.cpu().tolist(), rp.cpu(), k_ref, v_ref, nq, nkv)
        assert not torch.isnan(out.float()).any()
        assert (out.float() - want.float()).abs().max().item() <= 2e-2 * want.float().abs().max().item()
        return qkv, rs, rp, out

    # fill the caches: every sequence's history, in chunks of rows at consecutive positions (a prompt chunk)
    for slot, n in enumerate(lengths):
        for lo in range(0, n, 48):
            hi = min(n, lo + 48)
            run([slot] * (hi - lo), list(range(lo, hi)))
    # the cache pages hold what the restatement holds (keys rotated, values verbatim)
    for slot, n in enumerate(lengths):
        for p in range(0, n, 97):
            page = int(pages[slot, p // ops.PAGE])
            assert torch.equal(k_pages[page, :, p % ops.PAGE], k_ref[slot, p]) and torch.equal(v_pages[page, :, p % ops.PAGE], v_ref[slot, p])
    # one decode step for all sequences at once, then a speculative-verify shaped step: 3 rows per sequence
    qkv, rs, rp, out = run(list(range(slots)), lengths)
    lengths = [n + 1 for n in lengths]
    run([s for s in range(slots) for _ in range(3)], [lengths[s] + j for s in range(slots) for j in range(3)])
    # batch invariance: a row computed alone gives the same bits as inside the batch (appends are idempotent)
    solo = torch.empty(1, nq * 128, device=dev, dtype=torch.bfloat16)
    attn(qkv[3:4], cos, sin, rs[3:4], rp[3:4], pages, k_pages, v_pages, solo)
    assert np.array_equal(_bits(solo), _bits(out[3:4]))
