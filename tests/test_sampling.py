"""Temperature / nucleus sampling and speculative acceptance (georefine_b200/sampling.py), on the CPU.

The session-level behaviour they mirror is the reference's ``FastSession._probs`` / ``_sample`` / the sampling branch of
``_spec_cycle`` (glc_serve/fastserve.py:308-395): the nucleus keeps a token while the mass ranked above it does not exceed
top_p; a draft is kept with the target's probability of it and the first refusal is redrawn without it.
"""
import numpy as np
import pytest
import torch

from georefine_b200 import sampling


def test_probabilities_are_a_tempered_softmax():
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(3, 50, generator=g).to(torch.bfloat16)
    for t in (0.5, 1.0, 2.0):
        p = sampling.probabilities(logits, t)
        want = torch.softmax(logits.double() / t, dim=-1)
        assert p.dtype == torch.float32
        assert torch.allclose(p.double(), want, atol=1e-6)
        assert torch.allclose(p.sum(-1), torch.ones(3), atol=1e-5)


def test_nucleus_keeps_the_smallest_head_that_reaches_top_p():
    p_in = torch.tensor([[0.5, 0.25, 0.15, 0.07, 0.03]])
    logits = p_in.log()
    # 0.5 + 0.25 = 0.75 < 0.8, so the third token (mass above it 0.75 <= 0.8) is still kept; the fourth (0.9 above) is not
    p = sampling.probabilities(logits, 1.0, 0.8)
    assert torch.allclose(p, torch.tensor([[0.5, 0.25, 0.15, 0.0, 0.0]]) / 0.9, atol=1e-6)
    # the first token is always kept, however small top_p is
    p = sampling.probabilities(logits, 1.0, 1e-9)
    assert p.tolist() == [[1.0, 0.0, 0.0, 0.0, 0.0]]
    # rows are filtered independently, and the order of the tokens does not matter
    perm = torch.tensor([3, 0, 4, 2, 1])
    p = sampling.probabilities(torch.cat([logits, logits[:, perm]]), 1.0, 0.8)
    assert torch.allclose(p[1], p[0][perm])


def test_ties_rank_by_token_id_like_the_argmax_kernel():
    logits = torch.tensor([[1.0, 3.0, 3.0, 0.0, 3.0]])
    p = sampling.probabilities(logits, 1.0, 1e-6)
    assert p.argmax().item() == 1 and p[0, 1] == 1.0 and p.sum() == 1.0


def test_arguments_are_checked():
    x = torch.zeros(1, 4)
    for t, tp in ((0.0, 1.0), (-1.0, 1.0), (1.0, 0.0), (1.0, 1.5)):
        with pytest.raises(ValueError):
            sampling.probabilities(x, t, tp)
    with pytest.raises(ValueError):
        sampling.Sampler(0.0)
    with pytest.raises(ValueError):
        sampling.accept_drafts(torch.full((2, 4), 0.25), [1, 2, 3])


def test_draws_are_reproducible_and_follow_the_distribution():
    p = torch.tensor([[0.1, 0.2, 0.3, 0.4]]).repeat(20000, 1)
    a = sampling.draw(p, sampling.make_generator("cpu", 11))
    b = sampling.draw(p, sampling.make_generator("cpu", 11))
    c = sampling.draw(p, sampling.make_generator("cpu", 12))
    assert torch.equal(a, b) and not torch.equal(a, c)
    freq = torch.bincount(a, minlength=4).double() / len(a)
    assert torch.allclose(freq, p[0].double(), atol=0.015)


def test_sure_drafts_are_all_kept_and_impossible_ones_never():
    k, vocab = 4, 6
    drafts = [2, 0, 5, 1]
    p = torch.zeros(k + 1, vocab)
    for i, d in enumerate(drafts):
        p[i, d] = 1.0
    p[k] = torch.tensor([0.0, 0.0, 0.0, 1.0, 0.0, 0.0])
    assert sampling.accept_drafts(p, drafts, sampling.make_generator("cpu", 1)) == drafts + [3]
    # the target gives the second draft no mass: one kept, then a token that is not the draft, nothing after it
    p[1] = torch.tensor([0.0, 0.5, 0.0, 0.0, 0.5, 0.0])
    for seed in range(20):
        out = sampling.accept_drafts(p, drafts, sampling.make_generator("cpu", seed))
        assert len(out) == 2 and out[0] == 2 and out[1] in (1, 4)
    # no drafts: one plain draw
    out = sampling.accept_drafts(p[k:], [], sampling.make_generator("cpu", 3))
    assert out == [3]


def test_speculative_sampling_leaves_the_target_distribution_alone():
    """Whatever the drafter proposes, the first emitted token is distributed as p[0], and the second - given that the
    first draft was kept - as p[1]."""
    g = torch.Generator().manual_seed(3)
    vocab, k, trials = 5, 2, 30000
    p = torch.softmax(torch.randn(k + 1, vocab, generator=g), dim=-1)
    drafts = [int(p[0].argmin()), int(p[1].argmax())]           # a poor first guess, a good second one
    gen = sampling.make_generator("cpu", 99)
    first = np.zeros(vocab)
    second = np.zeros(vocab)
    lengths = np.zeros(k + 2)
    for _ in range(trials):
        out = sampling.accept_drafts(p, drafts, gen)
        lengths[len(out)] += 1
        first[out[0]] += 1
        if len(out) > 1:
            assert out[0] == drafts[0]
            second[out[1]] += 1
    assert np.allclose(first / trials, p[0].numpy(), atol=0.012)
    assert np.allclose(second / second.sum(), p[1].numpy(), atol=0.04)
    # P(keep the first draft) = p[0, d0]; P(all kept) = p[0, d0] * p[1, d1]
    keep0 = float(p[0, drafts[0]])
    assert abs((lengths[2] + lengths[3]) / trials - keep0) < 0.01
    assert abs(lengths[3] / trials - keep0 * float(p[1, drafts[1]])) < 0.01


def test_sampler_binds_temperature_nucleus_and_generator():
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0]] * 3)
    s1, s2 = sampling.Sampler(0.7, 0.9, seed=4), sampling.Sampler(0.7, 0.9, seed=4)
    assert torch.equal(s1.draw(logits), s2.draw(logits))
    assert torch.allclose(s1.probabilities(logits), sampling.probabilities(logits, 0.7, 0.9))
    assert s1.accept(logits, [3, 3]) == s2.accept(logits, [3, 3])
    greedy = sampling.Sampler(1.0, 1e-9, seed=0)
    assert greedy.draw(logits).tolist() == [3, 3, 3]
    assert greedy.accept(logits, [3, 3]) == [3, 3, 3]
    assert greedy.accept(logits, [3, 1]) == [3, 3]
