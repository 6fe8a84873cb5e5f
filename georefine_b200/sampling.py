"""Token sampling for the decode engine: temperature, nucleus (top-p) filtering, and speculative sampling against a
drafter that proposes one definite token per position.

Host-side torch arithmetic over the logits a step leaves on the device - plumbing beside the path, as in the reference's
session (``glc_serve/fastserve.py:308-395``: ``_probs``, ``_sample`` and the sampling branch of ``_spec_cycle``).  Every
function works on any device and takes the ``torch.Generator`` the caller seeded, so a run is reproducible and the ranks
of a tensor-parallel decoder, seeded alike and holding the same logits, draw the same tokens.
"""
from __future__ import annotations


def _check(temperature: float, top_p: float) -> None:
    if not temperature > 0:
        raise ValueError("temperature must be positive; temperature 0 is the arg-max path")
    if not 0 < top_p <= 1:
        raise ValueError("top_p must be in (0, 1]")


def probabilities(logits, temperature: float, top_p: float = 1.0):
    """Rows of logits -> rows of FP32 probabilities at ``temperature`` > 0, restricted to the nucleus when ``top_p`` < 1:
    the tokens in descending order of probability up to and including the one that brings the running mass to ``top_p``
    (a token is dropped when the mass of the tokens ranked above it already exceeds ``top_p``; the first is always kept),
    renormalised.  Equal probabilities rank by token id, lowest first, which is also how the arg-max kernel breaks ties."""
    import torch

    _check(temperature, top_p)
    p = torch.softmax(logits.float() / float(temperature), dim=-1)
    if top_p < 1.0:
        ranked, order = torch.sort(p, dim=-1, descending=True, stable=True)
        above = torch.cumsum(ranked, dim=-1) - ranked            # mass of the tokens ranked before this one
        ranked = torch.where(above > top_p, torch.zeros_like(ranked), ranked)
        p = torch.zeros_like(p).scatter_(-1, order, ranked)
        p = p / p.sum(dim=-1, keepdim=True)
    return p


def draw(p, generator=None):
    """One token id per row of probabilities (int64 tensor on p's device)."""
    import torch

    return torch.multinomial(p, 1, generator=generator).reshape(-1)


def accept_drafts(p, drafts, generator=None):
    """Speculative sampling for one sequence.  ``p``: k + 1 rows of target probabilities - row i is the distribution of
    the token after the first i drafts; ``drafts``: the k tokens a deterministic drafter proposed.  Draft i is kept with
    probability p[i, draft]; the first one refused is replaced by a draw from p[i] with that token struck out, and
    nothing behind it is used; if all k are kept, one more token is drawn from row k.  Each emitted token is then
    distributed exactly as if it had been drawn from the target alone: P(t) = p[d]*[t = d] + (1 - p[d]) * p[t] / (1 - p[d])
    for t != d.  Returns the emitted tokens (1 to k + 1 of them)."""
    import torch

    k = len(drafts)
    if p.shape[0] != k + 1:
        raise ValueError("one row of probabilities per draft, and one more")
    u = torch.rand(k + 1, generator=generator, device=p.device).tolist()
    kept = p[torch.arange(k, device=p.device), torch.as_tensor(list(drafts), device=p.device, dtype=torch.long)].tolist() if k else []
    out = []
    for i, d in enumerate(drafts):
        if u[i] < kept[i]:
            out.append(int(d))
            continue
        rest = p[i].clone()
        rest[int(d)] = 0
        mass = float(rest.sum())
        out.append(int(draw((rest / mass)[None], generator)[0]) if mass > 0 else int(d))
        return out
    out.append(int(draw(p[k][None], generator)[0]))
    return out


class Sampler:
    """Temperature, nucleus and generator of one generation call, as the engine passes them around."""

    def __init__(self, temperature: float, top_p: float = 1.0, *, device="cpu", seed=None):
        self.temperature, self.top_p = float(temperature), float(top_p)
        _check(self.temperature, self.top_p)
        self.generator = make_generator(device, seed)

    def probabilities(self, logits):
        return probabilities(logits, self.temperature, self.top_p)

    def draw(self, logits):
        """One token per row of logits."""
        return draw(self.probabilities(logits), self.generator)

    def accept(self, logits, drafts):
        """``logits``: len(drafts) + 1 rows of one sequence's verify pass."""
        return accept_drafts(self.probabilities(logits), drafts, self.generator)


def make_generator(device, seed=None):
    """A generator on ``device``; seeded when a seed is given, else from the system's entropy."""
    import torch

    g = torch.Generator(device=device)
    if seed is None:
        g.seed()
    else:
        g.manual_seed(int(seed))
    return g
