"""Sampling semantics on CPU: top-k and top-p are sequential filters (top-k first, nucleus on the distribution
renormalised over the survivors), checked against a step-by-step transcription of the reference's algorithm
(batchgen/sampling.py:417-461: sort, rank mask, softmax of the masked logits, shifted cumulative mask)."""
import torch

from batchgen_b200.ops import ref


def _sequential_keep(logits, temp, top_k, top_p):
    """Set of tokens that survive: mask to top-k on the scaled logits, then the nucleus of the softmax over
    the survivors, where the token that crosses the threshold stays and the best token always stays."""
    V = logits.numel()
    x = logits.double() / temp
    order = torch.argsort(x, descending=True, stable=True)
    k = V if top_k <= 0 else min(top_k, V)
    x_sorted = x[order].clone()
    x_sorted[k:] = float("-inf")
    keep_sorted = torch.isfinite(x_sorted)
    if top_p < 1.0:
        cum = torch.softmax(x_sorted, -1).cumsum(-1)
        mask = cum > top_p
        mask[1:] = mask[:-1].clone()
        mask[0] = False
        keep_sorted &= ~mask
    return set(order[keep_sorted].tolist())


def test_topk_then_topp_example():
    # p = [.3, .2, .1 x 5], k = 2, top_p = .5: after top-k the survivors renormalise to (.6, .4); the mass before
    # token 1 is .6 > .5, so only token 0 remains.  Taking the nucleus on the full distribution would keep both.
    p = torch.tensor([0.3, 0.2, 0.1, 0.1, 0.1, 0.1, 0.1])
    logits = p.log().unsqueeze(0).repeat(64, 1)
    u = torch.linspace(0, 0.999, 64)
    tok = ref.sample(logits, torch.ones(64), torch.full((64,), 2), torch.full((64,), 0.5), uniform=u)
    assert set(tok.tolist()) == {0}
    assert _sequential_keep(p.log(), 1.0, 2, 0.5) == {0}


def test_kept_set_matches_sequential_transcription():
    g = torch.Generator().manual_seed(5)
    V, N = 40, 400
    for trial in range(12):
        logits = torch.randn(V, generator=g) * 2.0
        temp = float(torch.rand(1, generator=g)) * 1.5 + 0.2
        top_k = [0, 3, 7, 15][trial % 4]
        top_p = [1.0, 0.9, 0.6, 0.3][(trial // 4) % 4 if trial < 12 else 0]
        want = _sequential_keep(logits, temp, top_k, top_p)
        u = (torch.arange(N) + 0.5) / N
        tok = ref.sample(logits.unsqueeze(0).repeat(N, 1), torch.full((N,), temp), torch.full((N,), top_k),
                         torch.full((N,), top_p), uniform=u)
        got = set(tok.tolist())
        assert got <= want, (trial, got - want)
        # every survivor with a visible share of the kept mass must be drawn by a dense uniform grid
        probs = torch.softmax(logits.double() / temp, -1)
        mass = sum(float(probs[i]) for i in want)
        for i in want:
            if float(probs[i]) / mass > 2.5 / N:
                assert i in got, (trial, i)
