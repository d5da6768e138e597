"""The analytic backward sweeps against numerical differentiation (central
differences in float64) -- independent of the oracle: every autograd Function of
the package is checked on small shapes with non-trivial boundaries, for the three
recursion types where they apply.

torch.autograd.gradcheck itself cannot be used: it runs backward twice on one
graph, and the mutual-information Function rescales its saved occupancies in
place on every backward, exactly as the reference's does
(fast_rnnt/python/fast_rnnt/mutual_information.py:176-181).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def fr():
    import fast_rnnt_b200
    return fast_rnnt_b200


def _inputs(rnnt_type, seed, B=2, S=4, T=6, C=5):
    g = torch.Generator().manual_seed(seed)
    symbols = torch.randint(1, C, (B, S), generator=g)
    if rnnt_type == "regular":
        rows = [[0, 0, S, T], [0, 0, S - 1, T - 2]]
    else:  # the modified recursions need T_b >= S_b
        rows = [[0, 0, S, T], [0, 0, S - 2, T - 1]]
    boundary = torch.tensor(rows[:B], dtype=torch.int64)
    return g, symbols.cuda(), boundary.cuda()


def _check(fn, inputs, eps=1e-6, atol=2e-6, rtol=1e-5):
    """d/dx of sum_b w_b * fn(x)[b] (fixed weights w): one backward against central
    differences over every entry of every input, a fresh forward per evaluation."""
    out = fn(*inputs)
    w = torch.linspace(0.5, 1.5, out.numel(), dtype=out.dtype, device=out.device).reshape(out.shape)
    analytic = torch.autograd.grad((out * w).sum(), inputs)
    for x, ga in zip(inputs, analytic):
        flat = x.detach().reshape(-1)
        numeric = torch.empty_like(flat)
        for i in range(flat.numel()):
            keep = flat[i].item()
            with torch.no_grad():
                flat[i] = keep + eps
                up = (fn(*inputs) * w).sum().item()
                flat[i] = keep - eps
                down = (fn(*inputs) * w).sum().item()
                flat[i] = keep
            numeric[i] = (up - down) / (2 * eps)
        torch.testing.assert_close(ga.reshape(-1), numeric, atol=atol, rtol=rtol)


@pytest.mark.parametrize("modified", [False, True])
def test_mutual_information_recursion(modified):
    g = torch.Generator().manual_seed(3)
    B, S, T = 2, 4, 6
    px = (torch.rand(B, S, T + (0 if modified else 1), generator=g, dtype=torch.float64) * -3).cuda()
    py = (torch.rand(B, S + 1, T, generator=g, dtype=torch.float64) * -3).cuda()
    boundary = torch.tensor([[0, 0, S, T], [1, 1, S - 1, T - 1]], dtype=torch.int64).cuda()
    px.requires_grad_(True)
    py.requires_grad_(True)
    _check(lambda a, b: fr().mutual_information_recursion(a, b, boundary), (px, py))
    _check(lambda a, b: fr().mutual_information_recursion(a, b, None), (px, py))


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
@pytest.mark.parametrize("smoothed", [False, True])
def test_simple_losses(rnnt_type, smoothed):
    g, symbols, boundary = _inputs(rnnt_type, 11)
    B, S = symbols.shape
    T, C = 6, 5
    lm = torch.randn(B, S + 1, C, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    am = torch.randn(B, T, C, generator=g, dtype=torch.float64).cuda().requires_grad_(True)

    def loss(lm_, am_):
        if smoothed:
            return fr().rnnt_loss_smoothed(lm=lm_, am=am_, symbols=symbols, termination_symbol=0,
                                           lm_only_scale=0.25, am_only_scale=0.15, boundary=boundary,
                                           rnnt_type=rnnt_type, delay_penalty=0.1, reduction="none")
        return fr().rnnt_loss_simple(lm=lm_, am=am_, symbols=symbols, termination_symbol=0,
                                     boundary=boundary, rnnt_type=rnnt_type, delay_penalty=0.1,
                                     reduction="none")

    _check(loss, (lm, am))


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_unpruned_loss(rnnt_type):
    g, symbols, boundary = _inputs(rnnt_type, 17)
    B, S = symbols.shape
    T, C = 6, 5
    logits = torch.randn(B, T, S + 1, C, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    _check(lambda x: fr().rnnt_loss(logits=x, symbols=symbols, termination_symbol=0, boundary=boundary,
                                    rnnt_type=rnnt_type, reduction="none"), (logits,))


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_pruned_loss_and_pruning(rnnt_type):
    g, symbols, boundary = _inputs(rnnt_type, 23)
    B, S = symbols.shape
    T, C, R, D = 6, 5, 3, 4
    start = torch.sort(torch.randint(0, S + 2 - R, (B, T), generator=g), dim=1)[0]
    ranges = (start.unsqueeze(-1) + torch.arange(R)).cuda()
    logits = torch.randn(B, T, R, C, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    _check(lambda x: fr().rnnt_loss_pruned(logits=x, symbols=symbols, ranges=ranges, termination_symbol=0,
                                           boundary=boundary, rnnt_type=rnnt_type, reduction="none"),
           (logits,))
    enc = torch.randn(B, T, D, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    dec = torch.randn(B, S + 1, D, generator=g, dtype=torch.float64).cuda().requires_grad_(True)

    def pruned_sum(a, l):
        a_p, l_p = fr().do_rnnt_pruning(am=a, lm=l, ranges=ranges)
        return (a_p * l_p).sum(-1)

    _check(pruned_sum, (enc, dec))
