"""The delay penalty of the loss functions (reference rnnt_loss.py:309-324 and its three
copies) is added to px by the kernels that write the lattices.  Every loss with
delay_penalty > 0 must equal, bit for bit, the same lattices from the public
get_rnnt_logprobs* function plus the reference's torch expression for the penalty, run
through the same recursion."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference_penalty(px, boundary, rnnt_type, delay_penalty):
    """The reference's lines, verbatim in meaning (rnnt_loss.py:309-324)."""
    B, S, T0 = px.shape
    T = T0 if rnnt_type != "regular" else T0 - 1
    if boundary is None:
        offset = torch.tensor((T - 1) / 2, dtype=px.dtype, device=px.device).expand(B, 1, 1)
    else:
        offset = (boundary[:, 3] - 1) / 2
    penalty = offset.reshape(B, 1, 1) - torch.arange(T0, device=px.device).reshape(1, 1, T0)
    penalty = penalty * delay_penalty
    return px + penalty.to(px.dtype)


def make(B, S, T, C, dtype, with_boundary, rnnt_type, seed):
    g = torch.Generator().manual_seed(seed)
    lm = torch.randn(B, S + 1, C, generator=g, dtype=dtype).cuda()
    am = torch.randn(B, T, C, generator=g, dtype=dtype).cuda()
    symbols = torch.randint(1, C, (B, S), generator=g).cuda()
    boundary = None
    if with_boundary:
        Sb = torch.randint(max(1, S // 2), S + 1, (B,), generator=g)
        Tb = torch.randint(max(S, T // 2), T + 1, (B,), generator=g)
        z = torch.zeros(B, dtype=torch.int64)
        boundary = torch.stack([z, z, Sb, Tb], dim=1).cuda()
    return lm, am, symbols, boundary


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("with_boundary", [False, True])
@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
@pytest.mark.parametrize("smoothed", [False, True])
def test_simple_losses(dtype, with_boundary, rnnt_type, smoothed):
    import fast_rnnt_b200 as fr
    dp = 0.0123
    lm, am, symbols, boundary = make(3, 11, 29, 24, dtype, with_boundary, rnnt_type, 5)
    if smoothed:
        loss = fr.rnnt_loss_smoothed(lm=lm, am=am, symbols=symbols, termination_symbol=0,
                                     lm_only_scale=0.2, am_only_scale=0.1, boundary=boundary,
                                     rnnt_type=rnnt_type, delay_penalty=dp, reduction="none")
        px, py = fr.get_rnnt_logprobs_smoothed(lm=lm, am=am, symbols=symbols, termination_symbol=0,
                                               lm_only_scale=0.2, am_only_scale=0.1, boundary=boundary,
                                               rnnt_type=rnnt_type)
    else:
        loss = fr.rnnt_loss_simple(lm=lm, am=am, symbols=symbols, termination_symbol=0, boundary=boundary,
                                   rnnt_type=rnnt_type, delay_penalty=dp, reduction="none")
        px, py = fr.get_rnnt_logprobs(lm=lm, am=am, symbols=symbols, termination_symbol=0,
                                      boundary=boundary, rnnt_type=rnnt_type)
    want = -fr.mutual_information_recursion(px=reference_penalty(px, boundary, rnnt_type, dp), py=py,
                                            boundary=boundary)
    assert torch.equal(loss, want), (loss, want)
    # and it does something
    plain = -fr.mutual_information_recursion(px=px, py=py, boundary=boundary)
    assert not torch.equal(loss, plain)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("with_boundary", [False, True])
@pytest.mark.parametrize("rnnt_type", ["regular", "modified"])
def test_joint_and_pruned_losses(dtype, with_boundary, rnnt_type):
    import fast_rnnt_b200 as fr
    dp = 0.05
    B, S, T, C, R = 2, 9, 23, 16, 4
    lm, am, symbols, boundary = make(B, S, T, C, dtype, with_boundary, rnnt_type, 9)
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(B, T, S + 1, C, generator=g, dtype=dtype).cuda()
    loss = fr.rnnt_loss(logits=logits, symbols=symbols, termination_symbol=0, boundary=boundary,
                        rnnt_type=rnnt_type, delay_penalty=dp, reduction="none")
    px, py = fr.get_rnnt_logprobs_joint(logits=logits, symbols=symbols, termination_symbol=0,
                                        boundary=boundary, rnnt_type=rnnt_type)
    want = -fr.mutual_information_recursion(px=reference_penalty(px, boundary, rnnt_type, dp), py=py,
                                            boundary=boundary)
    assert torch.equal(loss, want)

    start = torch.sort(torch.randint(0, S + 1 - R + 1, (B, T), generator=g), dim=1)[0]
    ranges = (start.unsqueeze(-1) + torch.arange(R)).cuda()
    plog = torch.randn(B, T, R, C, generator=g, dtype=dtype).cuda()
    loss = fr.rnnt_loss_pruned(logits=plog, symbols=symbols, ranges=ranges, termination_symbol=0,
                               boundary=boundary, rnnt_type=rnnt_type, delay_penalty=dp, reduction="none")
    px, py = fr.get_rnnt_logprobs_pruned(logits=plog, symbols=symbols, ranges=ranges, termination_symbol=0,
                                         boundary=boundary, rnnt_type=rnnt_type)
    want = -fr.mutual_information_recursion(px=reference_penalty(px, boundary, rnnt_type, dp), py=py,
                                            boundary=boundary)
    assert torch.equal(loss, want)

    if dtype == torch.float32:
        D = 16
        enc = torch.randn(B, T, D, generator=g).cuda()
        dec = torch.randn(B, S + 1, D, generator=g).cuda()
        W = (torch.randn(C, D, generator=g) * 0.2).cuda()
        bias = torch.randn(C, generator=g).cuda()
        loss = fr.rnnt_loss_pruned_joiner(am=enc, lm=dec, ranges=ranges, joiner_weight=W, joiner_bias=bias,
                                          symbols=symbols, termination_symbol=0, boundary=boundary,
                                          rnnt_type=rnnt_type, delay_penalty=dp, reduction="none")
        px, py = fr.get_rnnt_logprobs_pruned_joiner(am=enc, lm=dec, ranges=ranges, joiner_weight=W,
                                                    joiner_bias=bias, symbols=symbols, termination_symbol=0,
                                                    boundary=boundary, rnnt_type=rnnt_type)
        want = -fr.mutual_information_recursion(px=reference_penalty(px, boundary, rnnt_type, dp), py=py,
                                                boundary=boundary)
        assert torch.equal(loss, want)
