"""float16 / bfloat16 inputs.  The reference dispatches float and double only
(fast_rnnt/csrc/mutual_information_cuda.cu:37-38), so the definition is this library's:
the result equals the float32 call on the inputs converted to float32 -- lattices and
losses bit for bit (they are float32), gradients equal to the float32 gradients rounded to
the input's type (autograd's cast)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

HALVES = [torch.float16, torch.bfloat16]


def make(B, S, T, C, seed):
    g = torch.Generator().manual_seed(seed)
    lm = torch.randn(B, S + 1, C, generator=g)
    am = torch.randn(B, T, C, generator=g)
    symbols = torch.randint(1, C, (B, S), generator=g).cuda()
    Sb = torch.randint(max(1, S // 2), S + 1, (B,), generator=g)
    Tb = torch.randint(max(S, T // 2), T + 1, (B,), generator=g)
    z = torch.zeros(B, dtype=torch.int64)
    boundary = torch.stack([z, z, Sb, Tb], dim=1).cuda()
    return lm, am, symbols, boundary


def run_both(fn, tensors16):
    """fn(*tensors) -> loss; once on the 16-bit leaves, once on float32 copies of them."""
    out = []
    for cast in (False, True):
        leaves = [(t.float() if cast else t).clone().requires_grad_(True) for t in tensors16]
        loss = fn(*leaves)
        loss.sum().backward()
        out.append((loss.detach(), [x.grad for x in leaves]))
    (l16, g16), (l32, g32) = out
    assert l16.dtype == torch.float32
    assert torch.equal(l16, l32), (l16, l32)
    for a, b, t in zip(g16, g32, tensors16):
        assert a.dtype == t.dtype
        assert torch.equal(a, b.to(t.dtype))


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
@pytest.mark.parametrize("am_only_scale", [0.0, 0.1])   # kernels read 16 bits / inputs converted first
def test_smoothed_loss(dtype, rnnt_type, am_only_scale):
    import fast_rnnt_b200 as fr
    lm, am, symbols, boundary = make(3, 13, 37, 40, 21)

    def fn(lm_, am_):
        return fr.rnnt_loss_smoothed(lm=lm_, am=am_, symbols=symbols, termination_symbol=0, lm_only_scale=0.25,
                                     am_only_scale=am_only_scale, boundary=boundary, rnnt_type=rnnt_type,
                                     delay_penalty=0.01, reduction="none")
    run_both(fn, [lm.to(dtype).cuda(), am.to(dtype).cuda()])


@pytest.mark.parametrize("dtype", HALVES)
@pytest.mark.parametrize("C", [40, 37])   # tensor-core path / odd vocabulary (converted first)
def test_simple_loss_and_occupancies(dtype, C):
    import fast_rnnt_b200 as fr
    lm, am, symbols, boundary = make(2, 9, 30, C, 5)
    l16, a16 = lm.to(dtype).cuda(), am.to(dtype).cuda()
    r16 = fr.rnnt_loss_simple(lm=l16, am=a16, symbols=symbols, termination_symbol=0, boundary=boundary,
                              reduction="sum", return_grad=True)
    r32 = fr.rnnt_loss_simple(lm=l16.float(), am=a16.float(), symbols=symbols, termination_symbol=0,
                              boundary=boundary, reduction="sum", return_grad=True)
    assert torch.equal(r16[0], r32[0])
    assert torch.equal(r16[1][0], r32[1][0]) and torch.equal(r16[1][1], r32[1][1])


@pytest.mark.parametrize("dtype", HALVES)
def test_fused_joiner_and_pruned_losses(dtype):
    import fast_rnnt_b200 as fr
    B, S, T, C, D, R = 3, 12, 41, 24, 32, 4
    _, _, symbols, boundary = make(B, S, T, C, 8)
    g = torch.Generator().manual_seed(2)
    enc = torch.randn(B, T, D, generator=g).to(dtype).cuda()
    dec = torch.randn(B, S + 1, D, generator=g).to(dtype).cuda()
    W = (torch.randn(C, D, generator=g) * 0.2).cuda()
    bias = torch.randn(C, generator=g).cuda()
    start = torch.sort(torch.randint(0, S + 1 - R + 1, (B, T), generator=g), dim=1)[0]
    ranges = (start.unsqueeze(-1) + torch.arange(R)).cuda()

    def fused(enc_, dec_):
        return fr.rnnt_loss_pruned_joiner(am=enc_, lm=dec_, ranges=ranges, joiner_weight=W, joiner_bias=bias,
                                          symbols=symbols, termination_symbol=0, boundary=boundary,
                                          reduction="none")
    run_both(fused, [enc, dec])

    logits = torch.randn(B, T, R, C, generator=g).to(dtype).cuda()

    def pruned(logits_):
        return fr.rnnt_loss_pruned(logits=logits_, symbols=symbols, ranges=ranges, termination_symbol=0,
                                   boundary=boundary, reduction="none")
    run_both(pruned, [logits])
