"""The 3xTF32 tensor-core linear layer (csrc/linear_umma.cu, TMA-fed) against a
float64 torch reference: fp32-level accuracy is required, i.e. errors no larger
than a few times those of torch's own float32 linear on the same inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", [(1, 4, 4), (128, 32, 128), (200, 64, 100), (333, 516, 500),
                                   (1000, 512, 500), (4097, 128, 260)])
def test_linear_forward_backward(M, K, N):
    from fast_rnnt_b200.linear import linear
    torch.manual_seed(M + K + N)
    x = torch.randn(M, K, device="cuda", requires_grad=True)
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).requires_grad_(True)
    b = torch.randn(N, device="cuda", requires_grad=True)
    y = linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xd, wd, bd, gd = x.detach().double(), w.detach().double(), b.detach().double(), g.double()
    y_ref, gx_ref, gw_ref, gb_ref = xd @ wd.t() + bd, gd @ wd, gd.t() @ xd, gd.sum(0)
    x2, w2, b2 = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    y32 = torch.nn.functional.linear(x2, w2, b2)
    y32.backward(g)

    def check(ours, ref, torch32, what):
        err = (ours.double() - ref).abs().max().item()
        base = (torch32.double() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err <= max(4 * base, 2e-6 * scale), (what, err, base, scale)

    check(y, y_ref, y32, "y")
    check(x.grad, gx_ref, x2.grad, "grad_input")
    check(w.grad, gw_ref, w2.grad, "grad_weight")
    check(b.grad, gb_ref, b2.grad, "grad_bias")


def test_linear_on_pruned_shapes_matches_torch():
    """[B][T][R][D] activations as the joiner sees them."""
    from fast_rnnt_b200.linear import linear
    torch.manual_seed(1)
    a = torch.randn(3, 17, 5, 64, device="cuda")
    w = torch.randn(20, 64, device="cuda") / 8
    b = torch.randn(20, device="cuda")
    y = linear(torch.tanh(a), w, b)
    assert y.shape == (3, 17, 5, 20)
    torch.testing.assert_close(y, torch.nn.functional.linear(torch.tanh(a), w, b), rtol=1e-5,
                               atol=1e-5)


def test_linear_rejects_unaligned_rows():
    from fast_rnnt_b200 import FrnntError
    from fast_rnnt_b200.linear import linear
    with pytest.raises(FrnntError):
        linear(torch.randn(8, 6, device="cuda"), torch.randn(4, 6, device="cuda"))


@pytest.mark.parametrize("shape,monotone", [((3, 19, 9, 4, 64, 36), True),
                                            ((2, 70, 33, 5, 128, 36), True),
                                            ((2, 37, 60, 5, 64, 20), False),
                                            # more rows per frame than the kernels keep in registers,
                                            # the narrowest rows TMA accepts
                                            ((2, 21, 14, 9, 8, 12), True)])
def test_pruned_joiner_matches_the_torch_composition(shape, monotone):
    """pruned_joiner == linear(tanh(am_pruned + lm_pruned)) of the reference's usage,
    values and all five gradients."""
    import fast_rnnt_b200 as fr
    torch.manual_seed(5)
    B, T, S1, R, D, C = shape
    enc = torch.randn(B, T, D, device="cuda", requires_grad=True)
    dec = torch.randn(B, S1, D, device="cuda", requires_grad=True)
    w = (torch.randn(C, D, device="cuda") / 8).requires_grad_(True)
    b = torch.randn(C, device="cuda", requires_grad=True)
    if monotone:   # what get_rnnt_prune_ranges produces: a window that only moves forward
        start = torch.sort(torch.randint(0, S1 - R + 1, (B, T), device="cuda"), dim=1)[0]
        ranges = start.unsqueeze(-1) + torch.arange(R, device="cuda")
    else:          # any rows at all (the input gradients then fall back to atomic adds)
        ranges = torch.randint(0, S1, (B, T, R), device="cuda")
    y = fr.pruned_joiner(enc, dec, ranges, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    ours = [y.detach(), enc.grad, dec.grad, w.grad, b.grad]
    e2, d2, w2, b2 = (t.detach().double().requires_grad_(True) for t in (enc, dec, w, b))
    a_p = e2.unsqueeze(2).expand(B, T, R, D)
    l_p = torch.gather(d2, 1, ranges.reshape(B, T * R, 1).expand(B, T * R, D)).reshape(B, T, R, D)
    y_ref = torch.nn.functional.linear(torch.tanh(a_p + l_p), w2, b2)
    y_ref.backward(g.double())
    ref = [y_ref.detach(), e2.grad, d2.grad, w2.grad, b2.grad]
    for o, r, what in zip(ours, ref, ("logits", "enc", "dec", "weight", "bias")):
        # fp32-level accuracy: a few ulps of the largest entry (sums of hundreds of terms)
        atol = 2e-5 * max(1.0, float(r.abs().max()) / 8)
        torch.testing.assert_close(o.double(), r, rtol=1e-5, atol=atol, msg=lambda m: what + m)
