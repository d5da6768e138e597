"""The fused pruned-joiner operator (csrc/joiner_pairs.cu, csrc/umma_pairs.cuh):
get_rnnt_logprobs_pruned_joiner / rnnt_loss_pruned_joiner against the composition
they replace -- do_rnnt_pruning, Linear(tanh(.)), get_rnnt_logprobs_pruned -- evaluated
in float64 by torch on the CPU oracle's formulas.

Tolerances: lattices 1e-5 absolute, loss 1e-5 relative, gradients 1e-4 absolute plus
1e-5 of the tensor's largest entry (sums over all joiner rows).
"""
import pytest
import torch

from oracle import rnnt_oracle as orc
from tests.test_mi_gpu import assert_close

pytestmark = pytest.mark.gpu


def fr():
    import fast_rnnt_b200
    return fast_rnnt_b200


def make_case(B, T, S, R, D, C, rnnt_type, seed, wscale=1.0, escale=1.0):
    g = torch.Generator().manual_seed(seed)
    enc = torch.randn(B, T, D, generator=g) * escale
    dec = torch.randn(B, S + 1, D, generator=g) * escale
    W = torch.randn(C, D, generator=g) * (wscale / D ** 0.5)
    bias = torch.randn(C, generator=g) * 0.1
    symbols = torch.randint(1, C, (B, S), generator=g)
    Sb = torch.randint(max(1, S // 2), S + 1, (B,), generator=g)
    lo = max(2, T // 2)
    Tb = torch.randint(lo, T + 1, (B,), generator=g)
    if rnnt_type != "regular":
        Tb = torch.maximum(Tb, Sb)
    z = torch.zeros(B, dtype=torch.int64)
    boundary = torch.stack([z, z, Sb, Tb], dim=1)
    # windows that only move forward, as get_rnnt_prune_ranges writes them
    start = torch.sort(torch.randint(0, S + 1 - R + 1, (B, T), generator=g), dim=1)[0]
    ranges = start.unsqueeze(-1) + torch.arange(R)
    return enc, dec, W, bias, symbols, boundary, ranges


def reference_f64(enc, dec, W, bias, symbols, boundary, ranges, rnnt_type, w_px, w_py):
    e, d, w, b = (t.double().clone().requires_grad_(True) for t in (enc, dec, W, bias))
    am_p, lm_p = orc.prune(e, d, ranges)
    logits = torch.nn.functional.linear(torch.tanh(am_p + lm_p), w, b)
    px, py = orc.pruned_logprobs(logits, symbols, ranges, 0, boundary, rnnt_type)
    fx, fy = torch.isfinite(px), torch.isfinite(py)
    loss = (torch.where(fx, px, torch.zeros_like(px)) * w_px.double()).sum() + \
           (torch.where(fy, py, torch.zeros_like(py)) * w_py.double()).sum()
    loss.backward()
    return px.detach(), py.detach(), e.grad, d.grad, w.grad, b.grad


CASES = [
    # B, T, S, R, D, C
    (3, 19, 8, 4, 64, 36),
    (2, 70, 32, 5, 128, 36),
    (2, 33, 12, 5, 512, 500),      # the joiner of the benchmark: four column tiles, ragged last one
    (1, 40, 9, 3, 72, 1032),       # more than eight column tiles, D not a multiple of the K slice
    (2, 21, 14, 9, 8, 12),         # the narrowest activations, more rows per frame than registers hold
    (2, 150, 20, 2, 40, 4),        # the smallest vocabulary
    # several tiles per persistent CTA (the two fold sets take turns), with one, three and
    # five K slices per tile (odd group counts walk through both accumulators)
    (16, 500, 50, 5, 64, 200),
    (12, 400, 40, 5, 192, 264),
    (10, 300, 30, 5, 320, 136),
]


@pytest.mark.parametrize("shape", CASES)
@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_fused_lattices_and_gradients_match_float64(shape, rnnt_type):
    B, T, S, R, D, C = shape
    if rnnt_type != "regular" and T < S:
        pytest.skip("modified recursion needs T >= S")
    enc, dec, W, bias, symbols, boundary, ranges = make_case(B, T, S, R, D, C, rnnt_type, seed=sum(shape))
    f = fr()
    ce, cd, cw, cb = (t.cuda().requires_grad_(True) for t in (enc, dec, W, bias))
    px, py = f.get_rnnt_logprobs_pruned_joiner(am=ce, lm=cd, ranges=ranges.cuda(), joiner_weight=cw,
                                               joiner_bias=cb, symbols=symbols.cuda(),
                                               termination_symbol=0, boundary=boundary.cuda(),
                                               rnnt_type=rnnt_type)
    g = torch.Generator().manual_seed(7)
    w_px = torch.randn(px.shape, generator=g)
    w_py = torch.randn(py.shape, generator=g)
    fx, fy = torch.isfinite(px), torch.isfinite(py)
    loss = (torch.where(fx, px, torch.zeros_like(px)) * w_px.cuda()).sum() + \
           (torch.where(fy, py, torch.zeros_like(py)) * w_py.cuda()).sum()
    loss.backward()
    rpx, rpy, ge, gd, gw, gb = reference_f64(enc, dec, W, bias, symbols, boundary, ranges, rnnt_type,
                                             w_px, w_py)
    assert_close(px, rpx, 0, 1e-5, "px")
    assert_close(py, rpy, 0, 1e-5, "py")
    for ours, ref, what in ((ce.grad, ge, "enc"), (cd.grad, gd, "dec"), (cw.grad, gw, "weight"),
                            (cb.grad, gb, "bias")):
        assert_close(ours, ref, 0, 1e-4 + 1e-5 * float(ref.abs().max()), what + " grad")


@pytest.mark.parametrize("wscale,escale", [(1e-6, 1.0), (3e4, 1.0), (1.0, 1e-4), (1.0, 30.0)])
def test_fused_operator_is_scale_safe(wscale, escale):
    """Weights and activations far from unit scale: the fp16 planes carry a per-operand
    power-of-two scale, so neither overflow nor loss of small values may show."""
    B, T, S, R, D, C = 2, 25, 10, 4, 64, 40
    enc, dec, W, bias, symbols, boundary, ranges = make_case(B, T, S, R, D, C, "regular", 3, wscale, escale)
    f = fr()
    ce, cd, cw, cb = (t.cuda().requires_grad_(True) for t in (enc, dec, W, bias))
    loss = f.rnnt_loss_pruned_joiner(am=ce, lm=cd, ranges=ranges.cuda(), joiner_weight=cw, joiner_bias=cb,
                                     symbols=symbols.cuda(), termination_symbol=0,
                                     boundary=boundary.cuda(), reduction="sum")
    loss.backward()
    e, d, w, b = (t.double().clone().requires_grad_(True) for t in (enc, dec, W, bias))
    am_p, lm_p = orc.prune(e, d, ranges)
    logits = torch.nn.functional.linear(torch.tanh(am_p + lm_p), w, b)
    ref = orc.loss_pruned(logits, symbols, ranges, 0, boundary, "regular", 0.0, "sum")
    ref.backward()
    assert_close(loss, ref.detach(), 1e-5, 1e-5, "loss")
    for ours, r, what in ((ce.grad, e.grad, "enc"), (cd.grad, d.grad, "dec"), (cw.grad, w.grad, "weight"),
                          (cb.grad, b.grad, "bias")):
        assert torch.isfinite(ours).all(), what
        assert_close(ours, r, 1e-4, 1e-4 + 1e-5 * float(r.abs().max()), what + " grad")


def test_fused_operator_equals_the_unfused_path_and_is_deterministic():
    """Same numbers (to float32 rounding) as pruned_joiner + rnnt_loss_pruned, bit-identical
    from run to run (no atomics anywhere on the path), gradients only where asked."""
    B, T, S, R, D, C = 4, 60, 25, 5, 256, 200
    enc, dec, W, bias, symbols, boundary, ranges = make_case(B, T, S, R, D, C, "regular", 11)
    f = fr()
    runs = []
    for _ in range(2):
        ce, cd, cw = (t.cuda().requires_grad_(True) for t in (enc, dec, W))
        loss = f.rnnt_loss_pruned_joiner(am=ce, lm=cd, ranges=ranges.cuda(), joiner_weight=cw,
                                         joiner_bias=None, symbols=symbols.cuda(),
                                         termination_symbol=0, boundary=boundary.cuda(),
                                         delay_penalty=0.01, reduction="none")
        loss.sum().backward()
        runs.append((loss.detach(), ce.grad, cd.grad, cw.grad))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    ce, cd, cw = (t.cuda().requires_grad_(True) for t in (enc, dec, W))
    logits = f.pruned_joiner(ce, cd, ranges.cuda(), cw, None)
    ref = f.rnnt_loss_pruned(logits=logits, symbols=symbols.cuda(), ranges=ranges.cuda(),
                             termination_symbol=0, boundary=boundary.cuda(), delay_penalty=0.01,
                             reduction="none")
    ref.sum().backward()
    assert_close(runs[0][0], ref.detach(), 1e-5, 1e-5, "loss")
    for ours, r, what in zip(runs[0][1:], (ce.grad, cd.grad, cw.grad), ("enc", "dec", "weight")):
        assert_close(ours, r, 1e-4, 1e-4, what + " grad")
    # weights only: no input gradients are computed or returned
    cw = W.cuda().requires_grad_(True)
    loss = f.rnnt_loss_pruned_joiner(am=enc.cuda(), lm=dec.cuda(), ranges=ranges.cuda(), joiner_weight=cw,
                                     joiner_bias=None, symbols=symbols.cuda(), termination_symbol=0,
                                     boundary=boundary.cuda(), reduction="sum")
    loss.backward()
    assert_close(cw.grad, runs[0][3] * 0 + cw.grad, 0, 0, "shape")
    assert cw.grad.shape == W.shape


def test_fused_operator_rejects_unsupported_sizes():
    f = fr()
    enc, dec, W, bias, symbols, boundary, ranges = make_case(1, 10, 4, 2, 12, 8, "regular", 1)
    with pytest.raises(f.FrnntError):   # D = 12 is not a multiple of 8
        f.get_rnnt_logprobs_pruned_joiner(am=enc.cuda(), lm=dec.cuda(), ranges=ranges.cuda(),
                                          joiner_weight=W.cuda(), joiner_bias=None,
                                          symbols=symbols.cuda(), termination_symbol=0,
                                          boundary=boundary.cuda())
