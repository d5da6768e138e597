"""GPU parity of the loss pipeline (csrc/simple.cu, lsm.cu, prune.cu, mi.cu through
the C ABI) against the reference-written golden vectors and the CPU oracle.

Stage-wise protocol: because the prune-range argmax is decided by one-ulp
margins, every stage is also checked with the REFERENCE's tensors of the
previous stage injected (ranges on the reference's occupancies: bit-exact;
pruned lattices on the reference's ranges and logits).

float32 tolerances: lattices px/py 1e-5 abs, loss 1e-5 rel, occupancies and
all gradients 1e-4 abs.
"""
import pytest
import torch

from oracle import rnnt_oracle as orc
from tests import workloads
from tests.conftest import load_golden
from tests.test_mi_gpu import assert_close

pytestmark = pytest.mark.gpu

LATTICE_ATOL = 1e-5
GRAD_ATOL = 1e-4
LOSS_RTOL = 1e-5


def fr():
    import fast_rnnt_b200
    return fast_rnnt_b200


def cu(x):
    return x.cuda() if isinstance(x, torch.Tensor) else x


def test_basic_known_answers():
    g = load_golden("basic")
    lm, am, symbols, blank = [cu(x) for x in workloads.reference_basic_tensors()]
    px, py = fr().get_rnnt_logprobs(lm=lm, am=am, symbols=symbols, termination_symbol=blank)
    assert px.shape == (1, 3, 5) and py.shape == (1, 4, 4)
    assert_close(px, g["px"], 0, LATTICE_ATOL, "px")
    assert_close(py, g["py"], 0, LATTICE_ATOL, "py")
    m = fr().mutual_information_recursion(px=px, py=py, boundary=None)
    assert_close(-m, g["neg_m"], LOSS_RTOL, 0, "mi")
    kw = dict(lm=lm, am=am, symbols=symbols, termination_symbol=blank, boundary=None,
              reduction="none")
    assert_close(fr().rnnt_loss_simple(**kw), g["simple"], LOSS_RTOL, 0, "simple")
    assert_close(fr().rnnt_loss_smoothed(lm_only_scale=0.0, am_only_scale=0.0, **kw),
                 g["smoothed0"], LOSS_RTOL, 0, "smoothed0")
    assert_close(fr().rnnt_loss_smoothed(lm_only_scale=0.0, am_only_scale=0.333, **kw),
                 g["smoothed_am0333"], LOSS_RTOL, 0, "smoothed_am")
    logits = am.unsqueeze(2) + lm.unsqueeze(1)
    assert_close(fr().rnnt_loss(logits=logits, symbols=symbols, termination_symbol=blank,
                                boundary=None, reduction="none"), g["joint"], LOSS_RTOL, 0, "joint")
    if "torchaudio" in g:
        assert_close(fr().rnnt_loss_simple(**kw), g["torchaudio"], LOSS_RTOL, 0, "torchaudio")
    # invariance to per-frame constants (reference rnnt_loss_test.py:155-189)
    torch.manual_seed(0)
    lm2 = lm + torch.randn(1, 4, 1, device="cuda")
    am2 = am + torch.randn(1, 4, 1, device="cuda")
    kw.update(lm=lm2, am=am2)
    assert_close(fr().rnnt_loss_simple(**kw), g["simple"], LOSS_RTOL, 1e-5, "simple shifted")
    assert_close(fr().rnnt_loss_smoothed(lm_only_scale=0.0, am_only_scale=0.0, **kw),
                 g["smoothed0"], LOSS_RTOL, 1e-5, "smoothed shifted")


def joiner_logits(kind, enc, dec, ranges, W, bias):
    """The joiner between do_rnnt_pruning and rnnt_loss_pruned: the reference's documented
    composition in torch ("torch"), or this library's pruned_joiner ("fused")."""
    f = fr()
    if kind == "fused":
        return f.pruned_joiner(enc, dec, ranges, W, bias)
    am_p, lm_p = f.do_rnnt_pruning(am=enc, lm=dec, ranges=ranges)
    return torch.nn.functional.linear(torch.tanh(am_p + lm_p), W, bias)


def samp(x):
    """The strided sample tests/golden/make_golden.py keeps of a full-size tensor."""
    flat = x.detach().reshape(-1)
    return flat[:: max(1, flat.numel() // 4096)]


def run_pipeline(wl, rnnt_type, dtype=torch.float32, joiner="torch"):
    f = fr()
    conv = lambda x: x.to(dtype).cuda() if x.is_floating_point() else x.cuda()  # noqa: E731
    am = conv(wl["am"]).requires_grad_(True)
    lm = conv(wl["lm"]).requires_grad_(True)
    enc = conv(wl["enc"]).requires_grad_(True)
    dec = conv(wl["dec"]).requires_grad_(True)
    W = conv(wl["joiner_w"]).requires_grad_(True)
    bias = conv(wl["joiner_b"]).requires_grad_(True)
    sym, bnd, blank = wl["symbols"].cuda(), wl["boundary"].cuda(), wl["blank"]
    ls, as_ = wl["lm_only_scale"], wl["am_only_scale"]
    px, py = f.get_rnnt_logprobs_smoothed(lm=lm.detach(), am=am.detach(), symbols=sym,
                                          termination_symbol=blank, lm_only_scale=ls,
                                          am_only_scale=as_, boundary=bnd, rnnt_type=rnnt_type)
    simple, (ox, oy) = f.rnnt_loss_smoothed(lm=lm, am=am, symbols=sym, termination_symbol=blank,
                                            lm_only_scale=ls, am_only_scale=as_, boundary=bnd,
                                            rnnt_type=rnnt_type, reduction="sum", return_grad=True)
    occ_x, occ_y = ox.clone(), oy.clone()
    ranges = f.get_rnnt_prune_ranges(px_grad=ox, py_grad=oy, boundary=bnd, s_range=wl["s_range"])
    logits = joiner_logits(joiner, enc, dec, ranges, W, bias)
    logits.retain_grad()
    ppx, ppy = f.get_rnnt_logprobs_pruned(logits=logits.detach(), symbols=sym, ranges=ranges,
                                          termination_symbol=blank, boundary=bnd,
                                          rnnt_type=rnnt_type)
    pruned = f.rnnt_loss_pruned(logits=logits, symbols=sym, ranges=ranges,
                                termination_symbol=blank, boundary=bnd, rnnt_type=rnnt_type,
                                reduction="sum")
    (simple + pruned).backward()
    return dict(simple=simple, pruned=pruned, ranges=ranges, px=px, py=py, occ_x=occ_x,
                occ_y=occ_y, pruned_px=ppx, pruned_py=ppy, am_grad=am.grad, lm_grad=lm.grad,
                enc_grad=enc.grad, dec_grad=dec.grad, logits=logits, logits_grad=logits.grad,
                w_grad=W.grad, b_grad=bias.grad)


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_mini_pipeline_stagewise(rnnt_type):
    g = load_golden("pipeline_mini_" + rnnt_type)
    wl = workloads.pipeline_workload("mini", rnnt_type=rnnt_type)
    out = run_pipeline(wl, rnnt_type)
    f = fr()
    bnd, sym = g["boundary"].cuda(), g["symbols"].cuda()
    # S1: simple/smoothed stage
    assert_close(out["px"], g["px"], 0, LATTICE_ATOL, "px")
    assert_close(out["py"], g["py"], 0, LATTICE_ATOL, "py")
    assert_close(out["simple"], g["simple"], LOSS_RTOL, 0, "simple loss")
    assert_close(out["occ_x"], g["occ_x"], 0, GRAD_ATOL, "occ_x")
    assert_close(out["occ_y"], g["occ_y"], 0, GRAD_ATOL, "occ_y")
    # S3: ranges on the reference's occupancies -> bit-exact
    r = f.get_rnnt_prune_ranges(px_grad=g["occ_x"].cuda(), py_grad=g["occ_y"].cuda(), boundary=bnd,
                                s_range=wl["s_range"])
    assert r.dtype == torch.int64 and r.shape[2] == g["s_range"]
    ref_ranges = g["s_begin"].to(torch.int64).unsqueeze(-1) + torch.arange(g["s_range"])
    assert torch.equal(r.cpu(), ref_ranges)
    # S4: pruned stage on the reference's ranges and logits
    ppx, ppy = f.get_rnnt_logprobs_pruned(logits=g["logits"].cuda(), symbols=sym,
                                          ranges=ref_ranges.cuda(), termination_symbol=0,
                                          boundary=bnd, rnnt_type=rnnt_type)
    assert_close(ppx, g["pruned_px"], 0, LATTICE_ATOL, "pruned px")
    assert_close(ppy, g["pruned_py"], 0, LATTICE_ATOL, "pruned py")
    logits = g["logits"].cuda().requires_grad_(True)
    loss = f.rnnt_loss_pruned(logits=logits, symbols=sym, ranges=ref_ranges.cuda(),
                              termination_symbol=0, boundary=bnd, rnnt_type=rnnt_type,
                              reduction="sum")
    assert_close(loss, g["pruned"], LOSS_RTOL, 0, "pruned loss")
    loss.backward()
    assert_close(logits.grad, g["logits_grad"], 0, GRAD_ATOL, "logits grad")
    # S5: end to end with our own ranges (they equal the reference's on this case)
    if torch.equal(out["ranges"].cpu(), ref_ranges):
        assert_close(out["pruned"], g["pruned"], LOSS_RTOL, 0, "pruned loss e2e")
        for k in ("am_grad", "lm_grad", "enc_grad", "dec_grad", "logits_grad", "w_grad", "b_grad"):
            assert_close(out[k], g[k], 1e-4, GRAD_ATOL, k)
    else:  # pragma: no cover - documented: a one-ulp argmax flip moves the ranges
        frac = (out["ranges"].cpu() != ref_ranges).float().mean().item()
        assert frac < 0.02, frac
        for k in ("am_grad", "lm_grad"):
            assert_close(out[k], g[k], 1e-4, GRAD_ATOL, k)


def test_simple_variants():
    g = load_golden("simple_variants_mini")
    wl = workloads.pipeline_workload("mini")
    f = fr()
    sym, bnd = wl["symbols"].cuda(), wl["boundary"].cuda()
    for rnnt_type in ("regular", "modified", "constrained"):
        am = wl["am"].cuda().requires_grad_(True)
        lm = wl["lm"].cuda().requires_grad_(True)
        loss = f.rnnt_loss_simple(lm=lm, am=am, symbols=sym, termination_symbol=0, boundary=bnd,
                                  rnnt_type=rnnt_type, delay_penalty=0.01, reduction="none")
        loss.sum().backward()
        assert_close(loss, g[f"simple_dp_{rnnt_type}"], LOSS_RTOL, 0, "dp loss " + rnnt_type)
        assert_close(am.grad, g[f"simple_dp_{rnnt_type}_am_grad"], 0, GRAD_ATOL, "am grad")
        assert_close(lm.grad, g[f"simple_dp_{rnnt_type}_lm_grad"], 0, GRAD_ATOL, "lm grad")
        am = wl["am"].cuda().requires_grad_(True)
        lm = wl["lm"].cuda().requires_grad_(True)
        loss = f.rnnt_loss_smoothed(lm=lm, am=am, symbols=sym, termination_symbol=0,
                                    lm_only_scale=0.1, am_only_scale=0.2, boundary=bnd,
                                    rnnt_type=rnnt_type, reduction="mean")
        loss.backward()
        assert_close(loss, g[f"smoothed_{rnnt_type}"], LOSS_RTOL, 0, "smoothed loss " + rnnt_type)
        assert_close(am.grad, g[f"smoothed_{rnnt_type}_am_grad"], 0, GRAD_ATOL, "am grad")
        assert_close(lm.grad, g[f"smoothed_{rnnt_type}_lm_grad"], 0, GRAD_ATOL, "lm grad")
    with pytest.raises(ValueError):
        f.rnnt_loss_simple(lm=wl["lm"].cuda(), am=wl["am"].cuda(), symbols=sym,
                           termination_symbol=0, boundary=bnd, reduction="bogus")


def test_c1_simple_loss():
    g = load_golden("c1_simple")
    wl = workloads.config_c1()
    f = fr()
    am = wl["am"].cuda().requires_grad_(True)
    lm = wl["lm"].cuda().requires_grad_(True)
    sym, bnd = wl["symbols"].cuda(), wl["boundary"].cuda()
    px, py = f.get_rnnt_logprobs(lm=lm.detach(), am=am.detach(), symbols=sym,
                                 termination_symbol=0, boundary=bnd)
    assert_close(px, g["px"], 0, LATTICE_ATOL, "px")
    assert_close(py, g["py"], 0, LATTICE_ATOL, "py")
    loss, (gx, gy) = f.rnnt_loss_simple(lm=lm, am=am, symbols=sym, termination_symbol=0,
                                        boundary=bnd, reduction="sum", return_grad=True)
    assert_close(loss, g["loss"], LOSS_RTOL, 0, "loss")
    assert_close(gx, g["occ_x"], 0, GRAD_ATOL, "occ_x")
    assert_close(gy, g["occ_y"], 0, GRAD_ATOL, "occ_y")
    loss.backward()
    assert_close(am.grad, g["am_grad"], 0, GRAD_ATOL, "am grad")
    assert_close(lm.grad, g["lm_grad"], 0, GRAD_ATOL, "lm grad")


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_joint_small(rnnt_type):
    g = load_golden("joint_small_" + rnnt_type)
    f = fr()
    logits = g["logits"].cuda().requires_grad_(True)
    sym, bnd = g["symbols"].cuda(), g["boundary"].cuda()
    px, py = f.get_rnnt_logprobs_joint(logits=logits.detach(), symbols=sym,
                                       termination_symbol=g["blank"], boundary=bnd,
                                       rnnt_type=rnnt_type)
    assert_close(px, g["px"], 0, LATTICE_ATOL, "px")
    assert_close(py, g["py"], 0, LATTICE_ATOL, "py")
    loss = f.rnnt_loss(logits=logits, symbols=sym, termination_symbol=g["blank"], boundary=bnd,
                       rnnt_type=rnnt_type, delay_penalty=0.02, reduction="none")
    loss.sum().backward()
    assert_close(loss, g["loss"], LOSS_RTOL, 0, "loss")
    assert_close(logits.grad, g["logits_grad"], 0, GRAD_ATOL, "logits grad")


def test_prune_range_edge_cases(capsys):
    g = load_golden("prune_edges")
    for tag in workloads.prune_edge_cases():
        r = fr().get_rnnt_prune_ranges(px_grad=g[tag + "_occ_x"].cuda(),
                                       py_grad=g[tag + "_occ_y"].cuda(),
                                       boundary=g[tag + "_boundary"].cuda(),
                                       s_range=int(g[tag + "_s_range_in"]))
        assert r.dtype == torch.int64
        assert torch.equal(r.cpu(), g[tag + "_ranges"]), tag
    assert "Adjusting to 6" in capsys.readouterr().out  # the s_range warning of the reference


def test_do_rnnt_pruning_forward_backward():
    torch.manual_seed(3)
    for (B, T, S1, R, D, dt) in [(2, 7, 5, 3, 16, torch.float32), (3, 11, 9, 4, 10, torch.float32),
                                 (2, 5, 6, 6, 7, torch.float64), (1, 33, 12, 5, 512, torch.float32)]:
        am = torch.randn(B, T, D, dtype=dt, device="cuda", requires_grad=True)
        lm = torch.randn(B, S1, D, dtype=dt, device="cuda", requires_grad=True)
        start = torch.randint(0, S1 - R + 1, (B, T, 1), device="cuda")
        ranges = start + torch.arange(R, device="cuda")
        a, l = fr().do_rnnt_pruning(am=am, lm=lm, ranges=ranges)
        ra, rl = orc.prune(am.detach().cpu(), lm.detach().cpu(), ranges.cpu())
        assert a.shape == (B, T, R, D) and a.stride(2) == 0
        assert torch.equal(a.cpu(), ra) and torch.equal(l.detach().cpu(), rl)
        w = torch.randn(B, T, R, D, dtype=dt, device="cuda")
        ((a + l) * w).sum().backward()
        lm_ref = lm.detach().cpu().clone().requires_grad_(True)
        am_ref = am.detach().cpu().clone().requires_grad_(True)
        ra, rl = orc.prune(am_ref, lm_ref, ranges.cpu())
        ((ra + rl) * w.cpu()).sum().backward()
        tol = 1e-5 if dt == torch.float32 else 1e-12
        assert_close(lm.grad, lm_ref.grad, tol, tol, "lm grad")
        assert_close(am.grad, am_ref.grad, tol, tol, "am grad")


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_small_pipeline_float64_vs_oracle(rnnt_type):
    """float64 leaves no room for rounding: every stage must agree to 1e-9."""
    wl = workloads.pipeline_workload("small", rnnt_type=rnnt_type, seed=4)
    out = run_pipeline(wl, rnnt_type, dtype=torch.float64)
    d = lambda x: x.double() if x.is_floating_point() else x  # noqa: E731
    am = d(wl["am"]).requires_grad_(True)
    lm = d(wl["lm"]).requires_grad_(True)
    enc = d(wl["enc"]).requires_grad_(True)
    dec = d(wl["dec"]).requires_grad_(True)
    W = d(wl["joiner_w"]).requires_grad_(True)
    bias = d(wl["joiner_b"]).requires_grad_(True)
    sym, bnd = wl["symbols"], wl["boundary"]
    ls, as_ = wl["lm_only_scale"], wl["am_only_scale"]
    px, py = orc.simple_logprobs(lm.detach(), am.detach(), sym, 0, rnnt_type, bnd, ls, as_)
    simple, (ox, oy) = orc.loss_smoothed(lm, am, sym, 0, ls, as_, bnd, rnnt_type, reduction="sum",
                                         return_grad=True)
    assert_close(out["px"], px, 1e-10, 1e-10, "px")
    assert_close(out["py"], py, 1e-10, 1e-10, "py")
    assert_close(out["occ_x"], ox, 0, 1e-9, "occ_x")
    assert_close(out["occ_y"], oy, 0, 1e-9, "occ_y")
    ranges = orc.prune_ranges(ox, oy, bnd, wl["s_range"])
    assert torch.equal(out["ranges"].cpu(), ranges)
    am_p, lm_p = orc.prune(enc, dec, ranges)
    logits = torch.nn.functional.linear(torch.tanh(am_p + lm_p), W, bias)
    logits.retain_grad()
    pruned = orc.loss_pruned(logits, sym, ranges, 0, bnd, rnnt_type, reduction="sum")
    (simple + pruned).backward()
    assert_close(out["simple"], simple, 1e-11, 0, "simple")
    assert_close(out["pruned"], pruned, 1e-11, 0, "pruned")
    for k, v in (("am_grad", am.grad), ("lm_grad", lm.grad), ("enc_grad", enc.grad),
                 ("dec_grad", dec.grad), ("logits_grad", logits.grad), ("w_grad", W.grad)):
        assert_close(out[k], v, 1e-8, 1e-9, k)


@pytest.mark.parametrize("joiner", ["torch", "fused"])
def test_c3_full_size_against_reference_summary(joiner):
    """The full pruned pipeline at B=64, T=500, S=100, C=500, s_range=5 against the
    summaries the reference wrote: losses, prune-range starts, strided samples; with the
    joiner in torch and on this library's pruned_joiner (what bench.py times)."""
    g = load_golden("c3_pipeline")
    wl = workloads.pipeline_workload("c3")
    out = run_pipeline(wl, "regular", joiner=joiner)
    assert_close(out["simple"], torch.tensor(g["simple"]), LOSS_RTOL, 0, "simple loss")

    assert_close(samp(out["px"]), g["px_sample"], 0, LATTICE_ATOL, "px")
    assert_close(samp(out["py"]), g["py_sample"], 0, LATTICE_ATOL, "py")
    assert_close(samp(out["occ_x"]), g["occ_x_sample"], 0, GRAD_ATOL, "occ_x")
    assert_close(samp(out["occ_y"]), g["occ_y_sample"], 0, GRAD_ATOL, "occ_y")
    assert_close(samp(out["am_grad"]), g["am_grad_sample"], 0, GRAD_ATOL, "am grad")
    assert_close(samp(out["lm_grad"]), g["lm_grad_sample"], 0, GRAD_ATOL, "lm grad")
    # end to end the ranges come from our own occupancies: a one-ulp difference
    # can move an argmax, so a small fraction of frames may differ (the
    # reference's own CPU and CUDA builds differ in the same way)
    s_begin = out["ranges"][:, :, 0].cpu()
    mismatch = (s_begin != g["s_begin"].to(torch.int64)).float().mean().item()
    assert mismatch < 0.01, mismatch
    assert_close(out["pruned"], torch.tensor(g["pruned"]), 5e-4, 0, "pruned loss (own ranges)")
    # ... and bit-exact on identical inputs: oracle on OUR occupancies
    ranges_oracle = orc.prune_ranges(out["occ_x"].cpu(), out["occ_y"].cpu(), wl["boundary"], 5)
    assert torch.equal(out["ranges"].cpu(), ranges_oracle)


def pruned_stage(wl, ranges, joiner):
    """Pruning -> joiner -> pruned loss -> backward on GIVEN ranges (regular type).
    joiner: "torch" (the reference's composition), "fused" (pruned_joiner) or "logprobs"
    (the single operator behind rnnt_loss_pruned_joiner, which never exposes logits)."""
    f = fr()
    enc = wl["enc"].cuda().requires_grad_(True)
    dec = wl["dec"].cuda().requires_grad_(True)
    W = wl["joiner_w"].cuda().requires_grad_(True)
    bias = wl["joiner_b"].cuda().requires_grad_(True)
    sym, bnd = wl["symbols"].cuda(), wl["boundary"].cuda()
    out = {}
    if joiner == "logprobs":
        ppx, ppy = f.get_rnnt_logprobs_pruned_joiner(
            am=enc.detach(), lm=dec.detach(), ranges=ranges, joiner_weight=W.detach(),
            joiner_bias=bias.detach(), symbols=sym, termination_symbol=0, boundary=bnd)
        pruned = f.rnnt_loss_pruned_joiner(am=enc, lm=dec, ranges=ranges, joiner_weight=W,
                                           joiner_bias=bias, symbols=sym, termination_symbol=0,
                                           boundary=bnd, reduction="sum")
        pruned.backward()
    else:
        logits = joiner_logits(joiner, enc, dec, ranges, W, bias)
        logits.retain_grad()
        ppx, ppy = f.get_rnnt_logprobs_pruned(logits=logits.detach(), symbols=sym, ranges=ranges,
                                              termination_symbol=0, boundary=bnd)
        pruned = f.rnnt_loss_pruned(logits=logits, symbols=sym, ranges=ranges,
                                    termination_symbol=0, boundary=bnd, reduction="sum")
        pruned.backward()
        out.update(logits=logits, logits_grad=logits.grad)
    out.update(pruned=pruned, pruned_px=ppx, pruned_py=ppy, enc_grad=enc.grad, dec_grad=dec.grad,
               w_grad=W.grad, b_grad=bias.grad)
    return out


def assert_as_close_as_the_reference(ours, g, key, atol):
    """ours against the reference's float32 sample of tensor `key`.  Where the reference
    also wrote a float64 sample, its own float32 rounding noise max|f32 - f64| is known;
    a difference from the float32 sample below twice that noise says nothing, so the
    bound is atol + 2 * noise (sums over all 160 000 joiner rows of a batch -- the
    weight, bias and decoder gradients -- carry noise far above 1e-4 in the reference
    itself)."""
    ref = g[key + "_sample"]
    noise = 0.0
    if key + "_f64_sample" in g:
        r64 = g[key + "_f64_sample"]
        fin = torch.isfinite(r64)
        noise = float((ref.double()[fin] - r64[fin]).abs().max())
    # ... plus float32 rounding of long sums in another order: 2e-6 of the largest entry
    scale = float(ref[torch.isfinite(ref)].abs().max())
    assert_close(samp(ours), ref, 0, atol + 2 * noise + 2e-6 * scale, key)
    return noise


def check_pruned_stage(out, g):
    """Pruned stage on the reference's own ranges: loss 1e-5 relative, lattices 1e-5,
    gradients 1e-4 absolute on top of the reference's own float32 noise."""
    assert_close(out["pruned"], torch.tensor(g["pruned"]), LOSS_RTOL, 0, "pruned loss")
    if "logits" in out:
        assert_close(samp(out["logits"]), g["logits_sample"], 0, LATTICE_ATOL, "logits")
    assert_close(samp(out["pruned_px"]), g["pruned_px_sample"], 0, LATTICE_ATOL, "pruned px")
    assert_close(samp(out["pruned_py"]), g["pruned_py_sample"], 0, LATTICE_ATOL, "pruned py")
    for k in ("logits_grad", "enc_grad", "dec_grad", "w_grad", "b_grad"):
        if k in out:
            assert_as_close_as_the_reference(out[k], g, k, GRAD_ATOL)


@pytest.mark.parametrize("joiner", ["torch", "fused", "logprobs"])
def test_c3_full_size_pruned_stage_on_reference_ranges(joiner):
    """Stage-wise at full size: with the reference's prune ranges injected the argmax
    no longer matters, so the pruned loss must agree to 1e-5 and the gradients of the
    logits, the encoder / decoder activations and the joiner's weights to 1e-4."""
    g = load_golden("c3_pipeline")
    wl = workloads.pipeline_workload("c3")
    ranges = (g["s_begin"].to(torch.int64).unsqueeze(-1) + torch.arange(g["s_range"])).cuda()
    check_pruned_stage(pruned_stage(wl, ranges, joiner), g)


@pytest.mark.parametrize("joiner", ["fused", "tensorcore"])
def test_c3_bench_step_matches_the_reference(joiner):
    """The step bench.py times (its make_step with the joiner it selects) on the same
    workload: loss and input gradients against the reference's summary."""
    import bench
    g = load_golden("c3_pipeline")
    wl = workloads.pipeline_workload("c3")
    step = bench.make_step(fr(), wl, joiner)
    t = {k: wl[k].cuda() for k in bench.TENSOR_KEYS}
    loss = step(t)
    # own ranges: a few frames may pick a neighbouring window (see the test above)
    assert_close(loss, torch.tensor(g["simple"] + g["pruned"]), 5e-4, 0, "simple + pruned")
    assert_as_close_as_the_reference(t["am"].grad, g, "am_grad", GRAD_ATOL)
    assert_as_close_as_the_reference(t["lm"].grad, g, "lm_grad", GRAD_ATOL)
    # a moved window changes the encoder gradient of its own frame only, and the decoder
    # gradient of the few rows it covers
    for k, allowed in (("enc", 0.02), ("dec", 0.3)):
        err = (samp(t[k].grad).cpu() - g[k + "_grad_sample"]).abs()
        assert (err > 1e-3).float().mean().item() < allowed, k


def test_c4_unpruned_against_reference_summary():
    g = load_golden("c4_unpruned")
    wl = workloads.config_c4()
    logits = wl["logits"].cuda().requires_grad_(True)
    loss = fr().rnnt_loss(logits=logits, symbols=wl["symbols"].cuda(), termination_symbol=0,
                          boundary=wl["boundary"].cuda(), reduction="sum")
    loss.backward()
    assert_close(loss, torch.tensor(g["loss"]), LOSS_RTOL, 0, "loss")
    if "torchaudio_loss" in g:
        assert_close(loss, torch.tensor(g["torchaudio_loss"]), LOSS_RTOL, 0, "loss vs torchaudio")
    flat = logits.grad.reshape(-1)
    assert_close(flat[:: max(1, flat.numel() // 4096)], g["logits_grad_sample"], 0, GRAD_ATOL,
                 "logits grad")


@pytest.mark.parametrize("joiner", ["torch", "fused", "logprobs"])
def test_c5_shape_against_reference_summary(joiner):
    """The large-vocabulary shape (T=400, S=60, C=5000, s_range=5, batch of 3) against
    vectors the reference itself wrote: simple stage, ranges bit for bit on the
    reference's occupancies, pruned stage on the reference's ranges.  Single lm
    gradients reach 3e2 here, where the reference's own float32 result is 1.2e-2 away
    from its float64 result: gradients are compared on top of that measured noise."""
    g = load_golden("c5_shape_pipeline")
    wl = workloads.pipeline_workload("c5", batch=3, seed=2)
    f = fr()
    sym, bnd = wl["symbols"].cuda(), wl["boundary"].cuda()
    am = wl["am"].cuda().requires_grad_(True)
    lm = wl["lm"].cuda().requires_grad_(True)
    px, py = f.get_rnnt_logprobs_smoothed(lm=lm.detach(), am=am.detach(), symbols=sym,
                                          termination_symbol=0, lm_only_scale=wl["lm_only_scale"],
                                          am_only_scale=wl["am_only_scale"], boundary=bnd)
    assert_close(samp(px), g["px_sample"], 0, LATTICE_ATOL, "px")
    assert_close(samp(py), g["py_sample"], 0, LATTICE_ATOL, "py")
    simple, (gx, gy) = f.rnnt_loss_smoothed(lm=lm, am=am, symbols=sym, termination_symbol=0,
                                            lm_only_scale=wl["lm_only_scale"],
                                            am_only_scale=wl["am_only_scale"], boundary=bnd,
                                            reduction="sum", return_grad=True)
    assert_close(simple, torch.tensor(g["simple"]), LOSS_RTOL, 0, "simple loss")
    assert_close(gx, g["occ_x"], 0, GRAD_ATOL, "occ_x")
    assert_close(gy, g["occ_y"], 0, GRAD_ATOL, "occ_y")
    simple.backward()
    assert_as_close_as_the_reference(am.grad, g, "am_grad", GRAD_ATOL)
    assert_as_close_as_the_reference(lm.grad, g, "lm_grad", GRAD_ATOL)
    ref_ranges = g["s_begin"].to(torch.int64).unsqueeze(-1) + torch.arange(g["s_range"])
    r = f.get_rnnt_prune_ranges(px_grad=g["occ_x"].cuda(), py_grad=g["occ_y"].cuda(), boundary=bnd,
                                s_range=wl["s_range"])
    assert torch.equal(r.cpu(), ref_ranges)
    check_pruned_stage(pruned_stage(wl, ref_ranges.cuda(), joiner), g)


def test_c5_shape_stagewise_vs_oracle():
    """The large-vocabulary shape (T=400, S=60, C=5000, s_range=5) on a batch of 2:
    large-vocabulary rows take the multi-warp log-softmax path.  Stage-wise
    against the CPU oracle with the oracle's occupancies, ranges and logits
    injected; gradients that reach 1e2 in magnitude are compared relatively."""
    wl = workloads.pipeline_workload("c5", batch=2, seed=2)
    f = fr()
    sym, bnd = wl["symbols"], wl["boundary"]
    ls, as_ = wl["lm_only_scale"], wl["am_only_scale"]
    am = wl["am"].clone().requires_grad_(True)
    lm = wl["lm"].clone().requires_grad_(True)
    ref_simple, (ox, oy) = orc.loss_smoothed(lm, am, sym, 0, ls, as_, bnd, reduction="sum",
                                             return_grad=True)
    ox, oy = ox.clone(), oy.clone()
    ref_simple.backward()
    cam = wl["am"].cuda().requires_grad_(True)
    clm = wl["lm"].cuda().requires_grad_(True)
    simple, (gx, gy) = f.rnnt_loss_smoothed(lm=clm, am=cam, symbols=sym.cuda(),
                                            termination_symbol=0, lm_only_scale=ls,
                                            am_only_scale=as_, boundary=bnd.cuda(),
                                            reduction="sum", return_grad=True)
    assert_close(simple, ref_simple.detach(), LOSS_RTOL, 0, "simple loss")
    assert_close(gx, ox, 0, GRAD_ATOL, "occ_x")
    assert_close(gy, oy, 0, GRAD_ATOL, "occ_y")
    simple.backward()
    assert_close(cam.grad, am.grad, 1e-4, GRAD_ATOL, "am grad")
    assert_close(clm.grad, lm.grad, 1e-4, GRAD_ATOL, "lm grad")
    # ranges on the oracle's occupancies: bit-exact
    ranges = orc.prune_ranges(ox, oy, bnd, wl["s_range"])
    r = f.get_rnnt_prune_ranges(px_grad=ox.cuda(), py_grad=oy.cuda(), boundary=bnd.cuda(),
                                s_range=wl["s_range"])
    assert torch.equal(r.cpu(), ranges)
    # pruned stage on the oracle's ranges and logits
    torch.manual_seed(9)
    logits = torch.randn(2, 400, 5, 5000).requires_grad_(True)
    ref_pruned = orc.loss_pruned(logits, sym, ranges, 0, bnd, reduction="sum")
    ref_pruned.backward()
    cl = logits.detach().cuda().requires_grad_(True)
    ppx, ppy = f.get_rnnt_logprobs_pruned(logits=cl.detach(), symbols=sym.cuda(), ranges=r,
                                          termination_symbol=0, boundary=bnd.cuda())
    rpx, rpy = orc.pruned_logprobs(logits.detach(), sym, ranges, 0, bnd)
    assert_close(ppx, rpx, 0, LATTICE_ATOL, "pruned px")
    assert_close(ppy, rpy, 0, LATTICE_ATOL, "pruned py")
    pruned = f.rnnt_loss_pruned(logits=cl, symbols=sym.cuda(), ranges=r, termination_symbol=0,
                                boundary=bnd.cuda(), reduction="sum")
    assert_close(pruned, ref_pruned.detach(), LOSS_RTOL, 0, "pruned loss")
    pruned.backward()
    assert_close(cl.grad, logits.grad, 0, GRAD_ATOL, "logits grad")


def test_provided_boundary_rows_skip_the_read_back():
    """provide_boundary_rows: same results, and the loss call does not synchronise
    on the boundary tensor (checked through torch's sync debug mode)."""
    wl = workloads.pipeline_workload("mini", "regular", seed=4)
    f = fr()
    lm, am, sym, bnd = (cu(wl[k]) for k in ("lm", "am", "symbols", "boundary"))
    ref = f.rnnt_loss_simple(lm=lm, am=am, symbols=sym, termination_symbol=0, boundary=bnd,
                             reduction="none")
    bnd2 = f.provide_boundary_rows(bnd.clone(), wl["boundary"])
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        out = f.rnnt_loss_simple(lm=lm, am=am, symbols=sym, termination_symbol=0, boundary=bnd2,
                                 reduction="none")
        r = f.get_rnnt_prune_ranges  # the s_range adjustment reads the rows too
    finally:
        torch.cuda.set_sync_debug_mode("default")
    assert torch.equal(out, ref)
    bnd2[0, 3] -= 1          # an in-place change drops the host copy
    from fast_rnnt_b200.mutual_information import _boundary_rows
    assert _boundary_rows(bnd2)[0][3] == int(wl["boundary"][0, 3]) - 1
