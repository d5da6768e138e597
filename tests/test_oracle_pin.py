"""Pins the CPU oracle (oracle/) to the reference: every function is checked
against golden vectors that the reference project itself produced
(tests/golden/make_golden.py), and the plain-C recursion is compared bit for
bit with the reference's compiled CPU extension where that exists."""
import random

import pytest
import torch

from oracle import rnnt_oracle as orc
from tests import workloads
from tests.conftest import load_golden, reference_extension

# float32 results of the same torch ops can differ in the last bits between
# CPU models (different GEMM kernels); on the machine that wrote the vectors the
# agreement is exact.
RTOL, ATOL = 2e-6, 2e-6


def close(a, b, rtol=RTOL, atol=ATOL):
    a, b = torch.as_tensor(a), torch.as_tensor(b)
    assert a.shape == b.shape, (a.shape, b.shape)
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin)
    assert torch.equal(a[~fin], b[~fin])
    torch.testing.assert_close(a[fin], b[fin], rtol=rtol, atol=atol)


def test_basic_known_answers():
    g = load_golden("basic")
    lm, am, symbols, blank = workloads.reference_basic_tensors()
    px, py = orc.simple_logprobs(lm, am, symbols, blank)
    close(px, g["px"])
    close(py, g["py"])
    close(-orc.mi_recursion(px, py), g["neg_m"])
    close(orc.loss_simple(lm, am, symbols, blank, reduction="none"), g["simple"])
    close(orc.loss_smoothed(lm, am, symbols, blank, 0.0, 0.0, reduction="none"), g["smoothed0"])
    close(orc.loss_smoothed(lm, am, symbols, blank, 0.0, 0.333, reduction="none"),
          g["smoothed_am0333"])
    logits = am.unsqueeze(2) + lm.unsqueeze(1)
    close(orc.loss_joint(logits, symbols, blank, reduction="none"), g["joint"])
    # the reference's own test requires all of these to agree with each other
    # and with torchaudio (rnnt_loss_test.py:97-153)
    for k in ("simple", "smoothed0", "joint", "torchaudio"):
        if k in g:
            torch.testing.assert_close(g[k], g["neg_m"], rtol=1e-5, atol=1e-8)


@pytest.mark.parametrize("name", list(workloads.MI_SMALL_CASES))
def test_mi_small(name):
    g = load_golden("mi_" + name)
    px, py = g["px"].clone().requires_grad_(True), g["py"].clone().requires_grad_(True)
    boundary = g["boundary"] if g["boundary"].numel() else None
    scores, (gx, gy) = orc.mi_recursion(px, py, boundary, return_grad=True)
    assert torch.equal(scores.detach(), g["scores"])
    assert torch.equal(gx, g["occ_x"]) and torch.equal(gy, g["occ_y"])
    (scores * g["w"]).sum().backward()
    assert torch.equal(px.grad, g["px_grad"]) and torch.equal(py.grad, g["py_grad"])
    # in-place rescaling of the returned occupancies (mutual_information.py:176-181)
    assert torch.equal(gx, g["px_grad"])
    j = orc.joint_mi((g["px"] * 0.25, g["px"] * 0.75), (g["py"] * 0.25, g["py"] * 0.75), boundary)
    close(j, g["joint"], rtol=1e-5, atol=1e-5)


def test_c_recursion_bitwise_vs_reference_extension():
    ext = reference_extension()
    if ext is None:
        pytest.skip("reference CPU extension not built here (make -C oracle ref)")
    rng = random.Random(3)
    torch.manual_seed(3)
    for it in range(40):
        B, S, T = rng.randint(1, 6), rng.randint(1, 20), rng.randint(1, 120)
        modified = rng.random() < 0.5
        if modified and T < S:
            T = S + rng.randint(0, 10)
        for dt in (torch.float32, torch.float64):
            px = torch.rand(B, S, T + (0 if modified else 1), dtype=dt) * -6
            py = torch.rand(B, S + 1, T, dtype=dt) * -6
            bnd = (workloads.random_mi_boundary(B, S, T, modified, rng)
                   if rng.random() < 0.7 else None)
            # -inf only where the total score stays finite (same rule as the
            # reference's own test, mutual_information_test.py:103-104): with a
            # -inf score the reference prints a diagnostic that crashes in this image.
            if S > 1 and bnd is None and not modified and rng.random() < 0.5:
                px[:, :, -1] = float("-inf")
            p, ans = orc.mi_forward_raw(px, py, bnd)
            ones = torch.ones(B, dtype=dt)
            gx, gy = orc.mi_backward_raw(px, py, bnd, p, ones)
            p2 = torch.empty(B, S + 1, T + 1, dtype=dt)
            ans2 = ext.mutual_information_forward(px, py, bnd, p2)
            gx2, gy2 = ext.mutual_information_backward(px, py, bnd, p2, ones)
            assert torch.equal(ans, ans2) and torch.equal(gx, gx2) and torch.equal(gy, gy2)


def _run_oracle_pipeline(wl, rnnt_type):
    am = wl["am"].clone().requires_grad_(True)
    lm = wl["lm"].clone().requires_grad_(True)
    enc = wl["enc"].clone().requires_grad_(True)
    dec = wl["dec"].clone().requires_grad_(True)
    W = wl["joiner_w"].clone().requires_grad_(True)
    bias = wl["joiner_b"].clone().requires_grad_(True)
    sym, bnd, blank = wl["symbols"], wl["boundary"], wl["blank"]
    ls, as_ = wl["lm_only_scale"], wl["am_only_scale"]
    px, py = orc.simple_logprobs(lm.detach(), am.detach(), sym, blank, rnnt_type, bnd, ls, as_)
    simple, (ox, oy) = orc.loss_smoothed(lm, am, sym, blank, ls, as_, bnd, rnnt_type,
                                         reduction="sum", return_grad=True)
    occ_x, occ_y = ox.clone(), oy.clone()
    ranges = orc.prune_ranges(ox, oy, bnd, wl["s_range"])
    am_p, lm_p = orc.prune(enc, dec, ranges)
    logits = torch.nn.functional.linear(torch.tanh(am_p + lm_p), W, bias)
    logits.retain_grad()
    ppx, ppy = orc.pruned_logprobs(logits.detach(), sym, ranges, blank, bnd, rnnt_type)
    pruned = orc.loss_pruned(logits, sym, ranges, blank, bnd, rnnt_type, reduction="sum")
    (simple + pruned).backward()
    return dict(simple=simple, pruned=pruned, s_begin=ranges[:, :, 0], s_range=ranges.shape[2],
                px=px, py=py, occ_x=occ_x, occ_y=occ_y, pruned_px=ppx, pruned_py=ppy,
                am_grad=am.grad, lm_grad=lm.grad, enc_grad=enc.grad, dec_grad=dec.grad,
                logits=logits, logits_grad=logits.grad, w_grad=W.grad, b_grad=bias.grad)


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_mini_pipeline_all_stages(rnnt_type):
    g = load_golden("pipeline_mini_" + rnnt_type)
    wl = workloads.pipeline_workload("mini", rnnt_type=rnnt_type)
    for k in ("am", "lm", "enc", "dec", "joiner_w", "symbols", "boundary"):
        assert torch.equal(wl[k], g[k]), f"seeded input {k} differs from the stored one"
    out = _run_oracle_pipeline(wl, rnnt_type)
    assert out["s_range"] == g["s_range"]
    for k in ("px", "py", "occ_x", "occ_y", "pruned_px", "pruned_py"):
        close(out[k], g[k], rtol=1e-5, atol=1e-5)
    close(out["simple"], g["simple"], rtol=1e-6, atol=1e-4)
    close(out["pruned"], g["pruned"], rtol=1e-6, atol=1e-4)
    for k in ("am_grad", "lm_grad", "enc_grad", "dec_grad", "logits_grad", "w_grad", "b_grad"):
        close(out[k], g[k], rtol=1e-4, atol=1e-5)
    # integer stage on the REFERENCE's own occupancies: bit-exact
    ranges = orc.prune_ranges(g["occ_x"], g["occ_y"], g["boundary"], wl["s_range"])
    assert torch.equal(ranges[:, :, 0], g["s_begin"].to(torch.int64))
    # pruned stage on the reference's ranges and logits
    rg = g["s_begin"].to(torch.int64).unsqueeze(-1) + torch.arange(g["s_range"])
    ppx, ppy = orc.pruned_logprobs(g["logits"], g["symbols"], rg, 0, g["boundary"], rnnt_type)
    close(ppx, g["pruned_px"])
    close(ppy, g["pruned_py"])


def test_simple_variants():
    g = load_golden("simple_variants_mini")
    wl = workloads.pipeline_workload("mini")
    for rnnt_type in ("regular", "modified", "constrained"):
        am = wl["am"].clone().requires_grad_(True)
        lm = wl["lm"].clone().requires_grad_(True)
        loss = orc.loss_simple(lm, am, wl["symbols"], 0, wl["boundary"], rnnt_type,
                               delay_penalty=0.01, reduction="none")
        loss.sum().backward()
        close(loss, g[f"simple_dp_{rnnt_type}"], rtol=1e-6, atol=1e-5)
        close(am.grad, g[f"simple_dp_{rnnt_type}_am_grad"], rtol=1e-4, atol=1e-5)
        close(lm.grad, g[f"simple_dp_{rnnt_type}_lm_grad"], rtol=1e-4, atol=1e-5)
        am = wl["am"].clone().requires_grad_(True)
        lm = wl["lm"].clone().requires_grad_(True)
        loss = orc.loss_smoothed(lm, am, wl["symbols"], 0, 0.1, 0.2, wl["boundary"], rnnt_type,
                                 reduction="mean")
        loss.backward()
        close(loss, g[f"smoothed_{rnnt_type}"], rtol=1e-6, atol=1e-5)
        close(am.grad, g[f"smoothed_{rnnt_type}_am_grad"], rtol=1e-4, atol=1e-6)
        close(lm.grad, g[f"smoothed_{rnnt_type}_lm_grad"], rtol=1e-4, atol=1e-6)


def test_c1_simple_loss():
    g = load_golden("c1_simple")
    wl = workloads.config_c1()
    assert torch.equal(wl["boundary"], g["boundary"]) and torch.equal(wl["symbols"], g["symbols"])
    am = wl["am"].clone().requires_grad_(True)
    lm = wl["lm"].clone().requires_grad_(True)
    px, py = orc.simple_logprobs(lm.detach(), am.detach(), wl["symbols"], 0, "regular",
                                 wl["boundary"])
    close(px, g["px"], rtol=1e-5, atol=1e-5)
    close(py, g["py"], rtol=1e-5, atol=1e-5)
    loss, (gx, gy) = orc.loss_simple(lm, am, wl["symbols"], 0, wl["boundary"], reduction="sum",
                                     return_grad=True)
    close(loss, g["loss"], rtol=1e-6, atol=1e-3)
    close(gx, g["occ_x"], rtol=1e-4, atol=1e-5)
    close(gy, g["occ_y"], rtol=1e-4, atol=1e-5)
    loss.backward()
    close(am.grad, g["am_grad"], rtol=1e-4, atol=1e-5)
    close(lm.grad, g["lm_grad"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("rnnt_type", ["regular", "modified", "constrained"])
def test_joint_small(rnnt_type):
    g = load_golden("joint_small_" + rnnt_type)
    logits = g["logits"].clone().requires_grad_(True)
    px, py = orc.joint_logprobs(logits.detach(), g["symbols"], g["blank"], g["boundary"], rnnt_type)
    close(px, g["px"])
    close(py, g["py"])
    loss = orc.loss_joint(logits, g["symbols"], g["blank"], g["boundary"], rnnt_type,
                          delay_penalty=0.02, reduction="none")
    loss.sum().backward()
    close(loss, g["loss"], rtol=1e-6, atol=1e-5)
    close(logits.grad, g["logits_grad"], rtol=1e-4, atol=1e-6)


def test_prune_range_edge_cases():
    g = load_golden("prune_edges")
    for tag in workloads.prune_edge_cases():
        r = orc.prune_ranges(g[tag + "_occ_x"], g[tag + "_occ_y"], g[tag + "_boundary"],
                             int(g[tag + "_s_range_in"]))
        assert r.dtype == torch.int64
        assert torch.equal(r, g[tag + "_ranges"]), tag


def test_c2_full_size_scores():
    g = load_golden("c2_mi")
    for tag, wb in (("full", False), ("bounded", True)):
        px, py, bnd = workloads.config_c2(wb)
        assert torch.equal(px.reshape(-1)[:: max(1, px.numel() // 4096)], g[tag + "_px_sample"])
        scores, (gx, gy) = orc.mi_recursion(px, py, bnd, return_grad=True)
        assert torch.equal(scores, g[tag + "_scores"])
        assert abs(gx.double().sum().item() - g[tag + "_occ_x_sum"]) < 1e-6
