"""GPU parity of the mutual-information recursion (csrc/mi.cu through the C ABI)
against the CPU oracle and the reference-written golden vectors.

Tolerances (float32): scores 1e-6 relative, occupancies / gradients 1e-5
absolute (the target for this stage; the end-to-end bar is 1e-4).  float64:
1e-12.
"""
import random

import pytest
import torch

from oracle import rnnt_oracle as orc
from tests import workloads
from tests.conftest import load_golden

pytestmark = pytest.mark.gpu


def fr():
    import fast_rnnt_b200
    return fast_rnnt_b200


def tol(dtype):
    return (1e-6, 1e-5) if dtype == torch.float32 else (1e-12, 1e-12)


def assert_close(a, b, rtol, atol, what=""):
    a, b = torch.as_tensor(a).detach().cpu(), torch.as_tensor(b).detach().cpu()
    b = b.to(a.dtype)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin), f"{what}: finiteness pattern differs"
    assert torch.equal(a[~fin], b[~fin]), f"{what}: non-finite values differ"
    err = (a[fin] - b[fin]).abs()
    bound = atol + rtol * b[fin].abs()
    if not bool((err <= bound).all()):
        idx = int((err - bound).argmax())
        raise AssertionError(f"{what}: max abs err {err.max().item():.3e}; worst: got "
                             f"{a[fin][idx].item()!r} want {b[fin][idx].item()!r}")


@pytest.mark.parametrize("name", list(workloads.MI_SMALL_CASES))
def test_mi_golden(name):
    g = load_golden("mi_" + name)
    dt = g["px"].dtype
    rtol, atol = tol(dt)
    px = g["px"].cuda().requires_grad_(True)
    py = g["py"].cuda().requires_grad_(True)
    boundary = g["boundary"].cuda() if g["boundary"].numel() else None
    scores, (gx, gy) = fr().mutual_information_recursion(px, py, boundary, return_grad=True)
    assert_close(scores, g["scores"], rtol, atol * 10, "scores")
    assert_close(gx, g["occ_x"], 0, atol, "occ_x")
    assert_close(gy, g["occ_y"], 0, atol, "occ_y")
    (scores * g["w"].cuda()).sum().backward()
    assert_close(px.grad, g["px_grad"], 0, 2 * atol, "px.grad")
    assert_close(py.grad, g["py_grad"], 0, 2 * atol, "py.grad")
    # the occupancies handed out by return_grad are rescaled in place by backward
    assert torch.equal(gx, px.grad)
    j = fr().joint_mutual_information_recursion(
        (g["px"].cuda() * 0.25, g["px"].cuda() * 0.75),
        (g["py"].cuda() * 0.25, g["py"].cuda() * 0.75), boundary)
    assert_close(j, g["joint"], 1e-5, 1e-4 if dt == torch.float32 else 1e-10, "joint")


SIZES = [(1, 1, 1), (2, 1, 7), (3, 5, 1), (2, 31, 40), (2, 32, 33), (3, 33, 31), (2, 63, 70),
         (2, 64, 64), (2, 65, 100), (1, 100, 37), (2, 127, 130), (1, 128, 20), (2, 200, 210),
         (1, 255, 256), (4, 17, 300), (2, 0, 9),
         # taller than one launch holds (256 float rows, 128 double rows): row blocks
         (2, 256, 40), (3, 300, 310), (1, 600, 100), (2, 513, 64)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("modified", [False, True])
def test_mi_random_vs_oracle(dtype, modified):
    rng = random.Random(17 + modified)
    torch.manual_seed(5)
    rtol, atol = tol(dtype)
    for (B, S, T) in SIZES:
        if modified and T < S:
            T = S + rng.randint(0, 5)
        for kind in ("none", "random", "full"):
            px = torch.rand(B, S, T + (0 if modified else 1), dtype=dtype) * -4
            py = torch.rand(B, S + 1, T, dtype=dtype) * -4
            if kind == "random":
                bnd = workloads.random_mi_boundary(B, S, T, modified, rng)
            elif kind == "full":
                bnd = torch.tensor([[0, 0, S, T]] * B, dtype=torch.int64)
            else:
                bnd = None
            if not modified and kind != "random" and S > 1:
                px[:, :, -1] = float("-inf")
            p_ref, ans_ref = orc.mi_forward_raw(px, py, bnd)
            w = torch.linspace(0.5, 1.5, B, dtype=dtype)
            gx_ref, gy_ref = orc.mi_backward_raw(px, py, bnd, p_ref, w)
            from fast_rnnt_b200 import mutual_information as mi
            cb = bnd.cuda() if bnd is not None else None
            ans, p, branch = mi.mi_forward(px.cuda(), py.cuda(), cb, want_p=True)
            what = f"B={B} S={S} T={T} mod={modified} bnd={kind} {dtype}"
            assert_close(ans, ans_ref, rtol, atol * 10, "ans " + what)
            # p is defined inside the boundary boxes only
            for b in range(B):
                s0, t0, s1, t1 = (0, 0, S, T) if bnd is None else bnd[b].tolist()
                assert_close(p[b, s0:s1 + 1, t0:t1 + 1], p_ref[b, s0:s1 + 1, t0:t1 + 1], rtol,
                             atol * 10, "p " + what)
            gx, gy = mi.mi_backward_from_lattice(px.cuda(), branch, cb, w.cuda(), py.shape)
            assert_close(gx, gx_ref, 0, 2 * atol, "px_grad " + what)
            assert_close(gy, gy_ref, 0, 2 * atol, "py_grad " + what)
            # the entry point that mirrors the reference's backward(px, py, boundary, p, ans_grad)
            gx2, gy2, origin = mi.mi_backward_from_p(px.cuda(), py.cuda(), cb, p_ref.cuda(), w.cuda(),
                                                     want_origin_grad=True)
            assert_close(gx2, gx_ref, 0, 2 * atol, "px_grad(p) " + what)
            assert_close(gy2, gy_ref, 0, 2 * atol, "py_grad(p) " + what)
            fin = torch.isfinite(ans_ref)
            assert_close(origin.cpu()[fin], w[fin], 1e-4 if dtype == torch.float32 else 1e-10, 0,
                         "origin grad " + what)
            # determinism: a second run is bit-identical
            ans_b, _, branch_b = mi.mi_forward(px.cuda(), py.cuda(), cb, want_p=False)
            gx_b, gy_b = mi.mi_backward_from_lattice(px.cuda(), branch_b, cb, w.cuda(), py.shape)
            assert torch.equal(ans, ans_b) and torch.equal(gx, gx_b) and torch.equal(gy, gy_b)


def test_mi_c2_full_size():
    g = load_golden("c2_mi")
    for tag, wb in (("full", False), ("bounded", True)):
        px, py, bnd = workloads.config_c2(wb)
        cb = bnd.cuda() if bnd is not None else None
        scores, (gx, gy) = fr().mutual_information_recursion(px.cuda(), py.cuda(), cb,
                                                            return_grad=True)
        assert_close(scores, g[tag + "_scores"], 1e-6, 0, "scores " + tag)
        step = max(1, gx.numel() // 4096)
        assert_close(gx.reshape(-1)[::step], g[tag + "_occ_x_sample"], 0, 1e-5, "occ_x " + tag)
        step = max(1, gy.numel() // 4096)
        assert_close(gy.reshape(-1)[::step], g[tag + "_occ_y_sample"], 0, 1e-5, "occ_y " + tag)
        # occupancy conservation: every path crosses each anti-diagonal once, so
        # per utterance sum(px_grad) = S_b and sum(py_grad) = T_b
        Sb = bnd[:, 2] if bnd is not None else torch.full((px.shape[0],), px.shape[1])
        Tb = bnd[:, 3] if bnd is not None else torch.full((px.shape[0],), py.shape[2])
        torch.testing.assert_close(gx.sum(dim=(1, 2)).cpu(), Sb.float(), rtol=1e-4, atol=1e-3)
        torch.testing.assert_close(gy.sum(dim=(1, 2)).cpu(), Tb.float(), rtol=1e-4, atol=1e-3)


def test_errors_are_reported():
    from fast_rnnt_b200 import FrnntError, mutual_information as mi
    from fast_rnnt_b200 import _lib
    px = torch.zeros(1, 300, 5, device="cuda")
    py = torch.zeros(1, 301, 4, device="cuda")
    ans = torch.zeros(1, device="cuda")
    # a lattice taller than one launch holds needs the scratch
    with pytest.raises(FrnntError, match="lattice scratch"):
        _lib.call("frnnt_mi_forward", 0, _lib.ptr(px), _lib.ptr(py), None, None, _lib.ptr(ans),
                  None, 1, 300, 4, 0, None)
    with pytest.raises(FrnntError, match="ans is NULL"):
        _lib.call("frnnt_mi_forward", 0, _lib.ptr(px), _lib.ptr(py), None, None, None,
                  None, 1, 300, 4, 0, None)
    with pytest.raises(TypeError):
        mi.mi_forward(px.half(), py.half(), None)
