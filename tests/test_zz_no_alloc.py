"""The entry point for hosts that cannot allocate device memory.

Some programs that embed this library own a fixed set of device buffers and may
not ask for another one (all memory was carved up at start-up, or cudaMalloc is
banned after initialisation because it stalls every stream).  For them
frnnt_mi_fwd_bwd_noalloc runs the recursion forward and backward with its
per-cell weights in a 32 MiB region that is part of the library image instead
of a caller-provided scratch.  This test calls it straight through the C ABI,
twice in a row with different lattices (the region still holds the first call's
weights when the second starts), and requires the same scores and gradients as
the two-call path with a caller-allocated scratch.

Collected last on purpose (file name), so a run that stops at the first
failure has already gone through every other test.
"""
import ctypes

import pytest
import torch

from tests import workloads

pytestmark = pytest.mark.gpu

LIMIT = 32 << 20


def _call_noalloc(lib, px, py, boundary, ans_grad):
    from fast_rnnt_b200 import _lib
    B, S, T1 = px.shape
    T = py.shape[2]
    ans = torch.empty(B, dtype=px.dtype, device=px.device)
    gx, gy = torch.empty_like(px), torch.empty_like(py)
    rc = lib.frnnt_mi_fwd_bwd_noalloc(
        ctypes.c_int(_lib.dtype_code(px.dtype)), _lib.ptr(px), _lib.ptr(py), _lib.ptr(boundary),
        _lib.ptr(ans_grad), _lib.ptr(ans), _lib.ptr(gx), _lib.ptr(gy), B, S, T, int(T1 == T),
        _lib.stream_ptr(px.device))
    return rc, ans, gx, gy


def _call_two_step(px, py, boundary, ans_grad):
    from fast_rnnt_b200 import mutual_information as mi
    ans, _, branch = mi.mi_forward(px, py, boundary)
    gx, gy = mi.mi_backward_from_lattice(px, branch, boundary, ans_grad, py.shape)
    return ans, gx, gy


def test_noalloc_matches_two_step_path_twice_in_a_row():
    from fast_rnnt_b200 import _lib
    lib = _lib.lib()
    cases = [
        # a large lattice first, then a smaller one of another dtype and recursion
        # type: the second call finds the first call's weights in the region
        dict(B=24, S=100, T=300, dtype=torch.float32, modified=False, seed=1),
        dict(B=5, S=40, T=77, dtype=torch.float64, modified=True, seed=2),
        # lattices taller than one launch sweeps (256 float / 128 double rows): the row
        # blocks hand their edge rows over through the same region, on top of what the
        # calls before left there
        dict(B=4, S=300, T=200, dtype=torch.float32, modified=False, seed=3),
        dict(B=3, S=150, T=170, dtype=torch.float64, modified=True, seed=4),
    ]
    for c in cases:
        torch.manual_seed(c["seed"])
        B, S, T = c["B"], c["S"], c["T"]
        px = (torch.rand(B, S, T + (0 if c["modified"] else 1), dtype=c["dtype"]) * -4).cuda()
        py = (torch.rand(B, S + 1, T, dtype=c["dtype"]) * -4).cuda()
        import random
        bnd = workloads.random_mi_boundary(B, S, T, c["modified"], random.Random(c["seed"]),
                                           allow_empty=False).cuda()
        w = torch.linspace(0.5, 1.5, B, dtype=c["dtype"]).cuda()
        assert lib.frnnt_mi_lattice_bytes(_lib.dtype_code(c["dtype"]), B, S, T) <= LIMIT
        assert (S + 1 > lib.frnnt_mi_rows_per_block(_lib.dtype_code(c["dtype"]))) == (c["seed"] >= 3)
        rc, ans, gx, gy = _call_noalloc(lib, px, py, bnd, w)
        assert rc == 0, lib.frnnt_last_error()
        # from the second call on nothing may be taken from the device: the free memory
        # the driver reports stays what it was (torch's caching allocator serves the
        # outputs of _call_noalloc, so they are allocated once more up front)
        torch.cuda.synchronize()
        spare = [torch.empty_like(ans), torch.empty_like(px), torch.empty_like(py)]
        del spare
        free0 = torch.cuda.mem_get_info()[0]
        rc2, ans_b, gx_b, gy_b = _call_noalloc(lib, px, py, bnd, w)
        torch.cuda.synchronize()
        assert rc2 == 0 and torch.cuda.mem_get_info()[0] == free0
        assert torch.equal(ans_b, ans) and torch.equal(gx_b, gx) and torch.equal(gy_b, gy)
        ans2, gx2, gy2 = _call_two_step(px, py, bnd, w)
        rtol, atol = (1e-6, 1e-5) if c["dtype"] == torch.float32 else (1e-12, 1e-12)
        torch.testing.assert_close(ans, ans2, rtol=rtol, atol=atol)
        torch.testing.assert_close(gx, gx2, rtol=0, atol=atol)
        torch.testing.assert_close(gy, gy2, rtol=0, atol=atol)
        assert torch.isfinite(ans).all()


def test_noalloc_empty_batch_and_null_outputs():
    from fast_rnnt_b200 import _lib
    lib = _lib.lib()
    x = torch.zeros(64, device="cuda")
    sp = _lib.stream_ptr(x.device)
    # B == 0: nothing to do, nothing touched
    assert lib.frnnt_mi_fwd_bwd_noalloc(ctypes.c_int(0), None, None, None, None, None, None, None,
                                        0, 3, 4, 0, sp) == 0
    # a missing gradient buffer is refused before the forward sweep is launched
    rc = lib.frnnt_mi_fwd_bwd_noalloc(ctypes.c_int(0), _lib.ptr(x), _lib.ptr(x), None, _lib.ptr(x),
                                      _lib.ptr(x), None, _lib.ptr(x), 1, 3, 4, 0, sp)
    assert rc == -1 and b"px_grad" in lib.frnnt_last_error()


def test_noalloc_refuses_lattices_beyond_the_region():
    from fast_rnnt_b200 import _lib
    lib = _lib.lib()
    B, S, T = 64, 200, 900  # needs far more than 32 MiB of weights
    assert lib.frnnt_mi_lattice_bytes(0, B, S, T) > LIMIT
    px = torch.zeros(1, device="cuda")
    # refused on the host before any launch, so the tiny buffers are never touched
    rc = lib.frnnt_mi_fwd_bwd_noalloc(ctypes.c_int(0), _lib.ptr(px), _lib.ptr(px), None,
                                      _lib.ptr(px), _lib.ptr(px), _lib.ptr(px), _lib.ptr(px),
                                      B, S, T, 0, _lib.stream_ptr(px.device))
    assert rc == -2
    assert b"built-in region" in lib.frnnt_last_error()
