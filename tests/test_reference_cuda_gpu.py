"""Our mutual-information kernels next to the reference's own CUDA kernels
(fast_rnnt/csrc/mutual_information_cuda.cu), compiled for sm_100a from the sources
where they lie by `make -C oracle ref_cuda` into oracle/_ref/cuda/ (a 14-minute nvcc
run, so it is not part of the regular build; the tests skip when the module is absent).

Scores must agree to float32 rounding.  The occupancies may differ by up to ~1e-3:
the reference's CUDA backward uses a different formulation from its CPU backward
(independent exps and product recurrences, mutual_information_cuda.cu:565-631, against
term2 = 1 - term1 style sums, mutual_information_cpu.cu:199-212), and this library
follows the CPU one, against which it is held to 1e-5.
"""
import importlib.util
import os

import pytest
import torch

from tests import workloads

pytestmark = pytest.mark.gpu

_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                   "cuda", "_fast_rnnt.so")


@pytest.fixture(scope="module")
def ref_cuda():
    if not os.path.exists(_SO):
        pytest.skip("the reference's CUDA extension has not been built (make -C oracle ref_cuda)")
    spec = importlib.util.spec_from_file_location("_fast_rnnt", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.with_cuda()
    return mod


def _ours(px, py, bnd):
    from fast_rnnt_b200 import mutual_information as mi
    ans, _, lattice = mi.mi_forward(px, py, bnd)
    ones = torch.ones(px.shape[0], device=px.device, dtype=px.dtype)
    gx, gy = mi.mi_backward_from_lattice(px, lattice, bnd, ones, py.shape)
    return ans, gx, gy


def _theirs(ref, px, py, bnd):
    B, S, _ = px.shape
    T = py.shape[2]
    p = torch.empty(B, S + 1, T + 1, device=px.device, dtype=px.dtype)
    ans = ref.mutual_information_forward(px, py, bnd, p)
    ones = torch.ones(B, device=px.device, dtype=px.dtype)
    gx, gy = ref.mutual_information_backward(px, py, bnd, p, ones)
    return ans, gx, gy


@pytest.mark.parametrize("with_boundary", [False, True])
def test_config2_against_the_reference_cuda_kernels(ref_cuda, with_boundary):
    px, py, bnd = workloads.config_c2(with_boundary)
    px, py = px.cuda(), py.cuda()
    bnd = bnd.cuda() if bnd is not None else None
    ans, gx, gy = _ours(px, py, bnd)
    ans_r, gx_r, gy_r = _theirs(ref_cuda, px, py, bnd)
    torch.testing.assert_close(ans, ans_r, rtol=1e-6, atol=0)
    torch.testing.assert_close(gx, gx_r, rtol=0, atol=3e-3)
    torch.testing.assert_close(gy, gy_r, rtol=0, atol=3e-3)
    # both are occupancies: every row s < S_b is crossed exactly once, every frame once
    if bnd is None:
        torch.testing.assert_close(gx.sum(dim=2), gx_r.sum(dim=2), rtol=0, atol=2e-3)


def test_modified_and_small_against_the_reference_cuda_kernels(ref_cuda):
    torch.manual_seed(3)
    for (B, S, T, modified) in ((3, 9, 13, True), (2, 40, 70, False), (2, 33, 33, True)):
        px = (torch.rand(B, S, T + (0 if modified else 1)) * -3).cuda()
        py = (torch.rand(B, S + 1, T) * -3).cuda()
        ans, gx, gy = _ours(px, py, None)
        ans_r, gx_r, gy_r = _theirs(ref_cuda, px, py, None)
        torch.testing.assert_close(ans, ans_r, rtol=1e-6, atol=0)
        torch.testing.assert_close(gx, gx_r, rtol=0, atol=3e-3)
        torch.testing.assert_close(gy, gy_r, rtol=0, atol=3e-3)
