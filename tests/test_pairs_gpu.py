"""The fp16-pair tensor-core products on their own (csrc/joiner_pairs.cu:
frnnt_pairs_from_f32, frnnt_pair_matmul_nt, frnnt_pair_matmul_tn) through the C ABI,
against float64 matrix products.  Bound: 2e-6 of the largest |a|·|b| row product sum,
i.e. fp32-level accuracy (an fp16 or tf32 product would miss it by three orders)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

_vp, _ll, _int = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int


def planes(lib_mod, x, pitch):
    """x [rows][cols] float32 on the GPU -> (hi, lo, inv_scale); rows `pitch` halves apart."""
    L = lib_mod.lib()
    L.frnnt_pairs_scratch_floats.restype = ctypes.c_size_t
    rows, cols = x.shape
    hi = torch.zeros(rows, pitch, dtype=torch.float16, device=x.device)
    lo = torch.zeros_like(hi)
    inv = torch.zeros(1, dtype=torch.float32, device=x.device)
    scratch = torch.zeros(L.frnnt_pairs_scratch_floats(), dtype=torch.float32, device=x.device)
    lib_mod.call("frnnt_pairs_from_f32", lib_mod.ptr(x), _ll(rows), _int(cols), _ll(pitch), lib_mod.ptr(hi),
                 lib_mod.ptr(lo), lib_mod.ptr(inv), lib_mod.ptr(scratch), lib_mod.stream_ptr(x.device))
    return hi, lo, inv


def up8(n):
    return (n + 7) // 8 * 8


def bound(a, b):
    return 2e-6 * float((a.abs().double() @ b.abs().double().t()).max())


# M, N, K: one tile; ragged edges; several row tiles per CTA, odd numbers of row tiles, several
# K groups.  Outputs wider than 128 columns run on 128 x 256 tiles, narrower ones with more
# than 128 rows on 256 x 128 tiles, the rest on 128 x 128 tiles.
NT_SHAPES = [(128, 128, 64), (100, 72, 200), (700, 136, 96), (600, 128, 200), (2048, 512, 512),
             (1300, 260, 328), (40000, 500, 512)]


@pytest.mark.parametrize("M,N,K", NT_SHAPES)
@pytest.mark.parametrize("with_bias", [False, True])
def test_pair_matmul_nt(M, N, K, with_bias):
    from fast_rnnt_b200 import _lib
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(N, K, generator=g) * 0.05
    bias = torch.randn(N, generator=g) if with_bias else None
    ca, cb = a.cuda(), b.cuda()
    ah, al, ia = planes(_lib, ca, up8(K))
    bh, bl, ib = planes(_lib, cb, up8(K))
    Np = (N + 3) // 4 * 4
    d = torch.full((M, Np), float("nan"), device="cuda")
    cbias = None
    if with_bias:
        cbias = torch.zeros(Np, device="cuda")
        cbias[:N] = bias.cuda()
    _lib.call("frnnt_pair_matmul_nt", _lib.ptr(ah), _lib.ptr(al), _lib.ptr(bh), _lib.ptr(bl), _lib.ptr(ia),
              _lib.ptr(ib), _lib.ptr(cbias), _lib.ptr(d), _int(M), _int(Np), _int(K), _ll(up8(K)), _ll(up8(K)),
              _lib.stream_ptr(d.device))
    ref = a.double() @ b.double().t()
    if with_bias:
        ref = ref + bias.double()
    got = d[:, :N].cpu().double()
    assert torch.isfinite(got).all()
    err = float((got - ref).abs().max())
    assert err <= bound(a, b), (err, bound(a, b))


# M, N, R: out [M][N] = a^T b over R rows (split over the CTAs when R is long)
TN_SHAPES = [(128, 128, 64), (72, 200, 1000), (500, 512, 40000), (264, 136, 5000), (300, 100, 3000)]


@pytest.mark.parametrize("M,N,R", TN_SHAPES)
def test_pair_matmul_tn(M, N, R):
    from fast_rnnt_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(M + N + R)
    a = torch.randn(R, M, generator=g)
    b = torch.randn(R, N, generator=g) * 0.05
    ca, cb = a.cuda(), b.cuda()
    ah, al, ia = planes(_lib, ca, up8(M))
    bh, bl, ib = planes(_lib, cb, up8(N))
    splits = L.frnnt_pair_matmul_tn_splits(_int(M), _int(N), _ll(R))
    Np = (N + 3) // 4 * 4
    d = torch.full((M, Np), float("nan"), device="cuda")
    partials = torch.zeros(max(1, splits) * M * Np, device="cuda")
    _lib.call("frnnt_pair_matmul_tn", _lib.ptr(ah), _lib.ptr(al), _lib.ptr(bh), _lib.ptr(bl), _lib.ptr(ia),
              _lib.ptr(ib), _lib.ptr(d), _lib.ptr(partials), _int(M), _int(Np), _ll(R), _ll(up8(M)), _ll(up8(N)),
              _lib.stream_ptr(d.device))
    ref = a.double().t() @ b.double()
    got = d[:, :N].cpu().double()
    assert torch.isfinite(got).all()
    err = float((got - ref).abs().max())
    bnd = 2e-6 * float((a.abs().double().t() @ b.abs().double()).max())
    assert err <= bnd, (err, bnd)
