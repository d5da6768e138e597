"""Mutual-information recursion on the GPU: drop-in for
fast_rnnt/python/fast_rnnt/mutual_information.py of the reference.

Same signatures and semantics (including the in-place rescaling of the
occupancies returned by ``return_grad=True`` when the loss is back-propagated,
reference mutual_information.py:165-181); the arithmetic runs in
libfrnnt_sm100.so (csrc/mi.cu).
"""
from typing import List, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor

from . import _lib
from ._lib import _c_int


def _boundary_rows(boundary: Tensor):
    """Host copy of the boundary rows, cached on the tensor so that the
    validations along one loss call share a single device-to-host copy."""
    key = (boundary.data_ptr(), boundary._version)
    cached = getattr(boundary, "_frnnt_rows", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    rows = boundary.tolist()
    try:
        boundary._frnnt_rows = (key, rows)
    except Exception:
        pass
    return rows


def provide_boundary_rows(boundary: Tensor, rows) -> Tensor:
    """Hands the library a host copy of ``boundary`` (a list of B rows
    ``[s_begin, t_begin, s_end, t_end]`` or a CPU tensor) that the caller already
    has -- a data loader builds the boundaries on the host before it uploads them.
    The range checks of the loss functions and the ``s_range`` adjustment of
    ``get_rnnt_prune_ranges`` (the reference reads the device tensor back for them,
    fast_rnnt/python/fast_rnnt/mutual_information.py:277-288, rnnt_loss.py:699-706)
    then need no device-to-host copy and no synchronisation.  The caller vouches
    that ``rows`` equals the tensor's content; the copy is dropped as soon as the
    tensor is modified in place.  No counterpart in the reference.  Returns
    ``boundary``."""
    rows = rows.tolist() if isinstance(rows, Tensor) else [[int(v) for v in r] for r in rows]
    assert len(rows) == boundary.shape[0] and all(len(r) == 4 for r in rows)
    boundary._frnnt_rows = ((boundary.data_ptr(), boundary._version), rows)
    return boundary


def mi_forward(px: Tensor, py: Tensor, boundary: Optional[Tensor], want_p: bool = False,
               want_lattice: bool = True):
    """Raw forward sweep: returns (ans [B], p or None, lattice scratch or None)."""
    B, S, T1 = px.shape
    T = py.shape[2]
    modified = int(T1 == T)
    dt = _lib.dtype_code(px.dtype)
    dev = px.device
    with torch.cuda.device(dev):
        ans = torch.empty(B, dtype=px.dtype, device=dev)
        p = torch.empty(B, S + 1, T + 1, dtype=px.dtype, device=dev) if want_p else None
        lattice = None
        # a lattice taller than one launch holds is swept in row blocks, which
        # hand the row above each block over through the scratch
        if want_lattice or S + 1 > _lib.lib().frnnt_mi_rows_per_block(dt):
            nbytes = _lib.lib().frnnt_mi_lattice_bytes(dt, B, S, T)
            lattice = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        _lib.call("frnnt_mi_forward", _c_int(dt), _lib.ptr(px), _lib.ptr(py), _lib.ptr(boundary),
                  _lib.ptr(p), _lib.ptr(ans), _lib.ptr(lattice), B, S, T, modified,
                  _lib.stream_ptr(dev))
    return ans, p, lattice


def mi_backward_from_lattice(px: Tensor, lattice: Tensor, boundary: Optional[Tensor],
                             ans_grad: Tensor, py_shape):
    """Reverse sweep from the diagonal-major lattice written by mi_forward."""
    B, S, T1 = px.shape
    T = py_shape[2]
    modified = int(T1 == T)
    dev = px.device
    with torch.cuda.device(dev):
        px_grad = torch.empty_like(px)
        py_grad = torch.empty(py_shape, dtype=px.dtype, device=dev)
        _lib.call("frnnt_mi_backward_from_lattice", _c_int(_lib.dtype_code(px.dtype)),
                  _lib.ptr(px), _lib.ptr(lattice), _lib.ptr(boundary), _lib.ptr(ans_grad),
                  _lib.ptr(px_grad), _lib.ptr(py_grad), None, B, S, T, modified,
                  _lib.stream_ptr(dev))
    return px_grad, py_grad


def mi_backward_from_p(px: Tensor, py: Tensor, boundary: Optional[Tensor], p: Tensor,
                       ans_grad: Tensor, want_origin_grad: bool = False):
    """Reverse sweep from a lattice ``p`` in the reference's layout (the
    counterpart of ``_fast_rnnt.mutual_information_backward``)."""
    B, S, T1 = px.shape
    T = py.shape[2]
    modified = int(T1 == T)
    dt = _lib.dtype_code(px.dtype)
    dev = px.device
    with torch.cuda.device(dev):
        nbytes = _lib.lib().frnnt_mi_lattice_bytes(dt, B, S, T)
        lattice = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
        px_grad = torch.empty_like(px)
        py_grad = torch.empty_like(py)
        origin = torch.zeros(B, dtype=px.dtype, device=dev) if want_origin_grad else None
        _lib.call("frnnt_mi_backward", _c_int(dt), _lib.ptr(px), _lib.ptr(py), _lib.ptr(boundary),
                  _lib.ptr(p), _lib.ptr(ans_grad), _lib.ptr(px_grad), _lib.ptr(py_grad),
                  _lib.ptr(origin), _lib.ptr(lattice), B, S, T, modified, _lib.stream_ptr(dev))
    return (px_grad, py_grad, origin) if want_origin_grad else (px_grad, py_grad)


class MutualInformationRecursionFunction(torch.autograd.Function):
    """Same contract as the reference's Function (mutual_information.py:24-181)."""

    @staticmethod
    def forward(ctx, px: Tensor, py: Tensor, pxy_grads: List[Optional[Tensor]],
                boundary: Optional[Tensor] = None, return_grad: bool = False) -> Tensor:
        (B, S, T1) = px.shape
        T = py.shape[-1]
        assert T1 in [T, T + 1]
        assert py.shape == (B, S + 1, T)
        if boundary is not None:
            assert boundary.shape == (B, 4)
        need_grad = return_grad or px.requires_grad or py.requires_grad
        ans, _, lattice = mi_forward(px, py, boundary, want_p=False, want_lattice=need_grad)
        px_grad, py_grad = None, None
        ctx.deferred = False
        if return_grad:
            # the reference's contract: the reverse sweep runs at once with ans_grad = 1, the
            # occupancies are handed out and rescaled in place when the loss is back-propagated
            ones = torch.ones(B, device=px.device, dtype=px.dtype)
            px_grad, py_grad = mi_backward_from_lattice(px, lattice, boundary, ones, py.shape)
            ctx.save_for_backward(px_grad, py_grad)
        elif need_grad:
            # nobody sees the occupancies: the reverse sweep waits for the real ans_grad, which
            # saves the two rescaling passes over the lattice gradients (same result up to
            # the rounding of one multiplication per entry)
            ctx.deferred = True
            ctx.py_shape = tuple(py.shape)
            ctx.save_for_backward(px, lattice, boundary)
        assert len(pxy_grads) == 2
        pxy_grads[0] = px_grad
        pxy_grads[1] = py_grad
        return ans

    @staticmethod
    def backward(ctx, ans_grad: Tensor) -> Tuple[Tensor, Tensor, None, None, None]:
        if ctx.deferred:
            px, lattice, boundary = ctx.saved_tensors
            px_grad, py_grad = mi_backward_from_lattice(px, lattice, boundary,
                                                        ans_grad.contiguous().to(px.dtype), ctx.py_shape)
            return (px_grad, py_grad, None, None, None)
        (px_grad, py_grad) = ctx.saved_tensors
        (B,) = ans_grad.shape
        ans_grad = ans_grad.reshape(B, 1, 1)
        px_grad *= ans_grad
        py_grad *= ans_grad
        return (px_grad, py_grad, None, None, None)


def _validate(px: Tensor, py: Tensor, boundary: Optional[Tensor]):
    assert px.ndim == 3
    B, S, T1 = px.shape
    T = py.shape[-1]
    assert px.shape[-1] in [T, T + 1]  # if T, then "modified".
    assert py.shape == (B, S + 1, T)
    assert px.dtype == py.dtype
    if boundary is not None:
        assert boundary.dtype == torch.int64
        assert boundary.shape == (B, 4)
        for s_begin, t_begin, s_end, t_end in _boundary_rows(boundary):
            assert 0 <= s_begin <= s_end <= S
            assert 0 <= t_begin <= t_end <= T


def mutual_information_recursion(
    px: Tensor, py: Tensor, boundary: Optional[Tensor] = None, return_grad: bool = False,
) -> Union[Tuple[Tensor, Tuple[Tensor, Tensor]], Tensor]:
    """See the reference's docstring (mutual_information.py:184-276); identical
    arguments and return values.  ``px`` is [B][S][T+1] (regular) or [B][S][T]
    (modified), ``py`` is [B][S+1][T], ``boundary`` is an optional int64
    [B][4] of (s_begin, t_begin, s_end, t_end)."""
    _validate(px, py, boundary)
    px, py = px.contiguous(), py.contiguous()
    if boundary is not None:
        boundary = boundary.contiguous()
    pxy_grads = [None, None]
    scores = MutualInformationRecursionFunction.apply(px, py, pxy_grads, boundary, return_grad)
    px_grad, py_grad = pxy_grads
    return (scores, (px_grad, py_grad)) if return_grad else scores


def _inner_product(a: Tensor, b: Tensor) -> Tensor:
    assert a.shape[-1] == b.shape[-1]
    return torch.matmul(a.unsqueeze(-2), b.unsqueeze(-1)).squeeze(-1).squeeze(-1)


def joint_mutual_information_recursion(
    px: Sequence[Tensor], py: Sequence[Tensor], boundary: Optional[Tensor] = None,
) -> Sequence[Tensor]:
    """Per-term breakdown of the recursion's total (reference
    mutual_information.py:314-425): returns [len(px)][B] whose sum over dim 0 is
    the total score; the first term carries the log-of-sum offset."""
    N = len(px)
    assert len(py) == N and N > 0
    B, S, T1 = px[0].shape
    T = py[0].shape[2]
    assert T1 in [T, T + 1]
    assert py[0].shape == (B, S + 1, T)
    assert px[0].dtype == py[0].dtype

    px_cat = torch.stack(list(px), dim=0)
    py_cat = torch.stack(list(py), dim=0)
    px_tot = px_cat.sum(dim=0).contiguous()
    py_tot = py_cat.sum(dim=0).contiguous()
    _validate(px_tot, py_tot, boundary)
    if boundary is not None:
        boundary = boundary.contiguous()

    with torch.no_grad():
        tot_probs, _, lattice = mi_forward(px_tot.detach(), py_tot.detach(), boundary)
        ones = torch.ones(B, device=px_tot.device, dtype=px_tot.dtype)
        px_grad, py_grad = mi_backward_from_lattice(px_tot.detach(), lattice, boundary, ones,
                                                    py_tot.shape)

    px_grad = px_grad.reshape(1, B, -1)
    py_grad = py_grad.reshape(1, B, -1)
    px_cat = px_cat.reshape(N, B, -1)
    py_cat = py_cat.reshape(N, B, -1)
    # -inf times a zero occupancy would be nan
    px_cat = px_cat.clamp(min=torch.finfo(px_cat.dtype).min)
    py_cat = py_cat.clamp(min=torch.finfo(py_cat.dtype).min)
    prods = _inner_product(px_grad, px_cat) + _inner_product(py_grad, py_cat)  # (N, B)
    with torch.no_grad():
        offset = tot_probs - prods.sum(dim=0)
    prods[0] += offset
    return prods
