"""TEST INFRASTRUCTURE ONLY -- the checker, never the product.

CPU restatement (torch CPU ops + the plain-C recursion in ``mi_oracle.c``) of
the pruned RNN-T loss path of k2-fsa/fast_rnnt.  Only ``tests/``, the smoke
check and the benchmark's CPU-baseline / reference leg may import this module.
The product package never does: it calls the CUDA library and raises when that
library is missing.

Parity status: PINNED.  ``tests/test_oracle_pin.py`` checks every function here
against golden vectors written by the reference project itself
(``tests/golden/make_golden.py`` imports the reference's python package and its
compiled CPU extension and dumps every stage of the pipeline), and, where the
reference's compiled CPU extension is present (``oracle/_ref``), against it
directly.

The arithmetic is kept in the reference's operation order so that float32
results agree to the last bit on the same torch build; the code structure is
ours (one normalizer helper shared by the simple and smoothed variants, one
``_finish`` shared by the four loss wrappers, a lattice "band placement" helper
shared by the pruned and unpruned variants).

Reference lines restated (paths inside the reference project):
  check_lengths            fast_rnnt/python/fast_rnnt/rnnt_loss.py:25-42
  simple_logprobs          rnnt_loss.py:66-227 (plain) and :1135-1369 (smoothed)
  joint_logprobs           rnnt_loss.py:343-449
  pruned_logprobs          rnnt_loss.py:821-853, :856-1024
  prune_ranges             rnnt_loss.py:550-632, :638-777
  prune                    rnnt_loss.py:780-818
  loss_* wrappers          rnnt_loss.py:230-340, :452-547, :1027-1132, :1372-1494
  mi_recursion, joint_mi   fast_rnnt/python/fast_rnnt/mutual_information.py:24-425
"""
import ctypes
import os
import subprocess
from typing import Optional, Sequence, Tuple

import torch
from torch import Tensor

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
NEG_INF = float("-inf")


def build_c_oracle() -> str:
    """Compile mi_oracle.c into liboracle_mi.so (gcc only, no dependencies)."""
    so = os.path.join(_HERE, "liboracle_mi.so")
    src = os.path.join(_HERE, "mi_oracle.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O2", "-fPIC", "-shared", "-fno-fast-math",
             "-ffp-contract=off", "-o", so, src, "-lm"])
    return so


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build_c_oracle())
    return _LIB


def _ptr(t: Optional[Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _sfx(dtype):
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.float64:
        return "f64"
    raise TypeError(f"oracle supports float32/float64 only, got {dtype}")


# --------------------------------------------------------------------------
# mutual-information recursion (mutual_information.py:24-298)
# --------------------------------------------------------------------------
def mi_forward_raw(px: Tensor, py: Tensor, boundary: Optional[Tensor]):
    """Returns (p, ans) exactly as the native CPU forward computes them."""
    B, S, T1 = px.shape
    T = py.shape[2]
    modified = int(T1 == T)
    px, py = px.contiguous(), py.contiguous()
    if boundary is not None:
        boundary = boundary.contiguous()
    p = torch.empty(B, S + 1, T + 1, dtype=px.dtype)
    ans = torch.empty(B, dtype=px.dtype)
    fn = getattr(_lib(), "mi_oracle_forward_" + _sfx(px.dtype))
    rc = fn(_ptr(px), _ptr(py), _ptr(boundary), _ptr(p), _ptr(ans), B, S, T, modified)
    assert rc == 0
    return p, ans


def mi_backward_raw(px, py, boundary, p, ans_grad):
    B, S, T1 = px.shape
    T = py.shape[2]
    modified = int(T1 == T)
    px, py, p = px.contiguous(), py.contiguous(), p.contiguous()
    if boundary is not None:
        boundary = boundary.contiguous()
    gx, gy = torch.empty_like(px), torch.empty_like(py)
    fn = getattr(_lib(), "mi_oracle_backward_" + _sfx(px.dtype))
    rc = fn(_ptr(px), _ptr(py), _ptr(boundary), _ptr(p), _ptr(ans_grad.contiguous()),
            _ptr(gx), _ptr(gy), B, S, T, modified)
    assert rc == 0
    return gx, gy


class _MiFn(torch.autograd.Function):
    # mutual_information.py:24-181: backward is run eagerly with ans_grad = 1
    # and the saved occupancies are rescaled IN PLACE by the upstream gradient.
    @staticmethod
    def forward(ctx, px, py, out, boundary, return_grad):
        p, ans = mi_forward_raw(px, py, boundary)
        if return_grad or px.requires_grad or py.requires_grad:
            ones = torch.ones(px.shape[0], dtype=px.dtype)
            gx, gy = mi_backward_raw(px, py, boundary, p, ones)
            ctx.save_for_backward(gx, gy)
            out[0], out[1] = gx, gy
        return ans

    @staticmethod
    def backward(ctx, g):
        gx, gy = ctx.saved_tensors
        g = g.reshape(-1, 1, 1)
        gx *= g
        gy *= g
        return gx, gy, None, None, None


def _check_boundary(boundary, B, S, T):
    assert boundary.dtype == torch.int64 and boundary.shape == (B, 4)
    for s0, t0, s1, t1 in boundary.tolist():
        assert 0 <= s0 <= s1 <= S
        assert 0 <= t0 <= t1 <= T


def mi_recursion(px: Tensor, py: Tensor, boundary: Optional[Tensor] = None,
                 return_grad: bool = False):
    """mutual_information.py:184-298."""
    assert px.ndim == 3
    B, S, T1 = px.shape
    T = py.shape[-1]
    assert T1 in (T, T + 1) and py.shape == (B, S + 1, T) and px.dtype == py.dtype
    if boundary is not None:
        _check_boundary(boundary, B, S, T)
    out = [None, None]
    scores = _MiFn.apply(px.contiguous(), py.contiguous(), out, boundary, return_grad)
    return (scores, (out[0], out[1])) if return_grad else scores


def joint_mi(px: Sequence[Tensor], py: Sequence[Tensor],
             boundary: Optional[Tensor] = None) -> Tensor:
    """mutual_information.py:314-425: per-term breakdown of the total score."""
    N = len(px)
    assert N > 0 and len(py) == N
    B, S, T1 = px[0].shape
    T = py[0].shape[2]
    assert T1 in (T, T + 1) and py[0].shape == (B, S + 1, T)
    xs, ys = torch.stack(list(px)), torch.stack(list(py))
    x_tot, y_tot = xs.sum(0).contiguous(), ys.sum(0).contiguous()
    if boundary is not None:
        _check_boundary(boundary, B, S, T)
    p, tot = mi_forward_raw(x_tot.detach(), y_tot.detach(), boundary)
    gx, gy = mi_backward_raw(x_tot.detach(), y_tot.detach(), boundary, p,
                             torch.ones(B, dtype=x_tot.dtype))
    lo = torch.finfo(xs.dtype).min
    xs = xs.reshape(N, B, -1).clamp(min=lo)
    ys = ys.reshape(N, B, -1).clamp(min=lo)

    def dot(a, b):  # mutual_information.py:301-311
        return torch.matmul(a.unsqueeze(-2), b.unsqueeze(-1)).squeeze(-1).squeeze(-1)

    prods = dot(gx.reshape(1, B, -1), xs) + dot(gy.reshape(1, B, -1), ys)
    with torch.no_grad():
        offset = tot - prods.sum(0)
    prods[0] += offset
    return prods


# --------------------------------------------------------------------------
# log-prob lattices
# --------------------------------------------------------------------------
def check_lengths(S: int, T: int, regular: bool, boundary: Optional[Tensor]):
    if boundary is None:
        assert S >= 1, S
        assert regular or T >= S, (T, S)
    else:
        assert bool((boundary[:, 2] >= 1).all())
        assert regular or bool((boundary[:, 3] >= boundary[:, 2]).all())


def _mask_at_t_end(px: Tensor, boundary: Optional[Tensor]) -> Tensor:
    # rnnt_loss.py:45-63: px[b, :, t_end[b]] = -inf (in place, blocks the gradient)
    if boundary is None:
        return px
    B, S, T1 = px.shape
    return px.scatter_(2, boundary[:, 3].reshape(B, 1, 1).expand(B, S, T1), NEG_INF)


def _append_neg_inf_column(x: Tensor) -> Tensor:
    B, S, _ = x.shape
    return torch.cat((x, torch.full((B, S, 1), NEG_INF, dtype=x.dtype)), dim=2)


def simple_logprobs(lm: Tensor, am: Tensor, symbols: Tensor, blank: int,
                    rnnt_type: str = "regular", boundary: Optional[Tensor] = None,
                    lm_only_scale: Optional[float] = None,
                    am_only_scale: Optional[float] = None) -> Tuple[Tensor, Tensor]:
    """get_rnnt_logprobs (both scales None) / get_rnnt_logprobs_smoothed.

    rnnt_loss.py:160-227 and :1246-1369.
    """
    assert lm.ndim == 3 and am.ndim == 3
    assert lm.shape[0] == am.shape[0] and lm.shape[2] == am.shape[2]
    B, T, C = am.shape
    S = lm.shape[1] - 1
    assert symbols.shape == (B, S)
    assert rnnt_type in ("regular", "modified", "constrained"), rnnt_type
    check_lengths(S, T, rnnt_type == "regular", boundary)
    smoothed = lm_only_scale is not None

    tiny = torch.finfo(lm.dtype).tiny
    am_max = am.max(dim=2, keepdim=True)[0]
    lm_max = lm.max(dim=2, keepdim=True)[0]
    am_p = (am - am_max).exp()
    lm_p = (lm - lm_max).exp()
    norm = (torch.matmul(lm_p, am_p.transpose(1, 2)) + tiny).log()

    if smoothed:
        lm_den = lm_p.sum(dim=2, keepdim=True)                       # [B,S+1,1]
        unigram = torch.mean(lm_p / lm_den, dim=(0, 1), keepdim=True) + tiny
        am_only_norm = (torch.mv(am_p.reshape(-1, C), unigram.reshape(C))
                        .reshape(B, T, 1).log() + am_max).transpose(1, 2)  # [B,1,T]
        log_unigram = unigram.log()
        lm_only_norm = lm_den.log() + lm_max                           # [B,S+1,1]

    norm = norm + lm_max + am_max.transpose(1, 2)                      # [B,S+1,T]

    px_am = torch.gather(am.transpose(1, 2), 1, symbols.unsqueeze(2).expand(B, S, T))
    if rnnt_type == "regular":
        px_am = _append_neg_inf_column(px_am)
    px_lm = torch.gather(lm[:, :S], 2, symbols.unsqueeze(-1))          # [B,S,1]
    px = px_am + px_lm
    px[:, :, :T] -= norm[:, :S, :]

    py_am = am[:, :, blank].unsqueeze(1)                               # [B,1,T]
    py_lm = lm[:, :, blank].unsqueeze(2)                               # [B,S+1,1]
    py = py_am + py_lm - norm

    if smoothed:
        px_lm_uni = torch.gather(log_unigram.expand(B, S, C), 2, symbols.unsqueeze(-1))
        px_am_only = px_am + px_lm_uni
        px_am_only[:, :, :T] -= am_only_norm
        px_lm_only = px_lm - lm_only_norm[:, :S, :]
        py_am_only = py_am + log_unigram[0][0][blank] - am_only_norm
        py_lm_only = py_lm - lm_only_norm
        both = 1.0 - lm_only_scale - am_only_scale
        # exact zeros would turn -inf * 0 into nan (rnnt_loss.py:1346-1351)
        ls = 1.0e-20 if lm_only_scale == 0.0 else lm_only_scale
        as_ = 1.0e-20 if am_only_scale == 0.0 else am_only_scale
        px = px * both + px_lm_only * ls + px_am_only * as_
        py = py * both + py_lm_only * ls + py_am_only * as_

    if rnnt_type == "regular":
        px = _mask_at_t_end(px, boundary)
    elif rnnt_type == "constrained":
        px += py[:, 1:, :]
    return px, py


def joint_logprobs(logits: Tensor, symbols: Tensor, blank: int,
                   boundary: Optional[Tensor] = None,
                   rnnt_type: str = "regular") -> Tuple[Tensor, Tensor]:
    """get_rnnt_logprobs_joint, rnnt_loss.py:410-449."""
    assert logits.ndim == 4
    B, T, S1, C = logits.shape
    S = S1 - 1
    assert symbols.shape == (B, S)
    assert rnnt_type in ("regular", "modified", "constrained"), rnnt_type
    check_lengths(S, T, rnnt_type == "regular", boundary)
    norm = torch.logsumexp(logits, dim=3).permute(0, 2, 1)              # [B,S+1,T]
    px = torch.gather(logits, 3, symbols.reshape(B, 1, S, 1).expand(B, T, S, 1))
    px = px.squeeze(-1).permute(0, 2, 1)
    if rnnt_type == "regular":
        px = _append_neg_inf_column(px)
    px[:, :, :T] -= norm[:, :S, :]
    py = logits[:, :, :, blank].permute(0, 2, 1).clone()
    py -= norm
    if rnnt_type == "regular":
        px = _mask_at_t_end(px, boundary)
    elif rnnt_type == "constrained":
        px += py[:, 1:, :]
    return px, py


def _place_band(band: Tensor, shifts: Tensor, S1: int) -> Tensor:
    """[B,T,R] band values -> [B,T,S1] rows with the band starting at
    ``shifts[b,t]`` (cyclically) and -inf elsewhere (rnnt_loss.py:821-853 applied
    to the -inf padded tensor of :967-982 / :1000-1015)."""
    B, T, R = band.shape
    pad = torch.full((B, T, S1 - R), NEG_INF, dtype=band.dtype)
    src = torch.cat((band, pad), dim=2)
    idx = (torch.arange(S1).view(1, 1, S1) - shifts.reshape(B, T, 1)) % S1
    return torch.gather(src, 2, idx)


def pruned_logprobs(logits: Tensor, symbols: Tensor, ranges: Tensor, blank: int,
                    boundary: Optional[Tensor] = None,
                    rnnt_type: str = "regular") -> Tuple[Tensor, Tensor]:
    """get_rnnt_logprobs_pruned, rnnt_loss.py:925-1024."""
    assert logits.ndim == 4
    B, T, R, C = logits.shape
    assert ranges.shape == (B, T, R)
    S = symbols.shape[1]
    assert symbols.shape == (B, S)
    assert rnnt_type in ("regular", "modified", "constrained"), rnnt_type
    check_lengths(S, T, rnnt_type == "regular", boundary)
    norm = torch.logsumexp(logits, dim=3)                               # [B,T,R]
    sym_ext = torch.cat((symbols, torch.full((B, 1), blank, dtype=torch.int64)), dim=1)
    sym_band = torch.gather(sym_ext.unsqueeze(1).expand(B, T, S + 1), 2, ranges)
    px_band = torch.gather(logits, 3, sym_band.reshape(B, T, R, 1)).squeeze(-1) - norm
    px = _place_band(px_band, ranges[:, :, 0], S + 1)[:, :, :S].permute(0, 2, 1)
    if rnnt_type == "regular":
        px = _append_neg_inf_column(px)
    py_band = logits[:, :, :, blank].clone() - norm
    py = _place_band(py_band, ranges[:, :, 0], S + 1).permute(0, 2, 1)
    if rnnt_type == "regular":
        px = _mask_at_t_end(px, boundary)
    elif rnnt_type == "constrained":
        px += py[:, 1:, :]
    return px, py


# --------------------------------------------------------------------------
# pruning
# --------------------------------------------------------------------------
def _suffix_min(x: Tensor) -> Tensor:
    # rnnt_loss.py:578-581
    return torch.flip(torch.cummin(torch.flip(x, dims=(-1,)), dim=-1)[0], dims=(-1,))


def _fix_lower_bound(s_begin: Tensor, step: int) -> Tensor:
    # rnnt_loss.py:617-632: monotone, starts at 0, advances by < step per frame
    T = s_begin.shape[1]
    ramp = (step - 1) * torch.arange(0, T)
    x = _suffix_min(s_begin)
    x = -(x - ramp)
    x = torch.clamp(_suffix_min(x), min=0)
    return -(x - ramp)


def prune_ranges(px_grad: Tensor, py_grad: Tensor, boundary: Tensor, s_range: int,
                 quiet: bool = True) -> Tensor:
    """get_rnnt_prune_ranges, rnnt_loss.py:685-777.  int64 [B,T,s_range']."""
    B, S, T1 = px_grad.shape
    T = py_grad.shape[-1]
    assert T1 in (T, T + 1)
    regular = T1 != T
    S1 = S + 1
    assert py_grad.shape == (B, S1, T) and boundary.shape == (B, 4)
    check_lengths(S, T, regular, boundary)
    if regular:
        need = int(boundary[:, 2].sub(1).div(boundary[:, 3], rounding_mode="trunc")
                   .add(2).max().item())
        if s_range < need:
            if not quiet:
                print(f"Warning: get_rnnt_prune_ranges - got s_range={s_range} "
                      f"for boundaries S={boundary[:, 2]}, T={boundary[:, 3]}. "
                      f"Adjusting to {need}")
            s_range = need
    if s_range > S:
        s_range = S1
    assert s_range >= (2 if regular else 1)

    # Window sums over s_range consecutive rows of py_grad (rnnt_loss.py:726-734).
    # The reference calls torch.sum on a strided view; torch adds the s_range
    # terms in order k = 0, 1, ... for all but the last few (< 32) elements of
    # each utterance's flattened output, where its scalar tail loop uses a
    # 4-accumulator cascade whose extent depends on the thread split.  The
    # oracle fixes the in-order sum everywhere: it is machine independent and
    # reproduces the reference's ranges bit for bit on every golden case.
    n_win = S1 - s_range + 1
    win_sum = py_grad[:, 0:n_win, :].clone()
    for k in range(1, s_range):
        win_sum = win_sum + py_grad[:, k:k + n_win, :]
    px_shift = torch.cat((torch.zeros((B, 1, T1), dtype=px_grad.dtype), px_grad), dim=1)
    score = win_sum - px_shift[:, : S1 - s_range + 1, :T]
    s_begin = torch.argmax(score, axis=1)                               # [B,T]

    live = torch.arange(0, T).reshape(1, T).expand(B, T) < boundary[:, 3].reshape(B, 1) - 1
    tail = torch.clamp(boundary[:, 2].reshape(B, 1) - s_range + 1, min=0)
    s_begin = torch.where(live, s_begin, tail)
    s_begin = _fix_lower_bound(s_begin, 2 if T1 == T else s_range)
    return s_begin.reshape(B, T, 1).expand(B, T, s_range) + torch.arange(s_range)


def prune(am: Tensor, lm: Tensor, ranges: Tensor) -> Tuple[Tensor, Tensor]:
    """do_rnnt_pruning, rnnt_loss.py:799-818."""
    B, T, R = ranges.shape
    assert am.shape[0] == B and lm.shape[0] == B and am.shape[1] == T
    D = lm.shape[2]
    am_p = am.unsqueeze(2).expand(B, T, R, am.shape[2])
    lm_p = torch.gather(lm, 1, ranges.reshape(B, T * R, 1).expand(B, T * R, D))
    return am_p, lm_p.reshape(B, T, R, D)


# --------------------------------------------------------------------------
# loss wrappers
# --------------------------------------------------------------------------
def _finish(px, py, boundary, rnnt_type, delay_penalty, reduction, return_grad):
    # the tail shared by the four wrappers (e.g. rnnt_loss.py:309-340)
    if delay_penalty > 0.0:
        B, S, T0 = px.shape
        T = T0 if rnnt_type != "regular" else T0 - 1
        if boundary is None:
            offset = torch.tensor((T - 1) / 2, dtype=px.dtype).expand(B, 1, 1)
        else:
            offset = (boundary[:, 3] - 1) / 2
        penalty = offset.reshape(B, 1, 1) - torch.arange(T0).reshape(1, 1, T0)
        px += (penalty * delay_penalty).to(px.dtype)
    res = mi_recursion(px, py, boundary=boundary, return_grad=return_grad)
    scores = res[0] if return_grad else res
    if reduction == "none":
        loss = -scores
    elif reduction == "mean":
        loss = -torch.mean(scores)
    elif reduction == "sum":
        loss = -torch.sum(scores)
    else:
        raise ValueError(
            f"reduction should be ('none' | 'mean' | 'sum'), given {reduction}")
    return (loss, res[1]) if return_grad else loss


def loss_simple(lm, am, symbols, blank, boundary=None, rnnt_type="regular",
                delay_penalty=0.0, reduction="mean", return_grad=False):
    px, py = simple_logprobs(lm, am, symbols, blank, rnnt_type, boundary)
    return _finish(px, py, boundary, rnnt_type, delay_penalty, reduction, return_grad)


def loss_smoothed(lm, am, symbols, blank, lm_only_scale=0.1, am_only_scale=0.1,
                  boundary=None, rnnt_type="regular", delay_penalty=0.0,
                  reduction="mean", return_grad=False):
    px, py = simple_logprobs(lm, am, symbols, blank, rnnt_type, boundary,
                             lm_only_scale, am_only_scale)
    return _finish(px, py, boundary, rnnt_type, delay_penalty, reduction, return_grad)


def loss_joint(logits, symbols, blank, boundary=None, rnnt_type="regular",
               delay_penalty=0.0, reduction="mean", return_grad=False):
    px, py = joint_logprobs(logits, symbols, blank, boundary, rnnt_type)
    return _finish(px, py, boundary, rnnt_type, delay_penalty, reduction, return_grad)


def loss_pruned(logits, symbols, ranges, blank, boundary=None, rnnt_type="regular",
                delay_penalty=0.0, reduction="mean", return_grad=False):
    px, py = pruned_logprobs(logits, symbols, ranges, blank, boundary, rnnt_type)
    return _finish(px, py, boundary, rnnt_type, delay_penalty, reduction, return_grad)
