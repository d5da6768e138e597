"""Pruned RNN-T loss on the GPU: drop-in for
fast_rnnt/python/fast_rnnt/rnnt_loss.py of the reference.

Every public function keeps the reference's name, arguments, defaults and
return values; the work runs in libfrnnt_sm100.so through autograd Functions
(one fused forward and one analytic backward per function instead of the
reference's chains of ATen ops).  CUDA tensors of float32 / float64, as in the reference.

float16 / bfloat16 inputs (no counterpart in the reference, which dispatches float and
double only) are accepted with this definition: the result is that of the float32 call on
the inputs converted to float32 (an exact conversion) -- lattices and losses are float32,
bit-identical; gradients arrive as float32 and autograd rounds them to the input's type.
The two kernels that read the large inputs of the pruned pipeline read 16-bit values
directly (lm / am of the simple losses when the am-only branch is off, enc / dec of the
fused joiner); everywhere else the inputs are converted first.
"""
from typing import Optional, Tuple, Union

import torch
from torch import Tensor

from . import _lib
from ._lib import _c_int, _c_f64
from .mutual_information import _boundary_rows, mutual_information_recursion

_RNNT_TYPES = {"regular": 0, "modified": 1, "constrained": 2}


def _contig(t: Optional[Tensor]) -> Optional[Tensor]:
    return None if t is None else t.contiguous()


def _bytes(n: int, device) -> Tensor:
    return torch.empty(max(int(n), 1), dtype=torch.uint8, device=device)


def validate_st_lengths(S: int, T: int, is_rnnt_type_regular: bool,
                        boundary: Optional[Tensor] = None):
    """Same checks as the reference (rnnt_loss.py:25-42): S >= 1 and, unless the
    type is regular, T >= S, per utterance when a boundary is given."""
    if boundary is None:
        assert S >= 1, S
        assert (is_rnnt_type_regular or T >= S), \
            f"Modified transducer requires T >= S, but got T={T} and S={S}"
    else:
        rows = _boundary_rows(boundary)
        Ss = [r[2] for r in rows]
        Ts = [r[3] for r in rows]
        assert all(s >= 1 for s in Ss), Ss
        assert (is_rnnt_type_regular or all(t >= s for s, t in zip(Ss, Ts))), \
            f"Modified transducer requires T >= S, but got T={Ts} and S={Ss}"


def fix_for_boundary(px: Tensor, boundary: Optional[Tensor] = None) -> Tensor:
    """px[b, :, t_end[b]] = -inf, in place (reference rnnt_loss.py:45-63).  The
    fused kernels already do this; kept for callers that build px themselves."""
    if boundary is None:
        return px
    B, S, T1 = px.shape
    index = boundary[:, 3].reshape(B, 1, 1).expand(B, S, T1)
    return px.scatter_(dim=2, index=index, value=float("-inf"))


# ------------------------------------------------------------------------------
# lattices from factorised lm / am
# ------------------------------------------------------------------------------
class _SimpleLogprobs(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lm, am, symbols, boundary, blank, rnnt_type, smoothed, ls, as_, delay_penalty=0.0):
        B, T, C = am.shape
        S = lm.shape[1] - 1
        dev, dt = lm.device, _lib.input_code(lm.dtype)   # 16-bit lm / am: float32 everywhere else
        out_dtype = torch.float32 if _lib.is_16bit(lm) else lm.dtype
        T1 = T + 1 if rnnt_type == 0 else T
        lm, am, symbols, boundary = _contig(lm), _contig(am), _contig(symbols), _contig(boundary)
        with torch.cuda.device(dev):
            px = torch.empty(B, S, T1, dtype=out_dtype, device=dev)
            py = torch.empty(B, S + 1, T, dtype=out_dtype, device=dev)
            saved = _bytes(_lib.lib().frnnt_simple_saved_bytes(dt, B, S, T, C), dev)
            scratch = _bytes(_lib.lib().frnnt_simple_scratch_bytes(dt, B, S, T, C), dev)
            _lib.call("frnnt_simple_logprobs_forward", _c_int(dt), _lib.ptr(lm), _lib.ptr(am),
                      _lib.ptr(symbols), _lib.ptr(boundary), blank, rnnt_type, int(smoothed),
                      _c_f64(ls), _c_f64(as_), _c_f64(delay_penalty), _lib.ptr(px), _lib.ptr(py),
                      _lib.ptr(saved), _lib.ptr(scratch), B, S, T, C, _lib.stream_ptr(dev))
        ctx.save_for_backward(lm, am, symbols, boundary, saved)
        ctx.cfg = (blank, rnnt_type, int(smoothed), ls, as_)
        return px, py

    @staticmethod
    def backward(ctx, g_px, g_py):
        lm, am, symbols, boundary, saved = ctx.saved_tensors
        blank, rnnt_type, smoothed, ls, as_ = ctx.cfg
        B, T, C = am.shape
        S = lm.shape[1] - 1
        dev, dt = lm.device, _lib.input_code(lm.dtype)
        out_dtype = torch.float32 if _lib.is_16bit(lm) else lm.dtype
        T1 = T + 1 if rnnt_type == 0 else T
        with torch.cuda.device(dev):
            g_px = (torch.zeros(B, S, T1, dtype=out_dtype, device=dev) if g_px is None
                    else g_px.contiguous())
            g_py = (torch.zeros(B, S + 1, T, dtype=out_dtype, device=dev) if g_py is None
                    else g_py.contiguous())
            lm_grad = torch.empty(lm.shape, dtype=out_dtype, device=dev)   # autograd casts it
            am_grad = torch.empty(am.shape, dtype=out_dtype, device=dev)
            scratch = _bytes(_lib.lib().frnnt_simple_scratch_bytes(dt, B, S, T, C), dev)
            _lib.call("frnnt_simple_logprobs_backward", _c_int(dt), _lib.ptr(lm), _lib.ptr(am),
                      _lib.ptr(symbols), _lib.ptr(boundary), blank, rnnt_type, smoothed,
                      _c_f64(ls), _c_f64(as_), _lib.ptr(g_px), _lib.ptr(g_py), _lib.ptr(saved),
                      _lib.ptr(scratch), _lib.ptr(lm_grad), _lib.ptr(am_grad), B, S, T, C,
                      _lib.stream_ptr(dev))
        return lm_grad, am_grad, None, None, None, None, None, None, None, None


def _simple_logprobs(lm, am, symbols, termination_symbol, rnnt_type, boundary, smoothed,
                     lm_only_scale=0.0, am_only_scale=0.0, delay_penalty=0.0):
    assert lm.ndim == 3, lm.ndim
    assert am.ndim == 3, am.ndim
    assert lm.shape[0] == am.shape[0], (lm.shape[0], am.shape[0])
    assert lm.shape[2] == am.shape[2], (lm.shape[2], am.shape[2])
    (B, T, C) = am.shape
    S = lm.shape[1] - 1
    assert symbols.shape == (B, S), symbols.shape
    assert lm.dtype == am.dtype
    validate_st_lengths(S, T, rnnt_type == "regular", boundary)
    assert rnnt_type in ["regular", "modified", "constrained"], rnnt_type
    if _lib.is_16bit(lm) and not _lib.lib().frnnt_simple_reads_16bit_inputs(
            S, T, C, _RNNT_TYPES[rnnt_type], int(smoothed), _c_f64(float(am_only_scale))):
        lm, am = lm.float(), am.float()   # the am-only branch and the SIMT paths read float32
    return _SimpleLogprobs.apply(lm, am, symbols, boundary, int(termination_symbol),
                                 _RNNT_TYPES[rnnt_type], smoothed, float(lm_only_scale),
                                 float(am_only_scale), float(delay_penalty))


def get_rnnt_logprobs(lm: Tensor, am: Tensor, symbols: Tensor, termination_symbol: int,
                      rnnt_type: str = "regular",
                      boundary: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """(px, py) for the "simple" joiner that adds lm [B][S+1][C] and am [B][T][C]
    (reference rnnt_loss.py:66-227).  px is [B][S][T+1] for "regular" and
    [B][S][T] otherwise; py is [B][S+1][T]."""
    return _simple_logprobs(lm, am, symbols, termination_symbol, rnnt_type, boundary, False)


def get_rnnt_logprobs_smoothed(lm: Tensor, am: Tensor, symbols: Tensor, termination_symbol: int,
                               lm_only_scale: float = 0.1, am_only_scale: float = 0.1,
                               boundary: Optional[Tensor] = None,
                               rnnt_type: str = "regular") -> Tuple[Tensor, Tensor]:
    """As get_rnnt_logprobs, interpolated with lm-only and am-only log-probs
    (reference rnnt_loss.py:1135-1369)."""
    return _simple_logprobs(lm, am, symbols, termination_symbol, rnnt_type, boundary, True,
                            lm_only_scale, am_only_scale)


# ------------------------------------------------------------------------------
# lattices from joiner logits
# ------------------------------------------------------------------------------
class _LsmGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, symbols, ranges, boundary, blank, rnnt_type, delay_penalty=0.0):
        B, T, R, C = logits.shape
        S = symbols.shape[1]
        dev, dt = logits.device, _lib.dtype_code(logits.dtype)
        T1 = T + 1 if rnnt_type == 0 else T
        logits, symbols = _contig(logits), _contig(symbols)
        ranges, boundary = _contig(ranges), _contig(boundary)
        with torch.cuda.device(dev):
            px = torch.empty(B, S, T1, dtype=logits.dtype, device=dev)
            py = torch.empty(B, S + 1, T, dtype=logits.dtype, device=dev)
            lse = torch.empty(3, B, T, R, dtype=logits.dtype, device=dev)
            _lib.call("frnnt_lsm_gather_forward", _c_int(dt), _lib.ptr(logits), _lib.ptr(symbols),
                      _lib.ptr(ranges), _lib.ptr(boundary), _lib.ptr(lse[0]), _lib.ptr(lse[1]),
                      _lib.ptr(lse[2]), _lib.ptr(px), _lib.ptr(py), B, T, R, S, C, blank,
                      rnnt_type, _c_f64(delay_penalty), _lib.stream_ptr(dev))
        ctx.save_for_backward(logits, symbols, ranges, boundary, lse)
        ctx.cfg = (blank, rnnt_type)
        return px, py

    @staticmethod
    def backward(ctx, g_px, g_py):
        logits, symbols, ranges, boundary, lse = ctx.saved_tensors
        blank, rnnt_type = ctx.cfg
        B, T, R, C = logits.shape
        S = symbols.shape[1]
        dev, dt = logits.device, _lib.dtype_code(logits.dtype)
        T1 = T + 1 if rnnt_type == 0 else T
        with torch.cuda.device(dev):
            g_px = (torch.zeros(B, S, T1, dtype=logits.dtype, device=dev) if g_px is None
                    else g_px.contiguous())
            g_py = (torch.zeros(B, S + 1, T, dtype=logits.dtype, device=dev) if g_py is None
                    else g_py.contiguous())
            g_logits = torch.empty_like(logits)
            _lib.call("frnnt_lsm_gather_backward", _c_int(dt), _lib.ptr(logits),
                      _lib.ptr(symbols), _lib.ptr(ranges), _lib.ptr(boundary), _lib.ptr(lse[0]),
                      _lib.ptr(g_px), _lib.ptr(g_py), _lib.ptr(g_logits), B, T, R, S, C, blank,
                      rnnt_type, _lib.stream_ptr(dev))
        return g_logits, None, None, None, None, None, None


def get_rnnt_logprobs_joint(logits: Tensor, symbols: Tensor, termination_symbol: int,
                            boundary: Optional[Tensor] = None,
                            rnnt_type: str = "regular") -> Tuple[Tensor, Tensor]:
    """(px, py) from full joiner logits [B][T][S+1][C] (reference rnnt_loss.py:343-449)."""
    return _logprobs_joint(logits, symbols, termination_symbol, boundary, rnnt_type, 0.0)


def _logprobs_joint(logits, symbols, termination_symbol, boundary, rnnt_type, delay_penalty):
    """get_rnnt_logprobs_joint with the delay penalty of the loss functions added to px by
    the kernel that writes the lattices."""
    assert logits.ndim == 4, logits.ndim
    if _lib.is_16bit(logits):
        logits = logits.float()
    (B, T, S1, C) = logits.shape
    S = S1 - 1
    assert symbols.shape == (B, S), symbols.shape
    validate_st_lengths(S, T, rnnt_type == "regular", boundary)
    assert rnnt_type in ["regular", "modified", "constrained"], rnnt_type
    return _LsmGather.apply(logits, symbols, None, boundary, int(termination_symbol),
                            _RNNT_TYPES[rnnt_type], float(delay_penalty))


def get_rnnt_logprobs_pruned(logits: Tensor, symbols: Tensor, ranges: Tensor,
                             termination_symbol: int, boundary: Optional[Tensor] = None,
                             rnnt_type: str = "regular") -> Tuple[Tensor, Tensor]:
    """(px, py) from pruned joiner logits [B][T][s_range][C] and the ranges
    [B][T][s_range] they were computed on (reference rnnt_loss.py:856-1024)."""
    return _logprobs_pruned(logits, symbols, ranges, termination_symbol, boundary, rnnt_type, 0.0)


def _logprobs_pruned(logits, symbols, ranges, termination_symbol, boundary, rnnt_type, delay_penalty):
    assert logits.ndim == 4, logits.ndim
    if _lib.is_16bit(logits):
        logits = logits.float()
    (B, T, s_range, C) = logits.shape
    assert ranges.shape == (B, T, s_range), f"{ranges.shape} == ({B}, {T}, {s_range})"
    (B, S) = symbols.shape
    validate_st_lengths(S, T, rnnt_type == "regular", boundary)
    assert rnnt_type in ["regular", "modified", "constrained"], rnnt_type
    return _LsmGather.apply(logits, symbols, ranges, boundary, int(termination_symbol),
                            _RNNT_TYPES[rnnt_type], float(delay_penalty))


class _PrunedJoinerLogprobs(torch.autograd.Function):
    """(px, py) of the pruned loss from the joiner's inputs as one autograd node
    (csrc/joiner_pairs.cu): pruning gather + tanh, the joiner's projection and its two
    gradient products on the tensor cores, log-softmax and symbol / blank gather."""

    @staticmethod
    def forward(ctx, enc, dec, ranges, weight, bias, symbols, boundary, blank, rnnt_type, delay_penalty=0.0):
        B, T, D = enc.shape
        S = symbols.shape[1]
        R = ranges.shape[2]
        C = weight.shape[0]
        dev = enc.device
        T1 = T + 1 if rnnt_type == 0 else T
        enc, dec, ranges, weight = _contig(enc), _contig(dec), _contig(ranges), _contig(weight)
        bias, symbols, boundary = _contig(bias), _contig(symbols), _contig(boundary)
        lib = _lib.lib()
        with torch.cuda.device(dev):
            px = torch.empty(B, S, T1, dtype=torch.float32, device=dev)
            py = torch.empty(B, S + 1, T, dtype=torch.float32, device=dev)
            saved = _bytes(lib.frnnt_pruned_joiner_saved_bytes(B, T, R, S, C, D), dev)
            scratch = _bytes(lib.frnnt_pruned_joiner_forward_scratch_bytes(B, T, R, S, C, D), dev)
            _lib.call("frnnt_pruned_joiner_logprobs_forward", _c_int(_lib.input_code(enc.dtype)),
                      _lib.ptr(enc), _lib.ptr(dec),
                      _lib.ptr(ranges), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(symbols),
                      _lib.ptr(boundary), _lib.ptr(px), _lib.ptr(py), _lib.ptr(saved),
                      _lib.ptr(scratch), B, T, R, S, C, D, blank, rnnt_type, _c_f64(delay_penalty),
                      _lib.stream_ptr(dev))
        ctx.save_for_backward(ranges, symbols, boundary, saved)
        ctx.cfg = (B, T, R, S, C, D, blank, rnnt_type, bias is not None)
        return px, py

    @staticmethod
    def backward(ctx, g_px, g_py):
        ranges, symbols, boundary, saved = ctx.saved_tensors
        B, T, R, S, C, D, blank, rnnt_type, has_bias = ctx.cfg
        dev = saved.device
        T1 = T + 1 if rnnt_type == 0 else T
        need = ctx.needs_input_grad
        lib = _lib.lib()
        with torch.cuda.device(dev):
            g_px = (torch.zeros(B, S, T1, dtype=torch.float32, device=dev) if g_px is None
                    else g_px.contiguous())
            g_py = (torch.zeros(B, S + 1, T, dtype=torch.float32, device=dev) if g_py is None
                    else g_py.contiguous())
            want_in = need[0] or need[1]
            enc_grad = torch.empty(B, T, D, dtype=torch.float32, device=dev) if want_in else None
            dec_grad = torch.empty(B, S + 1, D, dtype=torch.float32, device=dev) if want_in else None
            w_grad = torch.empty(C, D, dtype=torch.float32, device=dev) if need[3] else None
            b_grad = (torch.empty(C, dtype=torch.float32, device=dev)
                      if has_bias and need[4] else None)
            scratch = _bytes(lib.frnnt_pruned_joiner_backward_scratch_bytes(B, T, R, S, C, D), dev)
            _lib.call("frnnt_pruned_joiner_logprobs_backward", _lib.ptr(g_px), _lib.ptr(g_py),
                      _lib.ptr(ranges), _lib.ptr(symbols), _lib.ptr(boundary), _lib.ptr(saved),
                      _lib.ptr(scratch), _lib.ptr(enc_grad), _lib.ptr(dec_grad), _lib.ptr(w_grad),
                      _lib.ptr(b_grad), B, T, R, S, C, D, blank, rnnt_type, _lib.stream_ptr(dev))
        return (enc_grad if need[0] else None, dec_grad if need[1] else None, None, w_grad, b_grad,
                None, None, None, None, None)


def get_rnnt_logprobs_pruned_joiner(am: Tensor, lm: Tensor, ranges: Tensor, joiner_weight: Tensor,
                                    joiner_bias: Optional[Tensor], symbols: Tensor,
                                    termination_symbol: int, boundary: Optional[Tensor] = None,
                                    rnnt_type: str = "regular") -> Tuple[Tensor, Tensor]:
    """(px, py) of the pruned loss for the joiner of the reference's documented usage
    (README.md:180-190), in one fused operator::

        am_pruned, lm_pruned = do_rnnt_pruning(am, lm, ranges)
        logits = linear(tanh(am_pruned + lm_pruned), joiner_weight, joiner_bias)
        px, py = get_rnnt_logprobs_pruned(logits, symbols, ranges, termination_symbol, ...)

    am [B][T][D], lm [B][S+1][D], ranges [B][T][s_range], joiner_weight [C][D]; float32
    CUDA tensors, D a multiple of 8 and C a multiple of 4.  No counterpart in the
    reference (which leaves the joiner to the caller); the pruned tensors, and a
    second pass over the logits for their log-sum-exp, never exist."""
    return _logprobs_pruned_joiner(am, lm, ranges, joiner_weight, joiner_bias, symbols,
                                   termination_symbol, boundary, rnnt_type, 0.0)


def _logprobs_pruned_joiner(am, lm, ranges, joiner_weight, joiner_bias, symbols, termination_symbol,
                            boundary, rnnt_type, delay_penalty):
    assert am.ndim == 3 and lm.ndim == 3 and ranges.ndim == 3, (am.shape, lm.shape, ranges.shape)
    (B, T, D) = am.shape
    (B2, S1, D2) = lm.shape
    assert B2 == B and D2 == D, (am.shape, lm.shape)
    s_range = ranges.shape[2]
    assert ranges.shape == (B, T, s_range), f"{ranges.shape} == ({B}, {T}, {s_range})"
    S = S1 - 1
    assert symbols.shape == (B, S), symbols.shape
    assert joiner_weight.ndim == 2 and joiner_weight.shape[1] == D, joiner_weight.shape
    assert am.dtype == lm.dtype and am.dtype in (torch.float32, torch.float16, torch.bfloat16), \
        (am.dtype, lm.dtype)
    if _lib.is_16bit(joiner_weight):
        joiner_weight = joiner_weight.float()
    if _lib.is_16bit(joiner_bias):
        joiner_bias = joiner_bias.float()
    assert joiner_weight.dtype == torch.float32
    validate_st_lengths(S, T, rnnt_type == "regular", boundary)
    assert rnnt_type in ["regular", "modified", "constrained"], rnnt_type
    return _PrunedJoinerLogprobs.apply(am, lm, ranges, joiner_weight, joiner_bias, symbols, boundary,
                                       int(termination_symbol), _RNNT_TYPES[rnnt_type],
                                       float(delay_penalty))


# ------------------------------------------------------------------------------
# pruning
# ------------------------------------------------------------------------------
def get_rnnt_prune_ranges(px_grad: Tensor, py_grad: Tensor, boundary: Tensor,
                          s_range: int) -> Tensor:
    """int64 ranges [B][T][s_range'] of the symbols kept per frame, from the
    occupancies returned by a ``return_grad=True`` loss (reference
    rnnt_loss.py:638-777, including the s_range adjustments of :699-724)."""
    (B, S, T1) = px_grad.shape
    T = py_grad.shape[-1]
    is_regular = T1 != T
    assert T1 in [T, T + 1], T1
    assert py_grad.shape == (B, S + 1, T), py_grad.shape
    assert boundary.shape == (B, 4), boundary.shape
    assert px_grad.dtype == py_grad.dtype
    validate_st_lengths(S, T, is_regular, boundary)

    if is_regular:
        rows = _boundary_rows(boundary)
        # trunc division as in the reference (all operands non-negative here)
        s_range_min = max((r[2] - 1) // r[3] + 2 for r in rows)
        if s_range < s_range_min:
            print(f"Warning: get_rnnt_prune_ranges - got s_range={s_range} "
                  f"for boundaries S={boundary[:, 2]}, T={boundary[:, 3]}. "
                  f"Adjusting to {s_range_min}")
            s_range = s_range_min
    if s_range > S:
        s_range = S + 1
    if is_regular:
        assert s_range >= 2, ("Pruning range for standard RNN-T should be equal to or greater "
                              "than 2, or no valid paths could survive pruning.")
    else:
        assert s_range >= 1, ("Pruning range for modified RNN-T should be equal to or greater "
                              "than 1, or no valid paths could survive pruning.")

    dev = px_grad.device
    px_grad, py_grad, boundary = px_grad.contiguous(), py_grad.contiguous(), boundary.contiguous()
    with torch.cuda.device(dev):
        ranges = torch.empty(B, T, s_range, dtype=torch.int64, device=dev)
        _lib.call("frnnt_prune_ranges", _c_int(_lib.dtype_code(px_grad.dtype)),
                  _lib.ptr(px_grad.detach()), _lib.ptr(py_grad.detach()), _lib.ptr(boundary),
                  _lib.ptr(ranges), B, S, T, T1, s_range, _lib.stream_ptr(dev))
    return ranges


class _PruneGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, lm, ranges):
        B, S1, D = lm.shape
        _, T, R = ranges.shape
        dev = lm.device
        lm, ranges = lm.contiguous(), ranges.contiguous()
        with torch.cuda.device(dev):
            out = torch.empty(B, T, R, D, dtype=lm.dtype, device=dev)
            _lib.call("frnnt_prune_gather", _c_int(_lib.dtype_code(lm.dtype)), _lib.ptr(lm),
                      _lib.ptr(ranges), _lib.ptr(out), B, S1, T, R, D, _lib.stream_ptr(dev))
        ctx.save_for_backward(ranges)
        ctx.lm_shape = (B, S1, D)
        return out

    @staticmethod
    def backward(ctx, g):
        (ranges,) = ctx.saved_tensors
        B, S1, D = ctx.lm_shape
        _, T, R = ranges.shape
        dev = g.device
        g = g.contiguous()
        with torch.cuda.device(dev):
            lm_grad = torch.empty(B, S1, D, dtype=g.dtype, device=dev)
            if g.dtype == torch.float32 and D % 4 == 0 and D <= 3200:
                # windowed partial sums per chunk of frames (one streaming pass)
                nbytes = _lib.lib().frnnt_joiner_input_grads_scratch_bytes(B, T, D)
                scratch = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
                _lib.call("frnnt_joiner_input_grads", _lib.ptr(g), _lib.ptr(ranges), None,
                          _lib.ptr(lm_grad), _lib.ptr(scratch), B, S1, T, R, D,
                          _lib.stream_ptr(dev))
            else:
                _lib.call("frnnt_prune_gather_backward", _c_int(_lib.dtype_code(g.dtype)),
                          _lib.ptr(g), _lib.ptr(ranges), _lib.ptr(lm_grad), B, S1, T, R, D,
                          _lib.stream_ptr(dev))
        return lm_grad, None


def do_rnnt_pruning(am: Tensor, lm: Tensor, ranges: Tensor) -> Tuple[Tensor, Tensor]:
    """am [B][T][D], lm [B][S+1][D], ranges [B][T][s_range] -> (am_pruned,
    lm_pruned), both [B][T][s_range][D] (reference rnnt_loss.py:780-818).
    am_pruned is a stride-0 view of am, exactly as in the reference."""
    assert ranges.shape[0] == am.shape[0], (ranges.shape[0], am.shape[0])
    assert ranges.shape[0] == lm.shape[0], (ranges.shape[0], lm.shape[0])
    assert am.shape[1] == ranges.shape[1], (am.shape[1], ranges.shape[1])
    (B, T, s_range) = ranges.shape
    (B, S1, C) = lm.shape
    am_pruning = am.unsqueeze(2).expand((B, T, s_range, am.shape[2]))
    lm_pruning = _PruneGather.apply(lm, ranges)
    return am_pruning, lm_pruning


# ------------------------------------------------------------------------------
# losses
# ------------------------------------------------------------------------------
def _penalty(delay_penalty: float) -> float:
    """The reference applies the delay penalty only when it is positive
    (rnnt_loss.py:309); the lattice-writing kernels add it to px."""
    return float(delay_penalty) if delay_penalty > 0.0 else 0.0


def _finish(px, py, boundary, reduction, return_grad):
    """recursion and reduction shared by the losses (reference rnnt_loss.py:326-340 and its
    three copies)."""
    scores_and_grads = mutual_information_recursion(px=px, py=py, boundary=boundary,
                                                    return_grad=return_grad)
    negated_loss = scores_and_grads[0] if return_grad else scores_and_grads
    if reduction == "none":
        loss = -negated_loss
    elif reduction == "mean":
        loss = -torch.mean(negated_loss)
    elif reduction == "sum":
        loss = -torch.sum(negated_loss)
    else:
        raise ValueError(f"reduction should be ('none' | 'mean' | 'sum'), given {reduction}")
    return (loss, scores_and_grads[1]) if return_grad else loss


def rnnt_loss_simple(lm: Tensor, am: Tensor, symbols: Tensor, termination_symbol: int,
                     boundary: Optional[Tensor] = None, rnnt_type: str = "regular",
                     delay_penalty: float = 0.0, reduction: Optional[str] = "mean",
                     return_grad: bool = False,
                     ) -> Union[Tensor, Tuple[Tensor, Tuple[Tensor, Tensor]]]:
    """RNN-T loss with the additive "simple" joiner (reference rnnt_loss.py:230-340)."""
    px, py = _simple_logprobs(lm, am, symbols, termination_symbol, rnnt_type, boundary, False,
                              delay_penalty=_penalty(delay_penalty))
    return _finish(px, py, boundary, reduction, return_grad)


def rnnt_loss_smoothed(lm: Tensor, am: Tensor, symbols: Tensor, termination_symbol: int,
                       lm_only_scale: float = 0.1, am_only_scale: float = 0.1,
                       boundary: Optional[Tensor] = None, rnnt_type: str = "regular",
                       delay_penalty: float = 0.0, reduction: Optional[str] = "mean",
                       return_grad: bool = False,
                       ) -> Union[Tuple[Tensor, Tuple[Tensor, Tensor]], Tensor]:
    """Smoothed "simple" loss (reference rnnt_loss.py:1372-1494)."""
    px, py = _simple_logprobs(lm, am, symbols, termination_symbol, rnnt_type, boundary, True,
                              lm_only_scale, am_only_scale, delay_penalty=_penalty(delay_penalty))
    return _finish(px, py, boundary, reduction, return_grad)


def rnnt_loss(logits: Tensor, symbols: Tensor, termination_symbol: int,
              boundary: Optional[Tensor] = None, rnnt_type: str = "regular",
              delay_penalty: float = 0.0, reduction: Optional[str] = "mean",
              return_grad: bool = False) -> Tensor:
    """Unpruned RNN-T loss on logits [B][T][S+1][C] (reference rnnt_loss.py:452-547)."""
    px, py = _logprobs_joint(logits, symbols, termination_symbol, boundary, rnnt_type,
                             _penalty(delay_penalty))
    return _finish(px, py, boundary, reduction, return_grad)


def rnnt_loss_pruned(logits: Tensor, symbols: Tensor, ranges: Tensor, termination_symbol: int,
                     boundary: Optional[Tensor] = None, rnnt_type: str = "regular",
                     delay_penalty: float = 0.0, reduction: Optional[str] = "mean",
                     return_grad: bool = False) -> Tensor:
    """Pruned RNN-T loss on logits [B][T][s_range][C] (reference rnnt_loss.py:1027-1132)."""
    px, py = _logprobs_pruned(logits, symbols, ranges, termination_symbol, boundary, rnnt_type,
                              _penalty(delay_penalty))
    return _finish(px, py, boundary, reduction, return_grad)


def rnnt_loss_pruned_joiner(am: Tensor, lm: Tensor, ranges: Tensor, joiner_weight: Tensor,
                            joiner_bias: Optional[Tensor], symbols: Tensor, termination_symbol: int,
                            boundary: Optional[Tensor] = None, rnnt_type: str = "regular",
                            delay_penalty: float = 0.0, reduction: Optional[str] = "mean",
                            return_grad: bool = False) -> Tensor:
    """rnnt_loss_pruned (reference rnnt_loss.py:1027-1132) on the logits of the joiner
    ``linear(tanh(am_pruned + lm_pruned))``, computed by the fused operator behind
    get_rnnt_logprobs_pruned_joiner instead of being passed in."""
    px, py = _logprobs_pruned_joiner(am, lm, ranges, joiner_weight, joiner_bias, symbols,
                                     termination_symbol, boundary, rnnt_type, _penalty(delay_penalty))
    return _finish(px, py, boundary, reduction, return_grad)
