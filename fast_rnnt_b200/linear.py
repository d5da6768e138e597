"""fp32-accurate linear layer on the B200 tensor cores (3xTF32, TMA-fed) for the
joiner that sits between do_rnnt_pruning and rnnt_loss_pruned.  The reference
leaves that network to the caller (README.md:180-190); this is an optional
replacement of torch.nn.functional.linear for float32 CUDA tensors."""
import torch

from . import _lib


def _matmul_nt(a, b, bias, M, N, K, tanh_out=None):
    out = torch.empty(M, N, dtype=torch.float32, device=a.device)
    _lib.call("frnnt_matmul_nt", _lib.ptr(a), _lib.ptr(b), _lib.ptr(bias), _lib.ptr(tanh_out),
              _lib.ptr(out), M, N, K, _lib.stream_ptr(a.device))
    return out


def _matmul_tn(a, b, M, N, R, want_colsum=False):
    """a[R][M]^T @ b[R][N]; with want_colsum also a.sum(0), taken from the operand
    tiles as they pass through the product (the bias gradient of a linear layer)."""
    out = torch.empty(M, N, dtype=torch.float32, device=a.device)
    colsum = torch.empty(M, dtype=torch.float32, device=a.device) if want_colsum else None
    nscratch = _lib.lib().frnnt_matmul_tn_scratch_floats(M, N, R)
    scratch = torch.empty(max(nscratch, 1), dtype=torch.float32, device=a.device)
    _lib.call("frnnt_matmul_tn_colsum", _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(colsum),
              _lib.ptr(scratch), M, N, R, _lib.stream_ptr(a.device))
    return (out, colsum) if want_colsum else out


class _Linear3xTF32(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        N, K = weight.shape
        x2 = x.reshape(-1, K).contiguous()
        weight = weight.contiguous()
        with torch.cuda.device(x.device):
            out = _matmul_nt(x2, weight, None if bias is None else bias.contiguous(),
                             x2.shape[0], N, K)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return out.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, g):
        x2, weight = ctx.saved_tensors
        N, K = weight.shape
        M = x2.shape[0]
        g2 = g.reshape(M, N).contiguous()
        gx = gw = gb = None
        with torch.cuda.device(g.device):
            if ctx.needs_input_grad[0]:
                wt = weight.t().contiguous()                      # [K][N]
                gx = _matmul_nt(g2, wt, None, M, K, N).reshape(ctx.x_shape)
            want_gb = ctx.has_bias and ctx.needs_input_grad[2]
            if ctx.needs_input_grad[1]:
                gw = _matmul_tn(g2, x2, N, K, M, want_colsum=want_gb)
                if want_gb:
                    gw, gb = gw
            elif want_gb:
                gb = g2.sum(dim=0)
        return gx, gw, gb


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor = None) -> torch.Tensor:
    """``x @ weight.T + bias`` like torch.nn.functional.linear, float32 on CUDA;
    weight is [out_features][in_features]; in_features and out_features must be
    multiples of 4."""
    assert x.is_cuda and x.dtype == torch.float32 and weight.dtype == torch.float32
    return _Linear3xTF32.apply(x, weight, bias)


class _PrunedJoiner(torch.autograd.Function):
    """logits = Linear(tanh(enc[b,t] + dec[b, ranges[b,t,k]])) as one autograd node:
    gather + add + tanh in one kernel, the three products on the tensor cores, the
    tanh derivative in the epilogue of the grad-input product."""

    @staticmethod
    def forward(ctx, enc, dec, ranges, weight, bias):
        B, T, D = enc.shape
        S1 = dec.shape[1]
        R = ranges.shape[2]
        N = weight.shape[0]
        enc, dec, ranges, weight = (enc.contiguous(), dec.contiguous(), ranges.contiguous(),
                                    weight.contiguous())
        dev = enc.device
        with torch.cuda.device(dev):
            act = torch.empty(B, T, R, D, dtype=torch.float32, device=dev)
            _lib.call("frnnt_pruned_tanh", 0, _lib.ptr(enc), _lib.ptr(dec), _lib.ptr(ranges),
                      _lib.ptr(act), B, S1, T, R, D, _lib.stream_ptr(dev))
            out = _matmul_nt(act, weight, None if bias is None else bias.contiguous(),
                             B * T * R, N, D)
        ctx.save_for_backward(act, weight, ranges)
        ctx.dims = (B, T, R, D, S1, N)
        ctx.has_bias = bias is not None
        return out.reshape(B, T, R, N)

    @staticmethod
    def backward(ctx, g):
        act, weight, ranges = ctx.saved_tensors
        B, T, R, D, S1, N = ctx.dims
        M = B * T * R
        dev = g.device
        g2 = g.reshape(M, N).contiguous()
        enc_grad = dec_grad = gw = gb = None
        with torch.cuda.device(dev):
            if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
                wt = weight.t().contiguous()
                gz = _matmul_nt(g2, wt, None, M, D, N, tanh_out=act)   # d loss / d (enc + dec)
                enc_grad = torch.empty(B, T, D, dtype=torch.float32, device=dev)
                dec_grad = torch.empty(B, S1, D, dtype=torch.float32, device=dev)
                if D % 4 == 0 and D <= 3200:
                    # both from one pass over gz
                    nbytes = _lib.lib().frnnt_joiner_input_grads_scratch_bytes(B, T, D)
                    scratch = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
                    _lib.call("frnnt_joiner_input_grads", _lib.ptr(gz), _lib.ptr(ranges),
                              _lib.ptr(enc_grad), _lib.ptr(dec_grad), _lib.ptr(scratch), B, S1, T, R,
                              D, _lib.stream_ptr(dev))
                else:
                    _lib.call("frnnt_sum_over_range", 0, _lib.ptr(gz), _lib.ptr(enc_grad),
                              _lib._c_longlong(B * T), R, D, _lib.stream_ptr(dev))
                    _lib.call("frnnt_prune_gather_backward", 0, _lib.ptr(gz), _lib.ptr(ranges),
                              _lib.ptr(dec_grad), B, S1, T, R, D, _lib.stream_ptr(dev))
            want_gb = ctx.has_bias and ctx.needs_input_grad[4]
            if ctx.needs_input_grad[3]:
                gw = _matmul_tn(g2, act.reshape(M, D), N, D, M, want_colsum=want_gb)
                if want_gb:
                    gw, gb = gw
            elif want_gb:
                gb = g2.sum(dim=0)
        return enc_grad, dec_grad, None, gw, gb


def pruned_joiner(enc: torch.Tensor, dec: torch.Tensor, ranges: torch.Tensor,
                  weight: torch.Tensor, bias: torch.Tensor = None) -> torch.Tensor:
    """``linear(tanh(am_pruned + lm_pruned), weight, bias)`` for
    ``am_pruned, lm_pruned = do_rnnt_pruning(enc, dec, ranges)`` -- the joiner of
    the reference's documented usage (README.md:180-190) -- without materialising
    the pruned tensors.  float32 CUDA tensors; enc [B][T][D], dec [B][S+1][D],
    ranges int64 [B][T][R], weight [C][D]; returns logits [B][T][R][C]."""
    assert enc.dtype == torch.float32 and dec.dtype == torch.float32
    return _PrunedJoiner.apply(enc, dec, ranges, weight, bias)
