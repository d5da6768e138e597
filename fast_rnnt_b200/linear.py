"""fp32-accurate linear layer on the B200 tensor cores (3xTF32, TMA-fed) for the
joiner that sits between do_rnnt_pruning and rnnt_loss_pruned.  The reference
leaves that network to the caller (README.md:180-190); this is an optional
replacement of torch.nn.functional.linear for float32 CUDA tensors."""
import torch

from . import _lib


def _matmul_nt(a, b, bias, M, N, K):
    out = torch.empty(M, N, dtype=torch.float32, device=a.device)
    _lib.call("frnnt_matmul_nt", _lib.ptr(a), _lib.ptr(b), _lib.ptr(bias), _lib.ptr(out), M, N, K,
              _lib.stream_ptr(a.device))
    return out


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
            if ctx.needs_input_grad[1]:
                splits = _lib.lib().frnnt_matmul_tn_splits(N, K, M)
                gw = torch.empty(N, K, dtype=torch.float32, device=g.device)
                partials = (torch.empty(splits, N, K, dtype=torch.float32, device=g.device)
                            if splits > 1 else None)
                _lib.call("frnnt_matmul_tn", _lib.ptr(g2), _lib.ptr(x2), _lib.ptr(gw),
                          _lib.ptr(partials), N, K, M, _lib.stream_ptr(g.device))
            if ctx.has_bias and ctx.needs_input_grad[2]:
                gb = g2.sum(dim=0)
        return gx, gw, gb


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor = None) -> torch.Tensor:
    """``x @ weight.T + bias`` like torch.nn.functional.linear, float32 on CUDA;
    weight is [out_features][in_features]; in_features and out_features must be
    multiples of 4."""
    assert x.is_cuda and x.dtype == torch.float32 and weight.dtype == torch.float32
    return _Linear3xTF32.apply(x, weight, bias)
