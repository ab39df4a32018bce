"""autograd Function for the per-crystal mean over atoms."""
import torch

from .. import _lib


class IrregularMeanCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/irregular_mean.py:19-69: ``x_ik (N,*)`` -> ``(B,*)``."""

    @staticmethod
    def forward(ctx, x_ik, batch_i, sizes):
        N = x_ik.shape[0]
        D = x_ik.numel() // max(N, 1)
        dev = x_ik.device
        if sizes is None:
            B = int(batch_i.max().item()) + 1
            sizes = torch.zeros(B, dtype=torch.long, device=dev)
            sizes.scatter_add_(0, batch_i, torch.ones_like(batch_i))
        B = sizes.shape[0]
        start = torch.zeros(B + 1, dtype=torch.int64, device=dev)
        start[1:] = torch.cumsum(sizes, 0)
        x = x_ik.detach().contiguous().float()
        out = torch.empty((B,) + tuple(x.shape[1:]), device=dev, dtype=torch.float32)
        _lib.invoke("cfb200_segment_mean_fwd", 1, dev, _lib.ptr(x), _lib.iptr(start), B, D, _lib.ptr(out))
        ctx.save_for_backward(start)
        ctx.shape = tuple(x.shape)
        return out

    @staticmethod
    def backward(ctx, go_nk):
        start, = ctx.saved_tensors
        B = start.shape[0] - 1
        go = go_nk.detach().contiguous().float()
        gx = torch.empty(ctx.shape, device=go.device, dtype=torch.float32)
        D = gx.numel() // max(gx.shape[0], 1)
        _lib.invoke("cfb200_segment_mean_bwd", 1, go.device, _lib.ptr(go), _lib.iptr(start), B, D, _lib.ptr(gx))
        return gx, None, None
