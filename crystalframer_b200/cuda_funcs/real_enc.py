"""autograd Function for the plain real-space encoding with un-projected values."""
import torch

from .. import _lib
from .common import csr_offsets, f32c
from .framed_proj import _w3
from .kernel_manager import current_config


def _selectors(H, hd, K, dev):
    """K / hd weight sets (H,hd,K) that pick basis functions [hd b, hd b + hd) unchanged."""
    out = []
    for b in range(K // hd):
        S = torch.zeros((H, hd, K), device=dev, dtype=torch.float32)
        r = torch.arange(hd, device=dev)
        S[:, r, hd * b + r] = 1.0
        out.append(S)
    return out


class RealPeriodicEncodingFuncCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/real_space_enc.py:17-245 (kernels real_enc_fwd.cu, real_enc_bwd.cu): lattice-sum
    logit ``z_ek (E,H)`` and, for ``K > 0``, the softmax-weighted sums of all ``K`` distance Gaussians per (pair, head)
    -- ``(E,H,K)`` when ``W_k`` is None, else projected by ``W_k`` to ``(E,H,head_dim)`` (what
    ``RealPeriodicEncodingWithProjFuncCUDA(frame_method="no")`` returns).  No branch of the reference module calls
    this Function; the un-projected form is served by the projecting kernel with K / head_dim selector weight sets,
    i.e. that many lattice sums -- a convenience, not a fast path.  Gradients: ``a_ik`` and ``W_k``."""

    @staticmethod
    def forward(ctx, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale, W_k, rvlen_n=None,
                cutoff_radius=None):
        cfg = current_config()
        N, H = a_ik.shape
        E = edge_ij_e.shape[1]
        dev = a_ik.device
        if abs(float(wscale) - cfg.dist_wscale) > 1e-6 * max(1.0, abs(cfg.dist_wscale)):
            raise RuntimeError("call-time scalars differ from those bound by compile_kernels")
        if K > 0 and K != cfg.dist_dim:
            raise RuntimeError(f"K={K}, but compile_kernels bound {cfg.dist_dim} distance Gaussians")
        a, pos, tv, rv = f32c(a_ik), f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
        batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
        cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
        W = _w3(W_k)
        hd = cfg.head_dim
        weights = [] if K <= 0 else ([W] if W is not None else _selectors(H, hd, K, dev))
        z = torch.empty((E, H), device=dev, dtype=torch.float32)
        p, ip = _lib.ptr, _lib.iptr
        parts = []
        for Wb in weights or [None]:
            v = torch.empty((E, H, hd), device=dev, dtype=torch.float32) if Wb is not None else None
            _lib.invoke("cfb200_proj_heads_fwd", 1, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), N, E, H,
                        float(dist_max), cutoff, p(Wb), p(z), p(v))
            parts.append(v)
        ctx.save_for_backward(a, pos, tv, batch, edges, rv, z, *weights)
        ctx.meta = (float(dist_max), cutoff, rvlen_n is not None, W is not None, None if W_k is None else tuple(W_k.shape))
        if K <= 0:
            return z,
        return z, (parts[0] if W is not None else torch.cat(parts, dim=-1))

    @staticmethod
    def backward(ctx, gz_ek, gv_ekd=None):
        a, pos, tv, batch, edges, rv, z = ctx.saved_tensors[:7]
        weights = ctx.saved_tensors[7:]
        dist_max, cutoff, has_rv, projected, shape_w = ctx.meta
        N, H = a.shape
        E = edges.shape[1]
        dev = a.device
        out = [None] * (12 if has_rv else 10)
        if not weights:
            raise NotImplementedError("backward without the value encoding (K <= 0) is not implemented")
        hd = weights[0].shape[-2]
        gz = f32c(gz_ek) if gz_ek is not None else torch.zeros_like(z)
        gv = f32c(gv_ekd) if gv_ekd is not None else None
        e_start = csr_offsets(edges, N)
        nbytes = int(_lib.lib().cfb200_proj_heads_bwd_workspace_bytes(N, E, H))
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        p, ip = _lib.ptr, _lib.iptr
        ga_total, gW = None, None
        zero_gz = torch.zeros_like(gz)
        for b, Wb in enumerate(weights):
            if gv is None:
                gvb = torch.zeros((E, H, hd), device=dev, dtype=torch.float32)
            else:
                gvb = gv if projected else gv[..., hd * b:hd * (b + 1)].contiguous()
            ga = torch.empty((N, H), device=dev, dtype=torch.float32)
            gWb = torch.empty_like(Wb)
            # the logit's gradient enters once; the other selector passes carry value gradients only
            _lib.invoke("cfb200_proj_heads_bwd", 3, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N,
                        E, H, dist_max, cutoff, p(Wb), p(z), p(gz if b == 0 else zero_gz), p(gvb), p(ga), p(gWb),
                        ws.data_ptr(), nbytes)
            ga_total = ga if ga_total is None else ga_total + ga
            gW = gWb
        out[0] = ga_total
        if projected:
            out[9] = gW.reshape(shape_w)
        return tuple(out)
