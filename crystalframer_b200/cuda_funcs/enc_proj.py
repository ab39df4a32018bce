"""autograd Function for the plain Crystalformer encoding (no frames, un-windowed Gaussians)."""
import torch

from .. import _lib
from .common import csr_offsets, f32c
from .framed_proj import _w3
from .kernel_manager import current_config


class RealPeriodicEncodingWithProjFuncCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/real_space_enc_proj.py:21-213 with ``frame_method="no"``:
    returns ``(z_ek, v_ekd, None, None)``; gradients for ``a_ik`` (slot 0) and ``W_k`` (slot 9).
    The weighted-PCA branch of the reference Function is not implemented."""

    @staticmethod
    def forward(ctx, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale, W_k,
                frame_method, rvlen_n=None, cutoff_radius=None):
        if frame_method != "no":
            raise NotImplementedError(f"frame_method={frame_method}: only 'no' is implemented here")
        cfg = current_config()
        N, H = a_ik.shape
        E = edge_ij_e.shape[1]
        if H != cfg.num_heads or abs(float(wscale) - cfg.dist_wscale) > 1e-6 * max(1.0, abs(cfg.dist_wscale)):
            raise RuntimeError("call-time scalars differ from those bound by compile_kernels")
        dev = a_ik.device
        a, pos, tv = f32c(a_ik), f32c(rpos_ij_e), f32c(tvecs_n)
        batch, edges, rv = batch_i.contiguous(), edge_ij_e.contiguous(), f32c(rvlen_n)
        cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
        Wd = _w3(W_k)
        want_v = K > 0 and Wd is not None
        z = torch.empty((E, H), device=dev, dtype=torch.float32)
        v = torch.empty((E, H, Wd.shape[-2]), device=dev, dtype=torch.float32) if want_v else None
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_proj_fwd", 1, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), N, E, float(dist_max),
                    cutoff, p(Wd), p(z), p(v))
        ctx.save_for_backward(a, pos, tv, batch, edges, rv, Wd, z)
        ctx.meta = (float(dist_max), cutoff, rvlen_n is not None, None if W_k is None else tuple(W_k.shape))
        ctx.mark_non_differentiable()
        if not want_v:
            return z,
        return z, v, None, None

    @staticmethod
    def backward(ctx, gz_ek, gv_ekd=None, g_sigma=None, g_sigma_max=None):
        a, pos, tv, batch, edges, rv, Wd, z = ctx.saved_tensors
        dist_max, cutoff, has_rv, shape_d = ctx.meta
        N, H = a.shape
        E = edges.shape[1]
        dev = a.device
        if Wd is None or gv_ekd is None:
            raise NotImplementedError("backward without the value encoding (K <= 0) is not implemented")
        gz = f32c(gz_ek) if gz_ek is not None else torch.zeros_like(z)
        gv = f32c(gv_ekd)
        ga = torch.empty((N, H), device=dev, dtype=torch.float32)
        gWd = torch.empty_like(Wd)
        e_start = csr_offsets(edges, N)
        nbytes = _lib.lib().cfb200_framed_proj_bwd_workspace_bytes(N, E)
        ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_proj_bwd", 3, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E,
                    dist_max, cutoff, p(Wd), p(z), p(gz), p(gv), p(ga), p(gWd), ws.data_ptr(), int(nbytes))
        out = [None] * (15 if has_rv else 13)
        out[0] = ga
        out[9] = gWd.reshape(shape_d)
        return tuple(out)
