"""autograd Function for the lattice-sum bias and the frame-projected value encoding."""
import torch

from .. import _lib
from .common import csr_offsets, f32c, pair_geometry
from .kernel_manager import current_config


def _w3(W):
    """Projection weights arrive as (1,H,hd,K) or (H,hd,K); per-pair or per-atom weights
    (leading extent > 1) exist in the reference interface but no caller uses them."""
    if W is None:
        return None
    if W.dim() == 4:
        if W.shape[0] != 1:
            raise NotImplementedError("per-atom / per-pair projection weights are not supported")
        W = W[0]
    return f32c(W)


class RealEncodingWithFramedProjFuncCUDA(torch.autograd.Function):
    """Drop-in for the reference Function of the same name
    (models/cuda_funcs/real_space_framed_proj.py:19-221): same positional arguments, same
    outputs ``(z_ek (E,H), v_ekd (E,H,hd))`` (or ``(z_ek,)`` when K <= 0), same gradient slots.
    The weight gradients come back already summed over atoms in the parameter's shape, where the
    reference returns per-atom (N,H,hd,K) tensors that autograd then sums."""

    @staticmethod
    def forward(ctx, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                W_k, W_k1, W_k2, W_k3, frame_vec_1, frame_vec_2, frame_vec_3, dim_angle_enc,
                value_pe_angle_scale, cos_abs, length_rbf_mul, angle_rbf_mul, rvlen_n=None, cutoff_radius=None):
        cfg = current_config()
        N, H = a_ik.shape
        E = edge_ij_e.shape[1]
        if H != cfg.num_heads:
            raise RuntimeError(f"configured for {cfg.num_heads} heads, got {H}")
        if abs(float(wscale) - cfg.dist_wscale) > 1e-6 * max(1.0, abs(cfg.dist_wscale)) or \
                abs(float(length_rbf_mul) - cfg.dist_coef) > 1e-6 or int(cos_abs) != cfg.cos_abs:
            raise RuntimeError("call-time scalars differ from those bound by compile_kernels")
        ang = W_k1 is not None
        if ang and (abs(float(value_pe_angle_scale) - cfg.angle_wscale) > 1e-6 or
                    abs(float(angle_rbf_mul) - cfg.angle_coef) > 1e-6 or int(dim_angle_enc) != cfg.angle_dim):
            raise RuntimeError("angle scalars differ from those bound by compile_kernels")
        dev = a_ik.device
        a = f32c(a_ik)
        pos = f32c(rpos_ij_e)
        tv = f32c(tvecs_n)
        batch = batch_i.contiguous()
        edges = edge_ij_e.contiguous()
        rv = f32c(rvlen_n)
        cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
        Wd, W1, W2, W3 = _w3(W_k), _w3(W_k1), _w3(W_k2), _w3(W_k3)
        f1, f2, f3 = (f32c(frame_vec_1), f32c(frame_vec_2), f32c(frame_vec_3)) if ang else (None, None, None)
        want_v = K > 0 and Wd is not None
        z = torch.empty((E, H), device=dev, dtype=torch.float32)
        v = torch.empty((E, H, Wd.shape[-2]), device=dev, dtype=torch.float32) if want_v else None
        p, ip = _lib.ptr, _lib.iptr
        pcache, plist, prange = pair_geometry(rpos_ij_e, tvecs_n, batch_i, edge_ij_e, cutoff)
        _lib.invoke("cfb200_framed_proj_fwd_cached", 1, dev,
                    p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), N, E, float(dist_max), cutoff,
                    p(Wd), p(W1), p(W2), p(W3), p(f1), p(f2), p(f3), p(z), p(v), p(pcache), p(plist), prange)
        ctx.save_for_backward(a, pos, tv, batch, edges, rv, Wd, W1, W2, W3, f1, f2, f3, z)
        ctx.pair_list = (plist, prange)
        ctx.meta = (float(dist_max), cutoff, rvlen_n is not None,
                    None if W_k is None else tuple(W_k.shape), None if W_k1 is None else tuple(W_k1.shape))
        if not want_v:
            return z,
        return z, v

    @staticmethod
    def backward(ctx, gz_ek, gv_ekd=None):
        a, pos, tv, batch, edges, rv, Wd, W1, W2, W3, f1, f2, f3, z = ctx.saved_tensors
        dist_max, cutoff, has_rv, shape_d, shape_a = ctx.meta
        N, H = a.shape
        E = edges.shape[1]
        dev = a.device
        n_slots = 26 if has_rv else 23
        out = [None] * n_slots
        ga = torch.empty((N, H), device=dev, dtype=torch.float32)
        if Wd is None or gv_ekd is None:
            raise NotImplementedError("backward without the value encoding (K <= 0) is not implemented")
        gz = f32c(gz_ek) if gz_ek is not None else torch.zeros_like(z)
        gv = f32c(gv_ekd)
        gWd = torch.empty_like(Wd)
        gW1 = torch.empty_like(W1) if W1 is not None else None
        gW2 = torch.empty_like(W2) if W2 is not None else None
        gW3 = torch.empty_like(W3) if W3 is not None else None
        e_start = csr_offsets(edges, N)
        lib = _lib.lib()
        nbytes = lib.cfb200_framed_proj_bwd_workspace_bytes(N, E)
        ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        p, ip = _lib.ptr, _lib.iptr
        plist, prange = ctx.pair_list
        _lib.invoke("cfb200_framed_proj_bwd_cached", 3, dev,
                    p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E, dist_max, cutoff,
                    p(Wd), p(W1), p(W2), p(W3), p(f1), p(f2), p(f3), p(z), p(gz), p(gv), p(ga),
                    p(gWd), p(gW1), p(gW2), p(gW3), ws.data_ptr(), int(nbytes), p(plist), prange)
        out[0] = ga
        out[9] = gWd.reshape(shape_d)
        if gW1 is not None:
            out[10], out[11], out[12] = gW1.reshape(shape_a), gW2.reshape(shape_a), gW3.reshape(shape_a)
        return tuple(out)
