"""autograd Function for the plain Crystalformer encoding (no frames, un-windowed Gaussians) and for the
per-pair second moments of the weighted-PCA frames."""
import torch

from .. import _lib
from .common import csr_offsets, f32c, pair_geometry
from .framed_proj import _w3
from .kernel_manager import current_config
from .max_frame import _draw_seed


def _sigma_records(a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius):
    """(E,H,11) per-pair records of cfb200_sigma_edges and the noise seed that was drawn for them."""
    N, H = a_ik.shape
    E = edge_ij_e.shape[1]
    dev = a_ik.device
    a, pos, tv, rv = f32c(a_ik), f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
    batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
    cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
    _draw_seed()                    # the reference draws one seed for select_edges.cu (its output is never read) ...
    seed_noise = _draw_seed()       # ... and one for real_enc_sigma_fwd.cu (models/cuda_funcs/real_space_enc_proj.py:88,98)
    rec = torch.empty((E, H, 11), device=dev, dtype=torch.float32)
    p, ip = _lib.ptr, _lib.iptr
    _, plist, prange = pair_geometry(rpos_ij_e, tvecs_n, batch_i, edge_ij_e, cutoff)
    _lib.invoke("cfb200_sigma_edges_cached", 1, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), N, E, cutoff,
                seed_noise, p(rec), p(plist), prange)
    return rec, seed_noise


class RealPeriodicEncodingWithProjFuncCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/real_space_enc_proj.py:21-213.

    ``frame_method="no"``: returns ``(z_ek, v_ekd, None, None)``; gradients for ``a_ik`` (slot 0) and ``W_k``
    (slot 9).

    Any other frame method (the reference's weighted-PCA branch, :80-125): returns
    ``(z_ek (E,H), v_ekd (E,H,head_dim), sigma_mat (E,H,6), sigma_mat_max (N,H,6))`` without gradients, like the
    reference.  ``sigma_mat`` holds each pair's weight-averaged second moments (xx, xy, xz, yy, yz, zz) and
    ``sigma_mat_max`` the same six entries of u u^T for the unit vector u to the atom's nearest non-zero image
    over all of its pairs (lowest pair index on ties; the reference lets the pairs of an atom race for this slot).
    Two departures, both on outputs the reference leaves undefined: ``z_ek`` is the lattice-sum logit
    log sum_n exp(a d_n^2) -- the reference returns ``torch.empty`` here and feeds it to the pooling attention as a
    bias -- and ``v_ekd``, which no caller reads in this mode, is zeros."""

    @staticmethod
    def forward(ctx, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale, W_k,
                frame_method, rvlen_n=None, cutoff_radius=None):
        if frame_method != "no":
            rec, _ = _sigma_records(a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius)
            N, H = a_ik.shape
            E = edge_ij_e.shape[1]
            z = rec[:, :, 0].contiguous()
            sigma_mat = rec[:, :, 1:7].contiguous()
            # the atom's nearest non-zero image: smallest record [7] over the atom's pairs, lowest pair index on ties
            e_start = csr_offsets(edge_ij_e.contiguous(), N)
            d2 = rec[:, :, 7]
            idx = edge_ij_e[0][:, None].expand(E, H)
            best = torch.full((N, H), float("inf"), device=d2.device).scatter_reduce(0, idx, d2, reduce="amin", include_self=True)
            ar = torch.arange(E, device=d2.device)[:, None].expand(E, H)
            cand = torch.where(d2 == best[edge_ij_e[0]], ar, torch.full_like(ar, E))
            arg = torch.full((N, H), E, dtype=torch.long, device=d2.device).scatter_reduce(0, idx, cand, reduce="amin", include_self=True)
            hh = torch.arange(H, device=d2.device)[None, :].expand(N, H)
            u = rec[arg.clamp_max(E - 1), hh, 8:11]
            sigma_mat_max = torch.stack([u[..., 0] * u[..., 0], u[..., 0] * u[..., 1], u[..., 0] * u[..., 2],
                                         u[..., 1] * u[..., 1], u[..., 1] * u[..., 2], u[..., 2] * u[..., 2]], dim=-1)
            ctx.frame_method = frame_method
            ctx.n_in = 13 if rvlen_n is None else 15
            ctx.mark_non_differentiable(z, sigma_mat, sigma_mat_max)
            if K <= 0:
                return z,
            W = _w3(W_k)
            v = torch.zeros((E, H, W.shape[-2] if W is not None else K), device=a_ik.device, dtype=torch.float32)
            ctx.mark_non_differentiable(v)
            return z, v, sigma_mat, sigma_mat_max
        ctx.frame_method = frame_method
        cfg = current_config()
        N, H = a_ik.shape
        E = edge_ij_e.shape[1]
        if abs(float(wscale) - cfg.dist_wscale) > 1e-6 * max(1.0, abs(cfg.dist_wscale)):
            raise RuntimeError("call-time scalars differ from those bound by compile_kernels")
        # H may be smaller than the bound head count: the "multihead" domain encodes half of the heads in real space
        # (models/indexed_lattice_multi_head_attention_cuda.py:953-963); the weights then have H heads as well
        dev = a_ik.device
        a, pos, tv = f32c(a_ik), f32c(rpos_ij_e), f32c(tvecs_n)
        batch, edges, rv = batch_i.contiguous(), edge_ij_e.contiguous(), f32c(rvlen_n)
        cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
        Wd = _w3(W_k)
        want_v = K > 0 and Wd is not None
        z = torch.empty((E, H), device=dev, dtype=torch.float32)
        v = torch.empty((E, H, Wd.shape[-2]), device=dev, dtype=torch.float32) if want_v else None
        p, ip = _lib.ptr, _lib.iptr
        if Wd is not None and Wd.shape[0] != H:
            raise RuntimeError(f"W_k has {Wd.shape[0]} heads, a_ik {H}")
        _lib.invoke("cfb200_proj_heads_fwd", 1, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), N, E, H,
                    float(dist_max), cutoff, p(Wd), p(z), p(v))
        ctx.save_for_backward(a, pos, tv, batch, edges, rv, Wd, z)
        ctx.meta = (float(dist_max), cutoff, rvlen_n is not None, None if W_k is None else tuple(W_k.shape))
        ctx.mark_non_differentiable()
        if not want_v:
            return z,
        return z, v, None, None

    @staticmethod
    def backward(ctx, gz_ek, gv_ekd=None, g_sigma=None, g_sigma_max=None):
        if ctx.frame_method != "no":
            return (None,) * ctx.n_in                    # no gradients in this mode (real_space_enc_proj.py:135-137)
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
        nbytes = _lib.lib().cfb200_proj_heads_bwd_workspace_bytes(N, E, H)
        ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_proj_heads_bwd", 3, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E,
                    H, dist_max, cutoff, p(Wd), p(z), p(gz), p(gv), p(ga), p(gWd), ws.data_ptr(), int(nbytes))
        out = [None] * (15 if has_rv else 13)
        out[0] = ga
        out[9] = gWd.reshape(shape_d)
        return tuple(out)
