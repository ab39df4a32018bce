"""autograd Functions for the dynamic "max" frames (all outputs are non-differentiable)."""
import numpy as np
import torch

from .. import _lib
from .common import csr_offsets, f32c, pair_geometry


def _draw_seed():
    """One draw from numpy's global generator per Function call, as the reference does
    (models/cuda_funcs/calc_maximum_frame.py:43,121), so that numpy's state advances alike."""
    return int(np.random.randint(np.iinfo(np.int64).min, np.iinfo(np.int64).max, dtype=np.int64)) & (2 ** 64 - 1)


def _frame_call(axis, q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1,
                want_selection=False):
    N, H = a_ik.shape
    E = edge_ij_e.shape[1]
    dev = a_ik.device
    a, qq, kk = f32c(a_ik), f32c(q), f32c(k)
    pos, tv, rv = f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
    batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
    e_start = csr_offsets(edges, N)
    cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
    seed = _draw_seed()
    out = torch.empty((N, H, 3), device=dev, dtype=torch.float32)
    sel_e = torch.empty((N, H), device=dev, dtype=torch.int64) if want_selection else None
    sel_i = torch.empty((N, H), device=dev, dtype=torch.int32) if want_selection else None
    p, ip = _lib.ptr, _lib.iptr
    # per-pair geometry shared by the heads, the two axes and the layers of a batch (kept on the input tensor)
    pcache, plist, prange = pair_geometry(rpos_ij_e, tvecs_n, batch_i, edge_ij_e, cutoff)
    _lib.invoke("cfb200_max_frame_cached", 1, dev,
                axis, p(qq), p(kk), p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E, cutoff, seed,
                p(f32c(frame1)), p(out), ip(sel_e), _lib.ptr(sel_i, torch.int32), p(pcache), p(plist), prange)
    return (out, sel_e, sel_i) if want_selection else out


class ComputeFrame1MaximumMethodCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/calc_maximum_frame.py:24-91: first axis (N,H,3), the unit
    vector to the nearest periodic image of the pair that maximises q.k + a d^2_min."""

    @staticmethod
    def forward(ctx, q, k, v, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                rvlen_n=None, cutoff_radius=None):
        return _frame_call(1, q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, None)

    @staticmethod
    def backward(ctx, gframevec):
        return (None,) * 14


class ComputeFrame2MaximumMethodCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/calc_maximum_frame.py:95-170: second axis (N,H,3), not yet
    orthogonalised against the first."""

    @staticmethod
    def forward(ctx, q, k, v, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                frame1, rvlen_n=None, cutoff_radius=None):
        return _frame_call(2, q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1)

    @staticmethod
    def backward(ctx, gframevec):
        return (None,) * 15


def max_frame3_with_selection(q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1, frame2):
    """Third axis of "max_wo_orthogonal" and the pair it was taken from: (frame3 (N,H,3), sel_edge (N,H))."""
    N, H = a_ik.shape
    E = edge_ij_e.shape[1]
    dev = a_ik.device
    a, qq, kk = f32c(a_ik), f32c(q), f32c(k)
    pos, tv, rv = f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
    batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
    e_start = csr_offsets(edges, N)
    cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
    seed = _draw_seed()
    f3 = torch.empty((N, H, 3), device=dev, dtype=torch.float32)
    sel = torch.empty((N, H), device=dev, dtype=torch.int64)
    nbytes = int(_lib.lib().cfb200_max_frame3_workspace_bytes(N, E))
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
    p, ip = _lib.ptr, _lib.iptr
    _lib.invoke("cfb200_max_frame3", 2, dev, p(qq), p(kk), p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start),
                N, E, cutoff, seed, p(f32c(frame1)), p(f32c(frame2)), p(f3), ip(sel), ws.data_ptr(), nbytes)
    return f3, sel


class ComputeFrame3MaximumMethodCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/calc_maximum_frame.py:173-245: third axis (N,H,3) of the frame method
    "max_wo_orthogonal", selected like the first two with the triple product of the three axes in the score."""

    @staticmethod
    def forward(ctx, q, k, v, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                frame1, frame2, rvlen_n=None, cutoff_radius=None):
        return max_frame3_with_selection(q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius,
                                         frame1, frame2)[0]

    @staticmethod
    def backward(ctx, gframevec):
        return (None,) * 16


def max_frame_with_selection(axis, q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius,
                             frame1=None):
    """Frame axis plus the integer selection behind it: (frame, pair index (N,H) int64,
    linear translation index (N,H) int32)."""
    return _frame_call(axis, q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1,
                       want_selection=True)


def max_frames_fused(q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius):
    """Both axes and the Gram-Schmidt completion in one launch; returns frame1, frame2, frame3.
    Draws two seeds, like the two reference Functions it stands for."""
    N, H = a_ik.shape
    E = edge_ij_e.shape[1]
    dev = a_ik.device
    a, qq, kk = f32c(a_ik), f32c(q), f32c(k)
    pos, tv, rv = f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
    batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
    e_start = csr_offsets(edges, N)
    cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
    s1, s2 = _draw_seed(), _draw_seed()
    f = torch.empty((3, N, H, 3), device=dev, dtype=torch.float32)
    p, ip = _lib.ptr, _lib.iptr
    pcache, plist, prange = pair_geometry(rpos_ij_e, tvecs_n, batch_i, edge_ij_e, cutoff)
    _lib.invoke("cfb200_max_frames_cached", 1, dev,
                p(qq), p(kk), p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E, cutoff, s1, s2,
                p(f[0]), p(f[1]), p(f[2]), p(pcache), p(plist), prange)
    return f[0], f[1], f[2]


def weighted_pca_frames(q, k, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius):
    """Weighted-PCA frames (frame1, frame2, frame3), non-differentiable.  ``q`` is q / sqrt(head_dim).
    Stands for the reference's RealPeriodicEncodingWithProjFuncCUDA(frame_method="weighted_pca"),
    FusedDotProductAttentionSigmaMatCUDA and the eigen-decomposition block of
    models/indexed_lattice_multi_head_attention_cuda.py:656-725.  Two seeds are drawn from numpy's
    global generator (the reference draws two for its kernels); the row signs, which the reference
    takes from torch.randint, use one more draw from torch's generator."""
    N, H = a_ik.shape
    E = edge_ij_e.shape[1]
    dev = a_ik.device
    a, qq, kk = f32c(a_ik), f32c(q), f32c(k)
    pos, tv, rv = f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
    batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
    e_start = csr_offsets(edges, N)
    cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
    _draw_seed()                                   # select_edges' seed in the reference (its output is never read)
    seed_noise = _draw_seed()
    seed_sign = int(torch.randint(0, 2 ** 62, (1,)).item())
    f = torch.empty((3, N, H, 3), device=dev, dtype=torch.float32)
    nbytes = int(_lib.lib().cfb200_sigma_frames_workspace_bytes(N, E))
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
    p, ip = _lib.ptr, _lib.iptr
    _, plist, prange = pair_geometry(rpos_ij_e, tvecs_n, batch_i, edge_ij_e, cutoff)
    _lib.invoke("cfb200_sigma_frames_cached", 2, dev, p(qq), p(kk), p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges),
                ip(e_start), N, E, cutoff, seed_noise, seed_sign, p(f[0]), p(f[1]), p(f[2]), ws.data_ptr(), nbytes,
                p(plist), prange)
    return f[0], f[1], f[2], seed_noise, seed_sign


def _static_call(axis, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1, want_selection=False):
    N, H = a_ik.shape
    E = edge_ij_e.shape[1]
    dev = a_ik.device
    a, pos, tv, rv = f32c(a_ik), f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
    batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
    e_start = csr_offsets(edges, N)
    cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
    seed = _draw_seed()
    out = torch.empty((N, H, 3), device=dev, dtype=torch.float32)
    sel_e = torch.empty((N, H), device=dev, dtype=torch.int64) if want_selection else None
    sel_i = torch.empty((N, H), device=dev, dtype=torch.int32) if want_selection else None
    p, ip = _lib.ptr, _lib.iptr
    _lib.invoke("cfb200_max_frame_static", 1, dev, axis, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E,
                cutoff, seed, p(f32c(frame1)), p(out), ip(sel_e), _lib.ptr(sel_i, torch.int32))
    return (out, sel_e, sel_i) if want_selection else out


class ComputeFrame1MaximumStaticMethodCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/calc_maximum_static_frame.py:24-91: first axis (N,H,3) of the "max_static"
    frames -- the unit vector to the nearest periodic image of the pair that maximises a d^2_min; queries and
    keys are accepted and ignored, as in the reference."""

    @staticmethod
    def forward(ctx, q, k, v, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                rvlen_n=None, cutoff_radius=None):
        return _static_call(1, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, None)

    @staticmethod
    def backward(ctx, gframevec):
        return (None,) * 14


class ComputeFrame2MaximumStaticMethodCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/calc_maximum_static_frame.py:95-170: second axis (N,H,3), not yet
    orthogonalised; its score is (d^2 - d^2_min) + log(max(1 - |cos|, 1e-5)) without the Gaussian coefficient."""

    @staticmethod
    def forward(ctx, q, k, v, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                frame1, rvlen_n=None, cutoff_radius=None):
        return _static_call(2, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1)

    @staticmethod
    def backward(ctx, gframevec):
        return (None,) * 15


def max_static_frame_with_selection(axis, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1=None):
    """Static frame axis plus the integer selection behind it (frame, pair index (N,H), translation index (N,H))."""
    return _static_call(axis, a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius, frame1, want_selection=True)


def max_static_frames_fused(a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, cutoff_radius):
    """Both static axes and the Gram-Schmidt completion in one launch; draws two seeds like the two Functions."""
    N, H = a_ik.shape
    E = edge_ij_e.shape[1]
    dev = a_ik.device
    a, pos, tv, rv = f32c(a_ik), f32c(rpos_ij_e), f32c(tvecs_n), f32c(rvlen_n)
    batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
    e_start = csr_offsets(edges, N)
    cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
    s1, s2 = _draw_seed(), _draw_seed()
    f = torch.empty((3, N, H, 3), device=dev, dtype=torch.float32)
    pcache, _, prange = pair_geometry(rpos_ij_e, tvecs_n, batch_i, edge_ij_e, cutoff)
    p, ip = _lib.ptr, _lib.iptr
    _lib.invoke("cfb200_max_frames_static", 1, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E, cutoff,
                s1, s2, p(f[0]), p(f[1]), p(f[2]), p(pcache), prange)
    return f[0], f[1], f[2]


class ComputeLatticeFrameCUDA(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/calc_lattice_frame.py:22-150: (frame_first, frame_second, frame_third), each
    (N,H,3): the directions of the three shortest lattice vectors of each atom's cell.  Three seeds are drawn from
    numpy's global generator, as the reference does."""

    @staticmethod
    def forward(ctx, q, k, v, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                rvlen_n=None, cutoff_radius=None):
        N, H = a_ik.shape
        E = edge_ij_e.shape[1]
        dev = a_ik.device
        a, tv, rv = f32c(a_ik), f32c(tvecs_n), f32c(rvlen_n)
        batch, edges = batch_i.contiguous(), edge_ij_e.contiguous()
        e_start = csr_offsets(edges, N)
        cutoff = 0.0 if cutoff_radius is None or rvlen_n is None else float(cutoff_radius)
        s1, s2, s3 = _draw_seed(), _draw_seed(), _draw_seed()
        f = torch.empty((3, N, H, 3), device=dev, dtype=torch.float32)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_lattice_frames", 1, dev, p(a), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E, cutoff, s1, s2,
                    s3, p(f[0]), p(f[1]), p(f[2]))
        ctx.mark_non_differentiable(f)
        return f[0], f[1], f[2]

    @staticmethod
    def backward(ctx, g1, g2, g3):
        return (None,) * 14


class ComputePCAFrame(torch.autograd.Function):
    """Drop-in for models/cuda_funcs/calc_pca_frame.py:22-80: frames from the principal axes of an atom's pair
    separations in the home cell -- (frame_first, frame_second, frame_third), each (N,H,3), by ascending eigenvalue,
    with a drawn sign per axis and head and the triple times its determinant.  The signs come from one draw of
    torch's generator hashed per (atom, head, axis) (the reference takes three torch.randint tensors), and the
    eigenvectors' own signs are fixed by "largest component positive" (the reference's are LAPACK's): the axes
    agree with the reference's up to sign."""

    @staticmethod
    def forward(ctx, q, k, v, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale,
                rvlen_n=None, cutoff_radius=None):
        N, H = a_ik.shape
        E = edge_ij_e.shape[1]
        dev = a_ik.device
        pos = f32c(rpos_ij_e)
        e_start = csr_offsets(edge_ij_e.contiguous(), N)
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())
        f = torch.empty((3, N, H, 3), device=dev, dtype=torch.float32)
        p, ip = _lib.ptr, _lib.iptr
        _lib.invoke("cfb200_pca_frames", 1, dev, p(pos), ip(e_start), N, E, seed, p(f[0]), p(f[1]), p(f[2]))
        return f[0], f[1], f[2]

    @staticmethod
    def backward(ctx, gframe_first, gframe_second, gframe_third):
        return (None,) * 14
