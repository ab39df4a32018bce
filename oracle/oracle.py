"""numpy front end of the CPU oracle (test infrastructure, never part of the product).

Only ``tests/``, the smoke check and the CPU-baseline leg of the benchmark import
this module.  It loads ``libcforacle.so`` (built by ``build_oracle.py`` from
``cf_oracle.c``) and exposes one function per routine of the restatement.  Each
function takes and returns numpy arrays; ``dtype=np.float64`` selects the double
build, which is used to decide which side of a float disagreement is closer to
the exact value.

The host-side glue of the reference that sits between its kernels (allocation,
argmax over an atom's pairs, Gram-Schmidt, scaling by the two coefficients) is
restated here and in ``cf_oracle.c``; each function cites the reference lines.
"""
import ctypes
import dataclasses
import math
import os

import numpy as np

from . import build_oracle

_lib = None


class _CConfig(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("H", "head_dim", "D_dist", "D_ang", "lattice_range", "minimum_range", "cos_abs",
                 "win_dist", "win_ang", "cut_sigma")] + \
               [(n, ctypes.c_float) for n in
                ("dist_max", "wscale_dist", "angle_sigma", "c_dist", "c_ang", "cutoff_radius",
                 "symm_break_noise")]


@dataclasses.dataclass
class Config:
    """Hyper-parameters the reference bakes into its kernels by text substitution
    (models/cuda_funcs/kernel_manager.py:116-149) plus the scalars its Functions pass
    at launch (models/cuda_funcs/real_space_framed_proj.py:35-40).  Defaults are those
    of params/crystalframer/default_jarvis.json."""
    H: int = 8
    head_dim: int = 16
    D_dist: int = 64
    D_ang: int = 64
    lattice_range: int = 2
    minimum_range: int = 2
    cos_abs: int = 0
    cut_sigma: int = 4
    dist_max: float = 14.0
    wscale_dist: float = 1.0
    wscale_ang: float = 4.0
    c_dist: float = 1.0
    c_ang: float = 1.0
    cutoff_radius: float = -3.5
    symm_break_noise: float = 0.0

    @property
    def win_dist(self):
        return math.ceil(2 * self.wscale_dist * self.cut_sigma + 1)

    @property
    def win_ang(self):
        return math.ceil(2 * self.wscale_ang * self.cut_sigma + 1)

    @property
    def angle_sigma(self):
        if self.D_ang <= 1:
            return 1.0
        span = 1.0 if self.cos_abs else 2.0
        return span * self.wscale_ang / (self.D_ang - 1)

    def c(self):
        return _CConfig(self.H, self.head_dim, self.D_dist, self.D_ang, self.lattice_range,
                        self.minimum_range, self.cos_abs, self.win_dist, self.win_ang, self.cut_sigma,
                        self.dist_max, self.wscale_dist, self.angle_sigma, self.c_dist, self.c_ang,
                        self.cutoff_radius, self.symm_break_noise)


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.LIB
        if not os.path.exists(path):
            build_oracle.build_restatement()
        _lib = ctypes.CDLL(path)
    return _lib


def _fn(name, dtype):
    f = getattr(lib(), name + ("_f64" if np.dtype(dtype) == np.float64 else "_f32"))
    f.restype = None
    return f


def _p(x):
    return None if x is None else x.ctypes.data_as(ctypes.c_void_p)


def _r(x, dtype):
    return None if x is None else np.ascontiguousarray(x, dtype=dtype)


def _i64(x):
    return np.ascontiguousarray(x, dtype=np.int64)


def _f32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def edge_index(sizes):
    """models/indexed_latticeformer_encoder.py:15-32 and the CSR offsets of
    models/cuda_funcs/fused_dpa.py:24-26."""
    sizes = _i64(sizes)
    N = int(sizes.sum())
    E = int((sizes * sizes).sum())
    edges = np.empty((2, E), np.int64)
    e_start = np.empty(N + 1, np.int64)
    _fn("cfo_edge_index", np.float32)(_p(sizes), ctypes.c_int64(len(sizes)), _p(edges), _p(e_start),
                                      ctypes.c_int64(E))
    return edges, e_start


def lattice_geometry(pos, trans_vec, sizes):
    """pos_ij, reciprocal vectors, cell volume, batch index:
    models/indexed_latticeformer_encoder.py:175-245 (float32, same operation order)."""
    sizes = _i64(sizes)
    pos = _f32(pos)
    T = _f32(trans_vec)
    edges, e_start = edge_index(sizes)
    batch = np.repeat(np.arange(len(sizes), dtype=np.int64), sizes)
    m = T
    vcell = (m[:, 0, 0] * m[:, 1, 1] * m[:, 2, 2] + m[:, 0, 1] * m[:, 1, 2] * m[:, 2, 0]
             + m[:, 0, 2] * m[:, 1, 0] * m[:, 2, 1] - m[:, 0, 2] * m[:, 1, 1] * m[:, 2, 0]
             - m[:, 0, 0] * m[:, 1, 2] * m[:, 2, 1] - m[:, 0, 1] * m[:, 1, 0] * m[:, 2, 2]).astype(np.float32)
    rec = np.stack([np.cross(T[:, 1], T[:, 2]), np.cross(T[:, 2], T[:, 0]), np.cross(T[:, 0], T[:, 1])],
                   axis=1).astype(np.float32)
    rec = (rec * (np.float32(2.0 * math.pi) / vcell)[:, None, None]).astype(np.float32)
    pos_ij = (pos[edges[1]] - pos[edges[0]]).astype(np.float32)
    rvlen = np.sqrt((rec * rec).sum(-1)).astype(np.float32)
    return dict(edges=edges, e_start=e_start, batch=batch, pos_ij=pos_ij, rvecs=rec, vcell=vcell, rvlen=rvlen)


def lattice_range(cfg, a_ik, rvlen, batch):
    a_ik = _f32(a_ik)
    N = a_ik.shape[0]
    R = np.empty((N, cfg.H, 3), np.int32)
    c = cfg.c()
    _fn("cfo_lattice_range", np.float32)(ctypes.byref(c), _p(a_ik), _p(_f32(rvlen)), _p(_i64(batch)),
                                         ctypes.c_int64(N), _p(R))
    return R


def framed_proj_fwd(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, W_d, W_a, frames, dtype=np.float32,
                    values=True):
    """z (E,H) and values (E,H,head_dim).  W_d (H,hd,D_dist); W_a (3,H,hd,D_ang) or None;
    frames (3,N,H,3) or None."""
    a = _r(a_ik, dtype)
    N, H = a.shape
    E = edges.shape[1]
    z = np.empty((E, H), dtype)
    v = np.empty((E, H, cfg.head_dim), dtype) if values else None
    c = cfg.c()
    _fn("cfo_framed_proj_fwd", dtype)(
        ctypes.byref(c), _p(a), _p(_r(pos_ij, dtype)), _p(_r(tvecs, dtype)), _p(_f32(rvlen)),
        _p(_i64(batch)), _p(_i64(edges)), ctypes.c_int64(N), ctypes.c_int64(E),
        _p(_r(W_d, dtype)), _p(_r(W_a, dtype)), _p(_r(frames, dtype)), _p(z), _p(v))
    return z, v


def framed_proj_bwd(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, e_start, W_d, W_a, frames, z, gz, gv,
                    dtype=np.float32):
    a = _r(a_ik, dtype)
    N, H = a.shape
    E = edges.shape[1]
    ga = np.empty((N, H), dtype)
    gW_d = np.empty((H, cfg.head_dim, cfg.D_dist), dtype)
    gW_a = np.empty((3, H, cfg.head_dim, cfg.D_ang), dtype) if W_a is not None else None
    c = cfg.c()
    _fn("cfo_framed_proj_bwd", dtype)(
        ctypes.byref(c), _p(a), _p(_r(pos_ij, dtype)), _p(_r(tvecs, dtype)), _p(_f32(rvlen)),
        _p(_i64(batch)), _p(_i64(edges)), _p(_i64(e_start)), ctypes.c_int64(N), ctypes.c_int64(E),
        _p(_r(W_d, dtype)), _p(_r(W_a, dtype)), _p(_r(frames, dtype)), _p(_r(z, dtype)), _p(_r(gz, dtype)),
        _p(_r(gv, dtype)), _p(ga), _p(gW_d), _p(gW_a))
    return ga, gW_d, gW_a


def _frame_edges(name, cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed, frame1, dtype):
    a = _r(a_ik, dtype)
    N, H = a.shape
    E = edges.shape[1]
    d = np.empty((E, H, 3), dtype)
    val = np.empty((E, H), dtype)
    img = np.empty((E, H), np.int32)
    c = cfg.c()
    args = [ctypes.byref(c), _p(a), _p(_r(pos_ij, dtype)), _p(_r(tvecs, dtype)), _p(_f32(rvlen)),
            _p(_i64(batch)), _p(_i64(edges)), ctypes.c_int64(N), ctypes.c_int64(E), ctypes.c_uint64(seed)]
    if frame1 is not None:
        for f in (frame1 if isinstance(frame1, (tuple, list)) else (frame1,)):
            args.append(_p(_r(f, dtype)))
    args += [_p(d), _p(val), _p(img)]
    _fn(name, dtype)(*args)
    return d, val, img


def frame1_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed=0, dtype=np.float32):
    return _frame_edges("cfo_frame1_edges", cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed, None, dtype)


def frame2_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, frame1, seed=0, dtype=np.float32):
    return _frame_edges("cfo_frame2_edges", cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed, frame1, dtype)


def frame2_static_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, frame1, seed=0, dtype=np.float32):
    return _frame_edges("cfo_frame2_static_edges", cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed, frame1, dtype)


def frame3_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, frame1, frame2, seed=0, dtype=np.float32):
    """Third-axis candidates of "max_wo_orthogonal" (models/kernels/compute_third_frame_each_edge.cu)."""
    return _frame_edges("cfo_frame3_edges", cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed, (frame1, frame2), dtype)


def max_frames_wo_orthogonal(cfg, q_scaled, k, a_ik, pos_ij, tvecs, rvlen, batch, edges, e_start, seeds=(0, 0, 0),
                             dtype=np.float32):
    """Frame method "max_wo_orthogonal" (models/indexed_lattice_multi_head_attention_cuda.py:449-461, :483-488):
    the first axis and the un-orthogonalised second axis of "max", and a third axis selected like them with the
    triple product in place of the collinearity term."""
    d1, v1, _ = frame1_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seeds[0], dtype)
    f1, sel1 = frame_select(cfg, q_scaled, k, edges, e_start, d1, v1, dtype)
    d2, v2, _ = frame2_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, f1, seeds[1], dtype)
    f2, sel2 = frame_select(cfg, q_scaled, k, edges, e_start, d2, v2, dtype)
    d3, v3, img3 = frame3_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, f1, f2, seeds[2], dtype)
    f3, sel3 = frame_select(cfg, q_scaled, k, edges, e_start, d3, v3, dtype)
    hh = np.arange(cfg.H)[None, :]
    return dict(frame1=f1, frame2=f2, frame3=f3, sel_edge1=sel1, sel_edge2=sel2, sel_edge3=sel3, sel_image3=img3[sel3, hh])


def frame_select(cfg, q, k, edges, e_start, direction, value, dtype=np.float32):
    q = _r(q, dtype)
    N, H = q.shape[:2]
    E = edges.shape[1]
    frame = np.empty((N, H, 3), dtype)
    sel = np.empty((N, H), np.int64)
    c = cfg.c()
    _fn("cfo_frame_select", dtype)(ctypes.byref(c), _p(q), _p(_r(k, dtype)), _p(_i64(edges)),
                                   _p(_i64(e_start)), ctypes.c_int64(N), ctypes.c_int64(E),
                                   _p(_r(direction, dtype)), _p(_r(value, dtype)), _p(frame), _p(sel))
    return frame, sel


def frame_complete(f1, f2max, dtype=np.float32):
    f1 = _r(f1, dtype)
    f2max = _r(f2max, dtype)
    f2 = np.empty_like(f1)
    f3 = np.empty_like(f1)
    _fn("cfo_frame_complete", dtype)(_p(f1), _p(f2max), ctypes.c_int64(f1.size // 3), _p(f2), _p(f3))
    return f2, f3


def max_frames(cfg, q_scaled, k, a_ik, pos_ij, tvecs, rvlen, batch, edges, e_start, seed1=0, seed2=0,
               dtype=np.float32):
    """The "max" frame method end to end
    (models/indexed_lattice_multi_head_attention_cuda.py:435-493): first axis, second
    axis, Gram-Schmidt.  ``q_scaled`` is q / sqrt(head_dim).  Returns the three frames
    and the integer selections (pair and image for both axes)."""
    d1, v1, img1 = frame1_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed1, dtype)
    f1, sel1 = frame_select(cfg, q_scaled, k, edges, e_start, d1, v1, dtype)
    d2, v2, img2 = frame2_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, f1, seed2, dtype)
    f2max, sel2 = frame_select(cfg, q_scaled, k, edges, e_start, d2, v2, dtype)
    f2, f3 = frame_complete(f1, f2max, dtype)
    H = cfg.H
    hh = np.arange(H)[None, :]
    return dict(frame1=f1, frame2_max=f2max, frame2=f2, frame3=f3, sel_edge1=sel1, sel_edge2=sel2,
                sel_image1=img1[sel1, hh], sel_image2=img2[sel2, hh])


def max_static_frames(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, e_start, seed1=0, seed2=0, dtype=np.float32):
    """The "max_static" frame method (models/cuda_funcs/calc_maximum_static_frame.py:24-170 with
    models/indexed_lattice_multi_head_attention_cuda.py:463-481): as "max", but queries and keys do not enter
    the selection and the second axis' score carries no Gaussian coefficient."""
    N, H = a_ik.shape
    zeros = np.zeros((N, H, cfg.head_dim), dtype)
    d1, v1, img1 = frame1_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed1, dtype)
    f1, sel1 = frame_select(cfg, zeros, zeros, edges, e_start, d1, v1, dtype)
    d2, v2, img2 = frame2_static_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, f1, seed2, dtype)
    f2max, sel2 = frame_select(cfg, zeros, zeros, edges, e_start, d2, v2, dtype)
    f2, f3 = frame_complete(f1, f2max, dtype)
    hh = np.arange(cfg.H)[None, :]
    return dict(frame1=f1, frame2_max=f2max, frame2=f2, frame3=f3, sel_edge1=sel1, sel_edge2=sel2,
                sel_image1=img1[sel1, hh], sel_image2=img2[sel2, hh])


def lattice_frames(cfg, a_ik, tvecs, rvlen, batch, edges, e_start, seeds=(0, 0, 0), dtype=np.float32):
    """The "lattice" frame method: per (atom, head) the directions of the three shortest lattice vectors
    (models/cuda_funcs/calc_lattice_frame.py:22-150).  Returns (frame1, frame2, frame3), each (N,H,3)."""
    a = _r(a_ik, dtype)
    N, H = a.shape
    # pair index of every atom's self pair (the reference's kernels run over all pairs and act on i == j only;
    # the noise stream is indexed by that pair)
    self_pair = np.empty(N, np.int64)
    for i in range(N):
        js = edges[1, e_start[i]:e_start[i + 1]]
        self_pair[i] = e_start[i] + int(np.nonzero(js == i)[0][0])
    f = [np.empty((N, H, 3), dtype) for _ in range(3)]
    sd = (ctypes.c_uint64 * 3)(*[int(x) & (2 ** 64 - 1) for x in seeds])
    c = cfg.c()
    _fn("cfo_lattice_frames", dtype)(ctypes.byref(c), _p(a), _p(_r(tvecs, dtype)), _p(_f32(rvlen)), _p(_i64(batch)),
                                     ctypes.c_int64(N), sd, _p(self_pair), _p(f[0]), _p(f[1]), _p(f[2]))
    return f[0], f[1], f[2]


def dpa_fwd(cfg, q, k, v, aij, bij, edges, e_start, dtype=np.float32):
    q = _r(q, dtype)
    N, H, hd = q.shape
    E = edges.shape[1]
    prob = np.empty((E, H), dtype)
    out = np.empty((N, H, hd), dtype)
    c = cfg.c()
    _fn("cfo_dpa_fwd", dtype)(ctypes.byref(c), _p(q), _p(_r(k, dtype)), _p(_r(v, dtype)), _p(_r(aij, dtype)),
                              _p(_r(bij, dtype)), _p(_i64(edges)), _p(_i64(e_start)), ctypes.c_int64(N),
                              ctypes.c_int64(E), _p(prob), _p(out))
    return out, prob


def dpa_bwd(cfg, q, k, v, bij, edges, e_start, prob, out, gout, dtype=np.float32):
    q = _r(q, dtype)
    N, H, hd = q.shape
    E = edges.shape[1]
    gq = np.empty((N, H, hd), dtype)
    gk = np.empty((N, H, hd), dtype)
    gv = np.empty((N, H, hd), dtype)
    ga = np.empty((E, H), dtype)
    gb = np.empty((E, H, hd), dtype) if bij is not None else None
    c = cfg.c()
    _fn("cfo_dpa_bwd", dtype)(ctypes.byref(c), _p(q), _p(_r(k, dtype)), _p(_r(v, dtype)), _p(_r(bij, dtype)),
                              _p(_i64(edges)), _p(_i64(e_start)), ctypes.c_int64(N), ctypes.c_int64(E),
                              _p(_r(prob, dtype)), _p(_r(out, dtype)), _p(_r(gout, dtype)),
                              _p(gq), _p(gk), _p(gv), _p(ga), _p(gb))
    return gq, gk, gv, ga, gb


def mean_fwd(x, sizes, dtype=np.float32):
    x = _r(x, dtype)
    sizes = _i64(sizes)
    start = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    D = x.size // x.shape[0]
    out = np.empty((len(sizes),) + x.shape[1:], dtype)
    _fn("cfo_mean_fwd", dtype)(_p(x), _p(start), ctypes.c_int64(len(sizes)), ctypes.c_int64(D), _p(out))
    return out


def mean_bwd(gout, sizes, dtype=np.float32):
    gout = _r(gout, dtype)
    sizes = _i64(sizes)
    start = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    D = gout.size // gout.shape[0]
    gx = np.empty((int(sizes.sum()),) + gout.shape[1:], dtype)
    _fn("cfo_mean_bwd", dtype)(_p(gout), _p(start), ctypes.c_int64(len(sizes)), ctypes.c_int64(D), _p(gx))
    return gx


def reciprocal_geometry(pos, cells, sizes, edges):
    """Reciprocal vectors, cell volumes and the phase base of every pair
    (models/indexed_latticeformer_encoder.py:198-205, :239-243): rvecs (B,3,3) = 2 pi cross / vcell,
    kr (E,3) = rvecs[crystal of i] @ (pos_j - pos_i)."""
    cells = np.asarray(cells, np.float32)
    pos = np.asarray(pos, np.float32)
    vcell = np.einsum("bi,bi->b", cells[:, 0], np.cross(cells[:, 1], cells[:, 2])).astype(np.float32)
    rvecs = np.stack([np.cross(cells[:, 1], cells[:, 2]), np.cross(cells[:, 2], cells[:, 0]),
                      np.cross(cells[:, 0], cells[:, 1])], axis=1).astype(np.float32)
    rvecs = (rvecs * (np.float32(2.0 * math.pi) / vcell)[:, None, None]).astype(np.float32)
    batch = np.repeat(np.arange(len(sizes)), np.asarray(sizes))
    pos_ij = pos[edges[1]] - pos[edges[0]]
    kr = np.einsum("eij,ej->ei", rvecs[batch[edges[0]]], pos_ij).astype(np.float32)
    return rvecs, vcell, kr


def reci_enc_fwd(a_ik, kr, rvecs, vcell, batch, edges, lattice_range=2, dtype=np.float32):
    """models/cuda_funcs/reci_space_enc.py:19-62: (z (E,H), sumexp (E,H))."""
    a_ik = _r(a_ik, dtype)
    N, H = a_ik.shape
    edges = _i64(edges)
    E = edges.shape[1]
    z = np.empty((E, H), dtype)
    sumexp = np.empty((E, H), dtype)
    _fn("cfo_reci_enc_fwd", dtype)(_p(a_ik), _p(_r(kr, dtype)), _p(_r(rvecs, dtype)), _p(_r(vcell, dtype)),
                                   _p(_i64(batch)), _p(edges), ctypes.c_int64(N), ctypes.c_int64(H), ctypes.c_int64(E),
                                   ctypes.c_int(lattice_range), _p(z), _p(sumexp))
    return z, sumexp


def reci_enc_bwd(a_ik, kr, rvecs, batch, edges, gz, sumexp, lattice_range=2, dtype=np.float32):
    """models/cuda_funcs/reci_space_enc.py:64-97: ga (N,H)."""
    a_ik = _r(a_ik, dtype)
    N, H = a_ik.shape
    edges = _i64(edges)
    e_start = np.concatenate([[0], np.cumsum(np.bincount(edges[0], minlength=N))]).astype(np.int64)
    ga = np.empty((N, H), dtype)
    _fn("cfo_reci_enc_bwd", dtype)(_p(a_ik), _p(_r(kr, dtype)), _p(_r(rvecs, dtype)), _p(_i64(batch)), _p(e_start),
                                   _p(_r(gz, dtype)), _p(_r(sumexp, dtype)), ctypes.c_int64(N), ctypes.c_int64(H),
                                   ctypes.c_int(lattice_range), _p(ga))
    return ga


# ---------------------------------------------------------------------------------------------
# Weighted-PCA frames (models/indexed_lattice_multi_head_attention_cuda.py:620-725)
# ---------------------------------------------------------------------------------------------
def sigma_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed=0, dtype=np.float32):
    a = _r(a_ik, dtype)
    N, H = a.shape
    E = edges.shape[1]
    z, sig = np.empty((E, H), dtype), np.empty((E, H, 6), dtype)
    nd2, ndir = np.empty((E, H), dtype), np.empty((E, H, 3), dtype)
    c = cfg.c()
    _fn("cfo_sigma_edges", dtype)(ctypes.byref(c), _p(a), _p(_r(pos_ij, dtype)), _p(_r(tvecs, dtype)), _p(_f32(rvlen)),
                                  _p(_i64(batch)), _p(_i64(edges)), ctypes.c_int64(N), ctypes.c_int64(E),
                                  ctypes.c_uint64(seed), _p(z), _p(sig), _p(nd2), _p(ndir))
    return z, sig, nd2, ndir


def hash_uniform(seed, tid, draw):
    """Python twin of cfo_uniform (the counter-based noise shared with the CUDA library)."""
    M = (1 << 64) - 1
    x = (seed ^ ((tid * 0x9E3779B97F4A7C15) & M) ^ ((draw * 0xD1B54A32D192ED03) & M)) & M
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & M
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & M
    x ^= x >> 31
    return np.float32(((x >> 40) + 1)) * np.float32(1.0 / 16777216.0)


def pca_frames(pos_ij, e_start, H, seed=0):
    """The "pca" frame method (models/cuda_funcs/calc_pca_frame.py:22-76 of the reference): per atom the scatter
    matrix of its pair separations in the home cell about their mean, sum_j (r_ij - mean)(r_ij - mean)^T, and its
    eigenvectors by ascending eigenvalue as the three axes (columns of the eigenvector matrix, :47-60), the same for
    every head; per (atom, head) a sign per axis and all three axes times the determinant of the signed triple
    (:52-66).  The reference draws the signs with torch.randint and inherits LAPACK's eigenvector signs; here, as in
    the library, an eigenvector's largest component is positive before a hash-drawn sign.  Returns frames (3,N,H,3)
    float32, the scatter matrices (N,3,3) and their eigenvalues (N,3) in float64."""
    pos_ij = np.asarray(pos_ij, np.float64)
    N = len(e_start) - 1
    frames = np.zeros((3, N, H, 3), np.float32)
    mats, evals = np.zeros((N, 3, 3)), np.zeros((N, 3))
    for i in range(N):
        r = pos_ij[int(e_start[i]):int(e_start[i + 1])]
        d = r - r.mean(0, keepdims=True) if len(r) else r
        M = d.T @ d
        w, V = np.linalg.eigh(M)
        for c in range(3):
            if V[int(np.argmax(np.abs(V[:, c]))), c] < 0:
                V[:, c] = -V[:, c]
        mats[i], evals[i] = M, w
        for h in range(H):
            F = np.stack([V[:, c] * (1.0 if hash_uniform(seed, i * H + h, c) > 0.5 else -1.0) for c in range(3)])
            F = F * np.linalg.det(F.T)
            for c in range(3):
                frames[c, i, h] = F[c]
    return frames, mats, evals


def weighted_pca_frames(cfg, q_scaled, k, a_ik, pos_ij, tvecs, rvlen, batch, edges, e_start, seed_noise=0,
                        seed_sign=0):
    """Per (atom, head): attention-pooled second-moment matrix (softmax over the atom's pairs of
    q.k + z, the intended bias), optional tie-breaking term sigma_max * det^(1/3) * noise, symmetric
    eigen-decomposition (ascending eigenvalues; each eigenvector signed so that its largest component
    is positive), frames = ROWS of the eigenvector matrix (as the reference indexes it, :693-695),
    hash-drawn row signs, and a final multiplication by the determinant so that the triad is
    right-handed.  Matrices with determinant <= 1e-5 give the identity.  Returns frames (3,N,H,3),
    the pooled matrices (N,H,3,3) and their eigenvalues (N,H,3)."""
    N, H = a_ik.shape
    z, sig, nd2, ndir = sigma_edges(cfg, a_ik, pos_ij, tvecs, rvlen, batch, edges, seed_noise)
    q_scaled, k = np.asarray(q_scaled, np.float64), np.asarray(k, np.float64)
    frames = np.zeros((3, N, H, 3), np.float32)
    mats = np.zeros((N, H, 3, 3), np.float64)
    evals = np.zeros((N, H, 3), np.float64)
    idx6 = [(0, 0), (0, 1), (0, 2), (1, 1), (1, 2), (2, 2)]
    for i in range(N):
        e0, e1 = int(e_start[i]), int(e_start[i + 1])
        js = edges[1, e0:e1]
        for h in range(H):
            logit = (q_scaled[i, h][None, :] * k[js, h]).sum(-1) + z[e0:e1, h].astype(np.float64)
            p = np.exp(logit - logit.max())
            p /= p.sum()
            s6 = (p[:, None] * sig[e0:e1, h].astype(np.float64)).sum(0)
            M = np.zeros((3, 3))
            for v, (r, c) in zip(s6, idx6):
                M[r, c] = M[c, r] = v
            M = M.astype(np.float32).astype(np.float64)
            det = np.linalg.det(M)
            if cfg.symm_break_noise > 0:
                jn = int(np.argmin(nd2[e0:e1, h]))
                u = ndir[e0 + jn, h].astype(np.float64)
                M = M + np.outer(u, u) * np.cbrt(det) * cfg.symm_break_noise
            V = np.eye(3)
            w = np.zeros(3)
            if det > 1e-5:
                w, V = np.linalg.eigh(M)
                for c in range(3):
                    if V[int(np.argmax(np.abs(V[:, c]))), c] < 0:
                        V[:, c] = -V[:, c]
            F = V.copy()                                            # frame r = row r of V
            for r in range(3):
                sgn = 1.0 if hash_uniform(seed_sign, i * H + h, r) > 0.5 else -1.0
                F[r] *= sgn
            F *= np.sign(np.linalg.det(F.T))
            mats[i, h], evals[i, h] = M, w
            for r in range(3):
                frames[r, i, h] = F[r]
    return frames, mats, evals
