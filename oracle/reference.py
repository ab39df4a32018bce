"""Driver for the reference project's own kernels compiled into oracle/_ref/.

Test infrastructure only.  ``RefKernels("cpu")`` runs the reference kernels on the host
cores through the g++ build; ``RefKernels("cuda")`` launches the nvcc build of the same
sources on the current GPU (the reference-on-the-same-GPU baseline).  Tensors are torch
tensors on the matching device; the host-side steps the reference performs in Python
between its kernels are restated here with the file and line they follow.  The grid and
block shapes are the reference's own.
"""
import ctypes
import json
import math
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available(device="cpu"):
    return os.path.exists(os.path.join(REF_DIR, "libcfref_gpu.so" if device == "cuda" else "libcfref_cpu.so"))


def segment_argmax(score, edge_i, N):
    """Row-wise argmax over an atom's pairs, lowest pair index on ties (the reference
    leaves ties to torch_scatter.scatter_max, models/cuda_funcs/calc_maximum_frame.py:76)."""
    E, H = score.shape
    idx = edge_i[:, None].expand(E, H)
    best = torch.full((N, H), -1e10, dtype=score.dtype, device=score.device)
    best = best.scatter_reduce(0, idx, score, reduce="amax", include_self=True)
    ar = torch.arange(E, device=score.device)[:, None].expand(E, H)
    cand = torch.where(score == best[edge_i], ar, torch.full_like(ar, E))
    arg = torch.full((N, H), E, dtype=torch.long, device=score.device)
    return arg.scatter_reduce(0, idx, cand, reduce="amin", include_self=True)


class RefKernels:
    PE_THREADS = 16   # KernelManager.PE_THREAD_NUM, models/cuda_funcs/kernel_manager.py:62

    def __init__(self, device="cpu", tag=""):
        self.device = device
        name = ("libcfref_gpu" if device == "cuda" else "libcfref_cpu") + tag + ".so"
        self.lib = ctypes.CDLL(os.path.join(REF_DIR, name))
        self.sigs = json.load(open(os.path.join(REF_DIR, f"signatures{tag}.json")))
        self.consts = json.loads(self.sigs["_consts"])
        self.prefix = "cfref_gpu_" if device == "cuda" else "cfref_cpu_"

    def launch(self, name, grid, block, *args):
        sig = self.sigs[name]
        assert len(sig) == len(args), (name, len(sig), len(args))
        conv = [ctypes.c_uint(int(grid)), ctypes.c_uint(int(block))]
        if self.device == "cuda":
            conv.append(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        for kind, a in zip(sig, args):
            if kind == "ptr":
                if a is None:
                    conv.append(ctypes.c_void_p(0))
                else:
                    assert a.is_contiguous() and a.device.type == self.device, name
                    conv.append(ctypes.c_void_p(a.data_ptr()))
            elif kind == "f32":
                conv.append(ctypes.c_float(float(a)))
            elif kind == "f64":
                conv.append(ctypes.c_double(float(a)))
            elif kind == "u8":
                conv.append(ctypes.c_ubyte(int(a)))
            elif kind == "u32":
                conv.append(ctypes.c_uint(int(a)))
            elif kind == "i32":
                conv.append(ctypes.c_int(int(a)))
            elif kind == "i64":
                conv.append(ctypes.c_longlong(int(a)))
            elif kind == "u64":
                conv.append(ctypes.c_ulonglong(int(a) & (2 ** 64 - 1)))
            else:
                raise TypeError(kind)
        fn = getattr(self.lib, self.prefix + name)
        fn.restype = ctypes.c_int if self.device == "cuda" else None
        rc = fn(*conv)
        if self.device == "cuda" and rc != 0:
            raise RuntimeError(f"reference kernel {name}: CUDA error {rc}")

    # ---- models/cuda_funcs/fused_dpa.py:24-26 -------------------------------------
    @staticmethod
    def e_start(edges, N):
        s = torch.zeros(N + 1, dtype=torch.long, device=edges.device)
        s.scatter_add_(0, edges[0] + 1, torch.ones_like(edges[0]))
        return s.cumsum(0)

    # ---- models/cuda_funcs/real_space_framed_proj.py:21-120 -------------------------
    def framed_proj_fwd(self, a_ik, rpos, tvecs, batch, edges, dist_max, wscale, W_k, W_ks, frames,
                        angle_sigma, c_dist, c_ang, rvlen, cutoff):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        hd = W_k.shape[-2]
        z = torch.empty((E, H), **kw)
        v = torch.empty((E, H, hd), **kw)
        d2min = torch.empty((E, H), **kw)
        b = self.PE_THREADS
        self.launch("real_enc_frame_proj_fwd_length", (E * H + b - 1) // b, b,
                    a_ik, rpos, None, tvecs, batch, edges, N, H, E, dist_max, wscale, W_k, 1, rvlen, cutoff,
                    z, v, d2min)
        v = v * c_dist
        if W_ks is not None:
            va = torch.empty((3, E, H, hd), **kw)
            self.launch("real_enc_frame_proj_fwd_angle", (3 * E * H + b - 1) // b, b,
                        a_ik, rpos, d2min, tvecs, batch, edges, N, H, E, angle_sigma, W_ks, frames, 1, rvlen,
                        cutoff, None, va)
            v = v + va.sum(dim=0) * c_ang
        return z, v

    # ---- models/cuda_funcs/real_space_framed_proj.py:123-221 ------------------------
    def framed_proj_bwd(self, a_ik, rpos, tvecs, batch, edges, dist_max, wscale, W_k, W_ks, frames,
                        angle_sigma, c_dist, c_ang, rvlen, cutoff, z, gz, gv):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        e_start = self.e_start(edges, N)
        ga = torch.empty((N, H), **kw)
        gW = torch.empty((N,) + tuple(W_k.shape[-3:]), **kw)
        b = self.PE_THREADS
        self.launch("real_enc_frame_proj_bwd_length", (N * H + b - 1) // b, b,
                    a_ik, rpos, tvecs, batch, edges, e_start, z, gz.contiguous(), gv.contiguous(), N, H, E,
                    dist_max, wscale, W_k, 1, rvlen, cutoff, ga, gW)
        ga = ga * c_dist
        gWs = None
        if W_ks is not None:
            gWs = torch.empty((3, N) + tuple(W_ks.shape[-3:]), **kw)
            ga3 = torch.empty((3, N, H), **kw)
            self.launch("real_enc_frame_proj_bwd_angle", (3 * N * H + b - 1) // b, b,
                        a_ik, rpos, tvecs, batch, edges, e_start, z, gz.contiguous(), gv.contiguous(), N, H, E,
                        angle_sigma, W_ks, frames, 1, rvlen, cutoff, ga3, gWs)
            ga = ga + ga3.sum(dim=0) * c_ang
            gWs = gWs.sum(dim=1) * c_ang          # autograd's sum_to_size over the atom axis
        return ga, gW.sum(dim=0), gWs

    # ---- models/cuda_funcs/real_space_enc_proj.py:21-213, frame_method "no" ---------------
    def proj_fwd(self, a_ik, rpos, tvecs, batch, edges, K, dist_max, wscale, W_k, rvlen, cutoff):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        z = torch.empty((E, H), **kw)
        v = torch.empty((E, H, W_k.shape[-2]), **kw)
        self.launch("real_enc_proj_fwd", (E * H + H - 1) // H, H, a_ik, rpos, None, tvecs, batch, edges, N, H, E, K,
                    dist_max, wscale, W_k, 1, rvlen, cutoff, z, v)
        return z, v

    def proj_bwd(self, a_ik, rpos, tvecs, batch, edges, dist_max, wscale, W_k, rvlen, cutoff, z, gz, gv):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        e_start = self.e_start(edges, N)
        ga = torch.empty((N, H), **kw)
        gW = torch.empty((N,) + tuple(W_k.shape[-3:]), **kw)
        self.launch("real_enc_proj_bwd", (N * H + H - 1) // H, H, a_ik, rpos, tvecs, batch, edges, e_start, z,
                    gz.contiguous(), gv.contiguous(), N, H, E, dist_max, wscale, W_k, 1, rvlen, cutoff, ga, gW)
        return ga, gW.sum(dim=0)

    # ---- models/cuda_funcs/reci_space_enc.py:17-97 -----------------------------------------
    def reci_fwd(self, a_ik, kr, rvecs, vcell, batch, edges):
        N, H = a_ik.shape
        E = edges.shape[1]
        z = torch.empty((E, H), device=a_ik.device, dtype=a_ik.dtype)
        sumexp = torch.empty_like(z)
        self.launch("reci_enc_fwd", (E * H + H - 1) // H, H, a_ik, kr, rvecs, vcell, batch, edges, N, H, E, z, sumexp)
        return z, sumexp

    def reci_bwd(self, a_ik, kr, rvecs, vcell, batch, edges, z, gz, sumexp):
        N, H = a_ik.shape
        E = edges.shape[1]
        ga = torch.empty_like(a_ik)
        self.launch("reci_enc_bwd", (N * H + H - 1) // H, H, a_ik, kr, rvecs, vcell, batch, edges,
                    self.e_start(edges, N), z, gz.contiguous(), sumexp, N, H, E, ga)
        return ga

    # ---- models/cuda_funcs/real_space_enc.py:17-245: logit and un-projected value sums ----
    def real_enc_fwd(self, a_ik, rpos, tvecs, batch, edges, K, dist_max, wscale, rvlen, cutoff):
        N, H = a_ik.shape
        E = edges.shape[1]
        z = torch.empty((E, H), device=a_ik.device, dtype=a_ik.dtype)
        v = torch.empty((E, H, K), device=a_ik.device, dtype=a_ik.dtype)
        self.launch("real_enc_fwd", (E * H + H - 1) // H, H, a_ik, rpos, None, tvecs, batch, edges, N, H, E, K, dist_max,
                    wscale, rvlen, cutoff, z, v)
        return z, v

    def real_enc_bwd(self, a_ik, rpos, tvecs, batch, edges, K, dist_max, wscale, rvlen, cutoff, z, gz, gv):
        N, H = a_ik.shape
        E = edges.shape[1]
        ga = torch.empty_like(a_ik)
        self.launch("real_enc_bwd", (N * H + H - 1) // H, H, a_ik, rpos, None, tvecs, batch, edges, self.e_start(edges, N),
                    z, gz.contiguous(), gv.contiguous(), N, H, E, K, dist_max, wscale, rvlen, cutoff, ga)
        return ga

    # ---- weighted PCA: models/cuda_funcs/real_space_enc_proj.py:80-125, fused_dpa_sigmamat.py ----
    def sigma_fwd(self, a_ik, rpos, tvecs, batch, edges, rvlen, cutoff, seed=0):
        N, H = a_ik.shape
        E = edges.shape[1]
        dev = a_ik.device
        sigma = torch.zeros(E, H, 6, dtype=torch.float32, device=dev)
        select = torch.zeros((E, H), dtype=torch.int, device=dev)
        state = torch.empty(E * H * 48, dtype=torch.uint8, device=dev)
        sigma_max = torch.zeros((N, H, 6), device=dev)
        self.launch("real_enc_sigma_fwd", (E * H + H - 1) // H, H, a_ik, rpos, None, tvecs, batch, edges, N, H, E,
                    64, 14.0, 1.0, 1, rvlen, cutoff, sigma, state, seed, select, sigma_max)
        return sigma, sigma_max

    def sigma_pool(self, q_scaled, k, z, sigma, edges):
        N, H, K = q_scaled.shape
        E = edges.shape[1]
        e_start = self.e_start(edges, N)
        v0 = torch.zeros((N, H, 6), device=q_scaled.device)
        out = torch.empty_like(v0)
        prob = torch.empty((E, H), dtype=q_scaled.dtype, device=q_scaled.device)
        self.launch("fused_dpa_sigmamat_fwd", (N * H + H - 1) // H, H, q_scaled, k, v0, z, sigma, edges, e_start, N, H, E,
                    prob, out)
        return out

    # ---- models/cuda_funcs/calc_maximum_frame.py:24-170 -----------------------------
    def _edge_scores(self, q, k, edges, value):
        E = edges.shape[1]
        H = q.shape[1]
        qk = (q[edges[0]].reshape(E, H, 1, -1) @ k[edges[1]].reshape(E, H, -1, 1))[:, :, 0, 0]
        return qk + value

    def frame1(self, q_scaled, k, a_ik, rpos, tvecs, batch, edges, rvlen, cutoff, seed=0):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        state = torch.empty(E * H * 48, dtype=torch.uint8, device=a_ik.device)
        dx, dy, dz = (torch.zeros(E, H, **kw) for _ in range(3))
        val = torch.ones((E, H), **kw) * 1e10
        self.launch("compute_maximum_frame_each_edge", (E * H + 31) // 32, 32,
                    a_ik, rpos, None, tvecs, batch, edges, N, H, E, rvlen, cutoff, state, seed, dx, dy, dz, val)
        arg = segment_argmax(self._edge_scores(q_scaled, k, edges, val), edges[0], N)
        hh = torch.arange(H, device=a_ik.device)[None, :].expand(N, H)
        return torch.stack([dx[arg, hh], dy[arg, hh], dz[arg, hh]], dim=-1), arg

    def frame2(self, q_scaled, k, a_ik, rpos, tvecs, batch, edges, rvlen, cutoff, frame1, seed=0):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        state = torch.empty(E * H * 48, dtype=torch.uint8, device=a_ik.device)
        f1 = [frame1[:, :, d].contiguous() for d in range(3)]
        dx, dy, dz, val = (torch.zeros(E, H, **kw) for _ in range(4))
        self.launch("compute_second_frame_each_edge", (E * H + 31) // 32, 32,
                    a_ik, rpos, None, tvecs, batch, edges, N, H, E, rvlen, cutoff, state, seed,
                    f1[0], f1[1], f1[2], dx, dy, dz, val)
        arg = segment_argmax(self._edge_scores(q_scaled, k, edges, val), edges[0], N)
        hh = torch.arange(H, device=a_ik.device)[None, :].expand(N, H)
        return torch.stack([dx[arg, hh], dy[arg, hh], dz[arg, hh]], dim=-1), arg

    # ---- models/cuda_funcs/calc_maximum_frame.py:173-245 (frame method "max_wo_orthogonal") ----
    def frame3(self, q_scaled, k, a_ik, rpos, tvecs, batch, edges, rvlen, cutoff, frame1, frame2, seed=0):
        """The reference allocates the per-pair outputs with torch.empty and its kernel leaves them unwritten where no
        image qualifies; here they start as zero directions with value -1e15, which the arg-max never picks."""
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        state = torch.empty(E * H * 48, dtype=torch.uint8, device=a_ik.device)
        f1 = [frame1[:, :, d].contiguous() for d in range(3)]
        f2 = [frame2[:, :, d].contiguous() for d in range(3)]
        dx, dy, dz = (torch.zeros(E, H, **kw) for _ in range(3))
        val = torch.full((E, H), -1e15, **kw)
        # the kernel takes the head from threadIdx.x: one block per pair (calc_maximum_frame.py:196,205)
        self.launch("compute_third_frame_each_edge", E, H, a_ik, rpos, None, tvecs, batch, edges, N, H, E, 64, 14.0, 1.0,
                    rvlen, cutoff, state, seed, f1[0], f1[1], f1[2], f2[0], f2[1], f2[2], dx, dy, dz, val)
        arg = segment_argmax(self._edge_scores(q_scaled, k, edges, val), edges[0], N)
        hh = torch.arange(H, device=a_ik.device)[None, :].expand(N, H)
        return torch.stack([dx[arg, hh], dy[arg, hh], dz[arg, hh]], dim=-1), arg

    # ---- models/cuda_funcs/calc_maximum_static_frame.py:24-170: as frame1 / frame2 without q.k, static second kernel ----
    def frame1_static(self, a_ik, rpos, tvecs, batch, edges, rvlen, cutoff, seed=0):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        state = torch.empty(E * H * 48, dtype=torch.uint8, device=a_ik.device)
        dx, dy, dz = (torch.zeros(E, H, **kw) for _ in range(3))
        val = torch.ones((E, H), **kw) * 1e10
        self.launch("compute_maximum_frame_each_edge", (E * H + 31) // 32, 32,
                    a_ik, rpos, None, tvecs, batch, edges, N, H, E, rvlen, cutoff, state, seed, dx, dy, dz, val)
        arg = segment_argmax(val, edges[0], N)
        hh = torch.arange(H, device=a_ik.device)[None, :].expand(N, H)
        return torch.stack([dx[arg, hh], dy[arg, hh], dz[arg, hh]], dim=-1), arg

    def frame2_static(self, a_ik, rpos, tvecs, batch, edges, rvlen, cutoff, frame1, seed=0):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        state = torch.empty(E * H * 48, dtype=torch.uint8, device=a_ik.device)
        f1 = [frame1[:, :, d].contiguous() for d in range(3)]
        dx, dy, dz, val = (torch.zeros(E, H, **kw) for _ in range(4))
        self.launch("compute_second_frame_static_each_edge", (E * H + 31) // 32, 32,
                    a_ik, rpos, None, tvecs, batch, edges, N, H, E, rvlen, cutoff, state, seed,
                    f1[0], f1[1], f1[2], dx, dy, dz, val)
        arg = segment_argmax(val, edges[0], N)
        hh = torch.arange(H, device=a_ik.device)[None, :].expand(N, H)
        return torch.stack([dx[arg, hh], dy[arg, hh], dz[arg, hh]], dim=-1), arg

    # ---- models/cuda_funcs/calc_lattice_frame.py:22-150 -------------------------------------
    def lattice_frames(self, a_ik, rpos, tvecs, batch, edges, rvlen, cutoff, seeds=(0, 0, 0)):
        N, H = a_ik.shape
        E = edges.shape[1]
        kw = dict(device=a_ik.device, dtype=a_ik.dtype)
        f = [[torch.zeros(N, H, **kw) for _ in range(3)] for _ in range(3)]
        common = (a_ik, rpos, None, tvecs, batch, edges, N, H, E, 64, 14.0, 1.0, rvlen, cutoff)
        state = torch.empty(E * H * 48, dtype=torch.uint8, device=a_ik.device)
        self.launch("compute_lattice_first_frame", E, H, *common, state, seeds[0], *f[0])
        self.launch("compute_lattice_second_frame", E, H, *common, state, seeds[1], *f[0], *f[1])
        self.launch("compute_lattice_third_frame", E, H, *common, state, seeds[2], *f[0], *f[1], *f[2])
        return tuple(torch.stack(f[x], dim=-1) for x in range(3))

    @staticmethod
    def complete(frame1, frame2_max):
        """models/indexed_lattice_multi_head_attention_cuda.py:475-481"""
        dot = (frame1 * frame2_max).sum(-1, keepdim=True)
        f2 = torch.nn.functional.normalize(frame2_max - dot * frame1, dim=2)
        return f2, torch.linalg.cross(frame1, f2)

    # ---- models/cuda_funcs/fused_dpa.py:17-168 --------------------------------------
    def dpa_fwd(self, q, k, v, aij, bij, edges):
        N, H, K = q.shape
        E = edges.shape[1]
        e_start = self.e_start(edges, N)
        out = torch.empty_like(v)
        prob = torch.empty((E, H), dtype=q.dtype, device=q.device)
        self.launch("fused_dpa_fwd", (N * H + H - 1) // H, H, q, k, v, aij, bij, edges, e_start, N, H, E, prob, out)
        return out, prob, e_start

    def _transpose(self, src, dst, C, upper_e, mat_sec, sizes_t):
        hE = upper_e.shape[0]
        bsz = min(32, C)
        self.launch("irregular_transpose", (hE * C + bsz - 1) // bsz, bsz, src, upper_e, mat_sec, sizes_t, hE, C, dst)

    def dpa_bwd(self, q, k, v, aij, bij, batch, edges, e_start, prob, out, gout):
        N, H, K = q.shape
        E = edges.shape[1]
        B = int(batch.max().item()) + 1
        sizes = torch.zeros(B, dtype=torch.long, device=q.device)
        sizes.scatter_add_(0, batch, torch.ones_like(batch))
        start = torch.constant_pad_nd((sizes * sizes).cumsum(0), (1, 0))
        gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ga = torch.empty_like(aij)
        gb = torch.empty_like(bij) if bij is not None else None
        tprob = torch.empty_like(prob)
        tb = torch.empty_like(bij) if bij is not None else None
        upper = edges[0] <= edges[1]
        upper_e = torch.arange(E, dtype=torch.long, device=q.device)[upper]
        ub = batch[edges[0, upper]]
        mat_sec, sizes_t = start[ub].contiguous(), sizes[ub].contiguous()
        self._transpose(prob, tprob, H, upper_e, mat_sec, sizes_t)
        if bij is not None:
            self._transpose(bij, tb, H * K, upper_e, mat_sec, sizes_t)
        self.launch("fused_dpa_bwd", (N * H + H - 1) // H, H, q, k, v, aij, tb, batch, edges, e_start, N, H, E,
                    tprob, out, gout.contiguous(), gq, gk, gv, ga, gb)
        self._transpose(ga, ga, H, upper_e, mat_sec, sizes_t)
        if gb is not None:
            self._transpose(gb, gb, H * K, upper_e, mat_sec, sizes_t)
        self.launch("fused_dpa_bwd_q", (N * H + H - 1) // H, H, k, ga, edges, e_start, N, H, E, gq)
        return gq, gk, gv, ga, gb

    # ---- models/cuda_funcs/irregular_mean.py:19-57 (CPU build only) ------------------
    def mean_fwd(self, x, sizes):
        N = x.shape[0]
        D = x.numel() // N
        B = sizes.shape[0]
        start = torch.constant_pad_nd(torch.cumsum(sizes, 0), (1, 0)).contiguous()
        out = torch.empty((B,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        bsz = min(32, D)
        self.launch("irregular_mean_fwd", (B * D + bsz - 1) // bsz, bsz, x.contiguous(), start, N, D, out)
        return out


def angle_sigma(value_pe_angle_scale, dim_angle_enc, cos_abs=0):
    """models/cuda_funcs/real_space_framed_proj.py:37-40"""
    return (2 if cos_abs == 0 else 1) * value_pe_angle_scale / (dim_angle_enc - 1)
