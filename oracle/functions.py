"""CPU autograd Functions over the oracle (test infrastructure, never part of the product).

They let the whole 4-layer model run forward and backward on the host cores -- for end-to-end
parity tests and for the CPU baseline of the benchmark.  ``backend="reference"`` executes the
reference project's own kernels compiled for the CPU (``oracle/_ref``), ``backend="port"`` the C
restatement in ``cf_oracle.c``.  Host glue between kernels follows the reference Functions
(models/cuda_funcs/*.py), cited in ``reference.py`` and ``oracle.py``.
"""
import numpy as np
import dataclasses

import torch

from . import oracle as O
from . import reference as R

_state = {"backend": None, "rk": None, "cfg": O.Config()}


def configure(cfg: O.Config, backend=None):
    """``backend``: "port" (C restatement, CPU), "reference" (the reference's kernels built for the CPU) or
    "reference_cuda" (the reference's kernels built with nvcc, tensors on the current GPU: the
    reference-on-the-same-GPU baseline)."""
    if backend is None:
        backend = "reference" if R.available("cpu") else "port"
    _state["cfg"] = cfg
    _state["rk"] = None
    if backend == "reference":
        _state["rk"] = R.RefKernels("cpu")
    elif backend == "reference_cuda":
        _state["rk"] = R.RefKernels("cuda")
        backend = "reference"            # same host glue; only the device of the tensors differs
    _state["backend"] = backend
    if backend == "reference":
        c = _state["rk"].consts
        assert (c["HEAD_NUM"], c["VPE_DIM"], c["ANGLE_ENC_DIM"], c["LATTICE_RANGE"]) == \
            (cfg.H, cfg.D_dist, cfg.D_ang, cfg.lattice_range), "oracle/_ref was built for other constants"
    return backend


def backend():
    return _state["backend"]


def _np(t):
    return None if t is None else t.detach().contiguous().numpy()


def _e_start(edges, N):
    return R.RefKernels.e_start(edges, N)


def max_frames(q_scaled, k, a, pos_ij, tvecs, batch, edges, rvlen, cutoff):
    cfg = _state["cfg"]
    if _state["backend"] == "reference":
        rk = _state["rk"]
        f1, _ = rk.frame1(q_scaled, k, a, pos_ij, tvecs, batch, edges, rvlen, cutoff)
        f2m, _ = rk.frame2(q_scaled, k, a, pos_ij, tvecs, batch, edges, rvlen, cutoff, f1)
        f2, f3 = rk.complete(f1, f2m)
        return f1, f2, f3
    N = a.shape[0]
    fr = O.max_frames(cfg, _np(q_scaled), _np(k), _np(a), _np(pos_ij), _np(tvecs), _np(rvlen), _np(batch),
                      _np(edges), _np(_e_start(edges, N)))
    return tuple(torch.from_numpy(fr[n]) for n in ("frame1", "frame2", "frame3"))


class FramedProj(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, pos_ij, tvecs, batch, edges, rvlen, cutoff, dist_max, Wd, W1, W2, W3, f1, f2, f3):
        cfg = dataclasses.replace(_state["cfg"], H=a.shape[1])      # the "multihead" domain passes half of the heads
        ang = W1 is not None
        a_, Wd_ = a.detach().contiguous(), Wd.detach().contiguous()
        Ws = torch.stack([W1, W2, W3]).detach().contiguous() if ang else None      # (3,1,H,hd,D)
        fr = torch.stack([f1, f2, f3]).detach().contiguous() if ang else None
        if _state["backend"] == "reference":
            z, v = _state["rk"].framed_proj_fwd(a_, pos_ij, tvecs, batch, edges, dist_max, cfg.wscale_dist, Wd_, Ws, fr,
                                                cfg.angle_sigma, cfg.c_dist, cfg.c_ang, rvlen, cutoff)
        else:
            z, v = O.framed_proj_fwd(cfg, _np(a_), _np(pos_ij), _np(tvecs), _np(rvlen), _np(batch), _np(edges),
                                     _np(Wd_[0]), _np(Ws[:, 0]) if ang else None, _np(fr))
            z, v = torch.from_numpy(z), torch.from_numpy(v)
        ctx.save_for_backward(a_, pos_ij, tvecs, batch, edges, rvlen, Wd_, Ws, fr, z)
        ctx.meta = (cutoff, dist_max)
        return z, v

    @staticmethod
    def backward(ctx, gz, gv):
        a, pos_ij, tvecs, batch, edges, rvlen, Wd, Ws, fr, z = ctx.saved_tensors
        cutoff, dist_max = ctx.meta
        cfg = dataclasses.replace(_state["cfg"], H=a.shape[1])
        ang = Ws is not None
        if _state["backend"] == "reference":
            ga, gWd, gWs = _state["rk"].framed_proj_bwd(a, pos_ij, tvecs, batch, edges, dist_max, cfg.wscale_dist, Wd,
                                                        Ws, fr, cfg.angle_sigma, cfg.c_dist, cfg.c_ang, rvlen, cutoff,
                                                        z, gz.contiguous(), gv.contiguous())
            gWd = gWd[None]
            gW = [gWs[x][None] for x in range(3)] if ang else [None] * 3
        else:
            N = a.shape[0]
            ga, gWd, gWa = O.framed_proj_bwd(cfg, _np(a), _np(pos_ij), _np(tvecs), _np(rvlen), _np(batch), _np(edges),
                                             _np(_e_start(edges, N)), _np(Wd[0]), _np(Ws[:, 0]) if ang else None,
                                             _np(fr), _np(z), _np(gz), _np(gv))
            ga, gWd = torch.from_numpy(ga), torch.from_numpy(gWd)[None]
            gW = [torch.from_numpy(gWa[x])[None] for x in range(3)] if ang else [None] * 3
        return (ga, None, None, None, None, None, None, None, gWd, gW[0], gW[1], gW[2], None, None, None)


class Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_scaled, k, v, z, b, batch, edges):
        cfg = _state["cfg"]
        q_, k_, v_, z_, b_ = (t.detach().contiguous() for t in (q_scaled, k, v, z, b))
        if _state["backend"] == "reference":
            out, prob, e_start = _state["rk"].dpa_fwd(q_, k_, v_, z_, b_, edges)
        else:
            e_start = _e_start(edges, q_.shape[0])
            out, prob = O.dpa_fwd(cfg, _np(q_), _np(k_), _np(v_), _np(z_), _np(b_), _np(edges), _np(e_start))
            out, prob = torch.from_numpy(out), torch.from_numpy(prob)
        ctx.save_for_backward(q_, k_, v_, z_, b_, batch, edges, e_start, prob, out)
        return out

    @staticmethod
    def backward(ctx, go):
        q, k, v, z, b, batch, edges, e_start, prob, out = ctx.saved_tensors
        cfg = _state["cfg"]
        if _state["backend"] == "reference":
            g = _state["rk"].dpa_bwd(q, k, v, z, b, batch, edges, e_start, prob, out, go.contiguous())
        else:
            g = O.dpa_bwd(cfg, _np(q), _np(k), _np(v), _np(b), _np(edges), _np(e_start), _np(prob), _np(out), _np(go))
            g = tuple(torch.from_numpy(x) for x in g)
        return g[0], g[1], g[2], g[3], g[4], None, None


class Reci(torch.autograd.Function):
    """models/cuda_funcs/reci_space_enc.py:17-97"""

    @staticmethod
    def forward(ctx, a, kr, rvecs, vcell, batch, edges, lattice_range):
        a_ = a.detach().contiguous()
        if _state["backend"] == "reference":
            z, sumexp = _state["rk"].reci_fwd(a_, kr, rvecs, vcell, batch, edges)
        else:
            z, sumexp = (torch.from_numpy(x) for x in O.reci_enc_fwd(_np(a_), _np(kr), _np(rvecs), _np(vcell), _np(batch),
                                                                     _np(edges), lattice_range))
        ctx.save_for_backward(a_, kr, rvecs, vcell, batch, edges, z, sumexp)
        ctx.lattice_range = lattice_range
        return z

    @staticmethod
    def backward(ctx, gz):
        a, kr, rvecs, vcell, batch, edges, z, sumexp = ctx.saved_tensors
        if _state["backend"] == "reference":
            ga = _state["rk"].reci_bwd(a, kr, rvecs, vcell, batch, edges, z, gz.contiguous(), sumexp)
        else:
            ga = torch.from_numpy(O.reci_enc_bwd(_np(a), _np(kr), _np(rvecs), _np(batch), _np(edges), _np(gz), _np(sumexp),
                                                 ctx.lattice_range))
        return ga, None, None, None, None, None, None


class Mean(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sizes):
        if x.is_cuda:
            # the reference's pooling kernel has no nvcc build (it calls an unqualified host template);
            # the same per-crystal mean with torch operations
            batch = torch.repeat_interleave(torch.arange(len(sizes), device=x.device), sizes)
            out = torch.zeros((len(sizes),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            out.index_add_(0, batch, x.detach())
            out = out / sizes[:, None].to(x.dtype)
        elif _state["backend"] == "reference":
            out = _state["rk"].mean_fwd(x.detach().contiguous(), sizes)
        else:
            out = torch.from_numpy(O.mean_fwd(_np(x), _np(sizes)))
        ctx.save_for_backward(sizes)
        return out

    @staticmethod
    def backward(ctx, go):
        sizes, = ctx.saved_tensors
        batch = torch.repeat_interleave(torch.arange(len(sizes), device=sizes.device), sizes)
        return (go / sizes[:, None].float())[batch], None
