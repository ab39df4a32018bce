"""Times the reference project's own CUDA kernels (oracle/_ref/libcfref_gpu.so, compiled from the
reference sources for sm_100a) on the operator-level workload, and checks the library's results
against them on the same GPU.  Test infrastructure: it is the reference-on-the-same-GPU baseline.

    python -m oracle.gpu_reference_bench [--crystals 256] [--iters 5]

The reference kernels are compiled with SYMM_BREAK_NOISE = 0 (curand is still initialised per
thread, as in the reference, which is part of its cost).
"""
import argparse
import json

import numpy as np
import torch

from crystalframer_b200 import cuda_funcs as F
from crystalframer_b200 import opbench
from . import oracle as O
from . import reference as R


def timed(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        out = fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters, out


def reference_operator_ms(I, iters=3):
    """CUDA-event milliseconds of the reference kernels' launch sequence for one forward + backward of the
    isolated attention operator on the inputs ``I`` (crystalframer_b200.opbench.make_inputs): first and second
    frame axis, lattice sums + value encoding forward, attention forward, attention backward, lattice sums backward."""
    rk = R.RefKernels("cuda")
    a, pos, tv, batch, edges, rv = I["a"], I["pos_ij"], I["tv"], I["batch"], I["edges"], I["rvlen"]
    qs, k, v = (I["q"] / 4.0).contiguous(), I["k"], I["v"]
    Wd = I["W"][0].contiguous()
    Ws = torch.stack(I["W"][1:]).contiguous()
    asig = R.angle_sigma(4.0, 64)
    res = {}
    res["frame1"], (f1, _) = timed(lambda: rk.frame1(qs, k, a, pos, tv, batch, edges, rv, -3.5), iters)
    res["frame2"], (f2m, _) = timed(lambda: rk.frame2(qs, k, a, pos, tv, batch, edges, rv, -3.5, f1), iters)
    f2, f3 = rk.complete(f1, f2m)
    frames = torch.stack([f1, f2, f3]).contiguous()
    res["framed_proj_fwd"], (z, val) = timed(lambda: rk.framed_proj_fwd(a, pos, tv, batch, edges, 14.0, 1.0, Wd, Ws, frames,
                                                                        asig, 1.0, 1.0, rv, -3.5), iters)
    res["dpa_fwd"], (out, prob, es) = timed(lambda: rk.dpa_fwd(qs, k, v, z, val, edges), iters)
    res["dpa_bwd"], (gq, gk, gv, gz, gb) = timed(lambda: rk.dpa_bwd(qs, k, v, z, val, batch, edges, es, prob, out, I["go"]), iters)
    res["framed_proj_bwd"], _ = timed(lambda: rk.framed_proj_bwd(a, pos, tv, batch, edges, 14.0, 1.0, Wd, Ws, frames, asig, 1.0,
                                                                 1.0, rv, -3.5, z, gz, gb), iters)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--crystals", type=int, default=None)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, 0.0)
    I = opbench.make_inputs(args.workload, args.crystals, dev)
    rk = R.RefKernels("cuda")
    a, pos, tv, batch, edges, rv = I["a"], I["pos_ij"], I["tv"], I["batch"], I["edges"], I["rvlen"]
    qs, k, v = (I["q"] / 4.0).contiguous(), I["k"], I["v"]
    Wd = I["W"][0].contiguous()
    Ws = torch.stack(I["W"][1:]).contiguous()
    asig = R.angle_sigma(4.0, 64)
    res = {}
    res["frame1"], (f1, _) = timed(lambda: rk.frame1(qs, k, a, pos, tv, batch, edges, rv, -3.5), args.iters)
    res["frame2"], (f2m, _) = timed(lambda: rk.frame2(qs, k, a, pos, tv, batch, edges, rv, -3.5, f1), args.iters)
    f2, f3 = rk.complete(f1, f2m)
    frames = torch.stack([f1, f2, f3]).contiguous()
    res["framed_proj_fwd"], (z, val) = timed(lambda: rk.framed_proj_fwd(a, pos, tv, batch, edges, 14.0, 1.0, Wd, Ws, frames,
                                                                        asig, 1.0, 1.0, rv, -3.5), args.iters)
    res["dpa_fwd"], (out, prob, es) = timed(lambda: rk.dpa_fwd(qs, k, v, z, val, edges), args.iters)
    go = I["go"]
    res["dpa_bwd"], (gq, gk, gv, gz, gb) = timed(lambda: rk.dpa_bwd(qs, k, v, z, val, batch, edges, es, prob, out, go), args.iters)
    res["framed_proj_bwd"], (ga, gWd, gWs) = timed(lambda: rk.framed_proj_bwd(a, pos, tv, batch, edges, 14.0, 1.0, Wd, Ws, frames,
                                                                              asig, 1.0, 1.0, rv, -3.5, z, gz, gb), args.iters)
    # the library on the same inputs
    g1, g2, g3 = F.max_frames_fused(qs, k, a, pos, tv, batch, edges, rv, -3.5)
    a_ = a.detach().requires_grad_(True)
    W_ = [w.detach().requires_grad_(True) for w in I["W"]]
    q_, k_, v_ = (t.detach().requires_grad_(True) for t in (qs, k, v))
    z2, val2 = F.RealEncodingWithFramedProjFuncCUDA.apply(a_, pos, None, tv, batch, edges, 64, 14.0, 1.0, W_[0], W_[1], W_[2],
                                                          W_[3], f1, f2, f3, 64, 4.0, 0, 1.0, 1.0, rv, -3.5)
    out2 = F.FusedDotProductAttentionCUDA.apply(q_, k_, v_, z2, val2, batch, edges)
    out2.backward(go)

    def viol(x, y, scale=1.0):
        err = (x - y).abs()
        return float((err > 1e-5 * scale + 1e-4 * y.abs()).float().mean()), float(err.max())

    checks = {
        "frame1_equal_frac": float((g1 == f1).all(-1).float().mean()),
        "frame2_close_frac": float(((g2 - f2).abs().max(-1)[0] < 1e-4).float().mean()),
        "z": viol(z2, z), "values": viol(val2, val), "out": viol(out2, out), "gq": viol(q_.grad, gq),
        "gk": viol(k_.grad, gk), "gv": viol(v_.grad, gv),
        "ga": viol(a_.grad, ga, max(1.0, float(ga.abs().max()))),
        "gW_dist": viol(W_[0].grad[0], gWd, max(1.0, float(gWd.abs().max()))),
        "gW_ang": viol(torch.stack([w.grad[0] for w in W_[1:]]), gWs, max(1.0, float(gWs.abs().max()))),
    }
    b = I["batch_obj"]
    # reciprocal-space logit bias (plain Crystalformer's "reci" domain): reference kernels and the library
    rvecs, vcell, kr = (torch.from_numpy(x).to(dev) for x in O.reciprocal_geometry(b.pos, b.trans_vec, b.sizes,
                                                                                     edges.cpu().numpy()))
    ar = (a * 9.5).contiguous()                        # -0.5 scale_reci^2 f against -0.5 scale_real^-2 f
    reci = {}
    reci["reference_fwd"], (zr, sr) = timed(lambda: rk.reci_fwd(ar, kr, rvecs, vcell, batch, edges), args.iters)
    gzr = (torch.randn_like(zr) * (sr > 1e-2)).contiguous()
    reci["reference_bwd"], gar = timed(lambda: rk.reci_bwd(ar, kr, rvecs, vcell, batch, edges, zr, gzr, sr), args.iters)
    ar_ = ar.detach().requires_grad_(True)
    reci["library_fwd"], zl = timed(lambda: F.ReciPeriodicEncodingFuncCUDA.apply(ar_, kr, rvecs, vcell, batch, edges), args.iters)
    reci["library_bwd"], _ = timed(lambda: zl.backward(gzr, retain_graph=True), args.iters)
    ar_.grad = None
    zl.backward(gzr)
    ok = sr > 1e-3
    checks["reci_z"] = viol(zl.detach()[ok], zr[ok], 10.0)
    checks["reci_ga"] = viol(ar_.grad, gar, max(1.0, float(gar.abs().max())))
    res_reci = {k_: round(v_, 4) for k_, v_ in reci.items()}
    print(json.dumps({"impl": "reference CUDA kernels (sm_100a build)", "workload": args.workload, "crystals": len(b.sizes),
                      "reciprocal_encoding_ms": res_reci,
                      "pairs": b.num_pairs, "ms": {k_: round(v_, 4) for k_, v_ in res.items()},
                      "ms_total": round(sum(res.values()), 4),
                      "parity_vs_library (violating fraction, max abs err)": checks}))


if __name__ == "__main__":
    main()
