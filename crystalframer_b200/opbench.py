"""Operator-level benchmark: the isolated attention path, forward + backward, on one synthetic
batch (256 crystals, log-normal sizes, q/k/v ~ N(0,1), upstream gradient ~ N(0,1)).

    python -m crystalframer_b200.opbench [--workload cfg2] [--crystals 256] [--iters 20] [--noise 1e-5] [--fused]

Prints one JSON line with the CUDA-event time of every entry point.  Also the small, fixed
workload used for single-kernel profiler captures (few iterations, < 1 GB on the device).
"""
import argparse
import json
import math

import numpy as np
import torch

from . import _lib, synth
from . import cuda_funcs as F
from .encoder import build_pair_list, det_3x3


def make_inputs(workload, crystals, dev, seed=None):
    b = synth.make_workload(workload, seed=seed, num_crystals=crystals)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    sizes, pos, tv = t(b.sizes), t(b.pos), t(b.trans_vec)
    edges, e_start, batch, _ = build_pair_list(sizes, (b.num_atoms, b.num_pairs))
    vcell = det_3x3(tv)
    rvecs = torch.stack([torch.linalg.cross(tv[:, 1], tv[:, 2]), torch.linalg.cross(tv[:, 2], tv[:, 0]),
                         torch.linalg.cross(tv[:, 0], tv[:, 1])], 1) * (2.0 * math.pi / vcell[:, None, None])
    rvlen = rvecs.norm(dim=-1).contiguous()
    pos_ij = (pos[edges[1]] - pos[edges[0]]).contiguous()
    g = torch.Generator(device="cpu").manual_seed(1 if seed is None else seed)
    N, H, hd = b.num_atoms, 8, 16
    q, k, v = (torch.randn(N, H, hd, generator=g).to(dev) for _ in range(3))
    w = (torch.randn(H, hd, generator=g) * hd ** -0.5).to(dev)
    alpha = (q * w[None]).sum(-1)
    alpha = (alpha - alpha.mean()) / alpha.std()
    a = ((0.5 * torch.nn.functional.elu(alpha * 0.2) + 1.0) * (-0.5 * 1.4 ** -2)).contiguous()
    bound = (64 ** -0.5) * math.sqrt(6.0 / (64 + H * hd))
    W = [((torch.rand(1, H, hd, 64, generator=g) * 2 - 1) * bound).to(dev) for _ in range(4)]
    go = torch.randn(N, H, hd, generator=g).to(dev)
    return dict(batch_obj=b, sizes=sizes, tv=tv, edges=edges, e_start=e_start, batch=batch, rvlen=rvlen, pos_ij=pos_ij,
                q=q, k=k, v=v, a=a, W=W, go=go)


def run_once(I):
    q, k, v, a = (I[n].detach().requires_grad_(True) for n in ("q", "k", "v", "a"))
    W = [w.detach().requires_grad_(True) for w in I["W"]]
    qs = q / 4.0
    f1, f2, f3 = F.max_frames_fused(qs.detach(), k.detach(), a.detach(), I["pos_ij"], I["tv"], I["batch"], I["edges"],
                                    I["rvlen"], -3.5)
    z, val = F.RealEncodingWithFramedProjFuncCUDA.apply(a, I["pos_ij"], None, I["tv"], I["batch"], I["edges"], 64, 14.0,
                                                        1.0, W[0], W[1], W[2], W[3], f1, f2, f3, 64, 4.0, 0, 1.0, 1.0,
                                                        I["rvlen"], -3.5)
    out = F.FusedDotProductAttentionCUDA.apply(qs, k, v, z, val, I["batch"], I["edges"])
    out.backward(I["go"])
    return out


def run_once_fused(I):
    """The same work through the fused entry points (lattice sums + value encoding + attention in one
    kernel per direction, as the one-node encoder layer calls them)."""
    from .cuda_funcs.common import pair_geometry
    dev = I["q"].device
    p, ip = _lib.ptr, _lib.iptr
    q, k, v, a = I["q"], I["k"], I["v"], I["a"]
    N, H, hd = q.shape
    E = I["edges"].shape[1]
    qs = q / 4.0
    f1, f2, f3 = F.max_frames_fused(qs, k, a, I["pos_ij"], I["tv"], I["batch"], I["edges"], I["rvlen"], -3.5)
    _, plist, prange = pair_geometry(I["pos_ij"], I["tv"], I["batch"], I["edges"], -3.5)
    if "order" not in I:
        n_i = (I["e_start"][1:] - I["e_start"][:-1]).float()
        vcell = (I["tv"][:, 0] * torch.linalg.cross(I["tv"][:, 1], I["tv"][:, 2])).sum(1).abs()
        I["order"] = torch.argsort(n_i * (7.0 + (2145.0 / vcell).clamp(1.0, 125.0)[I["batch"]]), descending=True,
                                   stable=True).to(torch.int32)
        I["counters"] = torch.zeros(H, dtype=torch.int32, device=dev)
    W = [w[0] for w in I["W"]]
    out, z, lse, spool = (torch.empty(s, device=dev) for s in ((N, H, hd), (E, H), (N, H), (N, H, 256)))
    # per-pair results the forward leaves for the backward (None: the backward recomputes the lattice sums)
    saved = [torch.empty(s, device=dev) for s in ((E, H, hd), (E, H), (N, H, hd))] if I.get("save_pairs", True) else [None] * 3
    common = (p(qs), p(k), p(v), p(a), p(I["pos_ij"]), p(I["tv"]), p(I["rvlen"]), ip(I["batch"]), ip(I["edges"]),
              ip(I["e_start"]), p(I["order"], torch.int32), p(I["counters"], torch.int32), N, E, 14.0, -3.5, p(W[0]),
              p(W[1]), p(W[2]), p(W[3]), p(f1), p(f2), p(f3), p(plist), prange)
    _lib.invoke("cfb200_attn_fused_fwd", 1, dev, *common, p(out), p(z), p(lse), p(spool), *[p(x) for x in saved], 0)
    gq, gk, gv, ga, gz = (torch.empty(s, device=dev) for s in ((N, H, hd), (N, H, hd), (N, H, hd), (N, H), (E, H)))
    _lib.invoke("cfb200_attn_fused_bwd", 2, dev, *common, p(out), p(z), p(lse), p(I["go"]), p(gq), p(gk), p(gv), p(ga),
                p(gz), *[p(x) for x in saved], 0)
    gW = torch.bmm(I["go"].permute(1, 2, 0), spool.permute(1, 0, 2))
    return out, gW


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--crystals", type=int, default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--noise", type=float, default=1e-5)
    ap.add_argument("--fused", action="store_true", help="time the fused attention entry points")
    ap.add_argument("--recompute", action="store_true",
                    help="with --fused: lighter forward, backward recomputes the lattice sums (no per-pair results kept)")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, args.noise)
    I = make_inputs(args.workload, args.crystals, dev)
    I["save_pairs"] = not args.recompute
    step = run_once_fused if args.fused else run_once
    for _ in range(args.warmup):
        step(I)
    torch.cuda.synchronize()
    with _lib.KernelTimer() as kt:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            step(I)
        e1.record()
        times = kt.summary()
    b = I["batch_obj"]
    line = {"workload": args.workload, "crystals": len(b.sizes), "atoms": b.num_atoms, "pairs": b.num_pairs,
            "iters": args.iters, "ms_per_iter": e0.elapsed_time(e1) / args.iters,
            "ms": {k_: round(v_[1] / v_[0], 4) for k_, v_ in times.items()}, "device_status": _lib.read_status(dev)}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
