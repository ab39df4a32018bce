"""Operator-level benchmark: the isolated attention path, forward + backward, on one synthetic
batch (256 crystals, log-normal sizes, q/k/v ~ N(0,1), upstream gradient ~ N(0,1)).

    python -m crystalframer_b200.opbench [--workload cfg2] [--crystals 256] [--iters 20] [--noise 1e-5]

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--crystals", type=int, default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--noise", type=float, default=1e-5)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, args.noise)
    I = make_inputs(args.workload, args.crystals, dev)
    for _ in range(args.warmup):
        run_once(I)
    torch.cuda.synchronize()
    with _lib.KernelTimer() as kt:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            run_once(I)
        e1.record()
        times = kt.summary()
    b = I["batch_obj"]
    line = {"workload": args.workload, "crystals": len(b.sizes), "atoms": b.num_atoms, "pairs": b.num_pairs,
            "iters": args.iters, "ms_per_iter": e0.elapsed_time(e1) / args.iters,
            "ms": {k_: round(v_[1] / v_[0], 4) for k_, v_ in times.items()}, "device_status": _lib.read_status(dev)}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
