"""Model-level timing of one training step for any workload and frame method.

    python -m crystalframer_b200.modelbench [--workload cfg4] [--frame-method max|max_static|lattice|pca|weighted_pca|no]
                                            [--layers 4] [--steps 5] [--crystals N]

``bench.py`` at the repository root times the benchmark configuration (cfg3, max frames); this tool
covers the others -- the large-cell stress test (cfg4: 64 crystals of 100-200 atoms, plain Crystalformer
with frame method "no" and the weighted-PCA frames).  One JSON line: CUDA-event milliseconds per step
(forward + backward + AdamW) and per library entry point.
"""
import argparse
import json

import numpy as np
import torch

from . import _lib, data, synth
from .latticeformer import Latticeformer, ModelParams


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg4")
    ap.add_argument("--frame-method", default="weighted_pca", choices=["max", "max_static", "lattice", "pca", "weighted_pca", "no"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--crystals", type=int, default=None)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.manual_seed(3)
    over = dict(num_layers=args.layers, frame_method=args.frame_method)
    if args.frame_method == "no":
        over["value_pe_angle_real"] = 0              # plain Crystalformer: distance encoding only
    model = Latticeformer(ModelParams(**over)).to(dev).train()
    opt = torch.optim.AdamW(model.parameters(), lr=5e-4, betas=(0.9, 0.98), weight_decay=1e-5, fused=True)
    b = synth.make_workload(args.workload, num_crystals=args.crystals)
    y = np.random.default_rng(0).normal(size=(len(b.sizes), 1)).astype(np.float32)
    tb = data.host_batch(b, y).to(dev, non_blocking=False)
    with torch.no_grad():
        model(tb)                                    # measures the coefficient statistics

    def step():
        opt.zero_grad(set_to_none=True)
        loss = (model(tb) - tb.y).abs().mean()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        return loss

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    with _lib.KernelTimer() as kt:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            loss = step()
        e1.record()
        times = kt.summary()
    print(json.dumps({"workload": args.workload, "frame_method": args.frame_method, "layers": args.layers,
                      "crystals": len(b.sizes), "atoms": b.num_atoms, "pairs": b.num_pairs, "steps": args.steps,
                      "ms_per_step": e0.elapsed_time(e1) / args.steps, "loss": float(loss),
                      "ms_per_call": {k: round(v[1] / v[0], 4) for k, v in times.items()},
                      "calls_per_step": {k: v[0] / args.steps for k, v in times.items()},
                      "device_status": _lib.read_status(dev)}))


if __name__ == "__main__":
    main()
