"""Epoch throughput of data-parallel training over a synthetic structure set, input pipeline included.

    python -m crystalframer_b200.epochbench [--structures 650000] [--batch 256] [--max-steps N]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m crystalframer_b200.epochbench --structures 650000

The 4-layer max-frame model is trained for one epoch over ``--structures`` crystals of the benchmark
distribution (atom counts log-normal, median 8, at most 64; cells 3-15 angstrom) at ``--batch`` crystals per GPU:
every rank holds the structure set in memory (flat arrays, about 270 bytes per structure), walks the same seeded
permutation, takes its cost-balanced share of each global batch, and feeds the model through
``data.EpochLoader`` -- collation on a background thread into pinned double buffers, host-to-device copies on a
copy stream one step ahead, the species one-hot built on the device.  ``bench.py`` times the training step on a
few resident or host batches; this tool times what an epoch costs with nothing prepared in advance except the
structure set itself.  One JSON line from rank 0: wall-clock seconds of the epoch loop (max over ranks, barrier on
both sides), structures per second, the loader's bytes per step, and the set's generation time (not in the epoch
time).
"""
import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from . import data, parallel
from .latticeformer import Latticeformer, ModelParams
from .optim import FlatAdamW


SEGMENT = 32


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--structures", type=int, default=65536)
    ap.add_argument("--batch", type=int, default=256, help="crystals per GPU and step")
    ap.add_argument("--max-steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--depth", type=int, default=2, help="batches the loader keeps in flight")
    ap.add_argument("--overlap-exchange", type=int, default=0,
                    help="several ranks: all-reduce each layer's gradient slices beside the backward of earlier layers")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    t0 = time.perf_counter()
    ds = data.StructureSet.synthetic(args.structures, seed=4)          # the same set on every rank
    gen_s = time.perf_counter() - t0
    torch.manual_seed(2)
    model = Latticeformer(ModelParams()).to(dev).train()
    decay = [p for n, p in model.named_parameters() if p.requires_grad and not n.endswith("bias")]
    no_decay = [p for n, p in model.named_parameters() if p.requires_grad and n.endswith("bias")]
    opt = FlatAdamW(decay, no_decay, lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-5, max_norm=1.0)
    if world > 1 and args.overlap_exchange:
        opt.overlap_exchange()
    global_batch = args.batch * world

    def train_step(tb):
        opt.zero_grad(set_to_none=True)
        loss = (model(tb) - tb.y).abs().sum() / float(global_batch)
        loss.backward()
        opt.step(world_sum=True)
        return loss

    # the first training batch fixes the Gaussian-coefficient statistics; all ranks take rank 0's
    warm = data.EpochLoader(ds, args.batch, rank, world, dev, epoch=1000, seed=4, depth=args.depth,
                            max_steps=max(args.warmup, 1) + 1)
    it = iter(warm)
    with torch.no_grad():
        model(next(it))
    parallel.broadcast_state(model)
    for tb in it:
        train_step(tb)
    loader = data.EpochLoader(ds, args.batch, rank, world, dev, epoch=0, seed=4, depth=args.depth, max_steps=args.max_steps)
    losses = torch.zeros(len(loader), dtype=torch.float32, device=dev)
    barrier()
    t0 = time.perf_counter()
    steps = 0
    marks = [torch.cuda.Event(enable_timing=True)]
    marks[0].record()
    for tb in loader:
        losses[steps] = train_step(tb).detach()
        steps += 1
        if steps % SEGMENT == 0:                     # device time of every SEGMENT steps: the step's cost moves with
            marks.append(torch.cuda.Event(enable_timing=True))      # the learned Gaussian widths as training goes on
            marks[-1].record()
    torch.cuda.synchronize()
    mine = time.perf_counter() - t0
    barrier()
    t = torch.tensor([mine], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(losses)                       # per-rank parts of the global-batch loss
    epoch_s = float(t.item())
    if rank == 0:
        trained = steps * global_batch
        print(json.dumps({
            "metric": "crystals/sec over one training epoch (4-layer max-frame, input pipeline included)",
            "value": trained / epoch_s, "unit": "crystals/s", "n_gpus": world, "structures": args.structures,
            "structures_trained": trained, "steps": steps, "crystals_per_gpu_per_step": args.batch,
            "epoch_s": epoch_s, "ms_per_step": epoch_s / max(steps, 1) * 1e3,
            "h2d_bytes_per_step": loader.h2d_bytes / max(steps, 1), "loader_depth": args.depth,
            "ms_per_step_by_segment": [round(a.elapsed_time(b) / SEGMENT, 3) for a, b in zip(marks[:-1], marks[1:])],
            "segment_steps": SEGMENT, "set_generation_s": gen_s, "first_loss": float(losses[0].item()) if steps else None,
            "last_loss": float(losses[steps - 1].item()) if steps else None, "dtype": "fp32", "data": "synthetic",
            "scaling": "weak"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
