"""Times the reference project's pure-PyTorch model on the host cores (test / baseline infrastructure).

    CF_REFERENCE_ROOT=/path/to/reference python -m oracle.pure_baseline [--layers 1] [--seconds 20]

The reference's own Python code is imported from the tree named by CF_REFERENCE_ROOT -- nothing of it is copied
here -- with stub modules for its GPU-only dependencies (torch_scatter, cupy, pytorch_pfn_extras), so its
``use_cuda_code=False`` path runs: ``Latticeformer`` (models/latticeformer.py:32-287) over
``IndexedLatticeformerEncoder`` (models/indexed_latticeformer_encoder.py:405) and
``IndexedLatticeMultiheadAttention`` (models/indexed_lattice_multi_head_attention.py:1112-1414).  That path
implements plain Crystalformer only -- fixed lattice range 2 (125 translations), un-windowed distance
Gaussians, no frames, no angle encoding -- and, as shipped, reads two attributes that
``LatticeformerParams`` does not define (``positive_func``, ``value_pe_width_scale``); they are set here to
the values the CUDA path uses ("elu=0.1", 1.0).

Workload: the CPU-runnable configuration -- 8 synthetic crystals of 4-16 atoms (seed 0), d_model 128,
8 heads, 64 distance Gaussians, scalar regression head, L1 loss on N(0,1) targets, AdamW; one training step =
forward + backward + clip + update.  Prints one JSON line.
"""
import argparse
import json
import os
import sys
import time
import types

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _import_reference(root):
    for name in ("torch_scatter", "cupy", "pytorch_pfn_extras"):
        sys.modules.setdefault(name, types.ModuleType(name))
    cr = types.ModuleType("cupy.random")
    cr.XORWOW = object
    sys.modules["cupy.random"] = cr
    sys.modules["cupy"].random = cr
    if root not in sys.path:
        sys.path.insert(0, root)
    cwd = os.getcwd()
    os.chdir(root)
    try:
        from models import latticeformer as ref_model
    finally:
        os.chdir(cwd)
    return ref_model


class _Batch:
    pass


def measure(root, budget_s=20.0, layers=1, crystals=None):
    from crystalframer_b200 import synth
    from crystalframer_b200.latticeformer import ModelParams
    ref_model = _import_reference(root)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    params = ModelParams(num_layers=layers, use_cuda_code=False, frame_method="no", value_pe_angle_real=0,
                         adaptive_cutoff_sigma=-3.5)
    import contextlib
    import io
    with contextlib.redirect_stdout(io.StringIO()):          # the reference prints its hyper-parameters
        model = ref_model.Latticeformer(params).train()
    for layer in model.encoder.layers:
        P = layer.self_attn.params
        if not hasattr(P, "positive_func"):
            P.positive_func = "elu=0.1"
        if not hasattr(P, "value_pe_width_scale"):
            P.value_pe_width_scale = 1.0
    b = synth.make_workload("cfg1", num_crystals=crystals)
    data = _Batch()
    data.x, data.pos = torch.from_numpy(b.x), torch.from_numpy(b.pos)
    data.batch, data.trans_vec, data.sizes = torch.from_numpy(b.batch), torch.from_numpy(b.trans_vec), torch.from_numpy(b.sizes)
    y = torch.from_numpy(np.random.default_rng(0).normal(size=(len(b.sizes), 1)).astype(np.float32))
    opt = torch.optim.AdamW(model.parameters(), lr=5e-4, betas=(0.9, 0.98), weight_decay=1e-5)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = (model(data) - y).abs().mean()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        return float(loss.detach())

    times = []
    with contextlib.redirect_stdout(io.StringIO()):          # the first training forward prints its statistics
        for _ in range(2):
            step()
        t_start = time.perf_counter()
        while len(times) < 5 or (time.perf_counter() - t_start < budget_s and len(times) < 200):
            t0 = time.perf_counter()
            loss = step()
            times.append(time.perf_counter() - t0)
    med = float(np.median(times))
    return {"value": len(b.sizes) / med, "unit": "crystals/s", "cores": threads, "kind": "reference pure-PyTorch (plain Crystalformer part)",
            "ms_per_step": med * 1e3, "steps": len(times), "layers": layers, "loss": loss,
            "sample": f"{len(b.sizes)} crystals of 4-16 atoms ({b.num_atoms} atoms, {b.num_pairs} pairs), 1 training step = fwd+bwd+clip+AdamW, "
                      f"median of {len(times)} steps after 2 warm-up"}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=1)
    ap.add_argument("--seconds", type=float, default=20.0)
    ap.add_argument("--crystals", type=int, default=None)
    args = ap.parse_args()
    from oracle import build_oracle
    root = build_oracle.reference_root()
    if root is None:
        raise SystemExit("set CF_REFERENCE_ROOT to the reference project's root")
    print(json.dumps(measure(root, args.seconds, args.layers, args.crystals)))
