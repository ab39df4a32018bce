"""The one-call batch preparation and encoder layer (cfb200_batch_geometry, cfb200_encoder_layer_fwd / _bwd)
and the flat optimiser with gradient sinks.

* batch geometry: integer outputs bit-exact against the oracle's restatement of the reference host code,
  floats to float32 rounding, work-queue order against the stable sort it stands for;
* the layer: outputs and every gradient against the operator-by-operator path of the same module
  (reference-signature Functions + torch linear layers), for the three frame methods, at odd sizes;
  the comparison with the CPU oracle at model level is tests/test_gpu_parity.py::test_whole_model_against_cpu_oracle;
* gradient sinks: a training step through FlatAdamW equals clip_grad_norm_ + torch AdamW on autograd's gradients;
  a batch split over two shards and summed equals the whole batch.
"""
import copy

import numpy as np
import pytest
import torch

from parity_util import close, cuda, to_dev

pytestmark = pytest.mark.gpu


def test_batch_geometry_against_oracle():
    dev = cuda()
    from crystalframer_b200 import cuda_funcs as F, fused_layer, synth
    from oracle import oracle as O
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, 0.0)
    for workload, nc in (("cfg1", None), ("cfg2", 64), ("cfg4", 2)):
        b = synth.make_workload(workload, num_crystals=nc)
        want = O.lattice_geometry(b.pos, b.trans_vec, b.sizes)
        pos, tv, sizes = to_dev(b.pos, dev), to_dev(b.trans_vec, dev), to_dev(b.sizes, dev)
        g = fused_layer.LayerGeometry.from_raw(pos, tv, sizes, b.num_atoms, b.num_pairs, -3.5)
        assert torch.equal(g.edges.cpu(), torch.from_numpy(want["edges"]))
        assert torch.equal(g.e_start.cpu(), torch.from_numpy(want["e_start"]))
        assert torch.equal(g.batch.cpu(), torch.from_numpy(want["batch"]))
        # pos_ij is one float subtraction per component: identical on any IEEE machine
        assert np.array_equal(g.pos_ij.cpu().numpy(), want["pos_ij"])
        close("rvlen", g.rvlen.cpu().numpy(), want["rvlen"], 4e-7, 0.0)
        # work queue: stable descending sort of the atoms by their crystal's key; a crystal cut into chunks appears once
        # per chunk, its atoms in their order each time, with disjoint slots for the partial results
        vol = np.abs(np.linalg.det(b.trans_vec.astype(np.float64)))
        key = (b.sizes * (350.0 + 70.0 * np.clip(2145.0 / np.maximum(vol, 1e-6), 1.0, 125.0))).astype(np.float32)
        N = b.num_atoms
        from crystalframer_b200 import _lib
        # the library's order lives inside the geometry's float buffer; locate it through its pointer
        fbuf = g._keep[1]
        off = (g.c.order - fbuf.data_ptr()) // 4
        split = g.split.cpu().numpy()
        S, SLOTS = int(split[0]), 4096                       # chunk entries in use; the atoms' entries follow the region
        assert 0 <= S <= SLOTS
        queue = fbuf[off:off + SLOTS + N].view(torch.int32).cpu().numpy()
        info_all = split[4:4 + 2 * (SLOTS + N):2]
        assert (info_all[S:SLOTS] == 0).all() and (info_all[:S] != 0).all() and (info_all[SLOTS:] != 0).all()
        first = queue[SLOTS:]
        assert sorted(first.tolist()) == list(range(N))
        k_atom = key[want["batch"]]
        assert (np.diff(k_atom[first]) <= 1e-3 * k_atom.max()).all()         # non-increasing up to float rounding of the key
        same_key = np.diff(k_atom[first]) == 0
        assert (np.diff(first)[same_key] > 0).all()                           # stable within equal keys
        got = np.concatenate([queue[:S], first])
        info = np.concatenate([info_all[:S], info_all[SLOTS:]])
        chunk, chunks, slot = info & 15, (info >> 4) & 15, info >> 8
        assert (chunk[S:] == 0).all() and (chunk[:S] >= 1).all()
        counts = np.bincount(got, minlength=N)
        per_atom_chunks = np.zeros(N, np.int64)
        per_atom_chunks[got] = chunks
        assert np.array_equal(counts, per_atom_chunks)                        # every chunk of every atom queued once
        assert (chunks >= 1).all() and (chunks <= 8).all() and (chunk < chunks).all()
        assert (chunks <= np.maximum(b.sizes[want["batch"]][got] // 4, 1)).all()
        taken = np.zeros(SLOTS, np.int64)
        for a in np.unique(got[chunks > 1]):
            rows = slot[got == a]
            assert (rows == rows[0]).all() and sorted(chunk[got == a].tolist()) == list(range(chunks[got == a][0]))
            taken[rows[0]:rows[0] + chunks[got == a][0]] += 1
        assert taken.max() <= 1 and int(split[2]) == (np.nonzero(taken)[0].max() + 1 if taken.any() else 0)
        inv_vol = np.concatenate([split[5:5 + 2 * S:2], split[5 + 2 * SLOTS:5 + 2 * (SLOTS + N):2]]).view(np.float32)
        assert np.allclose(inv_vol, 1.0 / np.maximum(vol, 1e-6)[want["batch"]][got], rtol=1e-5)
        # per-pair geometry equals what cfb200_pair_cache gives on the same inputs
        cache = torch.empty(b.num_pairs, 4, device=dev)
        plist = torch.empty(b.num_pairs, 5, 128, device=dev)
        _lib.invoke("cfb200_pair_cache", 2, dev, _lib.ptr(g.pos_ij.contiguous()), _lib.ptr(tv), _lib.iptr(g.batch.contiguous()),
                    _lib.iptr(g.edges.contiguous()), N, b.num_pairs, 2, _lib.ptr(cache), _lib.ptr(plist))
        off_pc = (g.c.pair_cache - fbuf.data_ptr()) // 4
        assert torch.equal(fbuf[off_pc:off_pc + 4 * b.num_pairs].view(-1, 4).view(torch.int32), cache.view(torch.int32))
        assert torch.equal(g._keep[2].view(torch.int32), plist.view(torch.int32))
        assert _lib.read_status(dev) == 0


@pytest.mark.parametrize("frame_method,workload,nc", [("max", "cfg2", 16), ("max", "cfg1", None), ("no", "cfg2", 16),
                                                      ("weighted_pca", "cfg1", None), ("max_static", "cfg1", None),
                                                      ("lattice", "cfg2", 16), ("pca", "cfg2", 16)])
def test_one_call_layer_matches_operator_path(frame_method, workload, nc):
    """Same model, same batch: operator by operator (reference-signature Functions, torch linear layers, autograd)
    against one library call per layer with hand-written backward."""
    dev = cuda()
    from crystalframer_b200 import _lib, data, encoder, fused_layer, synth
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    torch.manual_seed(3)
    mp = ModelParams(num_layers=2, symm_break_noise=0.0, frame_method=frame_method,
                     value_pe_angle_real=0 if frame_method == "no" else 64)
    model = Latticeformer(mp).to(dev).train()
    b = synth.make_workload(workload, num_crystals=nc)
    y = np.random.default_rng(1).normal(size=(len(b.sizes), 1)).astype(np.float32)
    tb = data.host_batch(b, y, pinned=False).to(dev, non_blocking=False)
    with torch.no_grad():
        model(tb)                                   # measures gauss_scale, after which the one-call path is eligible
    results = []
    for fused in (False, True):
        encoder.FUSED_LAYER = fused
        model.zero_grad(set_to_none=True)
        np.random.seed(11)
        torch.manual_seed(11)                       # frame seeds are drawn from the global generators
        calls = []
        orig = _lib.invoke
        _lib.invoke = lambda name, *a, **k: (calls.append(name), orig(name, *a, **k))[1]
        try:
            out = model(tb)
            (out - tb.y).abs().mean().backward()
        finally:
            _lib.invoke = orig
        assert ("cfb200_encoder_layer_fwd" in calls) == fused and ("cfb200_encoder_layer_bwd" in calls) == fused
        results.append((out.detach().clone(), {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}))
    encoder.FUSED_LAYER = True
    (o0, g0), (o1, g1) = results
    assert torch.allclose(o0, o1, rtol=1e-5, atol=1e-6), float((o0 - o1).abs().max())
    assert set(g0) == set(g1)
    for n in g0:
        scale = float(g0[n].abs().max()) + 1e-12
        assert float((g0[n] - g1[n]).abs().max()) <= 1e-4 * scale + 1e-9, (n, float((g0[n] - g1[n]).abs().max()), scale)
    assert _lib.read_status(dev) == 0


@pytest.mark.parametrize("save_pairs", [True, False])
def test_chunked_tasks_change_nothing_but_rounding(save_pairs):
    """A batch with dense 48-64 atom cells among small crystals: the work queue cuts their atoms' tasks into chunks
    (partial results merged in chunk order).  Outputs and gradients equal the uncut run to rounding, and two cut runs
    are bit-identical however the chunks were scheduled."""
    dev = cuda()
    from crystalframer_b200 import _lib, data, encoder, fused_layer, synth
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    torch.manual_seed(5)
    model = Latticeformer(ModelParams(num_layers=2, symm_break_noise=0.0)).to(dev).train()
    dense = synth.make_batch(3, 21, size_dist="uniform", size_lo=48, size_hi=64, len_lo=3.0, len_hi=5.0)
    small = synth.make_batch(61, 22, size_dist="uniform", size_lo=1, size_hi=6, len_lo=6.0, len_hi=15.0)
    b = synth.concat([small, dense])
    y = np.random.default_rng(1).normal(size=(len(b.sizes), 1)).astype(np.float32)
    tb = data.host_batch(b, y, pinned=False).to(dev, non_blocking=False)
    with torch.no_grad():
        model(tb)
    seen = []
    orig = fused_layer.LayerGeometry.from_raw.__func__

    def spy(cls, *a, **k):
        g = orig(cls, *a, **k)
        seen.append(g)
        return g
    fused_layer.LayerGeometry.from_raw = classmethod(spy)
    fused_layer.SAVE_PAIR_RESULTS = save_pairs         # backward from stored per-pair results, or by recomputation
    results = []
    try:
        for split in (False, True, True):
            fused_layer.SPLIT_TASKS = split
            model.zero_grad(set_to_none=True)
            np.random.seed(11)
            torch.manual_seed(11)
            out = model(tb)
            (out - tb.y).abs().mean().backward()
            results.append((out.detach().clone(), {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}))
    finally:
        fused_layer.SPLIT_TASKS = True
        fused_layer.SAVE_PAIR_RESULTS = True
        fused_layer.LayerGeometry.from_raw = classmethod(orig)
    assert len(seen) == 3 and seen[0].split is None
    header = seen[1].split[:4].cpu().numpy()
    assert header[0] > 0 and header[2] > 0                            # the dense cells got chunk entries and partial rows
    (o0, g0), (o1, g1), (o2, g2) = results
    assert torch.allclose(o0, o1, rtol=1e-5, atol=1e-6), float((o0 - o1).abs().max())
    for n in g0:
        scale = float(g0[n].abs().max()) + 1e-12
        assert float((g0[n] - g1[n]).abs().max()) <= 1e-4 * scale + 1e-9, (n, float((g0[n] - g1[n]).abs().max()), scale)
    assert torch.equal(o1, o2) and all(torch.equal(g1[n], g2[n]) for n in g1)
    assert _lib.read_status(dev) == 0


def test_chunked_geometry_without_task_table_is_the_plain_queue():
    """A geometry built with the chunked queue, layers given no task table: the kernels walk the atoms' entries of the
    queue (behind its chunk region) exactly as they walk the plain queue -- bit-identical results."""
    dev = cuda()
    from crystalframer_b200 import _lib, data, fused_layer, synth
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    torch.manual_seed(5)
    model = Latticeformer(ModelParams(num_layers=1, symm_break_noise=0.0)).to(dev).train()
    b = synth.make_workload("cfg2", num_crystals=24)
    y = np.random.default_rng(1).normal(size=(len(b.sizes), 1)).astype(np.float32)
    tb = data.host_batch(b, y, pinned=False).to(dev, non_blocking=False)
    with torch.no_grad():
        model(tb)
    results = []
    try:
        for split, table in ((False, True), (True, False)):
            fused_layer.SPLIT_TASKS, fused_layer.TASK_TABLE = split, table
            model.zero_grad(set_to_none=True)
            np.random.seed(11)
            torch.manual_seed(11)
            out = model(tb)
            (out - tb.y).abs().mean().backward()
            results.append((out.detach().clone(), {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}))
    finally:
        fused_layer.SPLIT_TASKS, fused_layer.TASK_TABLE = True, True
    (o0, g0), (o1, g1) = results
    assert torch.equal(o0, o1) and all(torch.equal(g0[n], g1[n]) for n in g0)
    assert _lib.read_status(dev) == 0


def _step_models(dev, sink):
    from crystalframer_b200 import data, synth
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    from crystalframer_b200.optim import FlatAdamW
    torch.manual_seed(4)
    ref = Latticeformer(ModelParams(num_layers=2, symm_break_noise=0.0)).to(dev).train()
    ours = copy.deepcopy(ref)
    b = synth.make_workload("cfg2", num_crystals=24)
    y = np.random.default_rng(2).normal(size=(len(b.sizes), 1)).astype(np.float32)
    tb = data.host_batch(b, y, pinned=False).to(dev, non_blocking=False)
    with torch.no_grad():
        ref(tb)
    for lr, lo in zip(ref.encoder.layers, ours.encoder.layers):
        with torch.no_grad():
            lo.self_attn.gauss_scale.copy_(lr.self_attn.gauss_scale)
    split = lambda m: ([p for n, p in m.named_parameters() if p.requires_grad and not n.endswith("bias")],
                       [p for n, p in m.named_parameters() if p.requires_grad and n.endswith("bias")])
    d, nd = split(ref)
    opt_ref = torch.optim.AdamW([{"params": d, "weight_decay": 1e-2}, {"params": nd, "weight_decay": 0.0}], lr=5e-4,
                                betas=(0.9, 0.98))
    d2, nd2 = split(ours)
    opt = FlatAdamW(iter(d2), iter(nd2), lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-2, max_norm=1.0, grad_sink=sink)
    return ref, ours, opt_ref, opt, b, y, tb


@pytest.mark.parametrize("sink", [True, False])
def test_training_step_with_gradient_sinks(sink):
    """Three training steps: autograd gradients + clip_grad_norm_ + torch AdamW against the one-call layers adding
    their weight gradients into FlatAdamW's flat buffer.  The parameter groups are passed as iterators."""
    dev = cuda()
    from crystalframer_b200 import encoder
    ref, ours, opt_ref, opt, b, y, tb = _step_models(dev, sink)
    for step in range(3):
        np.random.seed(20 + step)
        encoder.FUSED_LAYER = False
        opt_ref.zero_grad(set_to_none=True)
        (ref(tb) - tb.y).abs().mean().backward()
        norm_ref = torch.nn.utils.clip_grad_norm_(list(ref.parameters()), 1.0)
        opt_ref.step()
        np.random.seed(20 + step)
        encoder.FUSED_LAYER = True
        opt.zero_grad()
        (ours(tb) - tb.y).abs().mean().backward()
        if sink:
            layer_w = ours.encoder.layers[0].linear1.weight
            assert layer_w.grad is None and float(layer_w._cf_grad_sink.abs().max()) > 0.0
        # gradients first: the flat buffer against autograd's gradients of the operator path
        opt.gather_grads()
        by_param = {id(p): s_ for p, s_ in zip(opt.params, opt.sinks)}
        for (n, a), c in zip(ref.named_parameters(), ours.parameters()):
            if a.grad is None:
                continue
            scale = float(a.grad.abs().max()) + 1e-12
            err = float((by_param[id(c)] - a.grad).abs().max())
            assert err <= 1e-4 * scale + 1e-9, (step, n, err, scale)
        opt.step()
        assert abs(float(opt.grad_norm) - float(norm_ref)) <= 1e-4 * max(1.0, float(norm_ref))
        # Adam divides by the root of the squared gradient: an entry whose gradient is at rounding level may move
        # by up to the learning rate in either implementation, so a few entries may differ by that much
        for (n, a), c in zip(ref.named_parameters(), ours.parameters()):
            close(f"step {step} {n}", c.detach().cpu().numpy(), a.detach().cpu().numpy(), 1e-4, 2e-6, frac_ok=2e-3)
            assert float((c - a).abs().max()) <= 2.5 * 5e-4 * (step + 1)
        with torch.no_grad():                       # continue from identical weights
            for a, c in zip(ref.parameters(), ours.parameters()):
                c.copy_(a)


def test_weight_decay_applies_with_iterator_groups():
    """With zero gradients AdamW only shrinks the decayed parameters; groups given as generators must not
    silently lose their weight decay."""
    dev = cuda()
    from crystalframer_b200.optim import FlatAdamW
    torch.manual_seed(0)
    m = torch.nn.Linear(16, 8).to(dev)
    w0, b0 = m.weight.detach().clone(), m.bias.detach().clone()
    opt = FlatAdamW((p for n, p in m.named_parameters() if n == "weight"), (p for n, p in m.named_parameters() if n == "bias"),
                    lr=1e-1, weight_decay=0.5)
    opt.zero_grad()
    opt.step()
    assert torch.allclose(m.weight, w0 * (1 - 1e-1 * 0.5), rtol=1e-6, atol=1e-8)
    assert torch.equal(m.bias, b0)
    with pytest.raises(ValueError):
        FlatAdamW([m.weight, m.weight], [])


def test_running_average_of_weights_matches_torch_swa():
    """step(average=True) against torch.optim.swa_utils.AveragedModel.update_parameters after every step
    (models/regression.py:150-152 of the reference), then the exchange with the live weights."""
    dev = cuda()
    from torch.optim.swa_utils import AveragedModel
    from crystalframer_b200.optim import FlatAdamW
    torch.manual_seed(1)
    ours = torch.nn.Sequential(torch.nn.Linear(12, 9), torch.nn.ReLU(), torch.nn.Linear(9, 3)).to(dev)
    theirs = copy.deepcopy(ours)
    opt_o = FlatAdamW(ours.parameters(), (), lr=1e-2, betas=(0.9, 0.98), weight_decay=1e-5, max_norm=1.0)
    opt_t = torch.optim.AdamW(theirs.parameters(), lr=1e-2, betas=(0.9, 0.98), weight_decay=1e-5)
    swa = AveragedModel(theirs)
    for step in range(5):
        x = torch.randn(32, 12, device=dev)
        for m, o in ((ours, opt_o), (theirs, opt_t)):
            o.zero_grad()
            m(x).square().mean().backward()
        opt_o.step(average=step >= 1)                  # averaging starts at the second step
        torch.nn.utils.clip_grad_norm_(theirs.parameters(), 1.0)
        opt_t.step()
        if step >= 1:
            swa.update_parameters(theirs)
    assert opt_o.n_averaged == 4
    for a, b in zip(opt_o.averaged_parameters(), swa.module.parameters()):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-7), float((a - b).abs().max())
    live = [p.detach().clone() for p in ours.parameters()]
    opt_o.swap_averaged()
    for p, b in zip(ours.parameters(), swa.module.parameters()):
        assert torch.allclose(p, b, rtol=1e-5, atol=1e-7)
    opt_o.swap_averaged()
    assert all(torch.equal(p, l) for p, l in zip(ours.parameters(), live))


def test_sharded_step_equals_whole_batch():
    """One global batch dealt into two shards by attention cost, each shard's loss divided by the GLOBAL crystal
    count, gradient buffers added: the same gradients and the same update as one pass over the whole batch
    (what the multi-GPU benchmark does with an all-reduce in place of the addition)."""
    dev = cuda()
    from crystalframer_b200 import data, synth
    from crystalframer_b200.parallel import attention_cost, partition_by_pair_count
    ref, ours, _, opt, b, y, tb = _step_models(dev, True)
    from crystalframer_b200.optim import FlatAdamW
    split = lambda m: ([p for n, p in m.named_parameters() if p.requires_grad and not n.endswith("bias")],
                       [p for n, p in m.named_parameters() if p.requires_grad and n.endswith("bias")])
    opt_whole = FlatAdamW(*split(ref), lr=5e-4, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-2, max_norm=1.0)
    B = len(b.sizes)
    np.random.seed(5)
    opt_whole.zero_grad()
    ((ref(tb) - tb.y).abs().sum() / B).backward()
    g_whole = opt_whole.gather_grads().clone()
    parts = partition_by_pair_count(b.sizes, 2, attention_cost(b.sizes, b.trans_vec))
    assert sorted(np.concatenate(parts).tolist()) == list(range(B))
    opt.zero_grad()
    for idx in parts:
        idx = np.sort(idx)
        sb = data.host_batch(synth.select(b, idx), y[idx], pinned=False).to(dev, non_blocking=False)
        np.random.seed(5)
        ((ours(sb) - sb.y).abs().sum() / B).backward()        # sinks and .grad accumulate over the shards
    g_sum = opt.gather_grads()
    scale = float(g_whole.abs().max())
    assert float((g_sum - g_whole).abs().max()) <= 1e-4 * scale
    opt_whole.step()
    opt.step()
    # Adam divides by the root of the squared gradient: entries whose gradient is at rounding level may move by up
    # to the learning rate in either run, so a few entries may differ by that much
    diff = (opt.flat - opt_whole.flat).abs()
    assert float((diff > 2e-6).float().mean()) <= 1e-3 and float(diff.max()) <= 2.5 * 5e-4


@pytest.mark.parametrize("M,N,K,kn", [(300, 128, 128, 0), (2661, 512, 128, 0), (1000, 128, 512, 0), (517, 128, 128, 1),
                                      (129, 512, 128, 1), (64, 96, 36, 0)])
def test_dense_layer_kernels(M, N, K, kn):
    """cfb200_linear (the kernels behind the layer's dense parts) against float64 matmul: plain, with bias +
    residual + ReLU, for torch-layout and transposed weights, at sizes with ragged last tiles.  The last case has a
    shape the tensor-core kernel does not cover and runs on the FP32 pipe."""
    dev = cuda()
    from crystalframer_b200 import _lib, cuda_funcs as F
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, 0.0)
    g = torch.Generator(device="cpu").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g)
    w = torch.randn((K, N) if kn else (N, K), generator=g) * K ** -0.5
    b, r = torch.randn(N, generator=g), torch.randn(M, N, generator=g)
    ref = x.double() @ (w.double() if kn else w.double().t())
    xd, wd, bd, rd = x.to(dev), w.to(dev), b.to(dev), r.to(dev)
    y = torch.empty(M, N, device=dev)
    p = _lib.ptr
    _lib.invoke("cfb200_linear", 1, dev, p(xd), p(wd), None, None, M, N, K, 0, kn, p(y))
    close("x W", y.cpu().numpy(), ref.numpy(), 1e-5, 2e-5)
    _lib.invoke("cfb200_linear", 1, dev, p(xd), p(wd), p(bd), p(rd), M, N, K, 1, kn, p(y))
    close("relu(x W + b + r)", y.cpu().numpy(), torch.relu(ref + b.double() + r.double()).numpy(), 1e-5, 2e-5)
    assert _lib.read_status(dev) == 0


def test_training_steps_repeat_bit_for_bit():
    """Two runs of three training steps of the 4-layer model on the benchmark's batch (256 crystals: chunked tasks,
    blocks moving across heads, weight gradients on the side stream) from the same weights and optimiser state:
    every parameter must come out identical -- which warp or block computes what varies from run to run, the
    order of every sum does not."""
    dev = cuda()
    import copy
    from crystalframer_b200 import data, synth
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    from crystalframer_b200.optim import FlatAdamW
    torch.manual_seed(5)
    model = Latticeformer(ModelParams(symm_break_noise=0.0)).to(dev).train()
    b = synth.make_workload("cfg3", seed=2)
    y = np.random.default_rng(2).normal(size=(len(b.sizes), 1)).astype(np.float32)
    tb = data.host_batch(b, y, pinned=False).to(dev, non_blocking=False)
    with torch.no_grad():
        model(tb)                                   # coefficient statistics; later forwards take the one-call layers
    decay = [p for n, p in model.named_parameters() if p.requires_grad and not n.endswith("bias")]
    no_decay = [p for n, p in model.named_parameters() if p.requires_grad and n.endswith("bias")]
    opt = FlatAdamW(decay, no_decay, lr=5e-4, betas=(0.9, 0.98), weight_decay=1e-5, max_norm=1.0)
    start_model = {k: v.detach().clone() for k, v in model.state_dict().items()}
    start_opt = copy.deepcopy(opt.state_dict())
    runs = []
    for _ in range(2):
        model.load_state_dict(start_model)
        opt.load_state_dict(copy.deepcopy(start_opt))
        losses = []
        for step in range(3):
            opt.zero_grad()
            loss = (model(tb) - tb.y).abs().mean()
            loss.backward()
            opt.step()
            losses.append(loss.detach().clone())
        runs.append((torch.stack(losses), opt.flat.clone(), opt.grad.clone()))
    assert torch.equal(runs[0][0], runs[1][0]), (runs[0][0], runs[1][0])
    assert torch.equal(runs[0][2], runs[1][2])      # the last step's gradients
    assert torch.equal(runs[0][1], runs[1][1])      # all parameters
