"""Host-side logic on CPU: synthetic data, module parameters, data-parallel plumbing (gloo)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_synthetic_workloads_are_seeded_and_in_range():
    from crystalframer_b200 import synth
    a, b = synth.make_workload("cfg2"), synth.make_workload("cfg2")
    assert np.array_equal(a.pos, b.pos) and np.array_equal(a.sizes, b.sizes)
    assert len(a.sizes) == 256 and a.sizes.min() >= 1 and a.sizes.max() <= 64
    assert 6 <= np.median(a.sizes) <= 10
    lengths = np.linalg.norm(a.trans_vec, axis=-1)
    assert lengths.min() >= 3.0 - 1e-4 and lengths.max() <= 15.0 + 1e-4
    assert abs(np.linalg.det(a.trans_vec.astype(np.float64))).min() > 1.0
    c = synth.make_workload("cfg4", num_crystals=3)
    assert c.sizes.min() >= 100 and c.sizes.max() <= 200
    assert a.x.shape == (a.num_atoms, 98) and (a.x.sum(1) == 1).all()


def test_model_has_reference_parameter_set():
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    m = Latticeformer(ModelParams())
    assert sum(p.numel() for p in m.parameters() if p.requires_grad) == 951809
    sd = m.state_dict()
    pre = "encoder.layers.0.self_attn."
    shapes = {"q_proj_weight": (128, 128), "k_proj_weight": (128, 128), "v_proj_weight": (128, 128),
              "in_proj_bias": (384,), "out_proj.weight": (128, 128), "out_proj.bias": (128,),
              "lattice_pos_weights": (128,), "pe_dist_proj": (1, 8, 16, 64), "proj_angle1": (1, 8, 16, 64),
              "proj_angle2": (1, 8, 16, 64), "proj_angle3": (1, 8, 16, 64), "gauss_scale": (2,), "atten_scale": (1,)}
    for k, shp in shapes.items():
        assert tuple(sd[pre + k].shape) == shp, k


def test_partition_by_pair_count_balances():
    from crystalframer_b200 import synth
    from crystalframer_b200.parallel import partition_by_pair_count
    sizes = synth.make_workload("cfg2").sizes
    parts = partition_by_pair_count(sizes, 8)
    assert sorted(np.concatenate(parts).tolist()) == list(range(len(sizes)))
    loads = np.array([(sizes[p] ** 2).sum() for p in parts])
    assert loads.max() - loads.min() <= (sizes ** 2).max()
    # with the attention-cost estimate (pairs x translations in reach) the same rule balances that cost
    from crystalframer_b200.parallel import attention_cost
    b = synth.make_workload("cfg2")
    cost = attention_cost(b.sizes, b.trans_vec)
    assert cost.shape == b.sizes.shape and (cost >= 8.0 * b.sizes ** 2).all() and (cost <= 132.0 * b.sizes ** 2).all()
    parts = partition_by_pair_count(b.sizes, 8, cost)
    assert sorted(np.concatenate(parts).tolist()) == list(range(len(b.sizes)))
    loads = np.array([cost[p].sum() for p in parts])
    assert loads.max() - loads.min() <= cost.max()
    # the counted cost: per pair, the translations of the 5x5x5 block above the pruning threshold
    from crystalframer_b200.parallel import attention_cost_counted
    small = synth.make_workload("cfg2", num_crystals=32)
    counted = attention_cost_counted(small.pos, small.trans_vec, small.sizes)
    n2 = small.sizes.astype(np.float64) ** 2
    assert counted.shape == small.sizes.shape
    assert (counted >= (350.0 + 70.0) * n2).all() and (counted <= (350.0 + 70.0 * 125) * n2).all()
    one = attention_cost_counted(small.pos[:small.sizes[0]], small.trans_vec[:1], small.sizes[:1])
    assert one[0] == counted[0]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from crystalframer_b200 import parallel
    torch.manual_seed(100 + rank)                      # different initial weights per rank on purpose
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 1))
    parallel.broadcast_state(model)
    w0 = torch.cat([p.detach().flatten() for p in model.parameters()])
    x = torch.full((4, 6), float(rank + 1))
    model(x).sum().backward()
    local = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
    parallel.allreduce_gradients(list(model.parameters()))
    avg = torch.cat([p.grad.flatten() for p in model.parameters()])
    gathered = [torch.zeros_like(local) for _ in range(world)]
    dist.all_gather(gathered, local)
    # numpy arrays travel by value; a tensor would travel as a shared-memory handle that dies with this process
    q.put((rank, w0.numpy(), avg.numpy(), torch.stack(gathered).mean(0).numpy()))
    dist.destroy_process_group()


def test_gradient_allreduce_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda t: t[0])
    res = [(r,) + tuple(torch.from_numpy(x) for x in rest) for r, *rest in res]
    for p in procs:
        p.join(60)
    (_, w_a, g_a, m_a), (_, w_b, g_b, m_b) = res
    assert torch.equal(w_a, w_b)                       # broadcast made the weights identical
    assert torch.allclose(g_a, g_b) and torch.allclose(g_a, m_a, atol=1e-6)


def test_dealing_by_cost_is_the_reference_rule():
    """cfb200_deal_by_cost (host code of the library) against the rule written out as the reference has it
    (models/latticeformer.py:224-233): descending cost, each item to the group with the smallest total."""
    from crystalframer_b200.parallel import partition_by_pair_count

    def written_out(weight, parts):
        totals, groups = np.zeros(parts, np.float64), [[] for _ in range(parts)]
        for item in np.argsort(-weight, kind="stable"):
            g = int(np.argmin(totals))
            totals[g] += weight[item]
            groups[g].append(int(item))
        return groups

    rng = np.random.default_rng(0)
    for n, parts in ((2048, 8), (256, 2), (7, 3), (50, 1), (0, 4)):
        w = np.round(rng.lognormal(3, 1, n))                  # rounded: many equal costs
        got = partition_by_pair_count(np.zeros(n), parts, w)
        assert [g.tolist() for g in got] == written_out(w, parts), (n, parts)
    sizes = rng.integers(1, 65, 300)
    got = partition_by_pair_count(sizes, 4)                   # default cost: the pair count
    assert [g.tolist() for g in got] == written_out(sizes.astype(np.float64) ** 2, 4)


def test_epoch_loader_covers_the_set_once_and_collates_like_the_batch_functions():
    """Structure set + epoch schedule + per-rank shares, on the CPU: every structure of the epoch's full global
    batches appears exactly once over the ranks, each rank's batch equals the collation of its structures by the
    batch functions, the schedule is the same on every rank and changes with the epoch."""
    from crystalframer_b200 import data, synth
    ds = data.StructureSet.synthetic(1000, 3, chunk=256)
    assert len(ds) == 1000 and ds.start[-1] == len(ds.pos)
    first = synth.make_workload("cfg3", seed=3 * 100003, num_crystals=256)
    pick = np.array([7, 255, 0, 31])
    got, want = ds.collate(pick), synth.select(first, pick)
    for f in ("x", "pos", "batch", "trans_vec", "sizes", "z"):
        assert np.array_equal(getattr(got, f), getattr(want, f)), f
    world, per_rank = 3, 64
    seen = []
    for rank in range(world):
        loader = data.EpochLoader(ds, per_rank, rank=rank, world=world, device="cpu", epoch=1, seed=9)
        sched = data.epoch_schedule(len(ds), per_rank * world, 1, 9)
        assert len(loader) == len(sched) == 1000 // (per_rank * world)
        for step, tb in enumerate(loader):
            mine = data.rank_share(ds, sched[step], rank, world)
            seen.append(mine)
            want = ds.collate(mine)
            assert torch.equal(tb.x, torch.from_numpy(want.x)) and torch.equal(tb.pos, torch.from_numpy(want.pos))
            assert torch.equal(tb.batch, torch.from_numpy(want.batch)) and torch.equal(tb.sizes, torch.from_numpy(want.sizes))
            assert torch.equal(tb.trans_vec, torch.from_numpy(want.trans_vec)) and tb.num_pairs == want.num_pairs
            assert torch.equal(tb.y, torch.from_numpy(ds.y[mine]))
    seen = np.concatenate(seen)
    assert len(seen) == len(np.unique(seen)) == (1000 // (per_rank * world)) * per_rank * world
    assert not np.array_equal(data.epoch_schedule(len(ds), 192, 0, 9), data.epoch_schedule(len(ds), 192, 1, 9))


def _exchange_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from crystalframer_b200.parallel import GradientExchange
    g = torch.Generator().manual_seed(7 + rank)
    flat = torch.randn(1000, generator=g)
    whole = flat.clone()
    dist.all_reduce(whole)
    ex = GradientExchange(flat)
    ex.send([(640, 704), (128, 256)])            # "layer 3": two slices, given out of order
    ex.send([(256, 320), (704, 768), (0, 0)])     # "layer 2": adjacent to the first ones; an empty range
    untouched = flat[320:640].clone()            # not sent yet: still this rank's own values
    ex.finish()
    second = flat.clone()
    ex.finish()                                  # nothing sent since: reduces the whole buffer again
    q.put((rank, flat.numpy().copy(), whole.numpy().copy(), untouched.numpy().copy(), second.numpy().copy()))
    dist.destroy_process_group()


def test_gradient_exchange_in_pieces_equals_one_allreduce_two_ranks_gloo():
    from crystalframer_b200.parallel import GradientExchange
    assert GradientExchange.merge([(5, 9), (0, 3), (3, 4), (8, 12), (20, 20)]) == [(0, 4), (5, 12)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() + 17) % 1000
    procs = [ctx.Process(target=_exchange_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda t: t[0])
    for p in procs:
        p.join(60)
    for rank, flat, whole, untouched, second in res:
        g = torch.Generator().manual_seed(7 + rank)
        own = torch.randn(1000, generator=g).numpy()
        assert np.array_equal(untouched, own[320:640])                 # finish() had not run yet
        assert np.allclose(second, whole, rtol=0, atol=1e-6)           # pieces add up to the single all-reduce
        assert np.allclose(flat, 2 * whole, rtol=0, atol=2e-6)         # a finish() with nothing sent reduces everything
    assert np.array_equal(res[0][4], res[1][4])                       # both ranks hold the same sums


def test_reference_checkpoint_layout_round_trip():
    """A checkpoint in the layout of the reference's training module (model.*, swa_model.module.*, target_std,
    target_mean; models/regression.py:30-59) loads as demo.py:67-88 loads it: averaged weights by default, the last
    linear layer rescaled to the targets' units."""
    from crystalframer_b200 import checkpoint
    torch.manual_seed(0)
    src = checkpoint.build_model(num_layers=2)
    avg = {k: v + 0.01 for k, v in src.state_dict().items()}
    ck = checkpoint.reference_checkpoint_of(src, averaged_state=avg, target_std=[2.5], target_mean=[-0.75], n_averaged=7)
    keys = set(ck["state_dict"])
    assert {"target_std", "target_mean", "swa_model.n_averaged"} <= keys
    assert sum(k.startswith("model.") for k in keys) == sum(k.startswith("swa_model.module.") for k in keys) == len(avg)
    dst = checkpoint.build_model(num_layers=2)
    std, mean = checkpoint.load_reference_checkpoint(dst, ck)
    assert float(std) == 2.5 and float(mean) == -0.75
    for k, v in dst.state_dict().items():
        if k == "mlp.3.weight":
            assert torch.allclose(v, avg[k] * 2.5)
        elif k == "mlp.3.bias":
            assert torch.allclose(v, avg[k] * 2.5 - 0.75)
        else:
            assert torch.equal(v, avg[k]), k
    live = checkpoint.build_model(num_layers=2)
    checkpoint.load_reference_checkpoint(live, ck["state_dict"], prefix="model.", denormalize=False)
    for k, v in live.state_dict().items():
        assert torch.equal(v, src.state_dict()[k]), k
    with pytest.raises(KeyError):
        checkpoint.load_reference_checkpoint(live, ck, prefix="ema.")
