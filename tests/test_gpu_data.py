"""The epoch loader on the GPU: batches staged through pinned buffers and a copy stream by the background thread
are, byte for byte, the collation of the same structures on the host; a training step fed by the loader gives
the loss of the same step fed by a host batch."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_epoch_loader_batches_equal_host_collation():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    from crystalframer_b200 import data
    ds = data.StructureSet.synthetic(2000, 5, chunk=512)
    for rank, world in ((0, 1), (1, 2)):
        loader = data.EpochLoader(ds, 96, rank=rank, world=world, device=dev, epoch=2, seed=1, depth=2)
        sched = data.epoch_schedule(len(ds), 96 * world, 2, 1)
        got = []
        for step, tb in enumerate(loader):
            # keep the consumer slow on some steps and fast on others, so that slots are reused under both orders
            if step % 3 == 0:
                torch.cuda.synchronize()
            got.append(tb)
        torch.cuda.synchronize()
        assert len(got) == len(sched) == len(loader)
        for step, tb in enumerate(got):
            want = ds.collate(data.rank_share(ds, sched[step], rank, world))
            assert tb.x.device == dev and tb.num_pairs == want.num_pairs
            assert np.array_equal(tb.x.cpu().numpy(), want.x) and np.array_equal(tb.pos.cpu().numpy(), want.pos)
            assert np.array_equal(tb.batch.cpu().numpy(), want.batch) and np.array_equal(tb.sizes.cpu().numpy(), want.sizes)
            assert np.array_equal(tb.trans_vec.cpu().numpy(), want.trans_vec)
        assert loader.h2d_bytes > 0


def test_training_step_from_the_loader_equals_the_step_from_a_host_batch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    import copy
    from crystalframer_b200 import data
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    ds = data.StructureSet.synthetic(256, 6)
    torch.manual_seed(0)
    model = Latticeformer(ModelParams(num_layers=2, symm_break_noise=0.0)).to(dev).train()
    loader = data.EpochLoader(ds, 64, device=dev, epoch=0, seed=3)
    sched = data.epoch_schedule(len(ds), 64, 0, 3)
    first = next(iter(loader))
    with torch.no_grad():
        model(first)                                            # coefficient statistics
    twin = copy.deepcopy(model)
    for step, tb in enumerate(loader):
        hb = data.host_batch(ds.collate(sched[step]), ds.y[sched[step]]).to(dev, non_blocking=False)
        la = (model(tb) - tb.y).abs().mean()
        lb = (twin(hb) - hb.y).abs().mean()
        assert torch.equal(la, lb), step
        la.backward()
        lb.backward()
    for (n, p), (_, q) in zip(model.named_parameters(), twin.named_parameters()):
        assert (p.grad is None) == (q.grad is None), n
        if p.grad is not None:
            assert torch.equal(p.grad, q.grad), n


def test_inference_from_a_reference_layout_checkpoint():
    """A few training steps with the running weight average, exported in the reference's checkpoint layout, loaded
    into a fresh model the way the reference's demo loads it, evaluated without gradients: the predictions are the
    averaged model's, rescaled to the targets' units, and the eval forward (lighter kernels, no per-pair results
    kept) agrees with the training forward of the same weights."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    from crystalframer_b200 import checkpoint, data
    from crystalframer_b200.optim import FlatAdamW
    ds = data.StructureSet.synthetic(384, 8)
    torch.manual_seed(1)
    model = checkpoint.build_model(num_layers=2, symm_break_noise=0.0).to(dev).train()
    decay = [p for n, p in model.named_parameters() if not n.endswith("bias")]
    no_decay = [p for n, p in model.named_parameters() if n.endswith("bias")]
    opt = FlatAdamW(decay, no_decay, lr=5e-4, betas=(0.9, 0.98), weight_decay=1e-5, max_norm=1.0)
    for tb in data.EpochLoader(ds, 64, device=dev, epoch=0, seed=0):
        opt.zero_grad()
        ((model(tb) - tb.y).abs().mean()).backward()
        opt.step(average=True)
    avg_state = dict(model.state_dict())
    by_id = {id(p): a for p, a in zip(opt.params, opt.averaged_parameters())}
    for name, p in model.named_parameters():
        if id(p) in by_id:
            avg_state[name] = by_id[id(p)].detach().clone()
    ck = checkpoint.reference_checkpoint_of(model, averaged_state=avg_state, target_std=[3.0], target_mean=[0.5],
                                            n_averaged=opt.n_averaged)
    fresh = checkpoint.build_model(num_layers=2, symm_break_noise=0.0).to(dev)
    checkpoint.load_reference_checkpoint(fresh, ck)
    batches = list(data.EpochLoader(ds, 128, device=dev, epoch=5, seed=0))
    mae, pred = checkpoint.evaluate(fresh, batches)
    # the averaged model itself, un-rescaled, in training mode (the forward that keeps per-pair results)
    opt.swap_averaged()
    want = torch.cat([model(tb).detach() for tb in batches]) * 3.0 + 0.5
    opt.swap_averaged()
    assert pred.shape == want.shape and torch.allclose(pred, want, rtol=1e-4, atol=1e-5), float((pred - want).abs().max())
    y = torch.cat([tb.y for tb in batches])
    assert torch.allclose(mae, (pred - y).abs().mean(0))
    assert fresh.training                                       # evaluate() leaves the module's mode as it found it
