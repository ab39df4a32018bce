"""Data-parallel plumbing: one process per GPU, crystals sharded across ranks, one flat-buffer
all-reduce of the gradients per step.  Replaces the reference's in-forward
replicate / parallel_apply / gather over the encoder (models/latticeformer.py:211-273) and its
Lightning DDP mode (train.py:97-119); no kernel of this package communicates."""
import numpy as np
import torch
import torch.distributed as dist


def attention_cost(sizes, cells):
    """Estimated attention cost of each crystal: pairs x (a constant + the lattice translations within reach
    of a Gaussian of typical width, about a sphere of radius 8 A over the cell volume, between 1 and 125) --
    the same estimate that orders the work queue of the fused attention kernels."""
    vol = np.abs(np.linalg.det(np.asarray(cells, dtype=np.float64)))
    survivors = np.clip(2145.0 / np.maximum(vol, 1e-6), 1.0, 125.0)
    return np.asarray(sizes, dtype=np.float64) ** 2 * (7.0 + survivors)


def attention_cost_counted(pos, cells, sizes, a_typical=-0.255, prune=16.0, per_pair=350.0, per_term=70.0):
    """Attention cost of each crystal from a COUNT of the lattice translations the kernels will expand, instead of
    the cell-volume guess of ``attention_cost``: for every pair, the translations of the 5 x 5 x 5 block whose
    Gaussian weight exp(a (d^2 - d^2_min)) stays above exp(-prune) for a coefficient of typical size
    (a = -1/(2 * 1.4^2)).  cost = sum over pairs of (per_pair + per_term * survivors), the two constants being the
    measured instruction counts of the fused attention kernels per pair and per surviving translation.  ``pos`` (N,3)
    are the atoms' positions in crystal order; a few tens of milliseconds of numpy work for a 256-crystal batch."""
    pos = np.asarray(pos, dtype=np.float64)
    cells = np.asarray(cells, dtype=np.float64)
    sizes = np.asarray(sizes, dtype=np.int64)
    start = np.concatenate([[0], np.cumsum(sizes)])
    r = np.arange(-2, 3)
    n = np.stack(np.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 3).astype(np.float64)
    out = np.zeros(len(sizes), np.float64)
    for c in range(len(sizes)):
        p = pos[start[c]:start[c + 1]]
        t = n @ cells[c]                                       # (125,3)
        d = p[None, :, :] - p[:, None, :]
        d2 = ((d[:, :, None, :] + t[None, None]) ** 2).sum(-1)  # (n, n, 125)
        surv = (a_typical * (d2 - d2.min(-1, keepdims=True)) > -prune).sum(-1)
        out[c] = per_pair * surv.size + per_term * surv.sum()
    return out


def deal_by_cost(cost, n_parts):
    """Group (0..n_parts-1) of every item under the dealing rule of ``partition_by_pair_count``, as one call into the
    library's host code (cfb200_deal_by_cost): 2 048 crystals over 8 ranks take microseconds there and several
    milliseconds as a Python loop, and the call releases the interpreter lock, which matters to the epoch loader's
    background thread (data.EpochLoader)."""
    from . import _lib
    weight = np.ascontiguousarray(cost, dtype=np.float64)
    part_of = np.empty(len(weight), np.int32)
    rc = _lib.lib().cfb200_deal_by_cost(weight.ctypes.data, len(weight), int(n_parts), part_of.ctypes.data)
    if rc != 0:
        _lib.check(rc, "cfb200_deal_by_cost")
    return part_of


def partition_by_pair_count(sizes, n_parts, cost=None):
    """Greedy split of crystals into ``n_parts`` groups of nearly equal cost, largest first -- the rule of
    models/latticeformer.py:224-233, whose cost is the squared size (the pair count).  ``cost`` replaces the
    squared sizes by a better estimate (``attention_cost``).  Returns a list of index arrays."""
    weight = np.ascontiguousarray(np.asarray(sizes, dtype=np.float64) ** 2 if cost is None else cost, dtype=np.float64)
    part_of = deal_by_cost(weight, n_parts)
    order = np.argsort(-weight, kind="stable")
    dealt = part_of[order]
    return [order[dealt == g].astype(np.int64) for g in range(n_parts)]


def broadcast_state(module, src=0):
    """Initial weights and the data-dependent ``gauss_scale`` statistics must agree on all ranks
    (the reference initialises them from the first training batch,
    models/indexed_lattice_multi_head_attention_cuda.py:907-923)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return
    for t in list(module.parameters()) + list(module.buffers()):
        dist.broadcast(t.data, src)


def allreduce_gradients(params, average=True):
    """Sums (averages) ``p.grad`` of all parameters over the ranks with ONE collective on a
    flattened buffer (about 3.8 MB for the 4-layer model: latency-bound, so one launch beats
    per-tensor calls)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch._utils._flatten_dense_tensors(grads)
    dist.all_reduce(flat)
    if average:
        flat.div_(dist.get_world_size())
    torch._foreach_copy_(grads, list(torch._utils._unflatten_dense_tensors(flat, grads)))   # one launch, not one per tensor


class GradientExchange:
    """Sums a flat gradient buffer over the ranks in pieces.  ``send(ranges)`` starts an asynchronous all-reduce of
    element ranges whose gradients are final -- the communication library runs it on its own stream, ordered after
    the work already enqueued on the caller's stream, so it overlaps whatever the caller enqueues next (the backward
    pass of earlier layers); ``finish()`` sends every element not sent yet and makes the caller's stream wait for
    all of it.  Every rank must send the same ranges in the same order.  The reference exchanges nothing by hand:
    its replicas' gradients are reduced by nn.parallel / Lightning DDP after the backward pass
    (models/latticeformer.py:211-273, train.py:97-119)."""

    def __init__(self, flat):
        self.flat = flat
        self.sent, self.work = [], []

    @staticmethod
    def merge(ranges):
        out = []
        for a, b in sorted((int(a), int(b)) for a, b in ranges if b > a):
            if out and a <= out[-1][1]:
                out[-1][1] = max(out[-1][1], b)
            else:
                out.append([a, b])
        return [(a, b) for a, b in out]

    def send(self, ranges):
        for a, b in self.merge(ranges):
            self.work.append(dist.all_reduce(self.flat[a:b], async_op=True))
            self.sent.append((a, b))

    def finish(self):
        rest, at = [], 0
        for a, b in self.merge(self.sent):
            if a > at:
                rest.append((at, a))
            at = max(at, b)
        if at < self.flat.numel():
            rest.append((at, self.flat.numel()))
        self.send(rest)
        for w in self.work:
            w.wait()
        self.sent, self.work = [], []
