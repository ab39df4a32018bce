"""Host <-> device staging of crystal batches."""
import dataclasses

import numpy as np
import torch

from .synth import CrystalBatch


@dataclasses.dataclass
class TensorBatch:
    """The fields the model reads (x, pos, batch, trans_vec, sizes) as torch tensors, plus the
    pair count, which lets the pair-list kernel run without reading ``sizes`` back."""
    x: torch.Tensor
    pos: torch.Tensor
    batch: torch.Tensor
    trans_vec: torch.Tensor
    sizes: torch.Tensor
    y: torch.Tensor
    num_pairs: int

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.x, self.pos, self.batch, self.trans_vec, self.sizes, self.y))

    def to(self, device, non_blocking=True):
        return TensorBatch(*(t.to(device, non_blocking=non_blocking) for t in
                             (self.x, self.pos, self.batch, self.trans_vec, self.sizes, self.y)), self.num_pairs)


def host_batch(b: CrystalBatch, targets: np.ndarray, pinned=True) -> TensorBatch:
    ts = [torch.from_numpy(np.ascontiguousarray(a)) for a in (b.x, b.pos, b.batch, b.trans_vec, b.sizes, targets)]
    if pinned and torch.cuda.is_available():
        ts = [t.pin_memory() for t in ts]
    return TensorBatch(*ts, b.num_pairs)



# ---------------------------------------------------------------------------------------------
# Epoch pipeline: an in-memory structure set, per-rank batches collated on the fly by a background
# thread into pinned double buffers, copied to the device on a copy stream one step ahead.
# Stands where the reference has a PyG InMemoryDataset behind a torch DataLoader with the collate of
# dataloaders/dataset_latticeformer.py:11-38 (x, pos, batch, trans_vec, sizes per batch).
# ---------------------------------------------------------------------------------------------
@dataclasses.dataclass
class StructureSet:
    """Crystals in flat form: per structure its size, cell and target, per atom position and atomic number."""
    sizes: np.ndarray      # (M,) int64
    start: np.ndarray      # (M+1,) int64 first atom of each structure
    cells: np.ndarray      # (M,3,3) float32
    pos: np.ndarray        # (sum sizes, 3) float32
    z: np.ndarray          # (sum sizes,) int64 atomic numbers 1..98
    y: np.ndarray          # (M,1) float32 targets
    cost: np.ndarray       # (M,) float64 estimated attention cost (parallel.attention_cost)

    def __len__(self):
        return len(self.sizes)

    @classmethod
    def from_batches(cls, batches, targets):
        from .parallel import attention_cost
        sizes = np.concatenate([b.sizes for b in batches]).astype(np.int64)
        cells = np.concatenate([b.trans_vec for b in batches]).astype(np.float32)
        return cls(sizes=sizes, start=np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64), cells=cells,
                   pos=np.concatenate([b.pos for b in batches]).astype(np.float32),
                   z=np.concatenate([b.z for b in batches]).astype(np.int64),
                   y=np.concatenate(targets).astype(np.float32), cost=attention_cost(sizes, cells))

    @classmethod
    def synthetic(cls, num_structures, seed, workload="cfg3", chunk=4096):
        """``num_structures`` crystals of a synthetic workload's distribution with N(0,1) targets, drawn in chunks."""
        from . import synth
        batches, targets, done, i = [], [], 0, 0
        while done < num_structures:
            n = min(chunk, num_structures - done)
            batches.append(synth.make_workload(workload, seed=seed * 100003 + i, num_crystals=n))
            targets.append(np.random.default_rng(seed * 100003 + i).normal(size=(n, 1)).astype(np.float32))
            done += n
            i += 1
        return cls.from_batches(batches, targets)

    def atoms_of(self, idx):
        """Flat atom indices of the structures ``idx``, in order (vectorised ragged gather)."""
        idx = np.asarray(idx, dtype=np.int64)
        sizes = self.sizes[idx]
        total = int(sizes.sum())
        first = np.repeat(self.start[idx] - np.concatenate([[0], np.cumsum(sizes)[:-1]]), sizes)
        return first + np.arange(total, dtype=np.int64), sizes

    def collate(self, idx) -> CrystalBatch:
        """The batch made of structures ``idx`` with the fields of the reference's collated Data object."""
        atoms, sizes = self.atoms_of(idx)
        z = self.z[atoms]
        x = np.zeros((len(atoms), 98), np.float32)
        x[np.arange(len(atoms)), z - 1] = 1.0
        return CrystalBatch(x=x, pos=self.pos[atoms], batch=np.repeat(np.arange(len(sizes), dtype=np.int64), sizes),
                            trans_vec=self.cells[np.asarray(idx, dtype=np.int64)], sizes=sizes, z=z)


def epoch_schedule(num_structures, global_batch, epoch, seed):
    """Structure indices of every step of an epoch: a seeded permutation (the same on every rank) cut into
    global batches; the incomplete last batch is dropped."""
    perm = np.random.default_rng([seed, epoch]).permutation(num_structures)
    steps = num_structures // global_batch
    return perm[:steps * global_batch].reshape(steps, global_batch)


def rank_share(dataset, global_idx, rank, world):
    """This rank's structures of one global batch: dealt by estimated attention cost, most expensive first
    (the reference's rule for spreading a batch over devices, models/latticeformer.py:224-233, there by pair
    count), returned in ascending dataset order."""
    if world == 1:
        return np.asarray(global_idx, dtype=np.int64)
    from .parallel import deal_by_cost
    global_idx = np.asarray(global_idx, dtype=np.int64)
    return np.sort(global_idx[deal_by_cost(dataset.cost[global_idx], world) == rank])


class _Slot:
    """Pinned staging buffers of one in-flight batch."""

    def __init__(self, max_atoms, max_structures, pinned):
        mk = (lambda *s, dtype: torch.empty(*s, dtype=dtype).pin_memory()) if pinned else \
            (lambda *s, dtype: torch.empty(*s, dtype=dtype))
        self.pos = mk(max_atoms, 3, dtype=torch.float32)
        self.z = mk(max_atoms, dtype=torch.int64)
        self.batch = mk(max_atoms, dtype=torch.int64)
        self.cells = mk(max_structures, 3, 3, dtype=torch.float32)
        self.sizes = mk(max_structures, dtype=torch.int64)
        self.y = mk(max_structures, 1, dtype=torch.float32)
        self.copied = None                  # event: the last host-to-device copies out of this slot have finished


class EpochLoader:
    """Iterates over one rank's batches of an epoch as device-resident ``TensorBatch`` objects.

    A background thread collates step s+1 (ragged gather out of the structure set into pinned staging buffers)
    and enqueues its host-to-device copies on a copy stream while the caller's stream computes step s; ``depth``
    batches may be in flight.  The species one-hot ``x`` (N,98) is built on the device from the atomic numbers, so
    a step moves about 36 bytes per atom over PCIe instead of 428.  On the consumer side ``__next__`` makes the
    current stream wait for the batch's copy event; nothing blocks the host.  With ``device`` a CPU device the
    same schedule runs without streams or pinning (tests)."""

    def __init__(self, dataset, batch_per_rank, rank=0, world=1, device="cpu", epoch=0, seed=0, depth=2, max_steps=None):
        self.ds, self.rank, self.world = dataset, rank, world
        self.device = torch.device(device)
        self.schedule = epoch_schedule(len(dataset), batch_per_rank * world, epoch, seed)
        if max_steps is not None:
            self.schedule = self.schedule[:max_steps]
        self.depth = depth
        self.cuda = self.device.type == "cuda"
        biggest = int(np.sort(dataset.sizes)[::-1][:batch_per_rank * world].sum()) if len(dataset) else 0
        self.max_atoms, self.max_structures = biggest, batch_per_rank * world
        self.h2d_bytes = 0

    def __len__(self):
        return len(self.schedule)

    def _stage(self, slot, idx):
        ds = self.ds
        atoms, sizes = ds.atoms_of(idx)
        n, b = len(atoms), len(idx)
        np.take(ds.pos, atoms, axis=0, out=slot.pos.numpy()[:n])
        np.take(ds.z, atoms, out=slot.z.numpy()[:n])
        slot.batch.numpy()[:n] = np.repeat(np.arange(b, dtype=np.int64), sizes)
        np.take(ds.cells, idx, axis=0, out=slot.cells.numpy()[:b])
        slot.sizes.numpy()[:b] = sizes
        np.take(ds.y, idx, axis=0, out=slot.y.numpy()[:b])
        return n, b, int((sizes * sizes).sum())

    def _to_device(self, slot, n, b, num_pairs):
        dev = self.device
        pos, z, batch = (t[:n].to(dev, non_blocking=True) for t in (slot.pos, slot.z, slot.batch))
        cells, sizes, y = (t[:b].to(dev, non_blocking=True) for t in (slot.cells, slot.sizes, slot.y))
        x = torch.zeros((n, 98), dtype=torch.float32, device=dev)
        x.scatter_(1, (z - 1)[:, None], 1.0)
        self.h2d_bytes += sum(t.numel() * t.element_size() for t in (pos, z, batch, cells, sizes, y))
        return TensorBatch(x, pos, batch, cells, sizes, y, num_pairs)

    def __iter__(self):
        if not self.cuda:
            slot = _Slot(self.max_atoms, self.max_structures, pinned=False)
            for g in self.schedule:
                n, b, pairs = self._stage(slot, rank_share(self.ds, g, self.rank, self.world))
                tb = self._to_device(slot, n, b, pairs)
                yield TensorBatch(*(t.clone() for t in (tb.x, tb.pos, tb.batch, tb.trans_vec, tb.sizes, tb.y)), pairs)
            return
        import queue
        import threading
        ready = queue.Queue(maxsize=self.depth)
        stop = threading.Event()
        copy_stream = torch.cuda.Stream(self.device)
        # one more slot than batches in flight: a slot is refilled only after its copies have finished
        slots = [_Slot(self.max_atoms, self.max_structures, pinned=True) for _ in range(self.depth + 1)]

        def produce():
            try:
                torch.cuda.set_device(self.device)
                for s, g in enumerate(self.schedule):
                    if stop.is_set():
                        return
                    slot = slots[s % len(slots)]
                    if slot.copied is not None:
                        slot.copied.synchronize()
                    n, b, pairs = self._stage(slot, rank_share(self.ds, g, self.rank, self.world))
                    with torch.cuda.stream(copy_stream):
                        tb = self._to_device(slot, n, b, pairs)
                        slot.copied = torch.cuda.Event()
                        slot.copied.record(copy_stream)
                    while not stop.is_set():
                        try:
                            ready.put((tb, slot.copied), timeout=0.1)
                            break
                        except queue.Full:
                            pass
                ready.put(None)
            except BaseException as exc:          # hand the failure to the consumer instead of dying silently
                ready.put(exc)

        worker = threading.Thread(target=produce, daemon=True)
        worker.start()
        try:
            while True:
                item = ready.get()
                if item is None:
                    return
                if isinstance(item, BaseException):
                    raise item
                tb, copied = item
                cur = torch.cuda.current_stream(self.device)
                cur.wait_event(copied)
                for t in (tb.x, tb.pos, tb.batch, tb.trans_vec, tb.sizes, tb.y):
                    t.record_stream(cur)          # allocated on the copy stream, used on the caller's
                yield tb
        finally:
            stop.set()
            worker.join(timeout=10)
