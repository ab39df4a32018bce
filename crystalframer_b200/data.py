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

