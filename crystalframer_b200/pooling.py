"""Per-crystal pooling of atom features (models/pooling.py:13-24 of the reference)."""
import torch

from .cuda_funcs import IrregularMeanCUDA


def max_pool(x, batch, sizes):
    parts = torch.split_with_sizes(x, sizes.tolist(), 0)
    return torch.stack([p.max(dim=0)[0] for p in parts])


def avr_pool(x, batch, sizes):
    return IrregularMeanCUDA.apply(x, batch, sizes)
