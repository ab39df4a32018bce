"""Seeded synthetic crystal batches.

The public materials datasets the reference trains on (JARVIS-DFT, Materials Project,
OQMD) are not redistributable with this package, so benchmarks and tests draw batches
with the same fields and shapes as the reference's collated ``Data`` object
(``x, pos, batch, trans_vec, sizes``; dataloaders/dataset_latticeformer.py:11-38 of the
reference) from simple distributions:

* atom counts: ``uniform`` in [lo, hi] or ``lognormal`` (median, sigma) clipped to [lo, hi];
* cell lengths uniform in [len_lo, len_hi] angstrom, cell angles uniform in [60, 120] degrees,
  re-drawn until the cell is well conditioned;
* fractional coordinates uniform in [0, 1); atomic numbers uniform in 1..94, one-hot over
  98 species (models/latticeformer.py:112 of the reference).
"""
import dataclasses
import math

import numpy as np


@dataclasses.dataclass
class CrystalBatch:
    x: np.ndarray          # (N, 98) float32 one-hot species
    pos: np.ndarray        # (N, 3) float32 cartesian positions
    batch: np.ndarray      # (N,) int64 crystal index of each atom
    trans_vec: np.ndarray  # (B, 3, 3) float32 lattice vectors as rows
    sizes: np.ndarray      # (B,) int64 atoms per crystal
    z: np.ndarray          # (N,) int64 atomic numbers

    @property
    def num_atoms(self):
        return int(self.sizes.sum())

    @property
    def num_pairs(self):
        return int((self.sizes * self.sizes).sum())


def _cell(rng, len_lo, len_hi):
    a, b, c = rng.uniform(len_lo, len_hi, 3)
    while True:
        al, be, ga = np.deg2rad(rng.uniform(60.0, 120.0, 3))
        ca, cb, cg = math.cos(al), math.cos(be), math.cos(ga)
        vol2 = 1.0 - ca * ca - cb * cb - cg * cg + 2.0 * ca * cb * cg
        if vol2 > 0.05:
            break
    sg = math.sin(ga)
    va = [a, 0.0, 0.0]
    vb = [b * cg, b * sg, 0.0]
    cx = c * cb
    cy = c * (ca - cb * cg) / sg
    cz = c * math.sqrt(vol2) / sg
    return np.array([va, vb, [cx, cy, cz]], dtype=np.float64)


def make_batch(num_crystals, seed, size_dist="lognormal", size_lo=1, size_hi=64, size_median=8.0,
               size_sigma=0.75, len_lo=3.0, len_hi=15.0):
    rng = np.random.default_rng(seed)
    if size_dist == "lognormal":
        s = np.rint(rng.lognormal(math.log(size_median), size_sigma, num_crystals))
        sizes = np.clip(s, size_lo, size_hi).astype(np.int64)
    elif size_dist == "uniform":
        sizes = rng.integers(size_lo, size_hi + 1, num_crystals).astype(np.int64)
    else:
        raise ValueError(size_dist)
    cells = np.stack([_cell(rng, len_lo, len_hi) for _ in range(num_crystals)])
    N = int(sizes.sum())
    frac = rng.uniform(0.0, 1.0, (N, 3))
    batch = np.repeat(np.arange(num_crystals, dtype=np.int64), sizes)
    pos = np.einsum("nd,nde->ne", frac, cells[batch])
    z = rng.integers(1, 95, N).astype(np.int64)
    x = np.zeros((N, 98), np.float32)
    x[np.arange(N), z - 1] = 1.0
    return CrystalBatch(x=x, pos=pos.astype(np.float32), batch=batch, trans_vec=cells.astype(np.float32),
                        sizes=sizes, z=z)


# The five workloads the benchmarks and parity tests are quoted on.
WORKLOADS = {
    "cfg1": dict(num_crystals=8, seed=0, size_dist="uniform", size_lo=4, size_hi=16, len_lo=3.0, len_hi=10.0),
    "cfg2": dict(num_crystals=256, seed=1, size_dist="lognormal", size_lo=1, size_hi=64, len_lo=3.0, len_hi=15.0),
    "cfg3": dict(num_crystals=256, seed=2, size_dist="lognormal", size_lo=1, size_hi=64, len_lo=3.0, len_hi=15.0),
    "cfg4": dict(num_crystals=64, seed=3, size_dist="uniform", size_lo=100, size_hi=200, len_lo=10.0, len_hi=25.0),
    "cfg5": dict(num_crystals=256, seed=4, size_dist="lognormal", size_lo=1, size_hi=64, len_lo=3.0, len_hi=15.0),
}


def make_workload(name, seed=None, num_crystals=None):
    kw = dict(WORKLOADS[name])
    if seed is not None:
        kw["seed"] = seed
    if num_crystals is not None:
        kw["num_crystals"] = num_crystals
    return make_batch(**kw)


def select(b: CrystalBatch, crystal_idx) -> CrystalBatch:
    """Sub-batch made of the given crystals (in the given order)."""
    crystal_idx = np.asarray(crystal_idx, dtype=np.int64)
    start = np.concatenate([[0], np.cumsum(b.sizes)])
    atoms = np.concatenate([np.arange(start[c], start[c + 1]) for c in crystal_idx]) if len(crystal_idx) else np.zeros(0, np.int64)
    sizes = b.sizes[crystal_idx]
    return CrystalBatch(x=b.x[atoms], pos=b.pos[atoms], batch=np.repeat(np.arange(len(sizes), dtype=np.int64), sizes),
                        trans_vec=b.trans_vec[crystal_idx], sizes=sizes, z=b.z[atoms])


def concat(batches) -> CrystalBatch:
    """One batch holding the crystals of several, in order."""
    sizes = np.concatenate([b.sizes for b in batches])
    return CrystalBatch(x=np.concatenate([b.x for b in batches]), pos=np.concatenate([b.pos for b in batches]),
                        batch=np.repeat(np.arange(len(sizes), dtype=np.int64), sizes),
                        trans_vec=np.concatenate([b.trans_vec for b in batches]), sizes=sizes,
                        z=np.concatenate([b.z for b in batches]))
