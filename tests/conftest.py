import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def make_problem(workload="cfg1", num_crystals=None, seed=None, noise=0.0, H=8, hd=16):
    """Seeded inputs of the attention path for one synthetic batch: geometry from the oracle's
    restatement of the reference host code, q/k/v ~ N(0,1), Gaussian coefficients from the real
    coefficient pipeline (elu form) with per-batch normalisation, projection weights with the
    module's initialisation bounds."""
    from crystalframer_b200 import synth
    from oracle import oracle as O
    b = synth.make_workload(workload, seed=seed, num_crystals=num_crystals)
    geo = O.lattice_geometry(b.pos, b.trans_vec, b.sizes)
    rng = np.random.default_rng(1234 + (seed or 0))
    N = b.num_atoms
    q = rng.normal(size=(N, H, hd)).astype(np.float32)
    k = rng.normal(size=(N, H, hd)).astype(np.float32)
    v = rng.normal(size=(N, H, hd)).astype(np.float32)
    w = rng.normal(0, hd ** -0.5, size=(H, hd)).astype(np.float32)
    alpha = np.einsum("nhd,hd->nh", q, w)
    alpha = (alpha - alpha.mean()) / alpha.std()
    x = alpha * (0.1 / 0.5)
    pos = 0.5 * np.where(x > 0, x, np.expm1(np.minimum(x, 0))) + 1.0
    a = (pos * (-0.5 * 1.4 ** -2)).astype(np.float32)
    bound = (64 ** -0.5) * np.sqrt(6.0 / (64 + H * hd))
    W_d = rng.uniform(-bound, bound, size=(H, hd, 64)).astype(np.float32)
    W_a = rng.uniform(-bound, bound, size=(3, H, hd, 64)).astype(np.float32)
    cfg = O.Config(H=H, head_dim=hd, symm_break_noise=noise)
    return dict(batch=b, geo=geo, q=q, k=k, v=v, a=a, W_d=W_d, W_a=W_a, cfg=cfg, rng=rng)


@pytest.fixture(scope="session")
def problem_cfg1():
    return make_problem("cfg1")
