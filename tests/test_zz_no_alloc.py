"""cfb200_framed_proj_bwd_noalloc against cfb200_framed_proj_bwd, through the C ABI.

The no-allocation entry point exists for hosts that cannot pass scratch memory (a plugin that
only ever receives its input and output buffers, a service that may not allocate on the device
after start-up); its scratch is a fixed array inside the library, shared by all calls.  The test
makes two calls in a row on different problems -- the second smaller, so anything that wrongly
depended on what the first left in the array would show -- and requires the same results as the
regular entry point with a caller-provided workspace.  This file sorts last on purpose: a run
that stops at the first failure has then already executed every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import make_problem

pytestmark = pytest.mark.gpu


def _run_both(P, dev):
    from crystalframer_b200 import _lib
    from crystalframer_b200 import cuda_funcs as F
    from oracle import oracle as O
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, 0.0)
    geo, b = P["geo"], P["batch"]
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    fr = O.max_frames(P["cfg"], P["q"] / 4.0, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                      geo["edges"], geo["e_start"])
    a, pos, tv, rv = t(P["a"]), t(geo["pos_ij"]), t(b.trans_vec), t(geo["rvlen"])
    batch, edges, e_start = t(geo["batch"]), t(geo["edges"]), t(geo["e_start"])
    Wd, Wa = t(P["W_d"]), [t(P["W_a"][x]) for x in range(3)]
    f = [t(fr[n]) for n in ("frame1", "frame2", "frame3")]
    N, E = a.shape[0], edges.shape[1]
    z = torch.empty((E, 8), device=dev)
    val = torch.empty((E, 8, 16), device=dev)
    p, ip = _lib.ptr, _lib.iptr
    _lib.invoke("cfb200_framed_proj_fwd", 1, dev, p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), N, E, 14.0, -3.5,
                p(Wd), p(Wa[0]), p(Wa[1]), p(Wa[2]), p(f[0]), p(f[1]), p(f[2]), p(z), p(val))
    rng = np.random.default_rng(E)
    gz, gv = t(rng.normal(size=(E, 8)).astype(np.float32)), t(rng.normal(size=(E, 8, 16)).astype(np.float32))

    def outputs():
        return [torch.full((N, 8), float("nan"), device=dev)] + [torch.full((8, 16, 64), float("nan"), device=dev) for _ in range(4)]

    common = (p(a), p(pos), p(tv), p(rv), ip(batch), ip(edges), ip(e_start), N, E, 14.0, -3.5, p(Wd), p(Wa[0]),
              p(Wa[1]), p(Wa[2]), p(f[0]), p(f[1]), p(f[2]), p(z), p(gz), p(gv))
    ref = outputs()
    nbytes = _lib.lib().cfb200_framed_proj_bwd_workspace_bytes(N, E)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _lib.invoke("cfb200_framed_proj_bwd", 3, dev, *common, *[p(o) for o in ref], ws.data_ptr(), nbytes)
    got = outputs()
    _lib.invoke("cfb200_framed_proj_bwd_noalloc", 3, dev, *common, *[p(o) for o in got])
    torch.cuda.synchronize()
    return ref, got


def test_no_alloc_backward_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    for workload, nc in (("cfg2", 24), ("cfg1", None)):
        ref, got = _run_both(make_problem(workload, num_crystals=nc), dev)
        for name, r, g in zip(("ga", "gW_dist", "gW_ang1", "gW_ang2", "gW_ang3"), ref, got):
            r, g = r.cpu().numpy(), g.cpu().numpy()
            assert np.isfinite(g).all(), name
            assert np.all(np.abs(g - r) <= 1e-5 + 1e-4 * np.abs(r)), f"{name}: max abs diff {np.abs(g - r).max():.3e}"


def test_no_alloc_refuses_oversized_problems():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from crystalframer_b200 import _lib
    from crystalframer_b200 import cuda_funcs as F
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, 0.0)
    L = _lib.lib()
    E = 2_000_000                                     # scratch need far beyond the fixed array
    assert L.cfb200_framed_proj_bwd_workspace_bytes(1000, E) > 16 * 1024 * 1024
    rc = L.cfb200_framed_proj_bwd_noalloc(*([None] * 7), 1000, E, 14.0, -3.5, *([None] * 15), None)
    assert rc == -7 and b"scratch" in L.cfb200_error_string(rc)
