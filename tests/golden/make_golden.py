"""Generates the golden fixtures in this directory.  Run where the reference tree is mounted:

    python tests/golden/make_golden.py [reference_root]

The reference has no tests or golden vectors of its own for this path, so its code is executed
here on small seeded inputs and the inputs and outputs are committed:

* ``ref_kernels_small.npz`` -- the reference's CUDA kernel sources compiled for the CPU
  (oracle/_ref, built by oracle/ref_shim/gen_ref.py) driven with the reference's host logic:
  max frames, static max frames, lattice frames, lattice-sum bias z, value encoding, their gradients,
  ragged attention forward and backward, mean pooling.  Crystals: 1 atom, 3 atoms in a small cell (lattice range 3 and 4 occur),
  5 atoms, 2 atoms in a large cell.
* ``ref_pure_small.npz`` -- the reference's pure-PyTorch twin
  (models/indexed_lattice_multi_head_attention.py: LogSumExpXYFunc, AverageGaussiansBySoftmaxXYFunc_,
  _scaled_dot_product_attention; models/indexed_latticeformer_encoder.py: compute_lattice_distances)
  imported with stub modules for its missing GPU-only dependencies: fixed lattice range 2,
  un-windowed distance Gaussians, no frames.
* ``ref_reci_small.npz`` -- the reciprocal-space encoding: reciprocal vectors, volumes and phase bases from the
  reference's compute_lattice_distances_for_cuda, z / sumexp / ga from its reci_enc kernels (CPU build), and z and
  the gradient of the lattice sum from its pure-PyTorch twin (compute_reci_domain_attn with cos_kr, k2 from
  compute_lattice_distances).
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as O                     # noqa: E402
from oracle import reference as R                  # noqa: E402


def small_problem():
    rng = np.random.default_rng(20240607)
    sizes = np.array([1, 3, 5, 2], np.int64)
    cells = np.array([
        [[4.1, 0.0, 0.0], [0.3, 3.7, 0.0], [-0.5, 0.4, 5.2]],
        [[2.6, 0.0, 0.0], [0.9, 2.4, 0.0], [0.2, -0.6, 2.9]],          # small cell: ranges above 2
        [[6.5, 0.0, 0.0], [-1.8, 7.1, 0.0], [0.7, 1.1, 8.3]],
        [[14.0, 0.0, 0.0], [2.0, 12.5, 0.0], [-3.0, 1.0, 16.0]],
    ], np.float32)
    N = int(sizes.sum())
    batch = np.repeat(np.arange(len(sizes)), sizes)
    frac = rng.uniform(0, 1, (N, 3))
    pos = np.einsum("nd,nde->ne", frac, cells[batch].astype(np.float64)).astype(np.float32)
    H, hd = 8, 16
    q = rng.normal(size=(N, H, hd)).astype(np.float32)
    k = rng.normal(size=(N, H, hd)).astype(np.float32)
    v = rng.normal(size=(N, H, hd)).astype(np.float32)
    a = (-(0.5 + 1.2 * rng.uniform(size=(N, H))) * 0.255).astype(np.float32)
    bound = (64 ** -0.5) * np.sqrt(6.0 / (64 + H * hd))
    W_d = rng.uniform(-bound, bound, size=(H, hd, 64)).astype(np.float32)
    W_a = rng.uniform(-bound, bound, size=(3, H, hd, 64)).astype(np.float32)
    return dict(sizes=sizes, cells=cells, pos=pos, q=q, k=k, v=v, a=a, W_d=W_d, W_a=W_a)


def kernels_fixture(path):
    P = small_problem()
    g = O.lattice_geometry(P["pos"], P["cells"], P["sizes"])
    rk = R.RefKernels("cpu")
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    a, q, k, v = T(P["a"]), T(P["q"] / 4.0), T(P["k"]), T(P["v"])
    r, tv, b, e, rv = T(g["pos_ij"]), T(P["cells"]), T(g["batch"]), T(g["edges"]), T(g["rvlen"])
    f1, sel1 = rk.frame1(q, k, a, r, tv, b, e, rv, -3.5)
    f2m, sel2 = rk.frame2(q, k, a, r, tv, b, e, rv, -3.5, f1)
    f2, f3 = rk.complete(f1, f2m)
    frames = torch.stack([f1, f2, f3]).contiguous()
    asig = R.angle_sigma(4.0, 64)
    Wd, Wa = T(P["W_d"])[None].contiguous(), T(P["W_a"])[:, None].contiguous()
    z, val = rk.framed_proj_fwd(a, r, tv, b, e, 14.0, 1.0, Wd, Wa, frames, asig, 1.0, 1.0, rv, -3.5)
    rng = np.random.default_rng(5)
    gz = T(rng.normal(size=tuple(z.shape)).astype(np.float32))
    gv = T(rng.normal(size=tuple(val.shape)).astype(np.float32))
    ga, gWd, gWa = rk.framed_proj_bwd(a, r, tv, b, e, 14.0, 1.0, Wd, Wa, frames, asig, 1.0, 1.0, rv, -3.5, z, gz, gv)
    out, prob, es = rk.dpa_fwd(q, k, v, z, val, e)
    go = T(rng.normal(size=tuple(out.shape)).astype(np.float32))
    gq, gk, gvv, gaij, gbij = rk.dpa_bwd(q, k, v, z, val, b, e, es, prob, out, go)
    x = T(rng.normal(size=(a.shape[0], 32)).astype(np.float32))
    mean = rk.mean_fwd(x, T(P["sizes"]))
    # frame methods "max_static" and "lattice"
    fs1, ssel1 = rk.frame1_static(a, r, tv, b, e, rv, -3.5)
    fs2m, ssel2 = rk.frame2_static(a, r, tv, b, e, rv, -3.5, fs1)
    lat = rk.lattice_frames(a, r, tv, b, e, rv, -3.5)
    R_eh = O.lattice_range(O.Config(), P["a"], g["rvlen"], g["batch"])
    np.savez_compressed(
        path, **{k_: v_ for k_, v_ in P.items()}, edges=g["edges"], e_start=g["e_start"], R_ah=R_eh,
        frame1=f1.numpy(), frame2_max=f2m.numpy(), frame2=f2.numpy(), frame3=f3.numpy(), sel_edge1=sel1.numpy(),
        sel_edge2=sel2.numpy(), z=z.numpy(), values=val.numpy(), gz=gz.numpy(), gv=gv.numpy(), ga=ga.numpy(),
        gW_d=gWd.numpy(), gW_a=gWa.numpy(), dpa_out=out.numpy(), dpa_prob=prob.numpy(), go=go.numpy(), gq=gq.numpy(),
        gk=gk.numpy(), gvv=gvv.numpy(), gaij=gaij.numpy(), gbij=gbij.numpy(), mean_x=x.numpy(), mean=mean.numpy(),
        static_frame1=fs1.numpy(), static_frame2_max=fs2m.numpy(), static_sel_edge1=ssel1.numpy(),
        static_sel_edge2=ssel2.numpy(), lattice_frame1=lat[0].numpy(), lattice_frame2=lat[1].numpy(),
        lattice_frame3=lat[2].numpy())


def _import_reference_models(ref_root):
    for name in ("torch_scatter", "cupy", "pytorch_pfn_extras"):
        sys.modules.setdefault(name, types.ModuleType(name))
    cr = types.ModuleType("cupy.random")
    cr.XORWOW = object
    sys.modules["cupy.random"] = cr
    sys.modules["cupy"].random = cr
    sys.path.insert(0, ref_root)
    cwd = os.getcwd()
    os.chdir(ref_root)
    try:
        from models import indexed_lattice_multi_head_attention as pure
        from models import indexed_latticeformer_encoder as enc
    finally:
        os.chdir(cwd)
    return pure, enc


def reci_fixture(path, ref_root):
    pure, enc = _import_reference_models(ref_root)
    P = small_problem()
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    sizes = T(P["sizes"])
    batch = torch.repeat_interleave(torch.arange(len(sizes)), sizes)
    pos, cells = T(P["pos"]), T(P["cells"])
    _, _, kr, rvecs, vcell, edges = enc.compute_lattice_distances_for_cuda(pos, batch, cells, sizes, 2, -3.5, True, True)
    a = T(P["a"] * 8.0)                    # the reci domain's coefficients are -0.5 scale_reci^2 f: larger than real-space ones
    rk = R.RefKernels("cpu")
    z, sumexp = rk.reci_fwd(a, kr, rvecs, vcell, batch, edges)
    rng = np.random.default_rng(11)
    gz = T(rng.normal(size=tuple(z.shape)).astype(np.float32))
    ga = rk.reci_bwd(a, kr, rvecs, vcell, batch, edges, z, gz, sumexp)
    _, cos_kr, k2, vcell_p, _, edges_p, _ = enc.compute_lattice_distances(pos, batch, cells, sizes, 2, output_dis=False,
                                                                          output_rec=True)
    assert torch.equal(edges_p, edges)
    ap = a.clone().requires_grad_(True)
    z_pure = pure.compute_reci_domain_attn(ap, cos_kr, k2, vcell_p, edges[0], batch)
    (z_pure * gz).sum().backward()
    # the kernels leave out the gradient of the normaliser 1.5 log(-4 pi a), which is 1.5 / a per pair
    gsum = torch.zeros_like(a).index_add_(0, edges[0], gz)
    ga_pure = ap.grad - 1.5 / a * gsum
    np.savez_compressed(path, a=a.numpy(), kr=kr.numpy(), rvecs=rvecs.numpy(), vcell=vcell.numpy(), edges=edges.numpy(),
                        z=z.numpy(), sumexp=sumexp.numpy(), gz=gz.numpy(), ga=ga.numpy(), z_pure=z_pure.detach().numpy(),
                        ga_pure=ga_pure.numpy())


def pure_fixture(path, ref_root):
    pure, enc = _import_reference_models(ref_root)
    P = small_problem()
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    sizes = T(P["sizes"])
    batch = torch.repeat_interleave(torch.arange(len(sizes)), sizes)
    dist, _, _, _, _, edges, _ = enc.compute_lattice_distances(T(P["pos"]), batch, T(P["cells"]), sizes, 2)
    dist2 = dist * dist                                                        # (E, 125)
    a = T(P["a"])
    z = pure.LogSumExpXYFunc.apply(dist2[:, None, :], a[:, :, None][edges[0]], -1)            # (E,H)
    Wd = T(P["W_d"])[None]
    vals = pure.AverageGaussiansBySoftmaxXYFunc_.apply(14.0, 64, dist2[:, None, :, None],
                                                       a[:, :, None, None][edges[0]], -2, Wd, 1.0)
    out, attn, _ = pure._scaled_dot_product_attention(T(P["q"]), T(P["k"]), T(P["v"]), batch, batch, edges, z, vals, 0.0)
    np.savez_compressed(path, z=z.numpy(), values=vals.numpy(), out=out.numpy(), prob=attn.numpy(), edges=edges.numpy())


if __name__ == "__main__":
    from oracle import build_oracle
    ref_root = sys.argv[1] if len(sys.argv) > 1 else build_oracle.reference_root()
    if ref_root is None:
        raise SystemExit("reference tree not found: pass its root or set CF_REFERENCE_ROOT")
    kernels_fixture(os.path.join(HERE, "ref_kernels_small.npz"))
    pure_fixture(os.path.join(HERE, "ref_pure_small.npz"), ref_root)
    reci_fixture(os.path.join(HERE, "ref_reci_small.npz"), ref_root)
    print("fixtures written")
