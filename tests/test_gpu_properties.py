"""The CUDA path against the committed golden fixtures, on edge cases, and -- at the full size of
the benchmark workload, where the CPU oracle would take minutes -- through properties that do not
depend on the size: linearity in the projection weights, the adjoint identity between the forward
and the backward kernels, independence of the crystals of a batch, normalisation of the attention.
"""
import os

import numpy as np
import pytest
import torch

from conftest import make_problem

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _configure(noise=0.0):
    from crystalframer_b200 import cuda_funcs as F
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, noise)
    return F


def _t(x, dev):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def _close(name, got, want, rtol=1e-4, atol=1e-5):
    got = np.asarray(got.detach().cpu().numpy() if torch.is_tensor(got) else got, np.float64)
    want = np.asarray(want.detach().cpu().numpy() if torch.is_tensor(want) else want, np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert np.isfinite(got).all(), name
    err = np.abs(got - want)
    bad = err > atol + rtol * np.abs(want)
    assert not bad.any(), f"{name}: {bad.sum()} of {bad.size} outside tolerance, max abs err {err.max():.3e}"


def _device_problem(dev, workload, nc=None, seed=None):
    """Geometry and random operands of one synthetic batch, built on the device by the library's own
    pair-list kernel and the host code of the encoder."""
    from crystalframer_b200 import synth
    from crystalframer_b200.encoder import build_pair_list, compute_lattice_distances_for_cuda
    b = synth.make_workload(workload, seed=seed, num_crystals=nc)
    sizes, pos, tv = _t(b.sizes, dev), _t(b.pos, dev), _t(b.trans_vec, dev)
    edges, e_start, batch, _ = build_pair_list(sizes, (b.num_atoms, b.num_pairs))
    pos_ij, _, _, rvecs, _, edges2 = compute_lattice_distances_for_cuda(pos, batch, tv, sizes, 2, num_pairs=b.num_pairs)
    assert torch.equal(edges, edges2)
    rvlen = torch.norm(rvecs, 2, dim=-1)
    g = torch.Generator(device="cpu").manual_seed(11)
    N, H, hd = b.num_atoms, 8, 16
    q, k, v = (torch.randn(N, H, hd, generator=g).to(dev) for _ in range(3))
    a = (-(0.15 + 0.25 * torch.rand(N, H, generator=g))).to(dev)
    bound = (64 ** -0.5) * (6.0 / (64 + H * hd)) ** 0.5
    W = [((torch.rand(1, H, hd, 64, generator=g) * 2 - 1) * bound).to(dev) for _ in range(4)]
    return dict(b=b, sizes=sizes, tv=tv, edges=edges, e_start=e_start, batch=batch, pos_ij=pos_ij.contiguous(),
                rvlen=rvlen.contiguous(), q=q, k=k, v=v, a=a, W=W, gen=g)


def _encode(F, D, a, W, frames):
    return F.RealEncodingWithFramedProjFuncCUDA.apply(a, D["pos_ij"], None, D["tv"], D["batch"], D["edges"], 64, 14.0, 1.0,
                                                      W[0], W[1], W[2], W[3], *frames, 64, 4.0, 0, 1.0, 1.0, D["rvlen"],
                                                      -3.5)


def test_golden_fixture_of_the_reference_kernels():
    """Inputs and outputs of the reference's own kernels (tests/golden/make_golden.py) through the
    CUDA path: pair list and selections bit-exact, floats within the stated tolerance."""
    dev = _cuda()
    F = _configure()
    from crystalframer_b200.encoder import build_pair_list
    from oracle import oracle as O
    G = np.load(os.path.join(GOLD, "ref_kernels_small.npz"))
    sizes, tv = _t(G["sizes"], dev), _t(G["cells"], dev)
    N, E = G["pos"].shape[0], G["edges"].shape[1]
    edges, e_start, batch, _ = build_pair_list(sizes, (N, E))
    assert np.array_equal(edges.cpu().numpy(), G["edges"]) and np.array_equal(e_start.cpu().numpy(), G["e_start"])
    geo = O.lattice_geometry(G["pos"], G["cells"], G["sizes"])      # the reference's host arithmetic for pos_ij, |b_d|
    pos_ij, rvlen = _t(geo["pos_ij"], dev), _t(geo["rvlen"], dev)
    q, k, v, a = (_t(G[n], dev) for n in ("q", "k", "v", "a"))
    f1, e1, _ = F.max_frame_with_selection(1, q / 4.0, k, a, pos_ij, tv, batch, edges, rvlen, -3.5)
    assert np.array_equal(e1.cpu().numpy(), G["sel_edge1"])
    assert np.array_equal(f1.cpu().numpy(), G["frame1"])
    f2, e2, _ = F.max_frame_with_selection(2, q / 4.0, k, a, pos_ij, tv, batch, edges, rvlen, -3.5, f1)
    assert np.array_equal(e2.cpu().numpy(), G["sel_edge2"])
    _close("frame2_max", f2, G["frame2_max"], 1e-6, 1e-6)
    g1, g2, g3 = F.max_frames_fused(q / 4.0, k, a, pos_ij, tv, batch, edges, rvlen, -3.5)
    _close("frame2", g2, G["frame2"], 1e-5, 1e-6)
    _close("frame3", g3, G["frame3"], 1e-5, 1e-6)
    a_ = a.clone().requires_grad_(True)
    W = [_t(G["W_d"][None], dev).requires_grad_(True)] + [_t(G["W_a"][x][None], dev).requires_grad_(True) for x in range(3)]
    D = dict(pos_ij=pos_ij, tv=tv, batch=batch, edges=edges, rvlen=rvlen)
    z, val = _encode(F, D, a_, W, [_t(G[n], dev) for n in ("frame1", "frame2", "frame3")])
    _close("z", z, G["z"])
    _close("values", val, G["values"])
    # the reference's backward takes the forward's z; feed it the fixture's
    (z * _t(G["gz"], dev)).sum().add((val * _t(G["gv"], dev)).sum()).backward()
    _close("ga", a_.grad, G["ga"], 1e-4, 1e-5 * max(1.0, float(np.abs(G["ga"]).max())))
    _close("gW_d", W[0].grad[0], G["gW_d"])
    for x in range(3):
        _close(f"gW_a{x}", W[1 + x].grad[0], G["gW_a"][x])
    qs = (q / 4.0).requires_grad_(True)
    k_, v_ = k.clone().requires_grad_(True), v.clone().requires_grad_(True)
    zz, vv = _t(G["z"], dev).requires_grad_(True), _t(G["values"], dev).requires_grad_(True)
    out = F.FusedDotProductAttentionCUDA.apply(qs, k_, v_, zz, vv, batch, edges)
    _close("attention", out, G["dpa_out"])
    out.backward(_t(G["go"], dev))
    for n, t in (("gq", qs), ("gk", k_), ("gvv", v_), ("gaij", zz), ("gbij", vv)):
        _close(n, t.grad, G[n])
    m = F.IrregularMeanCUDA.apply(_t(G["mean_x"], dev), batch, sizes)
    _close("mean", m, G["mean"])
    # frame methods "max_static" and "lattice": outputs of the reference's kernels, bit for bit
    s1, se1, _ = F.max_static_frame_with_selection(1, a, pos_ij, tv, batch, edges, rvlen, -3.5)
    assert np.array_equal(se1.cpu().numpy(), G["static_sel_edge1"]) and np.array_equal(s1.cpu().numpy(), G["static_frame1"])
    s2, se2, _ = F.max_static_frame_with_selection(2, a, pos_ij, tv, batch, edges, rvlen, -3.5, s1)
    assert np.array_equal(se2.cpu().numpy(), G["static_sel_edge2"])
    _close("static frame2_max", s2, G["static_frame2_max"], 1e-6, 1e-6)
    lat = F.ComputeLatticeFrameCUDA.apply(q / 4.0, k, None, a, pos_ij, None, tv, batch, edges, 64, 14.0, 1.0, rvlen, -3.5)
    for x in range(3):
        assert np.array_equal(lat[x].cpu().numpy(), G[f"lattice_frame{x + 1}"])


def test_empty_batch_and_single_atoms():
    """No crystals at all, and crystals of one atom (the only pair is the atom with itself: no
    non-zero image inside a large cell's lattice range still yields finite outputs)."""
    dev = _cuda()
    F = _configure()
    from crystalframer_b200 import _lib
    from crystalframer_b200.encoder import build_pair_list
    H, hd = 8, 16
    sizes = torch.zeros(0, dtype=torch.int64, device=dev)
    edges, e_start, batch, _ = build_pair_list(sizes, (0, 0))
    assert edges.shape == (2, 0) and e_start.cpu().tolist() == [0] and batch.numel() == 0
    z0 = torch.zeros(0, H, device=dev)
    W = [torch.zeros(1, H, hd, 64, device=dev, requires_grad=True) for _ in range(4)]
    a0 = torch.zeros(0, H, device=dev, requires_grad=True)
    fr = [torch.zeros(0, H, 3, device=dev)] * 3
    D = dict(pos_ij=torch.zeros(0, 3, device=dev), tv=torch.zeros(0, 3, 3, device=dev), batch=batch, edges=edges,
             rvlen=torch.zeros(0, 3, device=dev))
    z, val = _encode(F, D, a0, W, fr)
    assert z.shape == (0, H) and val.shape == (0, H, hd)
    (z.sum() + val.sum()).backward()
    assert all(float(w.grad.abs().sum()) == 0.0 for w in W)
    out = F.FusedDotProductAttentionCUDA.apply(torch.zeros(0, H, hd, device=dev), torch.zeros(0, H, hd, device=dev),
                                               torch.zeros(0, H, hd, device=dev), z0, torch.zeros(0, H, hd, device=dev),
                                               batch, edges)
    assert out.shape == (0, H, hd)
    # three single-atom crystals
    from crystalframer_b200 import synth
    b = synth.make_batch(3, 5, size_dist="uniform", size_lo=1, size_hi=1)
    sizes = _t(b.sizes, dev)
    edges, e_start, batch, _ = build_pair_list(sizes, (3, 3))
    assert edges.cpu().tolist() == [[0, 1, 2], [0, 1, 2]]
    from oracle import oracle as O
    geo = O.lattice_geometry(b.pos, b.trans_vec, b.sizes)
    Pn = make_problem("cfg1")
    a = -0.2 * np.ones((3, H), np.float32)
    q = Pn["rng"].normal(size=(3, H, hd)).astype(np.float32)
    fr_w = O.max_frames(O.Config(), q, q, a, geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                        geo["e_start"])
    g = F.max_frames_fused(_t(q, dev), _t(q, dev), _t(a, dev), _t(geo["pos_ij"], dev), _t(b.trans_vec, dev), batch,
                           edges, _t(geo["rvlen"], dev), -3.5)
    for got, name in zip(g, ("frame1", "frame2", "frame3")):
        _close(name, got, fr_w[name], 1e-5, 1e-6)
    frames = np.stack([fr_w["frame1"], fr_w["frame2"], fr_w["frame3"]])
    z_w, v_w = O.framed_proj_fwd(O.Config(), a, geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 Pn["W_d"], Pn["W_a"], frames)
    D = dict(pos_ij=_t(geo["pos_ij"], dev), tv=_t(b.trans_vec, dev), batch=batch, edges=edges, rvlen=_t(geo["rvlen"], dev))
    W = [_t(Pn["W_d"][None], dev)] + [_t(Pn["W_a"][x][None], dev) for x in range(3)]
    z, val = _encode(F, D, _t(a, dev), W, [_t(frames[x], dev) for x in range(3)])
    _close("z", z, z_w)
    _close("values", val, v_w)
    assert _lib.read_status() == 0


def test_largest_cell_of_the_reference():
    """One crystal with 320 atoms, the reference's maximum per cell (102 400 pairs in one block of
    the pair list; an atom's pairs span several rounds of every per-atom kernel)."""
    dev = _cuda()
    F = _configure()
    from crystalframer_b200 import synth, _lib
    from crystalframer_b200.encoder import build_pair_list
    from oracle import oracle as O
    b = synth.make_batch(1, 9, size_dist="uniform", size_lo=320, size_hi=320, len_lo=18.0, len_hi=22.0)
    geo = O.lattice_geometry(b.pos, b.trans_vec, b.sizes)
    edges, e_start, batch, _ = build_pair_list(_t(b.sizes, dev), (320, 320 * 320))
    assert np.array_equal(edges.cpu().numpy(), geo["edges"]) and np.array_equal(e_start.cpu().numpy(), geo["e_start"])
    rng = np.random.default_rng(3)
    H, hd = 8, 16
    q, k, v = (rng.normal(size=(320, H, hd)).astype(np.float32) for _ in range(3))
    a = -(0.15 + 0.2 * rng.random((320, H))).astype(np.float32)
    cfg = O.Config()
    fr_w = O.max_frames(cfg, q / 4.0, k, a, geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                        geo["e_start"])
    tv, pos_ij, rvlen = _t(b.trans_vec, dev), _t(geo["pos_ij"], dev), _t(geo["rvlen"], dev)
    f1, e1, _ = F.max_frame_with_selection(1, _t(q / 4.0, dev), _t(k, dev), _t(a, dev), pos_ij, tv, batch, edges, rvlen, -3.5)
    assert np.array_equal(e1.cpu().numpy(), fr_w["sel_edge1"])
    assert np.array_equal(f1.cpu().numpy(), fr_w["frame1"])
    Pn = make_problem("cfg1")
    frames = np.stack([fr_w["frame1"], fr_w["frame2"], fr_w["frame3"]])
    z_w, v_w = O.framed_proj_fwd(cfg, a, geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], Pn["W_d"],
                                 Pn["W_a"], frames)
    D = dict(pos_ij=pos_ij, tv=tv, batch=batch, edges=edges, rvlen=rvlen)
    W = [_t(Pn["W_d"][None], dev)] + [_t(Pn["W_a"][x][None], dev) for x in range(3)]
    z, val = _encode(F, D, _t(a, dev), W, [_t(frames[x], dev) for x in range(3)])
    _close("z", z, z_w)
    _close("values", val, v_w)
    out_w, _ = O.dpa_fwd(cfg, q / 4.0, k, v, z_w, v_w, geo["edges"], geo["e_start"])
    out = F.FusedDotProductAttentionCUDA.apply(_t(q / 4.0, dev), _t(k, dev), _t(v, dev), z, val, batch, edges)
    _close("attention", out, out_w)
    assert _lib.read_status() == 0


def test_status_word_reports_bad_coefficients():
    """A non-negative Gaussian coefficient has no convergent lattice sum; the library reports it in
    the status word instead of trapping."""
    dev = _cuda()
    F = _configure()
    from crystalframer_b200 import _lib
    D = _device_problem(dev, "cfg1")
    _lib.read_status()
    a = D["a"].clone()
    a[0, 0] = 0.5
    fr = [torch.zeros(a.shape[0], 8, 3, device=dev) for _ in range(3)]
    _encode(F, D, a, D["W"], fr)
    st = _lib.read_status()
    assert st & 1, st                   # CFB200_STATUS_BAD_COEF
    _encode(F, D, D["a"], D["W"], fr)
    assert _lib.read_status() == 0      # reading clears the word


def test_status_word_reports_a_pair_list_that_is_not_dense():
    """The kernels read keys and per-pair rows of one atom as consecutive; a pair list whose columns are permuted
    inside an atom's block (still valid indices) is reported, not silently mis-summed."""
    dev = _cuda()
    F = _configure()
    from crystalframer_b200 import _lib
    D = _device_problem(dev, "cfg1")
    N, H = D["a"].shape
    gen = torch.Generator(device="cpu").manual_seed(0)
    q, k, v = (torch.randn(N, H, 16, generator=gen).to(dev) for _ in range(3))
    E = D["edges"].shape[1]
    z, val = torch.zeros(E, H, device=dev), torch.zeros(E, H, 16, device=dev)
    _lib.read_status()
    F.FusedDotProductAttentionCUDA.apply(q, k, v, z, val, D["batch"], D["edges"])
    assert _lib.read_status() == 0
    edges = D["edges"].clone()
    same = (edges[0, 1:] == edges[0, :-1]).nonzero()      # two consecutive pairs of one atom: swap their keys
    e = int(same[0])
    edges[1, e], edges[1, e + 1] = D["edges"][1, e + 1], D["edges"][1, e]
    F.FusedDotProductAttentionCUDA.apply(q, k, v, z, val, D["batch"], edges)
    assert _lib.read_status() & 16                        # CFB200_ST_PAIR_LAYOUT


def test_properties_at_benchmark_size():
    """cfg3 at its full size (256 crystals, about 50 000 pairs, 4*10^5 pair-heads)."""
    dev = _cuda()
    F = _configure()
    D = _device_problem(dev, "cfg3")
    g = D["gen"]
    E, N = D["edges"].shape[1], D["a"].shape[0]
    qs = D["q"] / 4.0
    frames = F.max_frames_fused(qs, D["k"], D["a"], D["pos_ij"], D["tv"], D["batch"], D["edges"], D["rvlen"], -3.5)
    for f in frames:                                       # unit vectors (or zero where no axis exists), orthogonal
        n = f.norm(dim=-1)
        assert bool((((n - 1).abs() < 1e-5) | (n == 0)).all())
    assert float((frames[0] * frames[1]).sum(-1).abs().max()) < 1e-5
    assert float((frames[0] * frames[2]).sum(-1).abs().max()) < 1e-5

    # linearity of the value encoding in the projection weights; z does not depend on them
    W1 = D["W"]
    W2 = [torch.randn(w.shape, generator=g).to(dev) * 0.05 for w in W1]
    z1, v1 = _encode(F, D, D["a"], W1, frames)
    z2, v2 = _encode(F, D, D["a"], W2, frames)
    z3, v3 = _encode(F, D, D["a"], [x + y for x, y in zip(W1, W2)], frames)
    assert torch.equal(z1, z2) and torch.equal(z1, z3)
    _close("values(W1 + W2)", v3, v1 + v2, 1e-4, 1e-5)

    # adjoint identity: <gW, dW> computed by the backward kernel equals <gv, values(dW)> computed by the
    # forward kernel, for a random direction dW
    Wg = [w.clone().requires_grad_(True) for w in W1]
    a_g = D["a"].clone().requires_grad_(True)
    z, v = _encode(F, D, a_g, Wg, frames)
    gv = torch.randn(v.shape, generator=g).to(dev)
    gz = torch.randn(z.shape, generator=g).to(dev)
    ((v * gv).sum() + (z * gz).sum()).backward()
    lhs = sum(float((w.grad.double() * d.double()).sum()) for w, d in zip(Wg, W2))
    rhs = float((gv.double() * v2.double()).sum())
    assert abs(lhs - rhs) <= 1e-4 * max(abs(lhs), abs(rhs)) + 1e-3, (lhs, rhs)

    # directional derivative in the Gaussian coefficient against a central difference of the forward kernel
    da = torch.randn(a_g.shape, generator=g).to(dev) * D["a"].abs()
    eps = 1e-3
    zp, vp = _encode(F, D, D["a"] + eps * da, W1, frames)
    zm, vm = _encode(F, D, D["a"] - eps * da, W1, frames)
    fd = float((((vp.double() - vm.double()) * gv.double()).sum() + ((zp.double() - zm.double()) * gz.double()).sum()) / (2 * eps))
    an = float((a_g.grad.double() * da.double()).sum())
    assert abs(fd - an) <= 2e-2 * max(abs(fd), abs(an)) + 1e-2, (fd, an)

    # crystals of a batch do not interact: the first 100 crystals alone give bit-identical rows
    nc = 100
    n_at = int(D["b"].sizes[:nc].sum())
    n_pr = int((D["b"].sizes[:nc] ** 2).sum())
    sub = dict(pos_ij=D["pos_ij"][:n_pr].contiguous(), tv=D["tv"][:nc].contiguous(), batch=D["batch"][:n_at].contiguous(),
               edges=D["edges"][:, :n_pr].contiguous(), rvlen=D["rvlen"][:nc].contiguous())
    fsub = F.max_frames_fused(qs[:n_at].contiguous(), D["k"][:n_at].contiguous(), D["a"][:n_at].contiguous(), sub["pos_ij"],
                              sub["tv"], sub["batch"], sub["edges"], sub["rvlen"], -3.5)
    for x in range(3):
        assert torch.equal(fsub[x], frames[x][:n_at])
    zs, vs = _encode(F, sub, D["a"][:n_at].contiguous(), W1, fsub)
    assert torch.equal(zs, z1[:n_pr]) and torch.equal(vs, v1[:n_pr])

    # attention rows are convex combinations: v = 1, values = 0 gives exactly-normalised outputs; the
    # gradient of sum(out) with respect to the logits is then zero
    ones = torch.ones_like(D["v"])
    zz = z1.clone().requires_grad_(True)
    out = F.FusedDotProductAttentionCUDA.apply(qs, D["k"], ones, zz, torch.zeros_like(v1), D["batch"], D["edges"])
    _close("rows sum to one", out, torch.ones_like(out), 1e-5, 1e-5)
    out.sum().backward()
    assert float(zz.grad.abs().max()) < 1e-5

    # mean pooling of ones is one; its backward spreads 1/n
    x = torch.ones(N, 32, device=dev, requires_grad=True)
    m = F.IrregularMeanCUDA.apply(x, D["batch"], D["sizes"])
    _close("mean of ones", m, torch.ones_like(m), 0, 1e-6)
    m.sum().backward()
    inv_n = (1.0 / D["sizes"].double())[D["batch"]].float()
    _close("mean backward", x.grad, inv_n[:, None].expand(N, 32), 1e-6, 1e-7)


@pytest.mark.parametrize("noise", [0.0, 1e-5])
def test_pair_cache_changes_no_bit(noise):
    """The per-pair geometry cache only spares work: frames, lattice-sum bias and value encoding come
    out bit-identical with and without it, on a batch that mixes cells at the cached lattice range with
    small cells whose range is larger (those take the uncached search)."""
    dev = _cuda()
    F = _configure(noise)
    from crystalframer_b200 import _lib
    D = _device_problem(dev, "cfg2", nc=48)
    D["tv"][:6] *= 0.45                                    # shrink a few cells: adaptive ranges above the minimum
    D["pos_ij"][: int((D["b"].sizes[:6] ** 2).sum())] *= 0.45
    from crystalframer_b200.encoder import det_3x3
    tv = D["tv"]
    rvecs = torch.stack([torch.linalg.cross(tv[:, 1], tv[:, 2]), torch.linalg.cross(tv[:, 2], tv[:, 0]),
                         torch.linalg.cross(tv[:, 0], tv[:, 1])], 1) * (2.0 * np.pi / det_3x3(tv)[:, None, None])
    rvlen = rvecs.norm(dim=-1).contiguous()
    N, E, H, hd = D["a"].shape[0], D["edges"].shape[1], 8, 16
    p, ip = _lib.ptr, _lib.iptr
    cache = torch.empty(E, 4, device=dev)
    plist = torch.empty(E, 5, 128, device=dev)
    _lib.invoke("cfb200_pair_cache", 2, dev, p(D["pos_ij"]), p(tv), ip(D["batch"]), ip(D["edges"]), N, E, 2, p(cache),
                p(plist))
    qs = (D["q"] / 4.0).contiguous()
    outs = []
    for use in (None, cache):
        f = torch.empty(3, N, H, 3, device=dev)
        _lib.invoke("cfb200_max_frames_cached", 1, dev, p(qs), p(D["k"]), p(D["a"]), p(D["pos_ij"]), p(tv), p(rvlen),
                    ip(D["batch"]), ip(D["edges"]), ip(D["e_start"]), N, E, -3.5, 17, 29, p(f[0]), p(f[1]), p(f[2]),
                    p(use), None, 2)
        z, val = torch.empty(E, H, device=dev), torch.empty(E, H, hd, device=dev)
        W = [w[0].contiguous() for w in D["W"]]
        _lib.invoke("cfb200_framed_proj_fwd_cached", 1, dev, p(D["a"]), p(D["pos_ij"]), p(tv), p(rvlen), ip(D["batch"]),
                    ip(D["edges"]), N, E, 14.0, -3.5, p(W[0]), p(W[1]), p(W[2]), p(W[3]), p(f[0]), p(f[1]), p(f[2]),
                    p(z), p(val), p(use), None, 2)
        outs.append((f, z, val))
    plain = torch.empty(3, N, H, 3, device=dev)
    _lib.invoke("cfb200_max_frames", 1, dev, p(qs), p(D["k"]), p(D["a"]), p(D["pos_ij"]), p(tv), p(rvlen), ip(D["batch"]),
                ip(D["edges"]), ip(D["e_start"]), N, E, -3.5, 17, 29, p(plain[0]), p(plain[1]), p(plain[2]))
    assert torch.equal(outs[0][0], plain)
    for a, b, name in zip(outs[0], outs[1], ("frames", "z", "values")):
        assert torch.equal(a, b), name
    assert bool(torch.isfinite(outs[1][2]).all())

    # sorted translation lists: ascending d^2, consistent vectors, 125 real entries; the lattice sums
    # accumulated nearest-first agree with the index-order sums to a few ulp, forward and backward
    d2l = plist[:, 0]
    assert bool((d2l[:, 1:] >= d2l[:, :-1]).all())
    assert bool((d2l[:, 125:] == 1e30).all()) and bool((d2l[:, :125] < 1e30).all())
    vec2 = (plist[:, 1:4, :125] ** 2).sum(1)
    codes = plist[:, 4, :125].contiguous().view(torch.int32)
    assert bool((codes >> 24 == ((codes & 255) * 5 + ((codes >> 8) & 255)) * 5 + ((codes >> 16) & 255)).all())
    assert bool((codes.sort(dim=1).values >> 24 == torch.arange(125, device=dev, dtype=torch.int32)[None]).all())
    flist = torch.empty(3, N, H, 3, device=dev)
    _lib.invoke("cfb200_max_frames_cached", 1, dev, p(qs), p(D["k"]), p(D["a"]), p(D["pos_ij"]), p(tv), p(rvlen),
                ip(D["batch"]), ip(D["edges"]), ip(D["e_start"]), N, E, -3.5, 17, 29, p(flist[0]), p(flist[1]),
                p(flist[2]), p(cache), p(plist), 2)
    assert torch.equal(flist, outs[0][0]), "frames searched nearest-first differ from the exhaustive search"
    assert float(((vec2 - d2l[:, :125]).abs() / (d2l[:, :125] + 1e-6)).max()) < 1e-5
    assert torch.equal(d2l[:, 0], cache[:, 3])
    f, z0, v0 = outs[0]
    W = [w[0].contiguous() for w in D["W"]]
    z1, v1 = torch.empty(E, H, device=dev), torch.empty(E, H, hd, device=dev)
    _lib.invoke("cfb200_framed_proj_fwd_cached", 1, dev, p(D["a"]), p(D["pos_ij"]), p(tv), p(rvlen), ip(D["batch"]),
                ip(D["edges"]), N, E, 14.0, -3.5, p(W[0]), p(W[1]), p(W[2]), p(W[3]), p(f[0]), p(f[1]), p(f[2]),
                p(z1), p(v1), p(cache), p(plist), 2)
    _close("z with lists", z1, z0, 1e-6, 1e-6)
    _close("values with lists", v1, v0, 1e-5, 1e-6)
    g = torch.Generator(device="cpu").manual_seed(5)
    gz, gv = torch.randn(E, H, generator=g).to(dev), torch.randn(E, H, hd, generator=g).to(dev)
    nbytes = int(_lib.lib().cfb200_framed_proj_bwd_workspace_bytes(N, E))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    res = []
    for use in (None, plist):
        ga = torch.empty(N, H, device=dev)
        gW = [torch.empty(H, hd, 64, device=dev) for _ in range(4)]
        _lib.invoke("cfb200_framed_proj_bwd_cached", 3, dev, p(D["a"]), p(D["pos_ij"]), p(tv), p(rvlen), ip(D["batch"]),
                    ip(D["edges"]), ip(D["e_start"]), N, E, 14.0, -3.5, p(W[0]), p(W[1]), p(W[2]), p(W[3]), p(f[0]),
                    p(f[1]), p(f[2]), p(z0), p(gz), p(gv), p(ga), p(gW[0]), p(gW[1]), p(gW[2]), p(gW[3]), ws.data_ptr(),
                    nbytes, p(use), 2)
        res.append([ga] + gW)
    for x, y, name in zip(res[0], res[1], ("ga", "gW_dist", "gW_ang1", "gW_ang2", "gW_ang3")):
        scale = max(1.0, float(x.abs().max()))
        _close(name + " with lists", y, x, 1e-4, 1e-5 * scale)
    assert _lib.read_status() == 0


def test_flat_adamw_matches_torch():
    """cfb200_adamw_clip_step (clip by global norm + AdamW on flat buffers) against
    torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW over several steps, with and without clipping active."""
    dev = _cuda()
    from crystalframer_b200.optim import FlatAdamW

    def make():
        torch.manual_seed(5)
        return torch.nn.Sequential(torch.nn.Linear(37, 64), torch.nn.ReLU(), torch.nn.Linear(64, 3)).to(dev)

    ref, ours = make(), make()
    split = lambda m: ([p for n, p in m.named_parameters() if not n.endswith("bias")],
                       [p for n, p in m.named_parameters() if n.endswith("bias")])
    d, nd = split(ref)
    opt_ref = torch.optim.AdamW([{"params": d, "weight_decay": 1e-2}, {"params": nd, "weight_decay": 0.0}], lr=3e-3,
                                betas=(0.9, 0.98))
    d2, nd2 = split(ours)
    opt = FlatAdamW(d2, nd2, lr=3e-3, betas=(0.9, 0.98), eps=1e-8, weight_decay=1e-2, max_norm=0.5)
    g = torch.Generator(device="cpu").manual_seed(1)
    for step in range(6):
        x = torch.randn(50, 37, generator=g).to(dev) * (10.0 if step % 2 == 0 else 0.01)   # large and tiny gradients
        for m, o in ((ref, opt_ref), (ours, opt)):
            o.zero_grad(set_to_none=True)
            m(x).square().mean().backward()
        norm_ref = torch.nn.utils.clip_grad_norm_(list(ref.parameters()), 0.5)
        opt_ref.step()
        opt.step()
        assert abs(float(opt.grad_norm) - float(norm_ref)) <= 1e-5 * max(1.0, float(norm_ref))
        for (n, a), b in zip(ref.named_parameters(), ours.parameters()):
            _close(f"step {step} {n}", b, a, 1e-5, 1e-7)
    # parameters stay views of the flat buffer, so state_dict round trips keep working
    ours.load_state_dict({k: v.clone() for k, v in ref.state_dict().items()})
    assert all(p.data_ptr() >= opt.flat.data_ptr() and p.data_ptr() < opt.flat.data_ptr() + 4 * opt.n for p in ours.parameters())
