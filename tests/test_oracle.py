"""The CPU oracle against everything that pins it (no GPU needed):

* committed golden fixtures produced by the reference's own code (tests/golden/make_golden.py);
* the reference kernels' CPU build, when oracle/_ref is present on this machine;
* finite differences of the float64 build;
* edge cases: single-atom crystal, small cells with lattice range above the minimum.
"""
import os

import numpy as np
import pytest
import torch

from conftest import make_problem
from oracle import oracle as O
from oracle import reference as R

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def close(name, got, want, rtol=1e-4, atol=1e-5):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, name
    err = np.abs(got - want)
    bad = err > atol + rtol * np.abs(want)
    assert not bad.any(), f"{name}: {bad.sum()} of {bad.size} outside tolerance, max abs {err.max():.3e}"


def test_golden_reference_kernels():
    G = np.load(os.path.join(GOLD, "ref_kernels_small.npz"))
    cfg = O.Config()
    g = O.lattice_geometry(G["pos"], G["cells"], G["sizes"])
    assert np.array_equal(g["edges"], G["edges"]) and np.array_equal(g["e_start"], G["e_start"])
    Rah = O.lattice_range(cfg, G["a"], g["rvlen"], g["batch"])
    assert np.array_equal(Rah, G["R_ah"]) and Rah.max() > 2       # the small cell exercises ranges above the minimum
    fr = O.max_frames(cfg, G["q"] / 4.0, G["k"], G["a"], g["pos_ij"], G["cells"], g["rvlen"], g["batch"], g["edges"],
                      g["e_start"])
    assert np.array_equal(fr["sel_edge1"], G["sel_edge1"]) and np.array_equal(fr["sel_edge2"], G["sel_edge2"])
    assert np.array_equal(fr["frame1"], G["frame1"]) and np.array_equal(fr["frame2_max"], G["frame2_max"])
    close("frame2", fr["frame2"], G["frame2"], 1e-6, 1e-6)
    close("frame3", fr["frame3"], G["frame3"], 1e-6, 1e-6)
    frames = np.stack([G["frame1"], G["frame2"], G["frame3"]])
    z, v = O.framed_proj_fwd(cfg, G["a"], g["pos_ij"], G["cells"], g["rvlen"], g["batch"], g["edges"], G["W_d"],
                             G["W_a"], frames)
    close("z", z, G["z"], 1e-6, 1e-6)
    close("values", v, G["values"], 1e-6, 1e-7)
    ga, gWd, gWa = O.framed_proj_bwd(cfg, G["a"], g["pos_ij"], G["cells"], g["rvlen"], g["batch"], g["edges"],
                                     g["e_start"], G["W_d"], G["W_a"], frames, G["z"], G["gz"], G["gv"])
    close("ga", ga, G["ga"], 1e-4, 1e-5 * max(1.0, np.abs(G["ga"]).max()))
    close("gW_d", gWd, G["gW_d"], 1e-4, 1e-5)
    close("gW_a", gWa, G["gW_a"], 1e-4, 1e-5)
    out, prob = O.dpa_fwd(cfg, G["q"] / 4.0, G["k"], G["v"], G["z"], G["values"], g["edges"], g["e_start"])
    close("attention out", out, G["dpa_out"])
    close("attention prob", prob, G["dpa_prob"])
    res = O.dpa_bwd(cfg, G["q"] / 4.0, G["k"], G["v"], G["values"], g["edges"], g["e_start"], G["dpa_prob"], G["dpa_out"],
                    G["go"])
    for n, x in zip(("gq", "gk", "gvv", "gaij", "gbij"), res):
        close(n, x, G[n])
    close("mean", O.mean_fwd(G["mean_x"], G["sizes"]), G["mean"])
    st = O.max_static_frames(cfg, G["a"], g["pos_ij"], G["cells"], g["rvlen"], g["batch"], g["edges"], g["e_start"])
    assert np.array_equal(st["sel_edge1"], G["static_sel_edge1"]) and np.array_equal(st["sel_edge2"], G["static_sel_edge2"])
    assert np.array_equal(st["frame1"], G["static_frame1"]) and np.array_equal(st["frame2_max"], G["static_frame2_max"])
    lat = O.lattice_frames(cfg, G["a"], G["cells"], g["rvlen"], g["batch"], g["edges"], g["e_start"])
    for x in range(3):
        assert np.array_equal(lat[x], G[f"lattice_frame{x + 1}"])


def test_golden_pure_pytorch_twin():
    """Fixed range 2, un-windowed Gaussians, no frames: the plain Crystalformer subset."""
    G = np.load(os.path.join(GOLD, "ref_pure_small.npz"))
    K = np.load(os.path.join(GOLD, "ref_kernels_small.npz"))
    cfg = O.Config(cut_sigma=32, cutoff_radius=0.0, D_ang=0)        # window >= 64 -> full range of Gaussians
    g = O.lattice_geometry(K["pos"], K["cells"], K["sizes"])
    assert np.array_equal(g["edges"], G["edges"])
    z, v = O.framed_proj_fwd(cfg, K["a"], g["pos_ij"], K["cells"], g["rvlen"], g["batch"], g["edges"], K["W_d"], None, None)
    close("z", z, G["z"])
    close("values", v, G["values"])
    out, prob = O.dpa_fwd(cfg, K["q"] / 4.0, K["k"], K["v"], G["z"], G["values"], g["edges"], g["e_start"])
    close("out", out, G["out"])
    close("prob", prob, G["prob"])


@pytest.mark.skipif(not R.available("cpu"), reason="oracle/_ref not built (reference tree absent)")
def test_against_reference_cpu_build(problem_cfg1):
    P = problem_cfg1
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    rk = R.RefKernels("cpu")
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    a, q, k, v = T(P["a"]), T(P["q"] / 4.0), T(P["k"]), T(P["v"])
    r, tv, bt, e, rv = T(geo["pos_ij"]), T(b.trans_vec), T(geo["batch"]), T(geo["edges"]), T(geo["rvlen"])
    f1, s1 = rk.frame1(q, k, a, r, tv, bt, e, rv, -3.5)
    f2m, s2 = rk.frame2(q, k, a, r, tv, bt, e, rv, -3.5, f1)
    f2, f3 = rk.complete(f1, f2m)
    fr = O.max_frames(cfg, P["q"] / 4.0, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                      geo["edges"], geo["e_start"])
    assert np.array_equal(fr["sel_edge1"], s1.numpy()) and np.array_equal(fr["sel_edge2"], s2.numpy())
    assert np.array_equal(fr["frame1"], f1.numpy())
    frames = torch.stack([f1, f2, f3]).contiguous()
    Wd, Wa = T(P["W_d"])[None].contiguous(), T(P["W_a"])[:, None].contiguous()
    z, val = rk.framed_proj_fwd(a, r, tv, bt, e, 14.0, 1.0, Wd, Wa, frames, cfg.angle_sigma, 1.0, 1.0, rv, -3.5)
    zo, vo = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                               P["W_d"], P["W_a"], frames.numpy())
    close("z", zo, z.numpy(), 1e-6, 1e-6)
    close("values", vo, val.numpy(), 1e-6, 1e-7)
    rng = np.random.default_rng(9)
    gz, gv = rng.normal(size=zo.shape).astype(np.float32), rng.normal(size=vo.shape).astype(np.float32)
    ga, gWd, gWa = rk.framed_proj_bwd(a, r, tv, bt, e, 14.0, 1.0, Wd, Wa, frames, cfg.angle_sigma, 1.0, 1.0, rv, -3.5,
                                      z, T(gz), T(gv))
    gao, gWdo, gWao = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                                        geo["edges"], geo["e_start"], P["W_d"], P["W_a"], frames.numpy(), z.numpy(), gz, gv)
    close("ga", gao, ga.numpy(), 1e-4, 1e-5 * max(1.0, float(ga.abs().max())))
    close("gW_d", gWdo, gWd.numpy(), 1e-4, 1e-5 * max(1.0, float(gWd.abs().max())))
    close("gW_a", gWao, gWa.numpy(), 1e-4, 1e-5 * max(1.0, float(gWa.abs().max())))


@pytest.mark.skipif(not R.available("cpu"), reason="oracle/_ref not built (reference tree absent)")
def test_unwindowed_encoding_against_reference_cpu_build(problem_cfg1):
    """frame_method "no": the reference's real_enc_proj kernels against the oracle with a window
    wide enough to cover every Gaussian."""
    P = problem_cfg1
    geo, b = P["geo"], P["batch"]
    cfg = O.Config(cut_sigma=32, D_ang=0)
    rk = R.RefKernels("cpu")
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    a, r, tv, bt, e, rv = T(P["a"]), T(geo["pos_ij"]), T(b.trans_vec), T(geo["batch"]), T(geo["edges"]), T(geo["rvlen"])
    Wd = T(P["W_d"])[None].contiguous()
    z, val = rk.proj_fwd(a, r, tv, bt, e, 64, 14.0, 1.0, Wd, rv, -3.5)
    zo, vo = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], P["W_d"],
                               None, None)
    close("z", zo, z.numpy(), 1e-6, 1e-6)
    close("values", vo, val.numpy(), 1e-5, 1e-6)
    rng = np.random.default_rng(19)
    gz, gv = rng.normal(size=zo.shape).astype(np.float32), rng.normal(size=vo.shape).astype(np.float32)
    ga, gW = rk.proj_bwd(a, r, tv, bt, e, 14.0, 1.0, Wd, rv, -3.5, z, T(gz), T(gv))
    gao, gWo, _ = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                    geo["e_start"], P["W_d"], None, None, z.numpy(), gz, gv)
    close("ga", gao, ga.numpy(), 1e-4, 1e-5 * max(1.0, float(ga.abs().max())))
    close("gW", gWo, gW.numpy(), 1e-4, 1e-5 * max(1.0, float(gW.abs().max())))


@pytest.mark.skipif(not R.available("cpu"), reason="oracle/_ref not built (reference tree absent)")
def test_weighted_pca_moments_against_reference_cpu_build(problem_cfg1):
    """Second-moment matrices per (pair, head) against real_enc_sigma_fwd, and their attention
    pooling against fused_dpa_sigmamat_fwd when both receive the same (true) bias z."""
    P = problem_cfg1
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    rk = R.RefKernels("cpu")
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    a, r, tv, bt, e, rv = T(P["a"]), T(geo["pos_ij"]), T(b.trans_vec), T(geo["batch"]), T(geo["edges"]), T(geo["rvlen"])
    sigma, sigma_max = rk.sigma_fwd(a, r, tv, bt, e, rv, -3.5)
    z, sig, nd2, ndir = O.sigma_edges(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"])
    close("sigma", sig, sigma.numpy(), 1e-5, 1e-6)
    # every pair's thread writes its nearest-image matrix into the same per-atom slot (a race in the
    # reference): whatever survived must be the matrix of one of the atom's pairs
    u = ndir
    cand = np.stack([u[..., 0] * u[..., 0], u[..., 0] * u[..., 1], u[..., 0] * u[..., 2], u[..., 1] * u[..., 1],
                     u[..., 1] * u[..., 2], u[..., 2] * u[..., 2]], -1)              # (E,H,6)
    sm = sigma_max.numpy()
    for i in range(sm.shape[0]):
        rows = cand[geo["e_start"][i]:geo["e_start"][i + 1]]                         # (n,H,6)
        err = np.abs(rows - sm[i][None]).max(-1)                                     # (n,H)
        assert (err.min(0) < 1e-5).all(), i
    pooled = rk.sigma_pool(T(P["q"] / 4.0), T(P["k"]), T(z), sigma, e)
    _, mats, _ = O.weighted_pca_frames(cfg, P["q"] / 4.0, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"],
                                       geo["batch"], geo["edges"], geo["e_start"])
    idx = [(0, 0), (0, 1), (0, 2), (1, 1), (1, 2), (2, 2)]
    got = np.stack([mats[:, :, r_, c_] for r_, c_ in idx], -1)
    close("pooled sigma", got, pooled.numpy(), 1e-4, 1e-5)


def test_finite_differences_float64(problem_cfg1):
    P = problem_cfg1
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    fr = O.max_frames(cfg, P["q"] / 4.0, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                      geo["edges"], geo["e_start"])
    frames = np.stack([fr["frame1"], fr["frame2"], fr["frame3"]])
    rng = np.random.default_rng(1)
    args = (geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"])

    def fwd(a, Wd, Wa):
        return O.framed_proj_fwd(cfg, a, *args, Wd, Wa, frames, dtype=np.float64)

    a0, Wd0, Wa0 = P["a"].astype(np.float64), P["W_d"].astype(np.float64), P["W_a"].astype(np.float64)
    z, v = fwd(a0, Wd0, Wa0)
    gz, gv = rng.normal(size=z.shape), rng.normal(size=v.shape)
    ga, gWd, gWa = O.framed_proj_bwd(cfg, a0, *args, geo["e_start"], Wd0, Wa0, frames, z, gz, gv, dtype=np.float64)
    loss = lambda a, Wd, Wa: sum((x * g).sum() for x, g in zip(fwd(a, Wd, Wa), (gz, gv)))
    eps = 1e-6
    for idx in [(0, 0), (17, 3), (40, 7)]:
        ap, am = a0.copy(), a0.copy()
        ap[idx] += eps
        am[idx] -= eps
        fd = (loss(ap, Wd0, Wa0) - loss(am, Wd0, Wa0)) / (2 * eps)
        assert abs(fd - ga[idx]) <= 1e-5 * max(1.0, abs(fd)), (idx, fd, ga[idx])
    for idx in [(0, 0, 0), (3, 5, 20), (7, 15, 63)]:
        Wp, Wm = Wd0.copy(), Wd0.copy()
        Wp[idx] += eps
        Wm[idx] -= eps
        fd = (loss(a0, Wp, Wa0) - loss(a0, Wm, Wa0)) / (2 * eps)
        assert abs(fd - gWd[idx]) <= 1e-5 * max(1.0, abs(fd)), (idx, fd, gWd[idx])
    for idx in [(0, 0, 0, 40), (2, 6, 9, 33)]:
        Wp, Wm = Wa0.copy(), Wa0.copy()
        Wp[idx] += eps
        Wm[idx] -= eps
        fd = (loss(a0, Wd0, Wp) - loss(a0, Wd0, Wm)) / (2 * eps)
        assert abs(fd - gWa[idx]) <= 1e-5 * max(1.0, abs(fd)), (idx, fd, gWa[idx])


def test_attention_gradients_float64():
    P = make_problem("cfg1")
    geo, cfg = P["geo"], P["cfg"]
    rng = np.random.default_rng(2)
    E = geo["edges"].shape[1]
    q, k, v = (P[n].astype(np.float64) for n in ("q", "k", "v"))
    zb, vb = rng.normal(size=(E, 8)), rng.normal(size=(E, 8, 16))
    out, prob = O.dpa_fwd(cfg, q, k, v, zb, vb, geo["edges"], geo["e_start"], dtype=np.float64)
    go = rng.normal(size=out.shape)
    gq, gk, gv, gz, gb = O.dpa_bwd(cfg, q, k, v, vb, geo["edges"], geo["e_start"], prob, out, go, dtype=np.float64)
    loss = lambda q_, k_, z_: (O.dpa_fwd(cfg, q_, k_, v, z_, vb, geo["edges"], geo["e_start"], dtype=np.float64)[0] * go).sum()
    eps = 1e-6
    for idx in [(0, 0, 0), (30, 4, 9)]:
        qp, qm = q.copy(), q.copy()
        qp[idx] += eps
        qm[idx] -= eps
        assert abs((loss(qp, k, zb) - loss(qm, k, zb)) / (2 * eps) - gq[idx]) < 1e-6
        kp, km = k.copy(), k.copy()
        kp[idx] += eps
        km[idx] -= eps
        assert abs((loss(q, kp, zb) - loss(q, km, zb)) / (2 * eps) - gk[idx]) < 1e-6
    zp, zm = zb.copy(), zb.copy()
    zp[5, 2] += eps
    zm[5, 2] -= eps
    assert abs((loss(q, k, zp) - loss(q, k, zm)) / (2 * eps) - gz[5, 2]) < 1e-6


def test_edge_cases():
    cfg = O.Config()
    # a single-atom crystal: one self pair; z is the lattice sum over the atom's own images
    cell = np.array([[[3.0, 0, 0], [0, 3.2, 0], [0, 0, 3.4]]], np.float32)
    g = O.lattice_geometry(np.zeros((1, 3), np.float32), cell, [1])
    assert g["edges"].tolist() == [[0], [0]] and g["e_start"].tolist() == [0, 1]
    a = np.full((1, 8), -0.2, np.float32)
    z, _ = O.framed_proj_fwd(cfg, a, g["pos_ij"], cell, g["rvlen"], g["batch"], g["edges"], np.zeros((8, 16, 64), np.float32),
                             None, None)
    Rr = O.lattice_range(cfg, a, g["rvlen"], g["batch"])[0, 0]
    n = [np.arange(-r, r + 1) for r in Rr]
    d2 = (n[0][:, None, None] * 3.0) ** 2 + (n[1][None, :, None] * 3.2) ** 2 + (n[2][None, None, :] * 3.4) ** 2
    assert abs(z[0, 0] - np.log(np.exp(-0.2 * d2).sum())) < 1e-5
    # empty batch
    e, s = O.edge_index(np.zeros(0, np.int64))
    assert e.shape == (2, 0) and s.tolist() == [0]
    # ragged sizes including 1
    e, s = O.edge_index([2, 1, 3])
    assert e.shape == (2, 14) and s.tolist() == [0, 2, 4, 5, 8, 11, 14]
    assert e[:, 4].tolist() == [2, 2]


def test_values_linear_in_weights(problem_cfg1):
    P = problem_cfg1
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    args = (cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"])
    W2 = np.random.default_rng(3).normal(size=P["W_d"].shape).astype(np.float32) * 0.01
    _, v1 = O.framed_proj_fwd(*args, P["W_d"], None, None)
    _, v2 = O.framed_proj_fwd(*args, W2, None, None)
    _, v12 = O.framed_proj_fwd(*args, P["W_d"] + W2, None, None)
    close("linearity", v12, v1 + v2, 1e-4, 1e-6)


def test_pooling_identity_behind_the_fused_attention(problem_cfg1):
    """The fused attention kernels never form the value encoding: they pool the 256 basis sums of an atom's
    pairs with the attention weights and project once per (atom, head).  The algebra, on the oracle in
    float64: with s_ij the basis sums of a pair (read off the oracle through one-hot projection weights),
      out_i = sum_j p_ij v_j + W (sum_j p_ij s_ij)          and          gW = sum_i gout_i (x) S_i,
    where S_i is the pooled basis (distance part unscaled, angle parts times the angle coefficient)."""
    P = problem_cfg1
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    fr = O.max_frames(cfg, P["q"] / 4.0, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                      geo["edges"], geo["e_start"])
    frames = np.stack([fr["frame1"], fr["frame2"], fr["frame3"]])
    args = (cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"])
    E, H, hd = geo["edges"].shape[1], 8, 16
    f64 = np.float64
    # basis sums (E,H,4,64): values with W = 16 one-hot rows at a time, distance then the three axes
    basis = np.zeros((E, H, 4, 64), f64)
    for blk in range(4):
        sel = np.zeros((H, hd, 64), f64)
        for o in range(hd):
            sel[:, o, blk * hd + o] = 1.0
        zero_a = np.zeros((3, H, hd, 64), f64)
        _, vd = O.framed_proj_fwd(*args, sel, zero_a, frames, dtype=f64)
        basis[:, :, 0, blk * hd:(blk + 1) * hd] = vd / cfg.c_dist
        for x in range(3):
            Wa = zero_a.copy()
            Wa[x] = sel
            _, va = O.framed_proj_fwd(*args, np.zeros((H, hd, 64), f64), Wa, frames, dtype=f64)
            basis[:, :, 1 + x, blk * hd:(blk + 1) * hd] = va
    Wd, Wa = P["W_d"].astype(f64), P["W_a"].astype(f64)
    z, values = O.framed_proj_fwd(*args, Wd, Wa, frames, dtype=f64)
    W_all = np.concatenate([Wd[:, :, None, :], np.moveaxis(Wa, 0, 2)], 2)                   # (H,16,4,64)
    close("values = W s", np.einsum("hobk,ehbk->eho", W_all, basis), values, 1e-9, 1e-10)
    qs, k, v = (P["q"] / 4.0).astype(f64), P["k"].astype(f64), P["v"].astype(f64)
    out, prob = O.dpa_fwd(cfg, qs, k, v, z, values, geo["edges"], geo["e_start"], dtype=f64)
    i_of, j_of = geo["edges"][0], geo["edges"][1]
    N = qs.shape[0]
    pooled_v = np.zeros((N, H, hd), f64)
    pooled_s = np.zeros((N, H, 4, 64), f64)
    np.add.at(pooled_v, i_of, prob[:, :, None] * v[j_of])
    np.add.at(pooled_s, i_of, prob[:, :, None, None] * basis)
    close("out = sum p v + W S", pooled_v + np.einsum("hobk,nhbk->nho", W_all, pooled_s), out, 1e-9, 1e-10)
    # weight gradients from the pooled basis
    rng = np.random.default_rng(9)
    go = rng.normal(size=out.shape)
    _, _, _, gz, gval = O.dpa_bwd(cfg, qs, k, v, values, geo["edges"], geo["e_start"], prob, out, go, dtype=f64)
    _, gWd, gWa = O.framed_proj_bwd(*args, geo["e_start"], Wd, Wa, frames, z, gz, gval, dtype=f64)
    gW_all = np.einsum("nho,nhbk->hobk", go, pooled_s)
    close("gW_dist = sum gout (x) S", gW_all[:, :, 0], gWd, 1e-8, 1e-10)
    for x in range(3):
        close(f"gW_ang{x + 1}", gW_all[:, :, 1 + x], gWa[x], 1e-8, 1e-10)


def test_static_and_lattice_frames_against_reference_kernels():
    """Frame methods "max_static" and "lattice": the restatement against the reference's own kernels compiled for the
    CPU (compute_second_frame_static_each_edge.cu, compute_lattice_{first,second,third}_frame.cu) with the reference's
    host logic: selections and frames bit for bit (symmetry-breaking noise off)."""
    from oracle import reference as R
    if not R.available("cpu"):
        pytest.skip("oracle/_ref is not built on this machine")
    import json
    sigs = json.load(open(os.path.join(R.REF_DIR, "signatures.json")))
    if "compute_lattice_third_frame" not in sigs:
        pytest.skip("oracle/_ref was built before the lattice kernels were added: rebuild it")
    from conftest import make_problem
    for workload, nc in (("cfg1", None), ("cfg2", 12)):
        P = make_problem(workload, num_crystals=nc)
        geo, b, cfg = P["geo"], P["batch"], P["cfg"]
        T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
        rk = R.RefKernels("cpu")
        a, r, tv, bt, e, rv = T(P["a"]), T(geo["pos_ij"]), T(b.trans_vec), T(geo["batch"]), T(geo["edges"]), T(geo["rvlen"])
        f1r, s1r = rk.frame1_static(a, r, tv, bt, e, rv, -3.5)
        f2r, s2r = rk.frame2_static(a, r, tv, bt, e, rv, -3.5, f1r)
        w = O.max_static_frames(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], geo["e_start"])
        assert np.array_equal(s1r.numpy(), w["sel_edge1"]) and np.array_equal(f1r.numpy(), w["frame1"])
        assert np.array_equal(s2r.numpy(), w["sel_edge2"]) and np.array_equal(f2r.numpy(), w["frame2_max"])
        got = rk.lattice_frames(a, r, tv, bt, e, rv, -3.5)
        want = O.lattice_frames(cfg, P["a"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], geo["e_start"])
        for x in range(3):
            assert np.array_equal(got[x].numpy(), want[x]), (workload, x)


def test_pca_frames_are_principal_axes():
    """oracle.pca_frames (models/cuda_funcs/calc_pca_frame.py:22-76): eigenvectors of the scatter matrix of each
    atom's pair separations, ascending eigenvalue, orthonormal, right-handed, heads differing by signs only."""
    from crystalframer_b200 import synth
    b = synth.make_workload("cfg1")
    g = O.lattice_geometry(b.pos, b.trans_vec, b.sizes)
    fr, mats, evals = O.pca_frames(g["pos_ij"], g["e_start"], 4, seed=3)
    N = b.num_atoms
    assert fr.shape == (3, N, 4, 3) and (np.diff(evals, axis=1) >= -1e-9).all()
    Fm = np.moveaxis(fr, 0, 2).astype(np.float64)
    assert np.abs(Fm @ np.swapaxes(Fm, -1, -2) - np.eye(3)).max() < 1e-5
    assert np.abs(np.linalg.det(Fm) - 1.0).max() < 1e-5
    for r in range(3):
        v = Fm[:, 0, r, :]
        assert np.abs(np.einsum("nij,nj->ni", mats, v) - evals[:, r, None] * v).max() < 1e-4 * max(1.0, evals.max())
        assert np.abs(np.abs((Fm[:, :1, r] * Fm[:, :, r]).sum(-1)) - 1.0).max() < 1e-5      # heads: same axis up to sign
    # by hand for one atom: scatter matrix about the mean of its separations
    e0, e1 = int(g["e_start"][5]), int(g["e_start"][6])
    r5 = g["pos_ij"][e0:e1].astype(np.float64)
    d = r5 - r5.mean(0)
    assert np.allclose(mats[5], d.T @ d)


def test_golden_reciprocal_encoding():
    """Reciprocal-space lattice sum: the oracle against the reference's reci_enc kernels and against its
    pure-PyTorch twin, on the committed fixture (geometry from the reference's own host code)."""
    G = np.load(os.path.join(GOLD, "ref_reci_small.npz"))
    small = np.load(os.path.join(GOLD, "ref_kernels_small.npz"))
    rvecs, vcell, kr = O.reciprocal_geometry(small["pos"], small["cells"], small["sizes"], G["edges"])
    close("rvecs", rvecs, G["rvecs"], 1e-6, 1e-7)
    close("vcell", vcell, G["vcell"], 1e-6, 1e-6)
    close("kr", kr, G["kr"], 1e-5, 1e-6)
    batch = np.repeat(np.arange(len(small["sizes"])), small["sizes"])
    z, sumexp = O.reci_enc_fwd(G["a"], G["kr"], G["rvecs"], G["vcell"], batch, G["edges"])
    close("sumexp", sumexp, G["sumexp"], 1e-5, 1e-6)
    close("z", z, G["z"], 1e-5, 1e-5)
    close("z (pure twin)", z, G["z_pure"], 1e-4, 1e-5)
    ga = O.reci_enc_bwd(G["a"], G["kr"], G["rvecs"], batch, G["edges"], G["gz"], G["sumexp"])
    close("ga", ga, G["ga"], 1e-5, 1e-5)
    close("ga (pure twin)", ga, G["ga_pure"], 1e-4, 1e-4)
    # the double build's sum differentiates to the double build's gradient
    a64 = G["a"].astype(np.float64)
    z64, s64 = O.reci_enc_fwd(a64, G["kr"], G["rvecs"], G["vcell"], batch, G["edges"], dtype=np.float64)
    ga64 = O.reci_enc_bwd(a64, G["kr"], G["rvecs"], batch, G["edges"], G["gz"], s64, dtype=np.float64)
    h = 1e-6
    _, sp = O.reci_enc_fwd(a64 + h, G["kr"], G["rvecs"], G["vcell"], batch, G["edges"], dtype=np.float64)
    _, sm = O.reci_enc_fwd(a64 - h, G["kr"], G["rvecs"], G["vcell"], batch, G["edges"], dtype=np.float64)
    fd = np.zeros_like(a64)
    np.add.at(fd, G["edges"][0], G["gz"] * (np.log(sp) - np.log(sm)) / (2 * h))
    close("ga (finite differences)", ga64, fd, 1e-6, 1e-6)


@pytest.mark.skipif(not R.available("cpu"), reason="oracle/_ref not built (reference tree absent)")
def test_reciprocal_encoding_against_reference_cpu_build(problem_cfg1):
    P = problem_cfg1
    geo, b = P["geo"], P["batch"]
    rvecs, vcell, kr = O.reciprocal_geometry(b.pos, b.trans_vec, b.sizes, geo["edges"])
    a = (P["a"] * 9.5).astype(np.float32)              # -0.5 scale_reci^2 f against -0.5 scale_real^-2 f
    rk = R.RefKernels("cpu")
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    z, sumexp = rk.reci_fwd(T(a), T(kr), T(rvecs), T(vcell), T(geo["batch"]), T(geo["edges"]))
    zo, so = O.reci_enc_fwd(a, kr, rvecs, vcell, geo["batch"], geo["edges"])
    close("sumexp", so, sumexp.numpy(), 1e-5, 1e-6)
    ok = sumexp.numpy() > 1e-3
    close("z", zo[ok], z.numpy()[ok], 1e-5, 1e-5)
    gz = np.random.default_rng(3).normal(size=zo.shape).astype(np.float32)
    ga = rk.reci_bwd(T(a), T(kr), T(rvecs), T(vcell), T(geo["batch"]), T(geo["edges"]), z, T(gz), sumexp)
    gao = O.reci_enc_bwd(a, kr, rvecs, geo["batch"], geo["edges"], gz, sumexp.numpy())
    close("ga", gao, ga.numpy(), 1e-4, 1e-5 * max(1.0, float(ga.abs().max())))


@pytest.mark.skipif(not R.available("cpu"), reason="oracle/_ref not built (reference tree absent)")
def test_third_axis_without_orthogonalisation_against_reference_cpu_build(problem_cfg1):
    """Frame method "max_wo_orthogonal": the third-axis search (triple product with the first two axes in place of
    the collinearity term) against the reference's compute_third_frame_each_edge kernel -- selected pair identical,
    direction bit-identical."""
    P = problem_cfg1
    geo, b = P["geo"], P["batch"]
    cfg = P["cfg"]
    rk = R.RefKernels("cpu")
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    qs = (P["q"] / 4.0).astype(np.float32)
    a, r, tv, bt, e, rv = T(P["a"]), T(geo["pos_ij"]), T(b.trans_vec), T(geo["batch"]), T(geo["edges"]), T(geo["rvlen"])
    fr = O.max_frames_wo_orthogonal(cfg, qs, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                                    geo["edges"], geo["e_start"])
    f1, _ = rk.frame1(T(qs), T(P["k"]), a, r, tv, bt, e, rv, -3.5)
    f2, _ = rk.frame2(T(qs), T(P["k"]), a, r, tv, bt, e, rv, -3.5, f1)
    assert np.array_equal(f1.numpy(), fr["frame1"]) and np.array_equal(f2.numpy(), fr["frame2"])
    f3, sel3 = rk.frame3(T(qs), T(P["k"]), a, r, tv, bt, e, rv, -3.5, f1, f2)
    assert np.array_equal(sel3.numpy(), fr["sel_edge3"])
    assert np.array_equal(f3.numpy(), fr["frame3"])
    # the three axes span space: |det| > 1e-5 by construction of the search
    M = np.stack([fr["frame1"], fr["frame2"], fr["frame3"]], axis=-2).astype(np.float64)
    assert (np.abs(np.linalg.det(M)) > 1e-5).all()


def _selector_weights(H, hd, K):
    out = []
    for b in range(K // hd):
        S = np.zeros((H, hd, K), np.float32)
        r = np.arange(hd)
        S[:, r, hd * b + r] = 1.0
        out.append(S)
    return out


@pytest.mark.skipif(not R.available("cpu"), reason="oracle/_ref not built (reference tree absent)")
def test_unprojected_value_sums_against_reference_cpu_build(problem_cfg1):
    """real_enc_fwd / real_enc_bwd (logit + the 64 un-projected value sums per (pair, head)) against the oracle's
    un-windowed encoding read out through selector weights (basis functions 16 b .. 16 b + 15 unchanged)."""
    P = problem_cfg1
    geo, b = P["geo"], P["batch"]
    cfg = O.Config(cut_sigma=32, D_ang=0)
    rk = R.RefKernels("cpu")
    T = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    a, r, tv, bt, e, rv = T(P["a"]), T(geo["pos_ij"]), T(b.trans_vec), T(geo["batch"]), T(geo["edges"]), T(geo["rvlen"])
    z, v = rk.real_enc_fwd(a, r, tv, bt, e, 64, 14.0, 1.0, rv, -3.5)
    rng = np.random.default_rng(23)
    gz = rng.normal(size=tuple(z.shape)).astype(np.float32)
    gv = rng.normal(size=tuple(v.shape)).astype(np.float32)
    ga = rk.real_enc_bwd(a, r, tv, bt, e, 64, 14.0, 1.0, rv, -3.5, z, T(gz), T(gv))
    ga_o = np.zeros_like(P["a"])
    for blk, S in enumerate(_selector_weights(8, 16, 64)):
        zo, vo = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], S, None, None)
        close("z", zo, z.numpy(), 1e-6, 1e-6)
        close(f"values {blk}", vo, v.numpy()[..., 16 * blk:16 * blk + 16], 1e-5, 1e-6)
        g, _, _ = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                    geo["e_start"], S, None, None, zo, gz if blk == 0 else np.zeros_like(gz),
                                    np.ascontiguousarray(gv[..., 16 * blk:16 * blk + 16]))
        ga_o += g
    close("ga", ga_o, ga.numpy(), 1e-4, 1e-5 * max(1.0, float(ga.abs().max())))
