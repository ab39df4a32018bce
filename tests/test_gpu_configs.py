"""Parity at the sizes of the stated workloads.

* the full operator-level batch (256 crystals, log-normal sizes) against the reference project's
  OWN CUDA kernels, compiled from their sources for sm_100a into oracle/_ref/libcfref_gpu.so, on
  the same GPU and the same inputs: both the reference-signature Functions and the fused entry
  points the training step uses;
* a slice of the large-cell workload (crystals of 100-200 atoms, cells of 10-25 angstrom) for the
  three frame methods against the CPU oracle;
* the Gaussian-coefficient kernels against the oracle's formula.

Integers (selected pair and image) are compared exactly; a differing second-axis selection must be a
tie at float32 resolution (parity_util.adjudicate_second_axis).  Floats within 1e-4 relative + 1e-5
absolute; the long cancelling sums (coefficient and weight gradients) with the absolute term scaled
by the largest entry.
"""
import math

import numpy as np
import pytest
import torch

from conftest import make_problem
from parity_util import (ATOL, RTOL, adjudicate_second_axis, close, close_reduction, cuda, geometry, to_dev)

pytestmark = pytest.mark.gpu


def _configure(noise=0.0, angle_dim=64):
    from crystalframer_b200 import cuda_funcs as F
    F.compile_kernels(2, 8, 16, 64, angle_dim, 16, True, 0, 1.0, 4.0, 1.0, 1.0, noise)
    return F


def _fused_call(dev, g, qs, k, v, a, W, frames, go, unwindowed=False, use_list=True):
    """cfb200_pair_cache + cfb200_attn_fused_fwd / _bwd through the C ABI, as the training step calls them.
    Returns dict of outputs; gW is the (H,16,256) weight gradient formed from the pooled basis sums."""
    from crystalframer_b200 import _lib
    p, ip = _lib.ptr, _lib.iptr
    N, H, hd = qs.shape
    E = g["edges"].shape[1]
    plist = None
    if use_list:
        plist = torch.empty(E, 5, 128, device=dev)
        _lib.invoke("cfb200_pair_cache", 2, dev, p(g["pos_ij"]), p(g["tvecs"]), ip(g["batch"]), ip(g["edges"]), N, E, 2,
                    None, p(plist))
    order = torch.argsort(g["e_start"][1:] - g["e_start"][:-1], descending=True, stable=True).to(torch.int32)
    counters = torch.zeros(64, dtype=torch.int32, device=dev)
    out, z, lse, spool = (torch.empty(s, device=dev) for s in ((N, H, hd), (E, H), (N, H), (N, H, 256)))
    Wp = [p(W[0])] + [p(W[x]) if not unwindowed else None for x in (1, 2, 3)]
    fp = [p(frames[x]) if not unwindowed else None for x in range(3)]
    common = (p(qs), p(k), p(v), p(a), p(g["pos_ij"]), p(g["tvecs"]), p(g["rvlen"]), ip(g["batch"]), ip(g["edges"]),
              ip(g["e_start"]), p(order, torch.int32), p(counters, torch.int32), N, E, 14.0, -3.5, *Wp, *fp, p(plist), 2)
    flag = 1 if unwindowed else 0
    results = []
    for saved in (False, True):
        # saved: the forward keeps per-pair results for the backward; else the backward recomputes the lattice sums
        keep = [torch.empty(s, device=dev) for s in ((E, H, hd), (E, H), (N, H, hd))] if saved else [None] * 3
        kp = [p(x) for x in keep]
        out, z, lse, spool = (torch.empty(s, device=dev) for s in ((N, H, hd), (E, H), (N, H), (N, H, 256)))
        _lib.invoke("cfb200_attn_fused_fwd", 1, dev, *common, p(out), p(z), p(lse), p(spool), *kp, flag)
        gq, gk, gv, ga, gz = (torch.empty(s, device=dev) for s in ((N, H, hd), (N, H, hd), (N, H, hd), (N, H), (E, H)))
        _lib.invoke("cfb200_attn_fused_bwd", 2, dev, *common, p(out), p(z), p(lse), p(go), p(gq), p(gk), p(gv), p(ga), p(gz),
                    *kp, flag)
        results.append(dict(out=out, z=z, gq=gq, gk=gk, gv=gv, ga=ga, gz=gz, spool=spool))
    for name in results[0]:           # the two ways agree to rounding (both are held to the oracle by the callers' checks)
        x, y = results[0][name], results[1][name]
        scale = float(x.abs().max()) + 1e-12
        assert float((x - y).abs().max()) <= 2e-4 * scale + 1e-6, (name, float((x - y).abs().max()), scale)
    out, z, gq, gk, gv, ga, gz, spool = (results[1][n] for n in ("out", "z", "gq", "gk", "gv", "ga", "gz", "spool"))
    gW = torch.bmm(go.permute(1, 2, 0), spool.permute(1, 0, 2))
    assert _lib.read_status(dev) == 0
    return dict(out=out, z=z, gq=gq, gk=gk, gv=gv, ga=ga, gz=gz, gW=gW)


def _viol(name, got, want, scale=1.0):
    err = (got - want).abs()
    bad = err > ATOL * scale + RTOL * want.abs()
    assert not bool(bad.any()), f"{name}: {int(bad.sum())} of {bad.numel()} outside tolerance, max abs err {float(err.max()):.3e}"


def test_operator_batch_against_reference_cuda_kernels():
    """BASELINE operator-level workload in full (256 crystals, 2 663 atoms, 38 320 pairs): frames, lattice-sum
    bias, value encoding, attention and every gradient against the reference's own kernels on this GPU."""
    dev = cuda()
    from oracle import reference as R
    if not R.available("cuda"):
        pytest.skip("oracle/_ref/libcfref_gpu.so is not built (python -m oracle.build_oracle with the reference tree)")
    from crystalframer_b200 import opbench
    F = _configure()
    I = opbench.make_inputs("cfg2", None, dev)
    rk = R.RefKernels("cuda")
    a, pos, tv, batch, edges, rv = I["a"], I["pos_ij"], I["tv"], I["batch"], I["edges"], I["rvlen"]
    qs, k, v, go = (I["q"] / 4.0).contiguous(), I["k"], I["v"], I["go"]
    N, H = a.shape
    assert len(I["batch_obj"].sizes) == 256
    # ---- frames: integer selections first, floats second --------------------------------------
    f1_ref, arg1_ref = rk.frame1(qs, k, a, pos, tv, batch, edges, rv, -3.5)
    f1, se1, _ = F.max_frame_with_selection(1, qs, k, a, pos, tv, batch, edges, rv, -3.5)
    assert torch.equal(se1, arg1_ref), f"first axis: selected pair differs on {int((se1 != arg1_ref).sum())} of {se1.numel()}"
    # The reference's nvcc build contracts d2 = dx*dx + dy*dy + dz*dz and the normalisation into fused
    # multiply-adds; the library evaluates them unfused (so that a CPU reproduces its selection bit for bit).
    # The unit vectors therefore agree to float32 rounding, not bit for bit; a different IMAGE of the
    # selected pair would move the vector by far more.
    assert float((f1 - f1_ref).abs().max()) <= 4 * np.finfo(np.float32).eps
    f2m_ref, arg2_ref = rk.frame2(qs, k, a, pos, tv, batch, edges, rv, -3.5, f1_ref)
    f2m, se2, _ = F.max_frame_with_selection(2, qs, k, a, pos, tv, batch, edges, rv, -3.5, f1_ref)
    same = se2 == arg2_ref
    n_diff = int((~same).sum())
    # a differing second-axis pair must be a tie: both implementations' candidates then score alike, which
    # the oracle-based test adjudicates in float64; here differing selections must stay isolated cases
    assert n_diff <= max(2, se2.numel() // 5000), f"second axis: selected pair differs on {n_diff} of {se2.numel()}"
    assert float((f2m - f2m_ref).abs().max(-1)[0][same].max()) <= 1e-6
    f2_ref, f3_ref = rk.complete(f1_ref, f2m_ref)
    g1, g2, g3 = F.max_frames_fused(qs, k, a, pos, tv, batch, edges, rv, -3.5)
    assert float((g1 - f1_ref).abs().max()) <= 4 * np.finfo(np.float32).eps
    assert float((g2 - f2_ref).abs().max(-1)[0][same].max()) <= 1e-5
    assert float((g3 - f3_ref).abs().max(-1)[0][same].max()) <= 1e-5
    # ---- forward and backward on the reference's frames --------------------------------------
    frames = torch.stack([f1_ref, f2_ref, f3_ref]).contiguous()
    Wd, Ws = I["W"][0].contiguous(), torch.stack(I["W"][1:]).contiguous()
    asig = R.angle_sigma(4.0, 64)
    z_r, val_r = rk.framed_proj_fwd(a, pos, tv, batch, edges, 14.0, 1.0, Wd, Ws, frames, asig, 1.0, 1.0, rv, -3.5)
    out_r, prob_r, es = rk.dpa_fwd(qs, k, v, z_r, val_r, edges)
    gq_r, gk_r, gv_r, gz_r, gb_r = rk.dpa_bwd(qs, k, v, z_r, val_r, batch, edges, es, prob_r, out_r, go)
    ga_r, gWd_r, gWs_r = rk.framed_proj_bwd(a, pos, tv, batch, edges, 14.0, 1.0, Wd, Ws, frames, asig, 1.0, 1.0, rv, -3.5,
                                            z_r, gz_r, gb_r)
    torch.cuda.synchronize()
    sc = lambda t: max(1.0, float(t.abs().max()))
    # (i) the reference-signature Functions
    a_ = a.detach().requires_grad_(True)
    W_ = [w.detach().requires_grad_(True) for w in I["W"]]
    q_, k_, v_ = (t.detach().requires_grad_(True) for t in (qs, k, v))
    z2, val2 = F.RealEncodingWithFramedProjFuncCUDA.apply(a_, pos, None, tv, batch, edges, 64, 14.0, 1.0, W_[0], W_[1], W_[2],
                                                          W_[3], f1_ref, f2_ref, f3_ref, 64, 4.0, 0, 1.0, 1.0, rv, -3.5)
    out2 = F.FusedDotProductAttentionCUDA.apply(q_, k_, v_, z2, val2, batch, edges)
    out2.backward(go)
    for name, got, want, s in (("z", z2, z_r, 1.0), ("values", val2, val_r, 1.0), ("out", out2, out_r, 1.0),
                               ("gq", q_.grad, gq_r, 1.0), ("gk", k_.grad, gk_r, 1.0), ("gv", v_.grad, gv_r, 1.0),
                               ("ga", a_.grad, ga_r, sc(ga_r)), ("gW_dist", W_[0].grad[0], gWd_r, sc(gWd_r)),
                               ("gW_ang", torch.stack([w.grad[0] for w in W_[1:]]), gWs_r, sc(gWs_r))):
        _viol("Functions: " + name, got.detach(), want, s)
    # (ii) the fused entry points of the training step
    g = dict(pos_ij=pos, tvecs=tv, batch=batch, edges=edges, rvlen=rv, e_start=I["e_start"])
    for use_list in (True, False):
        r = _fused_call(dev, g, qs, k, v, a, [w[0].contiguous() for w in I["W"]], frames, go, use_list=use_list)
        tag = "fused(list): " if use_list else "fused(sweep): "
        for name, want, s in (("z", z_r, 1.0), ("out", out_r, 1.0), ("gq", gq_r, 1.0), ("gk", gk_r, 1.0), ("gv", gv_r, 1.0),
                              ("gz", gz_r, 1.0), ("ga", ga_r, sc(ga_r))):
            _viol(tag + name, r[name], want, s)
        _viol(tag + "gW_dist", r["gW"][:, :, :64], gWd_r, sc(gWd_r))
        _viol(tag + "gW_ang", torch.stack([r["gW"][:, :, 64 * x:64 * (x + 1)] for x in (1, 2, 3)]), gWs_r, sc(gWs_r))


def _large_cell_problem(nc=4):
    """Slice of the large-cell workload: ``nc`` crystals of 100-200 atoms in cells of 10-25 angstrom."""
    return make_problem("cfg4", num_crystals=nc)


def test_large_cell_slice_max_frames_and_fused_attention():
    dev = cuda()
    from oracle import oracle as O
    F = _configure()
    P = _large_cell_problem()
    assert P["batch"].sizes.min() >= 100 and len(P["batch"].sizes) >= 4
    g = geometry(P, dev)
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    qs = (P["q"] / 4.0).astype(np.float32)
    want = O.max_frames(cfg, qs, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                        geo["e_start"])
    q, k, v, a = (to_dev(x, dev) for x in (qs, P["k"], P["v"], P["a"]))
    f1, se1, si1 = F.max_frame_with_selection(1, q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5)
    assert np.array_equal(se1.cpu().numpy(), want["sel_edge1"])
    assert np.array_equal(si1.cpu().numpy(), want["sel_image1"])
    assert np.array_equal(f1.cpu().numpy(), want["frame1"])
    f2, se2, si2 = F.max_frame_with_selection(2, q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5, f1)
    n_diff = adjudicate_second_axis(P, want["frame1"], se2.cpu().numpy(), si2.cpu().numpy(), want["sel_edge2"],
                                    want["sel_image2"])
    assert n_diff <= max(2, se2.numel() // 500)
    same = (se2.cpu().numpy() == want["sel_edge2"]) & (si2.cpu().numpy() == want["sel_image2"])
    close("frame2_max", f2.cpu().numpy()[same], want["frame2_max"][same], 1e-6, 1e-6)
    g1, g2, g3 = F.max_frames_fused(q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5)
    assert np.array_equal(g1.cpu().numpy(), want["frame1"])
    close("frame2", g2.cpu().numpy()[same], want["frame2"][same], 1e-5, 1e-6)
    close("frame3", g3.cpu().numpy()[same], want["frame3"][same], 1e-5, 1e-6)
    # fused attention on the oracle's frames
    frames = np.stack([want["frame1"], want["frame2"], want["frame3"]])
    _check_fused_against_oracle(dev, P, g, cfg, frames, unwindowed=False)


def test_large_cell_slice_plain_encoding():
    """frame_method "no" on large cells: the fused entry points with ``unwindowed=1`` and the
    reference-signature Function, against the oracle's un-windowed encoding."""
    dev = cuda()
    from oracle import oracle as O
    F = _configure(angle_dim=0)
    P = _large_cell_problem()
    P["cfg"] = O.Config(cut_sigma=32, D_ang=0)
    g = geometry(P, dev)
    _check_fused_against_oracle(dev, P, g, P["cfg"], None, unwindowed=True)
    geo, b = P["geo"], P["batch"]
    z_w, v_w = O.framed_proj_fwd(P["cfg"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 P["W_d"], None, None)
    a = to_dev(P["a"], dev)
    Wd = to_dev(P["W_d"][None], dev)
    z, v, _, _ = F.RealPeriodicEncodingWithProjFuncCUDA.apply(a, g["pos_ij"], None, g["tvecs"], g["batch"], g["edges"], 64,
                                                              14.0, 1.0, Wd, "no", g["rvlen"], -3.5)
    close("z", z.cpu().numpy(), z_w)
    close("values", v.cpu().numpy(), v_w)
    _configure()


def _check_fused_against_oracle(dev, P, g, cfg, frames, unwindowed):
    from oracle import oracle as O
    geo, b = P["geo"], P["batch"]
    qs = (P["q"] / 4.0).astype(np.float32)
    W_a = None if unwindowed else P["W_a"]
    z_w, v_w = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 P["W_d"], W_a, frames)
    out_w, prob_w = O.dpa_fwd(cfg, qs, P["k"], P["v"], z_w, v_w, geo["edges"], geo["e_start"])
    go = np.random.default_rng(11).normal(size=out_w.shape).astype(np.float32)
    gq_w, gk_w, gv_w, gz_w, gval_w = O.dpa_bwd(cfg, qs, P["k"], P["v"], v_w, geo["edges"], geo["e_start"], prob_w, out_w, go)
    ga_w, gWd_w, gWa_w = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                           geo["e_start"], P["W_d"], W_a, frames, z_w, gz_w, gval_w)
    z64, _ = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], P["W_d"],
                               W_a, frames, dtype=np.float64)
    ga_64, gWd_64, gWa_64 = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                                              geo["edges"], geo["e_start"], P["W_d"], W_a, frames, z64, gz_w, gval_w,
                                              dtype=np.float64)
    t = lambda x: to_dev(x, dev)
    W = [t(P["W_d"])] + [t(P["W_a"][x]) for x in range(3)]
    fr = None if unwindowed else [t(frames[x]) for x in range(3)]
    for use_list in (True, False):
        r = _fused_call(dev, g, t(qs), t(P["k"]), t(P["v"]), t(P["a"]), W, fr, t(go), unwindowed=unwindowed,
                        use_list=use_list)
        tag = ("list " if use_list else "sweep ")
        close(tag + "z", r["z"].cpu().numpy(), z_w)
        close(tag + "out", r["out"].cpu().numpy(), out_w)
        close(tag + "gq", r["gq"].cpu().numpy(), gq_w)
        close(tag + "gk", r["gk"].cpu().numpy(), gk_w)
        close(tag + "gv", r["gv"].cpu().numpy(), gv_w)
        close(tag + "gz", r["gz"].cpu().numpy(), gz_w)
        close_reduction(tag + "ga", r["ga"].cpu().numpy(), ga_w, ga_64)
        gW = r["gW"].cpu().numpy()
        close_reduction(tag + "gW_dist", gW[:, :, :64], gWd_w, gWd_64)
        if not unwindowed:
            for x in range(3):
                close_reduction(tag + f"gW_ang{x + 1}", gW[:, :, 64 * (x + 1):64 * (x + 2)], gWa_w[x], gWa_64[x])


def test_large_cell_slice_weighted_pca_frames():
    """Weighted-PCA frames on large cells: the per-pair second moments and their attention pooling are pinned
    by the reference kernels on the CPU (tests/test_oracle.py); here the library's pooled matrices must
    be diagonalised by its frames and agree with the oracle wherever the eigenvalues are separated."""
    dev = cuda()
    from oracle import oracle as O
    F = _configure()
    P = _large_cell_problem(nc=2)
    g = geometry(P, dev)
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    qs = (P["q"] / 4.0).astype(np.float32)
    q, k, a = (to_dev(x, dev) for x in (qs, P["k"], P["a"]))
    f1, f2, f3, seed_noise, seed_sign = F.weighted_pca_frames(q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"],
                                                              g["rvlen"], -3.5)
    Fg = torch.stack([f1, f2, f3], dim=-2).cpu().numpy().astype(np.float64)
    want, mats, evals = O.weighted_pca_frames(cfg, qs, P["k"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"],
                                              geo["batch"], geo["edges"], geo["e_start"], seed_noise, seed_sign)
    assert np.abs(np.einsum("nhrc,nhsc->nhrs", Fg, Fg) - np.eye(3)).max() < 1e-5
    assert np.abs(np.linalg.det(Fg) - 1.0).max() < 1e-5
    N, H = P["a"].shape
    S = np.array([[[1.0 if O.hash_uniform(seed_sign, i * H + h, r) > 0.5 else -1.0 for r in range(3)]
                   for h in range(H)] for i in range(N)])
    SMS = mats * S[..., :, None] * S[..., None, :]
    D = np.einsum("nhrc,nhrs,nhsd->nhcd", Fg, SMS, Fg)
    lam = np.einsum("nhcc->nhc", D)
    off = D - lam[..., None] * np.eye(3)
    # matrices with determinant <= 1e-5 (an atom that attends almost only to itself) are not decomposed: the
    # frame is the signed identity (models/indexed_lattice_multi_head_attention_cuda.py:683-690)
    flat = np.linalg.det(mats) <= 1e-5
    assert np.abs(np.abs(Fg[flat]) - np.eye(3)).max() < 1e-6 if flat.any() else True
    assert np.abs(off[~flat]).max() < 1e-4 * max(1.0, np.abs(mats).max())
    close("eigenvalues", lam[~flat], evals[~flat], 1e-4, 1e-4 * max(1.0, np.abs(evals).max()))
    gap = np.minimum(evals[..., 1] - evals[..., 0], evals[..., 2] - evals[..., 1]) / np.maximum(evals[..., 2], 1e-9)
    ok = (gap > 1e-2) & ~flat
    Fw = np.stack([want[0], want[1], want[2]], axis=-2).astype(np.float64)
    agree = np.abs(Fg - Fw).max(axis=(-1, -2)) < 1e-3
    assert ok.mean() > 0.5 and agree[ok].mean() > 0.97, (ok.mean(), agree[ok].mean())


def test_gauss_coefficient_kernels_against_oracle():
    """cfb200_gauss_coef_fwd / _bwd against the reference's chain of torch operations
    (models/indexed_lattice_multi_head_attention_cuda.py:896-940, :179), evaluated on the CPU in float64."""
    dev = cuda()
    from crystalframer_b200 import _lib
    _configure()
    rng = np.random.default_rng(5)
    N, H, hd = 777, 8, 16
    q = rng.normal(size=(N, H, hd)).astype(np.float32)
    w = rng.normal(0, hd ** -0.5, size=(H * hd)).astype(np.float32)
    lb, beta, r0 = 0.5, 0.1, 1.4
    dots = np.einsum("nhd,hd->nh", q.astype(np.float64), w.reshape(H, hd).astype(np.float64))
    gs = np.array([1.0 / dots.std(ddof=1), -dots.mean()], np.float32)
    ga = rng.normal(size=(N, H)).astype(np.float32)
    gqs = rng.normal(size=(N, H, hd)).astype(np.float32)
    q64 = torch.from_numpy(q).double().requires_grad_(True)
    w64 = torch.from_numpy(w).double().requires_grad_(True)
    alpha = (q64.reshape(N, H, 1, hd) @ w64.reshape(H, hd, 1)).view(N, H)
    alpha = (alpha + float(gs[1])) * float(gs[0])
    a64 = ((1.0 - lb) * torch.nn.functional.elu(alpha * (beta / (1.0 - lb))) + 1.0) * (-0.5 * r0 ** -2)
    qs64 = q64 / math.sqrt(hd)
    ((a64 * torch.from_numpy(ga).double()).sum() + (qs64 * torch.from_numpy(gqs).double()).sum()).backward()
    t = lambda x: to_dev(x, dev)
    p = _lib.ptr
    qd, wd, gsd = t(q), t(w), t(gs)
    a_out, qs_out = torch.empty(N, H, device=dev), torch.empty(N, H, hd, device=dev)
    _lib.invoke("cfb200_gauss_coef_fwd", 1, dev, p(qd), p(wd), p(gsd), N, lb, beta, r0, p(a_out), p(qs_out))
    close("a", a_out.cpu().numpy(), a64.detach().numpy())
    close("q scaled", qs_out.cpu().numpy(), qs64.detach().numpy())
    assert float(a_out.max()) < 0.0
    gq_out, gw_out = torch.empty(N, H, hd, device=dev), torch.empty(H * hd, device=dev)
    _lib.invoke("cfb200_gauss_coef_bwd", 1, dev, p(qd), p(wd), p(gsd), N, lb, beta, r0, p(t(ga)), p(t(gqs)), p(gq_out),
                p(gw_out))
    close("gq", gq_out.cpu().numpy(), q64.grad.numpy())
    close("gw", gw_out.cpu().numpy(), w64.grad.numpy(), RTOL, ATOL * max(1.0, float(w64.grad.abs().max())))


@pytest.mark.parametrize("workload,nc", [("cfg1", None), ("cfg2", 24)])
def test_static_and_lattice_frames(workload, nc):
    """Frame methods "max_static" and "lattice" against the oracle (which tests/test_oracle.py holds to the
    reference's own kernels): selections and first axes bit for bit; a differing static second-axis selection must be
    a tie at float32 resolution; lattice frames, which involve no transcendental function, bit for bit."""
    dev = cuda()
    from oracle import oracle as O
    F = _configure()
    P = make_problem(workload, num_crystals=nc)
    g = geometry(P, dev)
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    a = to_dev(P["a"], dev)
    want = O.max_static_frames(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], geo["e_start"])
    f1, se1, si1 = F.max_static_frame_with_selection(1, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5)
    assert np.array_equal(se1.cpu().numpy(), want["sel_edge1"]) and np.array_equal(si1.cpu().numpy(), want["sel_image1"])
    assert np.array_equal(f1.cpu().numpy(), want["frame1"])
    f2, se2, si2 = F.max_static_frame_with_selection(2, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5, f1)
    n_diff = adjudicate_second_axis(P, want["frame1"], se2.cpu().numpy(), si2.cpu().numpy(), want["sel_edge2"], want["sel_image2"],
                                    static=True)
    assert n_diff <= max(2, se2.numel() // 500)
    same = (se2.cpu().numpy() == want["sel_edge2"]) & (si2.cpu().numpy() == want["sel_image2"])
    close("static frame2_max", f2.cpu().numpy()[same], want["frame2_max"][same], 1e-6, 1e-6)
    g1, g2, g3 = F.max_static_frames_fused(a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5)
    assert np.array_equal(g1.cpu().numpy(), want["frame1"])
    close("static frame2", g2.cpu().numpy()[same], want["frame2"][same], 1e-5, 1e-6)
    close("static frame3", g3.cpu().numpy()[same], want["frame3"][same], 1e-5, 1e-6)
    # the drop-in Functions give the same axes
    q = to_dev(P["q"] / 4.0, dev)
    k = to_dev(P["k"], dev)
    h1 = F.ComputeFrame1MaximumStaticMethodCUDA.apply(q, k, None, a, g["pos_ij"], None, g["tvecs"], g["batch"], g["edges"], 64, 14.0,
                                                      1.0, g["rvlen"], -3.5)
    assert torch.equal(h1, f1)
    # lattice frames
    l_want = O.lattice_frames(cfg, P["a"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], geo["e_start"])
    l_got = F.ComputeLatticeFrameCUDA.apply(q, k, None, a, g["pos_ij"], None, g["tvecs"], g["batch"], g["edges"], 64, 14.0, 1.0,
                                            g["rvlen"], -3.5)
    for x in range(3):
        assert np.array_equal(l_got[x].cpu().numpy(), l_want[x]), f"lattice frame {x + 1}"
    from crystalframer_b200 import _lib
    assert _lib.read_status(dev) == 0
