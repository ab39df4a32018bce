"""Parity of the CUDA path (through the C ABI) with the CPU oracle on identical seeded inputs.

Tolerances: integer outputs (pair list, CSR offsets, selected pair / image) bit-exact; float
outputs and gradients within 1e-4 relative + 1e-5 absolute, the bound the specification of
this path states.
"""
import numpy as np
import pytest
import torch

from conftest import make_problem

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _close(name, got, want, rtol=RTOL, atol=ATOL, frac_ok=0.0):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert np.isfinite(got).all(), name
    err = np.abs(got - want)
    bad = err > atol + rtol * np.abs(want)
    assert bad.mean() <= frac_ok, f"{name}: {bad.sum()} of {bad.size} outside tolerance, max abs err {err.max():.3e}"


def _close_reduction(name, got, want32, want64):
    """Coefficient and weight gradients are sums over an atom's / the batch's pairs of terms that
    largely cancel; float32 accumulation noise alone
    (any summation order) reaches the elementwise bound on entries with heavy cancellation --
    the float32 oracle itself is that far from the float64 oracle.  So the absolute term scales
    with the largest entry, and the error against the float64 value must not exceed three times
    the float32 oracle's own error."""
    got = np.asarray(got, dtype=np.float64)
    scale = max(1.0, float(np.abs(want64).max()))
    _close(name, got, want32, RTOL, ATOL * scale)
    ours, theirs = np.abs(got - want64).max(), np.abs(want32.astype(np.float64) - want64).max()
    assert ours <= 3.0 * theirs + ATOL, f"{name}: error vs float64 {ours:.3e}, float32 oracle's {theirs:.3e}"


def _configure(noise=0.0, angle_dim=64, c_dist=1.0, c_ang=1.0, wscale_d=1.0, wscale_a=4.0):
    from crystalframer_b200 import cuda_funcs as F
    F.compile_kernels(2, 8, 16, 64, angle_dim, 16, True, 0, wscale_d, wscale_a, c_dist, c_ang, noise)
    return F


def _t(x, dev):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def _geometry(P, dev):
    g, b = P["geo"], P["batch"]
    return dict(pos_ij=_t(g["pos_ij"], dev), tvecs=_t(b.trans_vec, dev), batch=_t(g["batch"], dev),
                edges=_t(g["edges"], dev), rvlen=_t(g["rvlen"], dev), sizes=_t(b.sizes, dev))


@pytest.mark.parametrize("workload,nc", [("cfg1", None), ("cfg2", 24)])
def test_pair_list_bit_exact(workload, nc):
    dev = _cuda()
    from crystalframer_b200.encoder import build_pair_list
    from crystalframer_b200.cuda_funcs import csr_offsets
    P = make_problem(workload, num_crystals=nc)
    g = _geometry(P, dev)
    edges, e_start, batch, cstart = build_pair_list(g["sizes"])
    assert torch.equal(edges.cpu(), torch.from_numpy(P["geo"]["edges"]))
    assert torch.equal(e_start.cpu(), torch.from_numpy(P["geo"]["e_start"]))
    assert torch.equal(batch.cpu(), torch.from_numpy(P["geo"]["batch"]))
    assert cstart[-1].item() == P["batch"].num_atoms
    # CSR offsets rebuilt from a foreign pair list
    e2 = csr_offsets(g["edges"], P["batch"].num_atoms)
    assert torch.equal(e2.cpu(), torch.from_numpy(P["geo"]["e_start"]))


@pytest.mark.parametrize("workload,nc", [("cfg1", None), ("cfg2", 24)])
def test_max_frames(workload, nc):
    dev = _cuda()
    from oracle import oracle as O
    F = _configure()
    P = make_problem(workload, num_crystals=nc)
    g = _geometry(P, dev)
    qs = P["q"] / 4.0
    want = O.max_frames(P["cfg"], qs, P["k"], P["a"], P["geo"]["pos_ij"], P["batch"].trans_vec, P["geo"]["rvlen"],
                        P["geo"]["batch"], P["geo"]["edges"], P["geo"]["e_start"])
    q, k, a = _t(qs, dev), _t(P["k"], dev), _t(P["a"], dev)
    f1, se1, si1 = F.max_frame_with_selection(1, q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5)
    assert np.array_equal(se1.cpu().numpy(), want["sel_edge1"])
    assert np.array_equal(si1.cpu().numpy(), want["sel_image1"])
    assert np.array_equal(f1.cpu().numpy(), want["frame1"])          # bit-exact: same IEEE operations
    f2, se2, si2 = F.max_frame_with_selection(2, q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5, f1)
    same = (se2.cpu().numpy() == want["sel_edge2"]) & (si2.cpu().numpy() == want["sel_image2"])
    # the second axis' score contains logf, whose last bit differs between CUDA and glibc: a differing selection
    # must be a tie at float32 resolution (both candidates' float64 scores within rounding), and rare
    from parity_util import adjudicate_second_axis
    n_diff = adjudicate_second_axis(P, want["frame1"], se2.cpu().numpy(), si2.cpu().numpy(), want["sel_edge2"],
                                    want["sel_image2"])
    assert n_diff <= max(1, same.size // 1000), f"second-axis selection differs on {n_diff} of {same.size}"
    _close("frame2_max", f2.cpu().numpy()[same], want["frame2_max"][same], 1e-6, 1e-6)
    # fused launch: all three completed axes
    g1, g2, g3 = F.max_frames_fused(q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5)
    assert np.array_equal(g1.cpu().numpy(), want["frame1"])
    _close("frame2", g2.cpu().numpy()[same], want["frame2"][same], 1e-5, 1e-6)
    _close("frame3", g3.cpu().numpy()[same], want["frame3"][same], 1e-5, 1e-6)


def test_max_frames_with_symmetry_breaking_noise():
    """Noise on: the library and the oracle share the counter-based noise, so the selected pair and
    image must still agree (first axis exactly; second axis up to logf near-ties)."""
    dev = _cuda()
    from oracle import oracle as O
    F = _configure(noise=1e-5)
    P = make_problem("cfg1", noise=1e-5)
    g = _geometry(P, dev)
    qs = P["q"] / 4.0
    q, k, a = _t(qs, dev), _t(P["k"], dev), _t(P["a"], dev)
    np.random.seed(77)
    f1, se1, si1 = F.max_frame_with_selection(1, q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5)
    f2, se2, si2 = F.max_frame_with_selection(2, q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"], g["rvlen"], -3.5, f1)
    np.random.seed(77)
    draw = lambda: int(np.random.randint(np.iinfo(np.int64).min, np.iinfo(np.int64).max, dtype=np.int64)) & (2 ** 64 - 1)
    s1, s2 = draw(), draw()
    want = O.max_frames(P["cfg"], qs, P["k"], P["a"], P["geo"]["pos_ij"], P["batch"].trans_vec, P["geo"]["rvlen"],
                        P["geo"]["batch"], P["geo"]["edges"], P["geo"]["e_start"], seed1=s1, seed2=s2)
    assert np.array_equal(se1.cpu().numpy(), want["sel_edge1"]) and np.array_equal(si1.cpu().numpy(), want["sel_image1"])
    assert np.array_equal(f1.cpu().numpy(), want["frame1"])
    same = (se2.cpu().numpy() == want["sel_edge2"]) & (si2.cpu().numpy() == want["sel_image2"])
    assert same.mean() >= 0.995
    _configure(noise=0.0)


@pytest.mark.parametrize("noise", [0.0, 1e-5])
def test_weighted_pca_frames(noise):
    """Weighted-PCA frames: right-handed orthonormal triads whose un-signed rows diagonalise the
    pooled second-moment matrix of the oracle, and agreement with the oracle's frames wherever the
    eigenvalues are well separated (near-degenerate eigenvectors are not comparable)."""
    dev = _cuda()
    from oracle import oracle as O
    F = _configure(noise=noise)
    P = make_problem("cfg1", noise=noise)
    g = _geometry(P, dev)
    qs = P["q"] / 4.0
    q, k, a = _t(qs, dev), _t(P["k"], dev), _t(P["a"], dev)
    f1, f2, f3, seed_noise, seed_sign = F.weighted_pca_frames(q, k, a, g["pos_ij"], g["tvecs"], g["batch"], g["edges"],
                                                              g["rvlen"], -3.5)
    Fg = torch.stack([f1, f2, f3], dim=-2).cpu().numpy().astype(np.float64)          # (N,H,row,3)
    want, mats, evals = O.weighted_pca_frames(P["cfg"], qs, P["k"], P["a"], P["geo"]["pos_ij"], P["batch"].trans_vec,
                                              P["geo"]["rvlen"], P["geo"]["batch"], P["geo"]["edges"], P["geo"]["e_start"],
                                              seed_noise, seed_sign)
    assert np.abs(np.einsum("nhrc,nhsc->nhrs", Fg, Fg) - np.eye(3)).max() < 1e-5
    assert np.abs(np.linalg.det(Fg) - 1.0).max() < 1e-5
    # frame_r = s_r * (row r of V), the columns of V being eigenvectors of M; so with S = diag(s) the
    # matrix of frames F = S V satisfies F^T (S M S) F = diag(eigenvalues), ascending
    N, H = P["a"].shape
    S = np.array([[[1.0 if O.hash_uniform(seed_sign, i * H + h, r) > 0.5 else -1.0 for r in range(3)]
                   for h in range(H)] for i in range(N)])
    SMS = mats * S[..., :, None] * S[..., None, :]
    D = np.einsum("nhrc,nhrs,nhsd->nhcd", Fg, SMS, Fg)
    off = D - np.einsum("nhcc->nhc", D)[..., None] * np.eye(3)
    assert np.abs(off).max() < 1e-4 * max(1.0, np.abs(mats).max())
    lam = np.einsum("nhcc->nhc", D)
    assert (np.diff(lam, axis=-1) > -1e-4).all()
    _close("eigenvalues", lam, evals, 1e-4, 1e-4)
    gap = np.minimum(evals[..., 1] - evals[..., 0], evals[..., 2] - evals[..., 1]) / np.maximum(evals[..., 2], 1e-9)
    ok = gap > 1e-2
    Fw = np.stack([want[0], want[1], want[2]], axis=-2).astype(np.float64)
    agree = np.abs(Fg - Fw).max(axis=(-1, -2)) < 1e-3
    assert ok.mean() > 0.8 and agree[ok].mean() > 0.97, (ok.mean(), agree[ok].mean())
    _configure(noise=0.0)


def _frames(P):
    from oracle import oracle as O
    fr = O.max_frames(P["cfg"], P["q"] / 4.0, P["k"], P["a"], P["geo"]["pos_ij"], P["batch"].trans_vec,
                      P["geo"]["rvlen"], P["geo"]["batch"], P["geo"]["edges"], P["geo"]["e_start"])
    return np.stack([fr["frame1"], fr["frame2"], fr["frame3"]])


@pytest.mark.parametrize("workload,nc,angles,wscales,coefs", [
    ("cfg1", None, 64, (1.0, 4.0), (1.0, 1.0)), ("cfg2", 24, 64, (1.0, 4.0), (1.0, 1.0)), ("cfg1", None, 0, (1.0, 4.0), (1.0, 1.0)),
    ("cfg1", None, 64, (1.5, 3.0), (1.0, 1.0)),          # other window widths: 13 distance, 25 angle
    ("cfg1", None, 64, (8.0, 8.0), (1.0, 1.0)),          # windows wider than the bases: every Gaussian is evaluated
    # the reference's lightweight recipe (train_jarvis_time.sh:41-57): 16 angle Gaussians of width scale 1.0 (un-windowed),
    # distance coefficient 1.5, angle coefficient 6.0
    ("cfg1", None, 16, (1.0, 1.0), (1.5, 6.0)), ("cfg2", 24, 16, (1.0, 1.0), (1.5, 6.0)),
    ("cfg1", None, 48, (1.0, 4.0), (1.0, 1.0)),          # 48 angle Gaussians: windowed (33 of 48), second register slot half used
])
def test_framed_proj_forward_backward(workload, nc, angles, wscales, coefs):
    dev = _cuda()
    from oracle import oracle as O
    F = _configure(angle_dim=angles, wscale_d=wscales[0], wscale_a=wscales[1], c_dist=coefs[0], c_ang=coefs[1])
    P = make_problem(workload, num_crystals=nc)
    P["cfg"] = O.Config(wscale_dist=wscales[0], wscale_ang=wscales[1], D_ang=max(angles, 1), c_dist=coefs[0], c_ang=coefs[1])
    if angles not in (0, 64):
        bound = (angles ** -0.5) * np.sqrt(6.0 / (angles + 8 * 16))
        P["W_a"] = P["rng"].uniform(-bound, bound, size=(3, 8, 16, angles)).astype(np.float32)
    g = _geometry(P, dev)
    frames = _frames(P) if angles else None
    W_a = P["W_a"] if angles else None
    geo, b = P["geo"], P["batch"]
    z_w, v_w = O.framed_proj_fwd(P["cfg"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 P["W_d"], W_a, frames)
    a = _t(P["a"], dev).requires_grad_(True)
    Wd = _t(P["W_d"][None], dev).requires_grad_(True)
    if angles:
        Ws = [_t(P["W_a"][x][None], dev).requires_grad_(True) for x in range(3)]
        fs = [_t(frames[x], dev) for x in range(3)]
    else:
        Ws, fs = [None] * 3, [None] * 3
    z, v = F.RealEncodingWithFramedProjFuncCUDA.apply(
        a, g["pos_ij"], None, g["tvecs"], g["batch"], g["edges"], 64, 14.0, wscales[0], Wd, *Ws, *fs, angles, wscales[1], 0,
        coefs[0], coefs[1], g["rvlen"], -3.5)
    _close("z", z.detach().cpu().numpy(), z_w)
    _close("values", v.detach().cpu().numpy(), v_w)
    rng = np.random.default_rng(7)
    gz = rng.normal(size=z_w.shape).astype(np.float32)
    gv = rng.normal(size=v_w.shape).astype(np.float32)
    ga_w, gWd_w, gWa_w = O.framed_proj_bwd(P["cfg"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                                           geo["edges"], geo["e_start"], P["W_d"], W_a, frames, z_w, gz, gv)
    z64, v64 = O.framed_proj_fwd(P["cfg"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 P["W_d"], W_a, frames, dtype=np.float64)
    ga_64, gWd_64, gWa_64 = O.framed_proj_bwd(P["cfg"], P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                                          geo["edges"], geo["e_start"], P["W_d"], W_a, frames, z64, gz, gv,
                                          dtype=np.float64)
    (z * _t(gz, dev)).sum().add((v * _t(gv, dev)).sum()).backward()
    _close_reduction("ga", a.grad.cpu().numpy(), ga_w, ga_64)
    _close_reduction("gW_dist", Wd.grad.cpu().numpy()[0], gWd_w, gWd_64)
    if angles:
        for x in range(3):
            _close_reduction(f"gW_ang{x + 1}", Ws[x].grad.cpu().numpy()[0], gWa_w[x], gWa_64[x])
    from crystalframer_b200 import _lib
    assert _lib.read_status() == 0


def test_unwindowed_encoding_forward_backward():
    """frame_method "no" (plain Crystalformer, the baseline of the large-cell workload): every
    distance Gaussian, no frames."""
    dev = _cuda()
    from oracle import oracle as O
    F = _configure(angle_dim=0)
    P = make_problem("cfg1")
    cfg = O.Config(cut_sigma=32, D_ang=0)
    g = _geometry(P, dev)
    geo, b = P["geo"], P["batch"]
    z_w, v_w = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 P["W_d"], None, None)
    a = _t(P["a"], dev).requires_grad_(True)
    Wd = _t(P["W_d"][None], dev).requires_grad_(True)
    z, v, _, _ = F.RealPeriodicEncodingWithProjFuncCUDA.apply(a, g["pos_ij"], None, g["tvecs"], g["batch"], g["edges"], 64,
                                                              14.0, 1.0, Wd, "no", g["rvlen"], -3.5)
    _close("z", z.detach().cpu().numpy(), z_w)
    _close("values", v.detach().cpu().numpy(), v_w)
    rng = np.random.default_rng(23)
    gz, gv = rng.normal(size=z_w.shape).astype(np.float32), rng.normal(size=v_w.shape).astype(np.float32)
    ga_w, gW_w, _ = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                      geo["e_start"], P["W_d"], None, None, z_w, gz, gv)
    z64, _ = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"], P["W_d"],
                               None, None, dtype=np.float64)
    ga_64, gW_64, _ = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                        geo["e_start"], P["W_d"], None, None, z64, gz, gv, dtype=np.float64)
    (z * _t(gz, dev)).sum().add((v * _t(gv, dev)).sum()).backward()
    _close_reduction("ga", a.grad.cpu().numpy(), ga_w, ga_64)
    _close_reduction("gW", Wd.grad.cpu().numpy()[0], gW_w, gW_64)


@pytest.mark.parametrize("workload,nc", [("cfg1", None), ("cfg2", 24)])
def test_attention_forward_backward(workload, nc):
    dev = _cuda()
    from oracle import oracle as O
    F = _configure()
    P = make_problem(workload, num_crystals=nc)
    g = _geometry(P, dev)
    geo = P["geo"]
    rng = np.random.default_rng(11)
    E = geo["edges"].shape[1]
    zb = rng.normal(size=(E, 8)).astype(np.float32)
    vb = rng.normal(size=(E, 8, 16)).astype(np.float32) * 0.1
    qs = P["q"] / 4.0
    out_w, prob_w = O.dpa_fwd(P["cfg"], qs, P["k"], P["v"], zb, vb, geo["edges"], geo["e_start"])
    go = rng.normal(size=out_w.shape).astype(np.float32)
    want = O.dpa_bwd(P["cfg"], qs, P["k"], P["v"], vb, geo["edges"], geo["e_start"], prob_w, out_w, go)
    T = [_t(x, dev).requires_grad_(True) for x in (qs, P["k"], P["v"], zb, vb)]
    out = F.FusedDotProductAttentionCUDA.apply(*T, g["batch"], g["edges"])
    _close("out", out.detach().cpu().numpy(), out_w)
    out.backward(_t(go, dev))
    for name, t, w in zip(["gq", "gk", "gv", "gz", "gvalues"], T, want):
        _close(name, t.grad.cpu().numpy(), w)
    _, prob, _ = F.attention_probabilities(*[t.detach() for t in T], g["edges"])
    _close("prob", prob.cpu().numpy(), prob_w)
    # without biases
    out2_w, _ = O.dpa_fwd(P["cfg"], qs, P["k"], P["v"], None, None, geo["edges"], geo["e_start"])
    out2 = F.FusedDotProductAttentionCUDA.apply(T[0].detach(), T[1].detach(), T[2].detach(), None, None, g["batch"], g["edges"])
    _close("out(no bias)", out2.cpu().numpy(), out2_w)


def test_mean_pool():
    dev = _cuda()
    from oracle import oracle as O
    from crystalframer_b200.cuda_funcs import IrregularMeanCUDA
    P = make_problem("cfg2", num_crystals=40)
    N = P["batch"].num_atoms
    x = np.random.default_rng(3).normal(size=(N, 128)).astype(np.float32)
    xt = _t(x, dev).requires_grad_(True)
    g = _geometry(P, dev)
    out = IrregularMeanCUDA.apply(xt, g["batch"], g["sizes"])
    _close("mean", out.detach().cpu().numpy(), O.mean_fwd(x, P["batch"].sizes))
    go = np.random.default_rng(4).normal(size=(len(P["batch"].sizes), 128)).astype(np.float32)
    out.backward(_t(go, dev))
    _close("mean grad", xt.grad.cpu().numpy(), O.mean_bwd(go, P["batch"].sizes))
    out2 = IrregularMeanCUDA.apply(xt.detach(), g["batch"], None)
    assert torch.equal(out2, out.detach())


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("layers,frame_method", [(1, "max"), (4, "max"), (2, "no"), (2, "weighted_pca"), (2, "max_static"),
                                                 (2, "lattice"), (2, "pca")])
def test_whole_model_against_cpu_oracle(layers, frame_method, fused):
    _whole_model_check(layers, frame_method, fused)


def test_whole_model_with_head_options():
    """The reference's head options -- a per-atom projection before pooling, layer normalisation inside the head --
    around the one-call layers, against the CPU oracle."""
    _whole_model_check(1, "max", True, pre_pooling_op="w+relu", norm_type="ln", embedding_dim=[96, 64])


@pytest.mark.parametrize("gauss_state", ["x", "1"])
def test_whole_model_other_coefficient_sources(gauss_state):
    """Gaussian coefficients from the layer's input ("x") or one learned constant per head ("1") instead of the
    projected query: the whole model, operator by operator, against the CPU oracle."""
    _whole_model_check(1, "max", False, gauss_state=gauss_state)


def test_whole_model_without_orthogonalisation():
    """Frame method "max_wo_orthogonal" (second axis as selected, third axis selected with the triple product): the
    whole model against the CPU oracle; it runs operator by operator."""
    _whole_model_check(2, "max_wo_orthogonal", False)


@pytest.mark.parametrize("workload,nc", [("cfg1", None), ("cfg2", 24)])
def test_third_axis_selection(workload, nc):
    """cfb200_max_frame3 through the drop-in Function: selected pair and direction against the oracle (bit-exact but
    for the few atoms where the logarithm's last bit decides), all three axes linearly independent."""
    dev = _cuda()
    from oracle import oracle as O
    F = _configure()
    P = make_problem(workload, num_crystals=nc)
    g = _geometry(P, dev)
    qs = (P["q"] / 4.0).astype(np.float32)
    want = O.max_frames_wo_orthogonal(P["cfg"], qs, P["k"], P["a"], P["geo"]["pos_ij"], P["batch"].trans_vec,
                                      P["geo"]["rvlen"], P["geo"]["batch"], P["geo"]["edges"], P["geo"]["e_start"])
    f1, f2 = _t(want["frame1"], dev), _t(want["frame2"], dev)
    f3, sel = F.max_frame3_with_selection(_t(qs, dev), _t(P["k"], dev), _t(P["a"], dev), g["pos_ij"], g["tvecs"], g["batch"],
                                          g["edges"], g["rvlen"], -3.5, f1, f2)
    same = sel.cpu().numpy() == want["sel_edge3"]
    assert same.mean() >= 0.999, same.mean()
    assert np.array_equal(f3.cpu().numpy()[same], want["frame3"][same])
    M = np.stack([want["frame1"], want["frame2"], f3.cpu().numpy()], axis=-2).astype(np.float64)
    assert (np.abs(np.linalg.det(M)) > 1e-5).all()
    out = F.ComputeFrame3MaximumMethodCUDA.apply(_t(qs, dev), _t(P["k"], dev), None, _t(P["a"], dev), g["pos_ij"], None,
                                                 g["tvecs"], g["batch"], g["edges"], 64, 14.0, 1.0, f1, f2, g["rvlen"], -3.5)
    assert torch.equal(out, f3)


@pytest.mark.parametrize("fused", [False, True])
def test_whole_model_lightweight_recipe(fused):
    """The reference's second efficiency recipe (train_jarvis_time.sh:41-57): 16 angle Gaussians of width scale 1.0,
    distance coefficient 1.5, angle coefficient 6.0, max frames -- the whole model against the CPU oracle."""
    _whole_model_check(2, "max", fused, value_pe_angle_real=16, value_pe_angle_wscale=1.0, value_pe_dist_coef=1.5,
                       value_pe_angle_coef=6.0)


@pytest.mark.parametrize("domain,frame_method", [("real-reci", "max"), ("RECI", "no"), ("reci", "no"), ("multihead", "no")])
def test_whole_model_reciprocal_domains(domain, frame_method):
    """Layers with the reciprocal-space logit bias (alone, inverted, alternating with CrystalFramer layers, and on
    half of the heads beside the plain real-space encoding on the other half) in the whole model against the CPU
    oracle."""
    _whole_model_check(2, frame_method, False, domain=domain)


def _reciprocal_inputs(P, scale, H=None):
    from oracle import oracle as O
    geo, b = P["geo"], P["batch"]
    rvecs, vcell, kr = O.reciprocal_geometry(b.pos, b.trans_vec, b.sizes, geo["edges"])
    a = (P["a"] * scale).astype(np.float32)
    if H is not None:
        a = np.ascontiguousarray(np.tile(a, (1, 2))[:, :H] * np.linspace(0.7, 1.3, H, dtype=np.float32))
    return a, kr, rvecs, vcell


@pytest.mark.parametrize("H", [8, 4, 12])
def test_reciprocal_encoding(H):
    """cfb200_reci_enc_fwd / _bwd through the drop-in Function against the oracle (float32, and float64 as the
    judge of disagreements) on 24 crystals, for the configured head count, the half the "multihead" domain would
    pass, and one that needs two passes over the pairs.  The logit is compared where the lattice sum is not
    rounding noise (sum > 1e-3: below, log() amplifies the last bits of a sum of 75 terms of order one), the sum
    itself everywhere; the upstream gradient is zero on those pairs so that the coefficient gradient is
    well-conditioned too."""
    dev = _cuda()
    from oracle import oracle as O
    F = _configure()
    P = make_problem("cfg2", num_crystals=24)
    g = _geometry(P, dev)
    a, kr, rvecs, vcell = _reciprocal_inputs(P, 9.5, H)
    at = _t(a, dev).requires_grad_(True)
    z = F.ReciPeriodicEncodingFuncCUDA.apply(at, _t(kr, dev), _t(rvecs, dev), _t(vcell, dev), g["batch"], g["edges"])
    zo, so = O.reci_enc_fwd(a, kr, rvecs, vcell, P["geo"]["batch"], P["geo"]["edges"])
    z64, s64 = O.reci_enc_fwd(a, kr, rvecs, vcell, P["geo"]["batch"], P["geo"]["edges"], dtype=np.float64)
    ok = s64 > 1e-3
    assert ok.mean() > 0.5
    _close("z", z.detach().cpu().numpy()[ok], zo[ok], 1e-4, 1e-4)
    got_sum = np.exp(z.detach().cpu().numpy().astype(np.float64)
                     - (1.5 * np.log(-4 * np.pi * a.astype(np.float64)) - np.log(vcell.astype(np.float64))[P["geo"]["batch"], None])[P["geo"]["edges"][0]])
    assert np.abs(got_sum - np.maximum(s64, 1e-6))[ok].max() <= 3 * np.abs(so - s64)[ok].max() + 1e-5
    gz = (np.random.default_rng(5).normal(size=zo.shape) * (s64 > 1e-2)).astype(np.float32)
    z.backward(_t(gz, dev))
    gao = O.reci_enc_bwd(a, kr, rvecs, P["geo"]["batch"], P["geo"]["edges"], gz, so)
    ga64 = O.reci_enc_bwd(a, kr, rvecs, P["geo"]["batch"], P["geo"]["edges"], gz, s64, dtype=np.float64)
    _close_reduction("ga", at.grad.cpu().numpy(), gao, ga64)


def test_reciprocal_encoding_golden_and_reference_gpu():
    """The reciprocal encoding against the committed outputs of the reference's kernels and of its pure-PyTorch
    twin, and -- where the reference kernels' GPU build is present -- against those kernels on the same GPU."""
    import os
    dev = _cuda()
    F = _configure()
    G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_reci_small.npz"))
    small = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels_small.npz"))
    batch = _t(np.repeat(np.arange(len(small["sizes"])), small["sizes"]), dev)
    at = _t(G["a"], dev).requires_grad_(True)
    args = (_t(G["kr"], dev), _t(G["rvecs"], dev), _t(G["vcell"], dev), batch, _t(G["edges"], dev))
    z = F.ReciPeriodicEncodingFuncCUDA.apply(at, *args)
    _close("z", z.detach().cpu().numpy(), G["z"], 1e-5, 1e-5)
    _close("z (pure twin)", z.detach().cpu().numpy(), G["z_pure"], 1e-4, 1e-5)
    z.backward(_t(G["gz"], dev))
    _close("ga", at.grad.cpu().numpy(), G["ga"], 1e-4, 1e-4)
    _close("ga (pure twin)", at.grad.cpu().numpy(), G["ga_pure"], 1e-4, 1e-4)
    from oracle import reference as R
    if not R.available("cuda"):
        return
    P = make_problem("cfg2", num_crystals=24)
    g = _geometry(P, dev)
    a, kr, rvecs, vcell = _reciprocal_inputs(P, 9.5)
    rk = R.RefKernels("cuda")
    at = _t(a, dev).requires_grad_(True)
    targs = (_t(kr, dev), _t(rvecs, dev), _t(vcell, dev), g["batch"], g["edges"])
    z = F.ReciPeriodicEncodingFuncCUDA.apply(at, *targs)
    zr, sr = rk.reci_fwd(at.detach(), *targs)
    ok = (sr > 1e-3).cpu().numpy()
    _close("z vs reference kernels", z.detach().cpu().numpy()[ok], zr.cpu().numpy()[ok], 1e-4, 1e-4)
    gz = (torch.randn_like(zr) * (sr > 1e-2)).contiguous()
    z.backward(gz)
    gar = rk.reci_bwd(at.detach(), *targs, zr, gz, sr)
    _close("ga vs reference kernels", at.grad.cpu().numpy(), gar.cpu().numpy(), 1e-4, 1e-5 * max(1.0, float(gar.abs().max())))


def test_whole_model_largest_cell_and_single_atoms():
    """The one-call layers on a batch that holds the reference's largest cell (320 atoms, 102 400 pairs: its atoms'
    tasks are cut into chunks) beside single-atom crystals and a small one, against the CPU oracle."""
    from crystalframer_b200 import synth
    big = synth.make_batch(1, 9, size_dist="uniform", size_lo=320, size_hi=320, len_lo=18.0, len_hi=22.0)
    ones = synth.make_batch(3, 10, size_dist="uniform", size_lo=1, size_hi=1, len_lo=3.0, len_hi=6.0)
    small = synth.make_batch(1, 11, size_dist="uniform", size_lo=7, size_hi=7, len_lo=4.0, len_hi=8.0)
    _whole_model_check(1, "max", True, batch=synth.concat([ones, big, small]))


def _whole_model_check(layers, frame_method, fused, batch=None, **recipe):
    """Forward and backward of the whole model (species embedding, encoder layers, mean pooling,
    MLP head) on the GPU against the same weights run on the host cores through the oracle:
    8 crystals of 4-16 atoms, float32, symmetry-breaking noise off.

    ``fused=False``: the first training forward, which measures the coefficient statistics and runs
    operator by operator.  ``fused=True``: the statistics are in place, so every layer runs as the
    one-node fused layer -- the path the benchmark times; the test checks that it was taken.
    Weighted-PCA and pca frames are compared in their own tests (eigenvectors are not comparable where
    eigenvalues nearly coincide); here the CPU model receives the frames the GPU constructed, so
    everything downstream of the frames is compared."""
    dev = _cuda()
    import copy
    from crystalframer_b200 import _lib, data, encoder, fused_layer, synth
    from crystalframer_b200.latticeformer import Latticeformer, ModelParams
    from oracle import cpu_model
    torch.manual_seed(0)
    kw = dict(num_layers=layers, symm_break_noise=0.0, frame_method=frame_method,
              value_pe_angle_real=0 if frame_method == "no" else 64)
    kw.update(recipe)
    mp = ModelParams(**kw)
    cpu = Latticeformer(mp).train()
    gpu = copy.deepcopy(cpu).to(dev).train()
    from crystalframer_b200 import cuda_funcs as F
    F.compile_kernels(2, 8, 16, 64, mp.value_pe_angle_real, 16, True, 0, mp.value_pe_dist_wscale, mp.value_pe_angle_wscale,
                      mp.value_pe_dist_coef, mp.value_pe_angle_coef, 0.0)
    b = synth.make_workload("cfg1") if batch is None else batch
    y = np.random.default_rng(0).normal(size=(len(b.sizes), 1)).astype(np.float32)
    tb = data.host_batch(b, y, pinned=False).to(dev, non_blocking=False)
    if fused:
        with torch.no_grad():
            gpu(tb)                                   # measures gauss_scale; the next forward takes the fused layers
        for lg, lc in zip(gpu.encoder.layers, cpu.encoder.layers):
            with torch.no_grad():
                lc.self_attn.gauss_scale.copy_(lg.self_attn.gauss_scale.cpu())
    calls = []
    orig_invoke = _lib.invoke
    _lib.invoke = lambda name, *a, **k: (calls.append(name), orig_invoke(name, *a, **k))[1]
    fused_layer.FRAME_TAP = tap = []
    try:
        out = gpu(tb)
        loss = (out - tb.y).abs().mean()
        loss.backward()
    finally:
        _lib.invoke = orig_invoke
        fused_layer.FRAME_TAP = None
    n_fused = sum(1 for c in calls if c in fused_layer.FUSED_FORWARD_CALLS)
    assert n_fused == (layers if fused else 0), (n_fused, sorted(set(calls)))
    frames = None
    if frame_method in ("weighted_pca", "pca"):
        assert len(tap) == layers
        frames = [f.cpu() for f in tap]
    out_c = cpu_model.forward(cpu, b, backend="port", frames=frames)
    loss_c = (out_c - torch.from_numpy(y)).abs().mean()
    loss_c.backward()
    _close("prediction", out.detach().cpu().numpy(), out_c.detach().numpy(), 1e-4, 1e-5)
    for l in range(layers):
        assert torch.allclose(gpu.encoder.layers[l].self_attn.gauss_scale.cpu(), cpu.encoder.layers[l].self_attn.gauss_scale,
                              rtol=1e-4, atol=1e-6)
    for (n, pg), (_, pc) in zip(gpu.named_parameters(), cpu.named_parameters()):
        if pc.grad is None:
            assert pg.grad is None or float(pg.grad.abs().max()) == 0.0, n
            continue
        assert pg.grad is not None, n
        g, c = pg.grad.cpu().numpy().astype(np.float64), pc.grad.numpy().astype(np.float64)
        scale = max(np.abs(c).max(), 1e-8)
        bad = np.abs(g - c) > 2e-3 * scale + 1e-7
        # A ReLU unit whose pre-activation is within rounding of zero for some atom may be switched on in one
        # implementation and off in the other (the activations themselves agree: the unit's output is ~0 either
        # way).  That moves one atom's contribution in that unit's row of the feed-forward input weights and
        # bias -- about 1/atoms of the row's gradient.  Up to two such rows per layer are tolerated there, and
        # only there; everything else must agree entry by entry.
        if n.endswith("linear1.weight"):
            rows = bad.any(axis=1)
            assert rows.sum() <= 2 and np.abs(g - c).max() <= 5e-2 * scale, \
                f"{n}: {rows.sum()} rows differ, max abs diff {np.abs(g - c).max():.3e} at scale {scale:.3e}"
        elif n.endswith("linear1.bias"):
            assert bad.sum() <= 2 and np.abs(g - c).max() <= 5e-2 * scale, f"{n}: {bad.sum()} entries differ"
        else:
            assert not bad.any(), f"{n}: max abs diff {np.abs(g - c).max():.3e} at scale {scale:.3e}"


def test_pca_frames():
    """cfb200_pca_frames through the drop-in Function against the oracle: the axes are the eigenvectors of the
    scatter matrix of each atom's pair separations (ascending eigenvalue), identical for all heads up to the drawn
    signs, orthonormal and right-handed; where the eigenvalues are well separated the axes equal the oracle's, signs
    included."""
    dev = _cuda()
    from oracle import oracle as O
    F = _configure()
    P = make_problem("cfg2", num_crystals=24)
    g = _geometry(P, dev)
    N, H = P["a"].shape
    qs = _t((P["q"] / 4.0).astype(np.float32), dev)
    torch.manual_seed(7)
    f1, f2, f3 = F.ComputePCAFrame.apply(qs, _t(P["k"], dev), None, _t(P["a"], dev), g["pos_ij"], None, g["tvecs"], g["batch"],
                                         g["edges"], 64, 14.0, 1.0, g["rvlen"], -3.5)
    torch.manual_seed(7)
    seed = int(torch.randint(0, 2 ** 62, (1,)).item())
    want, mats, evals = O.pca_frames(P["geo"]["pos_ij"], P["geo"]["e_start"], H, seed)
    got = np.stack([f1.cpu().numpy(), f2.cpu().numpy(), f3.cpu().numpy()])          # (3,N,H,3)
    Fm = np.moveaxis(got, 0, 2).astype(np.float64)                                     # (N,H,axis,component)
    gram = Fm @ np.swapaxes(Fm, -1, -2)
    assert np.abs(gram - np.eye(3)).max() < 1e-4 and np.abs(np.linalg.det(Fm) - 1.0).max() < 1e-4
    scale = np.maximum(evals[:, 2], 1e-12)
    gaps = np.minimum(evals[:, 1] - evals[:, 0], evals[:, 2] - evals[:, 1]) / scale
    clear = gaps > 1e-2                                                                # atoms with three distinct axes
    assert clear.sum() > N // 2
    for r in range(3):                                                                  # eigenvector equation
        v = Fm[:, 0, r, :]
        resid = np.einsum("nij,nj->ni", mats, v) - evals[:, r, None] * v
        assert (np.abs(resid).max(1)[clear] <= 2e-4 * scale[clear]).all()
    dots = np.abs((got.astype(np.float64) * want.astype(np.float64)).sum(-1))            # (3,N,H)
    assert (dots[:, clear] > 1.0 - 1e-4).all()
    same = np.abs(got - want).max(axis=(0, 3)) < 1e-3                                   # (N,H): signs included
    assert same[clear].mean() > 0.9
    from crystalframer_b200 import _lib
    assert _lib.read_status(dev) == 0


@pytest.mark.parametrize("saved", [False, True])
@pytest.mark.parametrize("workload,nc,use_list", [("cfg1", None, True), ("cfg2", 24, True), ("cfg2", 24, False)])
def test_fused_attention_entry_points(workload, nc, use_list, saved):
    """cfb200_attn_fused_fwd / _bwd (lattice sums + value encoding + attention in one pass) against the CPU oracle's
    chain of the separate operators.  saved: the forward keeps per-pair results and the backward uses them; else the
    lighter forward, and the backward recomputes the lattice sums."""
    dev = _cuda()
    from oracle import oracle as O
    from crystalframer_b200 import _lib
    _configure()
    P = make_problem(workload, num_crystals=nc)
    g = _geometry(P, dev)
    geo, b, cfg = P["geo"], P["batch"], P["cfg"]
    frames = _frames(P)
    qs = (P["q"] / 4.0).astype(np.float32)
    z_w, v_w = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 P["W_d"], P["W_a"], frames)
    out_w, prob_w = O.dpa_fwd(cfg, qs, P["k"], P["v"], z_w, v_w, geo["edges"], geo["e_start"])
    rng = np.random.default_rng(11)
    go = rng.normal(size=out_w.shape).astype(np.float32)
    gq_w, gk_w, gv_w, gz_w, gval_w = O.dpa_bwd(cfg, qs, P["k"], P["v"], v_w, geo["edges"], geo["e_start"], prob_w, out_w, go)
    ga_w, gWd_w, gWa_w = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                                           geo["edges"], geo["e_start"], P["W_d"], P["W_a"], frames, z_w, gz_w, gval_w)
    z64, v64 = O.framed_proj_fwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"],
                                 P["W_d"], P["W_a"], frames, dtype=np.float64)
    ga_64, gWd_64, gWa_64 = O.framed_proj_bwd(cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"],
                                              geo["edges"], geo["e_start"], P["W_d"], P["W_a"], frames, z64, gz_w, gval_w,
                                              dtype=np.float64)
    N, E, H, hd = P["a"].shape[0], geo["edges"].shape[1], 8, 16
    p, ip = _lib.ptr, _lib.iptr
    t = lambda x: _t(x, dev)
    q_, k_, v_, a_ = t(qs), t(P["k"]), t(P["v"]), t(P["a"])
    e_start = t(geo["e_start"])
    W = [t(P["W_d"])] + [t(P["W_a"][x]) for x in range(3)]
    f = [t(frames[x]) for x in range(3)]
    plist = None
    if use_list:
        plist = torch.empty(E, 5, 128, device=dev)
        _lib.invoke("cfb200_pair_cache", 2, dev, p(g["pos_ij"]), p(g["tvecs"]), ip(g["batch"]), ip(g["edges"]), N, E, 2,
                    None, p(plist))
    order = torch.argsort(e_start[1:] - e_start[:-1], descending=True, stable=True).to(torch.int32)
    counters = torch.zeros(8, dtype=torch.int32, device=dev)
    out, z, lse, spool = (torch.empty(s, device=dev) for s in ((N, H, hd), (E, H), (N, H), (N, H, 256)))
    common = (p(q_), p(k_), p(v_), p(a_), p(g["pos_ij"]), p(g["tvecs"]), p(g["rvlen"]), ip(g["batch"]), ip(g["edges"]),
              ip(e_start), p(order, torch.int32), p(counters, torch.int32), N, E, 14.0, -3.5, p(W[0]), p(W[1]), p(W[2]),
              p(W[3]), p(f[0]), p(f[1]), p(f[2]), p(plist), 2)
    keep = [torch.empty(s, device=dev) for s in ((E, H, hd), (E, H), (N, H, hd))] if saved else [None] * 3
    kp = [p(x) for x in keep]
    _lib.invoke("cfb200_attn_fused_fwd", 1, dev, *common, p(out), p(z), p(lse), p(spool), *kp, 0)
    if saved:
        _close("values", keep[0].cpu().numpy(), v_w)         # the stored value encoding is the operator's output
    _close("z", z.cpu().numpy(), z_w)
    _close("out", out.cpu().numpy(), out_w)
    gq, gk, gv, ga, gz = (torch.empty(s, device=dev) for s in ((N, H, hd), (N, H, hd), (N, H, hd), (N, H), (E, H)))
    _lib.invoke("cfb200_attn_fused_bwd", 2, dev, *common, p(out), p(z), p(lse), p(t(go)), p(gq), p(gk), p(gv), p(ga), p(gz),
                *kp, 0)
    # atoms are drawn from a work queue, so which warp computes which atom varies from run to run; no sum
    # crosses atoms, hence every output must repeat bit for bit
    out_b, z_b, lse_b, spool_b = (torch.empty_like(x) for x in (out, z, lse, spool))
    keep_b = [torch.empty_like(x) for x in keep] if saved else [None] * 3
    _lib.invoke("cfb200_attn_fused_fwd", 1, dev, *common, p(out_b), p(z_b), p(lse_b), p(spool_b), *[p(x) for x in keep_b], 0)
    assert not saved or all(torch.equal(x, y) for x, y in zip(keep, keep_b))
    assert all(torch.equal(x, y) for x, y in ((out, out_b), (z, z_b), (lse, lse_b), (spool, spool_b)))
    again = [torch.empty_like(x) for x in (gq, gk, gv, ga, gz)]
    _lib.invoke("cfb200_attn_fused_bwd", 2, dev, *common, p(out), p(z), p(lse), p(t(go)), *[p(x) for x in again], *kp, 0)
    assert all(torch.equal(x, y) for x, y in zip((gq, gk, gv, ga, gz), again))
    _close("gq", gq.cpu().numpy(), gq_w)
    _close("gk", gk.cpu().numpy(), gk_w)
    _close("gv", gv.cpu().numpy(), gv_w)
    _close("gz", gz.cpu().numpy(), gz_w)
    _close_reduction("ga", ga.cpu().numpy(), ga_w, ga_64)
    gW = torch.bmm(t(go).permute(1, 2, 0), spool.permute(1, 0, 2)).cpu().numpy()       # (H,16,256)
    _close_reduction("gW_dist", gW[:, :, :64], gWd_w, gWd_64)
    for x in range(3):
        _close_reduction(f"gW_ang{x + 1}", gW[:, :, 64 * (x + 1):64 * (x + 2)], gWa_w[x], gWa_64[x])
    assert _lib.read_status() == 0


@pytest.mark.parametrize("noise", [0.0, 1e-5])
@pytest.mark.parametrize("workload,nc", [("cfg1", None), ("cfg2", 48)])
def test_second_moment_records_with_and_without_sorted_lists(workload, nc, noise):
    """cfb200_sigma_edges_cached -- warp per pair over the prefix of the pair's sorted translation list -- and the
    sweep over the whole box (no list) against the oracle: logit and the six weight-averaged second moments within
    tolerance (the list kernel leaves out translations below the pruning threshold of the lattice-sum kernels),
    the nearest non-zero image (its distance with the noise term, its direction) identical between the two kernels
    and equal to the oracle's.  The small cells of the second workload have boxes wider than the listed one."""
    dev = _cuda()
    from crystalframer_b200 import _lib
    from crystalframer_b200.cuda_funcs.common import pair_geometry
    from oracle import oracle as O
    _configure(noise=noise)
    P = make_problem(workload, num_crystals=nc, noise=noise)
    g = _geometry(P, dev)
    N, H = P["a"].shape
    E = P["geo"]["edges"].shape[1]
    a = _t(P["a"], dev)
    seed = 0x1234ABCD5678
    _, plist, prange = pair_geometry(g["pos_ij"], g["tvecs"], g["batch"], g["edges"], -3.5)
    assert plist is not None and prange == 2
    p, ip = _lib.ptr, _lib.iptr
    rec = {}
    for name, lst in (("list", plist), ("sweep", None)):
        out = torch.full((E, H, 11), float("nan"), device=dev)
        _lib.invoke("cfb200_sigma_edges_cached", 1, dev, p(a), p(g["pos_ij"]), p(g["tvecs"]), p(g["rvlen"]), ip(g["batch"]),
                    ip(g["edges"]), N, E, -3.5, seed, p(out), p(lst), prange)
        rec[name] = out.cpu().numpy()
        assert np.isfinite(rec[name]).all(), name
    cfg = O.Config(symm_break_noise=noise)
    z, sig, nd2, ndir = O.sigma_edges(cfg, P["a"], P["geo"]["pos_ij"], P["batch"].trans_vec, P["geo"]["rvlen"],
                                      P["geo"]["batch"], P["geo"]["edges"], seed=seed)
    scale = max(1.0, float(np.abs(sig).max()))
    for name in ("list", "sweep"):
        _close(f"z ({name})", rec[name][..., 0], z, 1e-4, 1e-5)
        _close(f"moments ({name})", rec[name][..., 1:7], sig, 1e-4, 1e-5 * scale)
        _close(f"nearest d2 ({name})", rec[name][..., 7], nd2, 1e-6, 1e-7)
        _close(f"nearest direction ({name})", rec[name][..., 8:11], ndir, 1e-5, 1e-6)
    assert np.array_equal(rec["list"][..., 7:11], rec["sweep"][..., 7:11])
    _configure(noise=0.0)


@pytest.mark.parametrize("projected", [False, True])
def test_plain_real_space_encoding_function(projected):
    """RealPeriodicEncodingFuncCUDA: logit and the value sums of all 64 distance Gaussians, un-projected (E,H,64) or
    projected by W_k (E,H,16), and the gradients of the coefficients (and of W_k), against the oracle's un-windowed
    encoding."""
    dev = _cuda()
    from oracle import oracle as O
    F = _configure(angle_dim=0)
    P = make_problem("cfg1")
    g = _geometry(P, dev)
    geo, b = P["geo"], P["batch"]
    cfg = O.Config(cut_sigma=32, D_ang=0)
    a = _t(P["a"], dev).requires_grad_(True)
    W = _t(P["W_d"][None], dev).requires_grad_(True) if projected else None
    z, v = F.RealPeriodicEncodingFuncCUDA.apply(a, g["pos_ij"], None, g["tvecs"], g["batch"], g["edges"], 64, 14.0, 1.0, W,
                                                g["rvlen"], -3.5)
    rng = np.random.default_rng(31)
    gz = rng.normal(size=tuple(z.shape)).astype(np.float32)
    gv = rng.normal(size=tuple(v.shape)).astype(np.float32)
    (z * _t(gz, dev)).sum().add((v * _t(gv, dev)).sum()).backward()
    args = (cfg, P["a"], geo["pos_ij"], b.trans_vec, geo["rvlen"], geo["batch"], geo["edges"])
    if projected:
        zo, vo = O.framed_proj_fwd(*args, P["W_d"], None, None)
        ga_o, gW_o, _ = O.framed_proj_bwd(*args, geo["e_start"], P["W_d"], None, None, zo, gz, gv)
        ga64, gW64, _ = O.framed_proj_bwd(*args, geo["e_start"], P["W_d"], None, None, zo, gz, gv, dtype=np.float64)
        _close_reduction("gW", W.grad.cpu().numpy()[0], gW_o, gW64)
    else:
        vo = np.empty((geo["edges"].shape[1], 8, 64), np.float32)
        ga_o = np.zeros_like(P["a"])
        ga64 = np.zeros(P["a"].shape, np.float64)
        for blk in range(4):
            S = np.zeros((8, 16, 64), np.float32)
            S[:, np.arange(16), 16 * blk + np.arange(16)] = 1.0
            zo, vb = O.framed_proj_fwd(*args, S, None, None)
            vo[..., 16 * blk:16 * blk + 16] = vb
            gzb = gz if blk == 0 else np.zeros_like(gz)
            gvb = np.ascontiguousarray(gv[..., 16 * blk:16 * blk + 16])
            ga_o += O.framed_proj_bwd(*args, geo["e_start"], S, None, None, zo, gzb, gvb)[0]
            ga64 += O.framed_proj_bwd(*args, geo["e_start"], S, None, None, zo, gzb, gvb, dtype=np.float64)[0]
    _close("z", z.detach().cpu().numpy(), zo)
    _close("values", v.detach().cpu().numpy(), vo)
    _close_reduction("ga", a.grad.cpu().numpy(), ga_o, ga64)
    _configure()
