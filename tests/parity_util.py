"""Helpers shared by the GPU parity tests: tolerances, device transfer, and the adjudication of
frame selections that differ from the oracle's.

Tolerances: integer outputs bit-exact; float outputs and gradients within 1e-4 relative + 1e-5
absolute.  A second-axis selection may legitimately differ from the float32 oracle's when two
candidates tie at float32 resolution (the score contains logf, whose last bit differs between
libm and the GPU); ``adjudicate_second_axis`` accepts a differing selection only if the two
candidates' scores, recomputed in float64, differ by less than float32 rounding of the score.
"""
import numpy as np
import pytest
import torch

RTOL, ATOL = 1e-4, 1e-5


def cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def to_dev(x, dev):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev)


def close(name, got, want, rtol=RTOL, atol=ATOL, frac_ok=0.0):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert np.isfinite(got).all(), name
    err = np.abs(got - want)
    bad = err > atol + rtol * np.abs(want)
    assert bad.mean() <= frac_ok, f"{name}: {bad.sum()} of {bad.size} outside tolerance, max abs err {err.max():.3e}"


def close_reduction(name, got, want32, want64):
    """Coefficient and weight gradients are long sums of terms that largely cancel; float32
    accumulation noise alone (any summation order) reaches the elementwise bound on entries with
    heavy cancellation -- the float32 oracle itself is that far from the float64 oracle.  So the
    absolute term scales with the largest entry, and the error against the float64 value must
    not exceed three times the float32 oracle's own error."""
    got = np.asarray(got, dtype=np.float64)
    scale = max(1.0, float(np.abs(want64).max()))
    close(name, got, want32, RTOL, ATOL * scale)
    ours, theirs = np.abs(got - want64).max(), np.abs(np.asarray(want32, np.float64) - want64).max()
    assert ours <= 3.0 * theirs + ATOL, f"{name}: error vs float64 {ours:.3e}, float32 oracle's {theirs:.3e}"


def geometry(P, dev):
    g, b = P["geo"], P["batch"]
    return dict(pos_ij=to_dev(g["pos_ij"], dev), tvecs=to_dev(b.trans_vec, dev), batch=to_dev(g["batch"], dev),
                edges=to_dev(g["edges"], dev), rvlen=to_dev(g["rvlen"], dev), sizes=to_dev(b.sizes, dev),
                e_start=to_dev(g["e_start"], dev))


def second_axis_score64(P, R, frame1, i, h, e, image, static=False):
    """float64 score of candidate (pair e, translation ``image``) for the second axis of (atom i,
    head h): q.k + a d^2 + log(max(1 - |cos(d, frame1)|, 1e-5))
    (models/kernels/compute_second_frame_each_edge.cu:100-135 plus the selection of
    models/cuda_funcs/calc_maximum_frame.py:146-152); None if the candidate is inadmissible."""
    geo, b = P["geo"], P["batch"]
    R1, R2, R3 = (int(x) for x in R[i, h])
    n3 = image % (2 * R3 + 1) - R3
    n2 = (image // (2 * R3 + 1)) % (2 * R2 + 1) - R2
    n1 = image // ((2 * R3 + 1) * (2 * R2 + 1)) - R1
    T = b.trans_vec[geo["batch"][i]].astype(np.float64)
    d = geo["pos_ij"][e].astype(np.float64) + n1 * T[0] + n2 * T[1] + n3 * T[2]
    d2 = float(d @ d)
    if d2 <= 1e-5:
        return None
    cosv = abs(float(d @ frame1[i, h].astype(np.float64)) / np.sqrt(d2))
    if cosv >= 0.9999:
        return None
    if static:          # no query-key term, no Gaussian coefficient (compute_second_frame_static_each_edge.cu:126,135)
        return d2 + np.log(max(1.0 - cosv, 1e-5))
    j = geo["edges"][1, e]
    qk = float((P["q"][i, h].astype(np.float64) / 4.0) @ P["k"][j, h].astype(np.float64))
    return qk + float(P["a"][i, h]) * d2 + np.log(max(1.0 - cosv, 1e-5))


def adjudicate_second_axis(P, frame1, sel_e, sel_i, want_e, want_i, static=False):
    """Every (atom, head) whose second-axis selection differs from the oracle's must be a tie at
    float32 resolution.  Returns the number of differing selections."""
    from oracle import oracle as O
    diff = np.argwhere((sel_e != want_e) | (sel_i != want_i))
    if len(diff) == 0:
        return 0
    R = O.lattice_range(P["cfg"], P["a"], P["geo"]["rvlen"], P["geo"]["batch"])
    for i, h in diff:
        s_got = second_axis_score64(P, R, frame1, i, h, int(sel_e[i, h]), int(sel_i[i, h]), static)
        s_want = second_axis_score64(P, R, frame1, i, h, int(want_e[i, h]), int(want_i[i, h]), static)
        assert s_got is not None and s_want is not None, f"atom {i} head {h}: inadmissible candidate selected"
        # float32 resolution of a score of this size, times the handful of roundings in its evaluation
        tol = 16 * np.finfo(np.float32).eps * max(1.0, abs(s_want))
        assert abs(s_got - s_want) <= tol, \
            f"atom {i} head {h}: selected score {s_got:.9g}, oracle's {s_want:.9g} (not a float32 tie)"
    return len(diff)
