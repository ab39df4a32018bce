"""The 4-layer model's forward pass on the host cores (test infrastructure only).

Takes a ``crystalframer_b200.latticeformer.Latticeformer`` instance that lives on the CPU (it
is used as a parameter container only -- its own forward needs the CUDA library) and replays
the reference's forward with the oracle Functions: species embedding, per layer the input
projections, Gaussian coefficients, max frames, lattice-sum bias + value encoding, ragged
attention, output projection, feed-forward; then mean pooling and the MLP head
(models/latticeformer.py:191-287, models/indexed_latticeformer_encoder.py:699-890,
models/indexed_lattice_multi_head_attention_cuda.py:737-996 of the reference).
"""
import math

import numpy as np
import torch
import torch.nn.functional as F

from . import functions as OF
from . import oracle as O


def oracle_config(model):
    p = model.encoder.lattice_params
    attn = model.encoder.layers[0].self_attn
    plain = p.frame_method == "no"
    # plain Crystalformer encoding (models/kernels/real_enc_proj_fwd.cu:127-134): every distance Gaussian
    # is evaluated (a window wider than the basis) and there is no angle basis
    return O.Config(H=attn.num_heads, head_dim=attn.head_dim, D_dist=p.value_pe_dist_real,
                    D_ang=0 if plain else p.value_pe_angle_real, cut_sigma=32 if plain else 4,
                    lattice_range=p.lattice_range,
                    minimum_range=p.lattice_range if p.minimum_range else 0, cos_abs=p.cos_abs,
                    dist_max=(-p.value_pe_dist_max) * attn.params.scale_real if p.value_pe_dist_max < 0 else p.value_pe_dist_max,
                    wscale_dist=p.value_pe_dist_wscale, wscale_ang=p.value_pe_angle_wscale,
                    c_dist=p.value_pe_dist_coef, c_ang=p.value_pe_angle_coef,
                    cutoff_radius=p.adaptive_cutoff_sigma, symm_break_noise=0.0)


def coefficients(attn, q, x=None):
    """models/indexed_lattice_multi_head_attention_cuda.py:896-940; ``x``: the layer's input, for gauss_state "x*"."""
    P = attn.params
    N, H, hd = q.shape
    if P.gauss_state.startswith("q"):
        alpha = (q.reshape(N, H, 1, hd) @ attn.lattice_pos_weights.reshape(H, hd, 1)).view(N, H)
    elif P.gauss_state == "1":
        alpha = (torch.ones_like(q).reshape(N, H, 1, hd) @ attn.lattice_pos_weights.reshape(H, hd, 1)).view(N, H)
    else:
        alpha = F.linear(x, attn.lattice_pos_weights).view(N, H)
    if P.normalize_gauss:
        if bool(attn.gauss_scale[0] > 0):
            scale, shift = attn.gauss_scale[0], attn.gauss_scale[1]
        else:
            scale = torch.reciprocal(alpha.detach().std())
            shift = -alpha.detach().mean()
            if attn.training:
                with torch.no_grad():
                    attn.gauss_scale[0] = scale
                    attn.gauss_scale[1] = shift
        alpha = (alpha + shift) * scale
    beta = P.positive_func_beta
    if P.domain == "multihead":               # :953-956
        a1, a2 = alpha.chunk(2, 1)
        lb1, lb2 = P.gauss_lb_real, P.gauss_lb_reci
        a1 = ((1.0 - lb1) * F.elu(a1 * (beta / (1.0 - lb1))) + 1.0) * (-0.5 * P.scale_real ** -2)
        a2 = ((1.0 - lb2) * F.elu(a2 * (beta / (1.0 - lb2))) + 1.0) * (-0.5 * P.scale_reci ** 2)
        return torch.cat([a1, a2], dim=1)
    if P.domain in ("reci", "RECI"):          # :946-952
        lb = P.gauss_lb_reci
        pos = (1.0 - lb) * F.elu(alpha * (beta / (1.0 - lb))) + 1.0
        return (1 / pos if P.domain == "RECI" else pos) * (-0.5 * P.scale_reci ** 2)
    lb = P.gauss_lb_real
    return ((1.0 - lb) * F.elu(alpha * (beta / (1.0 - lb))) + 1.0) * (-0.5 * P.scale_real ** -2)


def draw_frame_seeds(frame_method):
    """The draws the library's frame construction takes from the global generators, in its order
    (crystalframer_b200/cuda_funcs/max_frame.py): numpy for the noise seeds, torch for the row signs."""
    draw = lambda: int(np.random.randint(np.iinfo(np.int64).min, np.iinfo(np.int64).max, dtype=np.int64)) & (2 ** 64 - 1)
    if frame_method == "weighted_pca":
        draw()
        seed_noise = draw()
        return seed_noise, int(torch.randint(0, 2 ** 62, (1,)).item())
    if frame_method == "pca":          # no numpy draw (the reference's Function takes none); one torch draw for the signs
        return int(torch.randint(0, 2 ** 62, (1,)).item()), 0
    return draw(), draw()


def attention_layer(attn, x, geo, cfg, frames=None):
    """One attention block.  ``frames``: (3,N,H,3) tensor to use instead of constructing the frames here
    (for comparisons downstream of identical frames, e.g. weighted-PCA frames, whose eigenvectors are
    not comparable across implementations where eigenvalues nearly coincide)."""
    N = x.shape[0]
    H, hd = attn.num_heads, attn.head_dim
    bq, bk, bv = attn.in_proj_bias.split([attn.kdim, attn.kdim, attn.vdim])
    q = F.linear(x, attn.q_proj_weight, bq).view(N, H, hd)
    k = F.linear(x, attn.k_proj_weight, bk).view(N, H, hd)
    v = F.linear(x, attn.v_proj_weight, bv).view(N, H, hd)
    a = coefficients(attn, q, x)
    cutoff = attn.params.adaptive_cutoff_sigma
    qs = q / math.sqrt(hd)
    if attn.params.domain in ("reci", "RECI"):
        # reciprocal-space logit bias, no value encoding (:550-566)
        z = OF.Reci.apply(a, geo["kr"], geo["rvecs"], geo["vcell"], geo["batch"], geo["edges"], cfg.lattice_range)
        out = OF.Attention.apply(qs, k, v, z, torch.zeros((z.shape[0], H, hd), dtype=q.dtype, device=q.device), geo["batch"], geo["edges"])
        return F.linear(out.reshape(N, H * hd), attn.out_proj.weight, attn.out_proj.bias)
    method = attn.params.frame_method
    if attn.params.domain == "multihead":
        # first half of the heads: plain real-space encoding; second half: reciprocal-space bias, no values (:953-974)
        half = H // 2
        z1, v1 = OF.FramedProj.apply(a[:, :half].contiguous(), geo["pos_ij"], geo["tvecs"], geo["batch"], geo["edges"],
                                     geo["rvlen"], cutoff, cfg.dist_max, attn.pe_dist_proj[:, :half], None, None, None,
                                     None, None, None)
        z2 = OF.Reci.apply(a[:, half:].contiguous(), geo["kr"], geo["rvecs"], geo["vcell"], geo["batch"], geo["edges"],
                           cfg.lattice_range)
        out = OF.Attention.apply(qs, k, v, torch.cat([z1, z2], dim=1), torch.cat([v1, torch.zeros_like(v1)], dim=1),
                                 geo["batch"], geo["edges"])
        return F.linear(out.reshape(N, H * hd), attn.out_proj.weight, attn.out_proj.bias)
    if method == "no":
        f1 = f2 = f3 = None
    elif frames is not None:
        f1, f2, f3 = frames[0], frames[1], frames[2]
    elif method == "max":
        with torch.no_grad():
            f1, f2, f3 = OF.max_frames(qs.detach().contiguous(), k.detach().contiguous(), a.detach().contiguous(),
                                       geo["pos_ij"], geo["tvecs"], geo["batch"], geo["edges"], geo["rvlen"], cutoff)
    elif method == "max_wo_orthogonal":
        npy = lambda t: t.detach().contiguous().numpy()
        e_start = OF._e_start(geo["edges"], N)
        fr = O.max_frames_wo_orthogonal(cfg, npy(qs), npy(k), npy(a), npy(geo["pos_ij"]), npy(geo["tvecs"]), npy(geo["rvlen"]),
                                        npy(geo["batch"]), npy(geo["edges"]), npy(e_start))
        f1, f2, f3 = (torch.from_numpy(fr[n]) for n in ("frame1", "frame2", "frame3"))
    elif method in ("max_static", "lattice"):
        npy = lambda t: t.detach().contiguous().numpy()
        e_start = OF._e_start(geo["edges"], N)
        if method == "max_static":
            fr = O.max_static_frames(cfg, npy(a), npy(geo["pos_ij"]), npy(geo["tvecs"]), npy(geo["rvlen"]), npy(geo["batch"]),
                                     npy(geo["edges"]), npy(e_start))
            f1, f2, f3 = (torch.from_numpy(fr[n]) for n in ("frame1", "frame2", "frame3"))
        else:
            f1, f2, f3 = (torch.from_numpy(x) for x in O.lattice_frames(cfg, npy(a), npy(geo["tvecs"]), npy(geo["rvlen"]),
                                                                        npy(geo["batch"]), npy(geo["edges"]), npy(e_start)))
    elif method == "pca":
        seed, _ = draw_frame_seeds(method)
        e_start = OF._e_start(geo["edges"], N)
        fr, _, _ = O.pca_frames(geo["pos_ij"].detach().numpy(), e_start.numpy(), H, seed)
        f1, f2, f3 = (torch.from_numpy(fr[x]) for x in range(3))
    elif method == "weighted_pca":
        seed_noise, seed_sign = draw_frame_seeds(method)
        npy = lambda t: t.detach().contiguous().numpy()
        e_start = OF._e_start(geo["edges"], N)
        fr, _, _ = O.weighted_pca_frames(cfg, npy(qs), npy(k), npy(a), npy(geo["pos_ij"]), npy(geo["tvecs"]),
                                         npy(geo["rvlen"]), npy(geo["batch"]), npy(geo["edges"]), npy(e_start),
                                         seed_noise, seed_sign)
        f1, f2, f3 = (torch.from_numpy(fr[x]) for x in range(3))
    else:
        raise NotImplementedError(method)
    z, val = OF.FramedProj.apply(a, geo["pos_ij"], geo["tvecs"], geo["batch"], geo["edges"], geo["rvlen"], cutoff,
                                 cfg.dist_max, attn.pe_dist_proj, attn.proj_angle1, attn.proj_angle2,
                                 attn.proj_angle3, f1, f2, f3)
    out = OF.Attention.apply(qs, k, v, z, val, geo["batch"], geo["edges"])
    return F.linear(out.reshape(N, H * hd), attn.out_proj.weight, attn.out_proj.bias)


def forward(model, batch, backend=None, frames=None):
    """``batch``: crystalframer_b200.synth.CrystalBatch (numpy).  Returns the (B, 1) prediction.
    ``frames``: optional list with one (3,N,H,3) tensor per layer to use instead of constructing them.
    With ``backend="reference_cuda"`` the model's parameters must live on the GPU; the reference's own CUDA
    kernels then run there, with the reference's host glue between them."""
    cfg = oracle_config(model)
    OF.configure(cfg, backend)
    g = O.lattice_geometry(batch.pos, batch.trans_vec, batch.sizes)
    dev = next(model.parameters()).device
    t = lambda arr: torch.from_numpy(np.ascontiguousarray(arr)).to(dev)
    geo = dict(pos_ij=t(g["pos_ij"]), tvecs=t(batch.trans_vec), batch=t(g["batch"]), edges=t(g["edges"]),
               rvlen=t(g["rvlen"]))
    if any(d in ("reci", "RECI", "multihead") for d in model.encoder.lattice_params.domain.split("-")):
        rvecs, vcell, kr = O.reciprocal_geometry(batch.pos, batch.trans_vec, batch.sizes, g["edges"])
        geo.update(rvecs=t(rvecs), vcell=t(vcell), kr=t(kr))
    sizes = t(batch.sizes)
    x = model.input_embeddings(t(batch.x))
    for li, layer in enumerate(model.encoder.layers):
        x = layer.norm1(x + attention_layer(layer.self_attn, x, geo, cfg, None if frames is None else frames[li]))
        x = layer.norm2(x + layer.linear2(layer.activation(layer.linear1(x))))
    if model.encoder.norm is not None:
        x = model.encoder.norm(x)
    if getattr(model, "proj_before_pooling", None) is not None:
        x = model.proj_before_pooling(x)                    # models/latticeformer.py:282
    if getattr(model.params, "pooling", "avr") != "avr":
        raise NotImplementedError("the oracle model pools by the mean")
    x = OF.Mean.apply(x, sizes)
    return model.mlp(x)
