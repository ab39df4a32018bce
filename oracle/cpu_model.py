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
    return O.Config(H=attn.num_heads, head_dim=attn.head_dim, D_dist=p.value_pe_dist_real,
                    D_ang=p.value_pe_angle_real, lattice_range=p.lattice_range,
                    minimum_range=p.lattice_range if p.minimum_range else 0, cos_abs=p.cos_abs,
                    dist_max=(-p.value_pe_dist_max) * attn.params.scale_real if p.value_pe_dist_max < 0 else p.value_pe_dist_max,
                    wscale_dist=p.value_pe_dist_wscale, wscale_ang=p.value_pe_angle_wscale,
                    c_dist=p.value_pe_dist_coef, c_ang=p.value_pe_angle_coef,
                    cutoff_radius=p.adaptive_cutoff_sigma, symm_break_noise=0.0)


def coefficients(attn, q):
    """models/indexed_lattice_multi_head_attention_cuda.py:896-940"""
    P = attn.params
    N, H, hd = q.shape
    alpha = (q.reshape(N, H, 1, hd) @ attn.lattice_pos_weights.reshape(H, hd, 1)).view(N, H)
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
    lb, beta = P.gauss_lb_real, P.positive_func_beta
    return ((1.0 - lb) * F.elu(alpha * (beta / (1.0 - lb))) + 1.0) * (-0.5 * P.scale_real ** -2)


def attention_layer(attn, x, geo, cfg):
    N = x.shape[0]
    H, hd = attn.num_heads, attn.head_dim
    bq, bk, bv = attn.in_proj_bias.split([attn.kdim, attn.kdim, attn.vdim])
    q = F.linear(x, attn.q_proj_weight, bq).view(N, H, hd)
    k = F.linear(x, attn.k_proj_weight, bk).view(N, H, hd)
    v = F.linear(x, attn.v_proj_weight, bv).view(N, H, hd)
    a = coefficients(attn, q)
    cutoff = attn.params.adaptive_cutoff_sigma
    qs = q / math.sqrt(hd)
    with torch.no_grad():
        f1, f2, f3 = OF.max_frames(qs.detach().contiguous(), k.detach().contiguous(), a.detach().contiguous(),
                                   geo["pos_ij"], geo["tvecs"], geo["batch"], geo["edges"], geo["rvlen"], cutoff)
    z, val = OF.FramedProj.apply(a, geo["pos_ij"], geo["tvecs"], geo["batch"], geo["edges"], geo["rvlen"], cutoff,
                                 cfg.dist_max, attn.pe_dist_proj, attn.proj_angle1, attn.proj_angle2,
                                 attn.proj_angle3, f1, f2, f3)
    out = OF.Attention.apply(qs, k, v, z, val, geo["batch"], geo["edges"])
    return F.linear(out.reshape(N, H * hd), attn.out_proj.weight, attn.out_proj.bias)


def forward(model, batch, backend=None):
    """``batch``: crystalframer_b200.synth.CrystalBatch (numpy).  Returns the (B, 1) prediction."""
    cfg = oracle_config(model)
    OF.configure(cfg, backend)
    g = O.lattice_geometry(batch.pos, batch.trans_vec, batch.sizes)
    t = lambda arr: torch.from_numpy(np.ascontiguousarray(arr))
    geo = dict(pos_ij=t(g["pos_ij"]), tvecs=t(batch.trans_vec), batch=t(g["batch"]), edges=t(g["edges"]),
               rvlen=t(g["rvlen"]))
    sizes = t(batch.sizes)
    x = model.input_embeddings(t(batch.x))
    for layer in model.encoder.layers:
        x = layer.norm1(x + attention_layer(layer.self_attn, x, geo, cfg))
        x = layer.norm2(x + layer.linear2(layer.activation(layer.linear1(x))))
    if model.encoder.norm is not None:
        x = model.encoder.norm(x)
    x = OF.Mean.apply(x, sizes)
    return model.mlp(x)
