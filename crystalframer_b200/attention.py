"""Periodic lattice-sum multi-head attention: module and functional form.

Drop-in for ``CrystalformerMultiheadAttentionCUDA`` and
``crystalformer_multi_head_attention_forward_cuda`` of the reference
(models/indexed_lattice_multi_head_attention_cuda.py:737-1269): same constructor and forward
arguments, same parameter names, shapes and initialisation (so released checkpoints load), same
data-dependent ``gauss_scale`` state.  Input / output projections and the Gaussian-coefficient
pipeline stay in PyTorch; everything between them runs in libcfb200.

Domains: "real" with frame methods "max", "max_static", "max_wo_orthogonal", "lattice", "pca", "weighted_pca" (CrystalFramer)
and "no" (plain Crystalformer distance encoding); "reci" / "RECI" (plain Crystalformer's reciprocal-space
logit bias, no value encoding), also alternating by layer ("real-reci"); "multihead" (first half of the heads in
real space, second half in reciprocal space) for the plain Crystalformer encoding (frame_method "no").
"""
import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Module, Parameter
from torch.nn.init import constant_, normal_, xavier_uniform_
from torch.nn.modules.linear import NonDynamicallyQuantizableLinear

from .cuda_funcs import (ComputeFrame1MaximumMethodCUDA, ComputeFrame1MaximumStaticMethodCUDA, ComputeFrame3MaximumMethodCUDA,
                         ComputeFrame2MaximumMethodCUDA, ComputeFrame2MaximumStaticMethodCUDA, ComputeLatticeFrameCUDA, ComputePCAFrame,
                         FusedDotProductAttentionCUDA, RealEncodingWithFramedProjFuncCUDA,
                         RealPeriodicEncodingWithProjFuncCUDA, ReciPeriodicEncodingFuncCUDA, max_frames_fused, max_static_frames_fused,
                         weighted_pca_frames)
from .latticeformer_params import LatticeformerParams

# use the single-launch frame construction instead of the two Functions plus torch ops
FUSED_FRAMES = True


def _scaled_dot_product_attention(q, k, v, batch, batch_kv, edges, attn_weights=None, values=None, dropout_p=0.0):
    """models/indexed_lattice_multi_head_attention_cuda.py:144-185 (the fused branch)."""
    if dropout_p != 0.0 or batch is not batch_kv:
        raise NotImplementedError("only dropout-free self-attention is implemented")
    q = q / math.sqrt(q.shape[-1])
    return FusedDotProductAttentionCUDA.apply(q, k, v, attn_weights, values, batch, edges), None, None


def compute_frame_maximum_method_(q, k, v, alpha, pos, dist2_min, tvecs, batch, edges, proj, K, dist_max, wscale,
                                  frame_method, this_epoch=None, rvecs=None, cutoff=None):
    """models/indexed_lattice_multi_head_attention_cuda.py:435-493 for frame_method "max", "max_static" and
    "max_wo_orthogonal"."""
    if frame_method not in ("max", "max_static", "max_wo_orthogonal"):
        raise NotImplementedError(f"frame_method={frame_method}")
    if frame_method == "max_wo_orthogonal":
        # the second axis stays as selected, the third is selected like the first two (:449-455, :483-488)
        rvlen = torch.norm(rvecs, 2, dim=-1) if cutoff is not None else None
        adap = (rvlen, cutoff) if cutoff is not None else ()
        with torch.no_grad():
            qs = q / math.sqrt(q.shape[-1])
            f1 = ComputeFrame1MaximumMethodCUDA.apply(qs, k, v, alpha, pos, dist2_min, tvecs, batch, edges, K, dist_max, wscale, *adap)
            f2 = ComputeFrame2MaximumMethodCUDA.apply(qs, k, v, alpha, pos, dist2_min, tvecs, batch, edges, K, dist_max, wscale,
                                                      f1, *adap)
            f3 = ComputeFrame3MaximumMethodCUDA.apply(qs, k, v, alpha, pos, dist2_min, tvecs, batch, edges, K, dist_max, wscale,
                                                      f1, f2, *adap)
        return f1, f2, f3
    rvlen = torch.norm(rvecs, 2, dim=-1) if cutoff is not None else None
    qs = q / math.sqrt(q.shape[-1])
    if FUSED_FRAMES:
        with torch.no_grad():
            if frame_method == "max_static":
                return max_static_frames_fused(alpha, pos, tvecs, batch, edges, rvlen, cutoff)
            return max_frames_fused(qs, k, alpha, pos, tvecs, batch, edges, rvlen, cutoff)
    extra = (rvlen, cutoff) if cutoff is not None else ()
    F1, F2 = (ComputeFrame1MaximumMethodCUDA, ComputeFrame2MaximumMethodCUDA) if frame_method == "max" else \
        (ComputeFrame1MaximumStaticMethodCUDA, ComputeFrame2MaximumStaticMethodCUDA)
    f1 = F1.apply(qs, k, v, alpha, pos, dist2_min, tvecs, batch, edges, K, dist_max, wscale, *extra)
    f2m = F2.apply(qs, k, v, alpha, pos, dist2_min, tvecs, batch, edges, K, dist_max, wscale, f1, *extra)
    dot = (f1 * f2m).sum(dim=-1, keepdim=True)
    f2 = F.normalize(f2m - dot * f1, dim=2)
    return f1, f2, torch.linalg.cross(f1, f2)


def compute_real_domain_attn_frame_proj(q, k, v, batch_q, batch_kv, edges, pos, dist2_min, tvecs, rvecs,
                                        pe_dist_proj, proj_angle1, proj_angle2, proj_angle3, alpha,
                                        params: LatticeformerParams = None, this_epoch=None):
    """models/indexed_lattice_multi_head_attention_cuda.py:589-734: logit bias (E,H) and value
    bias (E,H,hd) of every pair."""
    K = params.value_pe_dist_real
    dist_max = params.value_pe_dist_max
    if dist_max < 0:
        dist_max = (-dist_max) * params.scale_real
    wscale = params.value_pe_dist_wscale
    adap = ()
    if params.adaptive_cutoff_sigma < 0:
        adap = (rvecs, params.adaptive_cutoff_sigma)
    elif params.adaptive_cutoff_sigma > 0:
        adap = (rvecs, params.scale_real * params.gauss_lb_real ** (-0.5) * params.adaptive_cutoff_sigma)
    rv_args = (torch.norm(adap[0], 2, dim=-1), adap[1]) if adap else ()
    if params.frame_method in ("max", "max_static", "max_wo_orthogonal"):
        f1, f2, f3 = compute_frame_maximum_method_(q, k, None, alpha, pos, dist2_min, tvecs, batch_q, edges,
                                                   pe_dist_proj, K, dist_max, wscale, params.frame_method, this_epoch, *adap)
        W1, W2, W3 = proj_angle1, proj_angle2, proj_angle3
    elif params.frame_method == "lattice":
        # models/indexed_lattice_multi_head_attention_cuda.py:496-520
        with torch.no_grad():
            f1, f2, f3 = ComputeLatticeFrameCUDA.apply(q / math.sqrt(q.shape[-1]), k, None, alpha, pos, dist2_min, tvecs,
                                                       batch_q, edges, K, dist_max, wscale, *rv_args)
        W1, W2, W3 = proj_angle1, proj_angle2, proj_angle3
    elif params.frame_method == "pca":
        # models/indexed_lattice_multi_head_attention_cuda.py:522-534
        with torch.no_grad():
            f1, f2, f3 = ComputePCAFrame.apply(q / math.sqrt(q.shape[-1]), k, None, alpha, pos, dist2_min, tvecs,
                                               batch_q, edges, K, dist_max, wscale, *rv_args)
        W1, W2, W3 = proj_angle1, proj_angle2, proj_angle3
        from . import fused_layer
        if fused_layer.FRAME_TAP is not None:
            fused_layer.FRAME_TAP.append(torch.stack([f1, f2, f3]).clone())
    elif params.frame_method == "weighted_pca":
        with torch.no_grad():
            qs = q / math.sqrt(q.shape[-1])
            f1, f2, f3 = weighted_pca_frames(qs, k, alpha, pos, tvecs, batch_q, edges, *(rv_args or (None, None)))[:3]
        W1, W2, W3 = proj_angle1, proj_angle2, proj_angle3
        from . import fused_layer
        if fused_layer.FRAME_TAP is not None:
            fused_layer.FRAME_TAP.append(torch.stack([f1, f2, f3]).clone())
    elif params.frame_method == "no":
        # plain Crystalformer: un-windowed distance encoding, no frames, no coefficients
        # (models/indexed_lattice_multi_head_attention_cuda.py:403-433, :620-624)
        out = RealPeriodicEncodingWithProjFuncCUDA.apply(alpha, pos, dist2_min, tvecs, batch_q, edges, K, dist_max,
                                                         wscale, pe_dist_proj, "no", *rv_args)
        return out[0], (out[1] if len(out) > 1 else None)
    else:
        raise NotImplementedError(f"frame_method={params.frame_method}")
    out = RealEncodingWithFramedProjFuncCUDA.apply(
        alpha, pos, dist2_min, tvecs, batch_q, edges, K, dist_max, wscale, pe_dist_proj, W1, W2, W3, f1, f2, f3,
        params.value_pe_angle_real, params.value_pe_angle_wscale, params.cos_abs, params.value_pe_dist_coef,
        params.value_pe_angle_coef, *rv_args)
    return out[0], (out[1] if len(out) > 1 else None)


def gauss_scale_ready(gauss_scale):
    """True once the coefficient statistics in ``gauss_scale`` are known to be set.  ``gauss_scale[0] > 0`` is a
    device-side fact; reading it every call would stall the host once per layer, so a positive answer is
    remembered on the tensor object TOGETHER with the tensor's version counter: any in-place write
    (load_state_dict, zero_, re-calibration) invalidates it and the value is read again."""
    if getattr(gauss_scale, "_cf_ready", None) == gauss_scale._version:
        return True
    if bool(gauss_scale[0] > 0):
        gauss_scale._cf_ready = gauss_scale._version
        return True
    return False


def reset_gauss_scale(module):
    """Forgets the measured coefficient statistics of every attention module below ``module``; the next training
    forward measures them again (as the reference does when gauss_scale is zero)."""
    for m in module.modules():
        gs = getattr(m, "gauss_scale", None)
        if gs is not None:
            with torch.no_grad():
                gs.zero_()


GAUSS_STATES = ("q", "q-headdim", "q-kdim", "1", "x", "x-norm", "x-xavier")


def gaussian_coefficients(q, lattice_pos_weights, gauss_scale, params, training, query=None):
    """models/indexed_lattice_multi_head_attention_cuda.py:896-940: per (atom, head) coefficient
    a < 0 of exp(a d^2), from q and the learned per-head direction, normalised with statistics
    that are measured once (first training forward) and then stored in ``gauss_scale``.  ``gauss_state`` "q*": from
    the projected query; "1": one learned constant per head; "x*": from the layer's input ``query`` (N, embed_dim)."""
    N, H, hd = q.shape
    if params.gauss_state not in GAUSS_STATES:
        raise NotImplementedError(f"gauss_state={params.gauss_state}")
    if params.gauss_state.startswith("q"):
        alpha = (q.reshape(N, H, 1, hd) @ lattice_pos_weights.reshape(H, hd, 1)).view(N, H)
    elif params.gauss_state == "1":
        alpha = (torch.ones_like(q).reshape(N, H, 1, hd) @ lattice_pos_weights.reshape(H, hd, 1)).view(N, H)
    else:
        alpha = F.linear(query, lattice_pos_weights).view(N, H)
    if params.normalize_gauss:
        if gauss_scale_ready(gauss_scale):
            scale, shift = gauss_scale[0], gauss_scale[1]
        else:
            scale = torch.reciprocal(alpha.detach().std())
            shift = -alpha.detach().mean()
            if training:
                with torch.no_grad():
                    gauss_scale[0] = scale
                    gauss_scale[1] = shift
                gauss_scale._cf_ready = gauss_scale._version
        alpha = (alpha + shift) * scale
    beta = params.positive_func_beta
    if params.domain == "multihead":
        # the first half of the heads attends in real space, the second half in reciprocal space
        # (models/indexed_lattice_multi_head_attention_cuda.py:953-956)
        a1, a2 = alpha.chunk(2, 1)
        lb1, lb2 = params.gauss_lb_real, params.gauss_lb_reci
        a1 = ((1.0 - lb1) * F.elu(a1 * (beta / (1.0 - lb1))) + 1.0) * (-0.5 * params.scale_real ** -2)
        a2 = ((1.0 - lb2) * F.elu(a2 * (beta / (1.0 - lb2))) + 1.0) * (-0.5 * params.scale_reci ** 2)
        return torch.cat([a1, a2], dim=1)
    if params.domain in ("reci", "RECI"):
        # reciprocal-space Gaussians widen where real-space ones narrow
        # (models/indexed_lattice_multi_head_attention_cuda.py:946-952)
        lb = params.gauss_lb_reci
        pos = (1.0 - lb) * F.elu(alpha * (beta / (1.0 - lb))) + 1.0
        if params.domain == "RECI":
            pos = 1 / pos
        return pos * (-0.5 * params.scale_reci ** 2)
    lb = params.gauss_lb_real
    pos = (1.0 - lb) * F.elu(alpha * (beta / (1.0 - lb))) + 1.0
    return pos * (-0.5 * params.scale_real ** -2)


def crystalformer_multi_head_attention_forward_cuda(
        query, key, value, batch_q, batch_kv, edges, pos, dist2_min, tvecs, kr_base, rvecs, vcell,
        lattice_pos_weights, embed_dim_to_check, num_heads, q_proj_weight, k_proj_weight, v_proj_weight,
        in_proj_bias, dropout_p, out_proj_weight, out_proj_bias, pe_dist_proj, pe_wave_proj, proj_angle1,
        proj_angle2, proj_angle3, training=True, need_weights=True, gauss_scale=None, atten_scale=None,
        onehot=None, params: LatticeformerParams = None, this_epoch=None) -> Tuple[Tensor, Optional[Tensor]]:
    """models/indexed_lattice_multi_head_attention_cuda.py:737-996, real-space domain."""
    N = query.shape[0]
    hq, hk, hv = (w.shape[0] // num_heads for w in (q_proj_weight, k_proj_weight, v_proj_weight))
    if in_proj_bias is None:
        bq = bk = bv = None
    else:
        bq, bk, bv = in_proj_bias.split([q_proj_weight.size(0), k_proj_weight.size(0), v_proj_weight.size(0)])
    q = F.linear(query, q_proj_weight, bq).view(N, num_heads, hq)
    k = F.linear(key, k_proj_weight, bk).view(key.shape[0], num_heads, hk)
    v = F.linear(value, v_proj_weight, bv).view(value.shape[0], num_heads, hv)
    attn_weights = values = None
    if params is not None and params.domain != "no":
        if params.domain not in ("real", "reci", "RECI", "multihead"):
            raise NotImplementedError(f"domain={params.domain}")
        alpha = gaussian_coefficients(q, lattice_pos_weights, gauss_scale, params, training, query)
        if params.domain == "multihead":
            # models/indexed_lattice_multi_head_attention_cuda.py:953-974
            half = num_heads // 2
            a1, a2 = alpha[:, :half].contiguous(), alpha[:, half:].contiguous()
            w1, v1 = compute_real_domain_attn_frame_proj(
                q, k, v, batch_q, batch_kv, edges, pos, dist2_min, tvecs, rvecs,
                None if pe_dist_proj is None else pe_dist_proj[:, :half], proj_angle1, proj_angle2, proj_angle3, a1,
                params, this_epoch)
            w2 = ReciPeriodicEncodingFuncCUDA.apply(a2, kr_base, rvecs, vcell, batch_q, edges)
            attn_weights = torch.cat([w1, w2], dim=1)
            values = None if v1 is None else torch.cat([v1, torch.zeros_like(v1)], dim=1)
        elif params.domain == "real":
            attn_weights, values = compute_real_domain_attn_frame_proj(
                q, k, v, batch_q, batch_kv, edges, pos, dist2_min, tvecs, rvecs, pe_dist_proj, proj_angle1,
                proj_angle2, proj_angle3, alpha, params, this_epoch)
        else:
            # models/indexed_lattice_multi_head_attention_cuda.py:550-566: logit bias only, no value encoding
            attn_weights = ReciPeriodicEncodingFuncCUDA.apply(alpha, kr_base, rvecs, vcell, batch_q, edges)
    if not training:
        dropout_p = 0.0
    out, _, _ = _scaled_dot_product_attention(q, k, v, batch_q, batch_kv, edges, attn_weights, values, dropout_p)
    out = F.linear(out.contiguous().view(N, hv * num_heads), out_proj_weight, out_proj_bias)
    if need_weights:
        raise NotImplementedError("need_weights=True: use cuda_funcs.attention_probabilities")
    return out, values


class CrystalformerMultiheadAttentionCUDA(Module):
    """models/indexed_lattice_multi_head_attention_cuda.py:998-1269.  Parameters:
    q_proj_weight, k_proj_weight, v_proj_weight, in_proj_bias, out_proj.{weight,bias},
    lattice_pos_weights (H*hd), pe_dist_proj (1,H,hd,D_dist), proj_angle1..3 (1,H,hd,D_ang),
    and the non-trainable gauss_scale (2), atten_scale (1)."""

    def __init__(self, embed_dim, num_heads, dropout=0., bias=True, kdim=None, vdim=None,
                 params=LatticeformerParams(), device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        if params.domain not in ("real", "reci", "RECI", "multihead", "no"):
            raise NotImplementedError(f"domain={params.domain}")
        if params.domain == "multihead" and (params.frame_method != "no" or num_heads % 2):
            # with frames the reference's CUDA module hands queries of all heads and coefficients of half of them to
            # its frame kernels (models/indexed_lattice_multi_head_attention_cuda.py:953-963); its README (:157)
            # limits CrystalFramer to the real domain.  Built for the plain Crystalformer encoding only.
            raise NotImplementedError("domain=multihead needs frame_method='no' and an even number of heads")
        self.embed_dim = embed_dim
        self.kdim = kdim * num_heads if kdim is not None and kdim > 0 else embed_dim
        self.vdim = vdim * num_heads if vdim is not None and vdim > 0 else embed_dim
        self.params = params
        self.num_heads = num_heads
        self.dropout = dropout
        self.head_dim = embed_dim // num_heads
        assert self.head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"
        self.gauss_scale = Parameter(torch.zeros(2, **kw), requires_grad=False)
        self.atten_scale = Parameter(torch.zeros(1, **kw), requires_grad=False)
        self.q_proj_weight = Parameter(torch.empty((self.kdim, embed_dim), **kw))
        self.k_proj_weight = Parameter(torch.empty((self.kdim, embed_dim), **kw))
        self.v_proj_weight = Parameter(torch.empty((self.vdim, embed_dim), **kw))
        if bias:
            self.in_proj_bias = Parameter(torch.empty(self.kdim * 2 + self.vdim, **kw))
        else:
            self.register_parameter("in_proj_bias", None)
        self.out_proj = NonDynamicallyQuantizableLinear(self.vdim, embed_dim, bias=bias, **kw)
        self.lattice_pos_weights = None
        self.pe_dist_proj = self.pe_wave_proj = self.proj_angle1 = self.proj_angle2 = self.proj_angle3 = None
        if params.domain in ("reci", "RECI"):
            # models/indexed_lattice_multi_head_attention_cuda.py:1100-1107
            if params.value_pe_dist_reci > 0 or params.value_pe_wave_reci > 0:
                raise NotImplementedError("value encodings of the reciprocal domain")
        if params.domain in ("real", "multihead", "reci", "RECI"):
            # models/indexed_lattice_multi_head_attention_cuda.py:1060-1071
            if params.gauss_state not in GAUSS_STATES:
                raise NotImplementedError(f"gauss_state={params.gauss_state}")
            shape = (num_heads, embed_dim) if params.gauss_state.startswith("x") else (self.kdim,)
            self.lattice_pos_weights = Parameter(torch.empty(*shape, **kw))
        if params.domain in ("real", "multihead"):
            if params.value_pe_dist_real > 0:
                self.pe_dist_proj = Parameter(torch.empty(1, num_heads, self.head_dim, params.value_pe_dist_real, **kw))
            if params.value_pe_angle_real > 0:
                # "multihead" keeps angle weights for its real-space half only (:1088-1097)
                shape = (1, num_heads if params.domain == "real" else num_heads // 2, self.head_dim, params.value_pe_angle_real)
                self.proj_angle1 = Parameter(torch.empty(*shape, **kw))
                self.proj_angle2 = Parameter(torch.empty(*shape, **kw))
                self.proj_angle3 = Parameter(torch.empty(*shape, **kw))
        self._reset_parameters()

    def _reset_parameters(self):
        for w in (self.q_proj_weight, self.k_proj_weight, self.v_proj_weight, self.out_proj.weight):
            xavier_uniform_(w)
        if self.in_proj_bias is not None:
            constant_(self.in_proj_bias, 0.)
            constant_(self.out_proj.bias, 0.)
        if self.lattice_pos_weights is not None:
            state = self.params.gauss_state                   # :1121-1130
            if state == "x-xavier":
                xavier_uniform_(self.lattice_pos_weights)
            else:
                std = self.kdim ** -0.5 if state == "q-kdim" else self.embed_dim ** -0.5 if state.startswith("x") else \
                    (self.kdim // self.num_heads) ** -0.5
                normal_(self.lattice_pos_weights, 0., std)
        with torch.no_grad():
            for P in (self.pe_dist_proj, self.proj_angle1, self.proj_angle2, self.proj_angle3):
                if P is not None:
                    for W in P:
                        W2 = W.view(-1, W.shape[-1])
                        xavier_uniform_(W2, W2.shape[1] ** -0.5)

    def forward(self, query, key, value, batch_q, batch_kv, edges, points, dist2_min, tvecs, kr_base=None,
                rvecs=None, vcell=None, onehot=None, need_weights=True, this_epoch=None):
        return crystalformer_multi_head_attention_forward_cuda(
            query, key, value, batch_q, batch_kv, edges, points, dist2_min, tvecs, kr_base, rvecs, vcell,
            self.lattice_pos_weights, self.embed_dim, self.num_heads, self.q_proj_weight, self.k_proj_weight,
            self.v_proj_weight, self.in_proj_bias, self.dropout, self.out_proj.weight, self.out_proj.bias,
            self.pe_dist_proj, self.pe_wave_proj, self.proj_angle1, self.proj_angle2, self.proj_angle3,
            training=self.training, need_weights=need_weights, gauss_scale=self.gauss_scale,
            atten_scale=self.atten_scale, onehot=onehot, params=self.params, this_epoch=this_epoch)
