"""Callers of the attention module: pair-list construction, lattice geometry and the encoder
stack (models/indexed_latticeformer_encoder.py of the reference: get_edge_index :15-32,
compute_lattice_distances_for_cuda :175-245, CrystalformerEncoderCUDA :611-742,
CrystalformerEncoderLayerCUDA :744-890).  Class names, constructor arguments and parameter
names are kept so that reference checkpoints load."""
import math
from typing import Callable, Union

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Dropout, Identity, LayerNorm, Linear, Module, ModuleList
from torch.nn.init import constant_, xavier_uniform_

from . import _lib
from . import fused_layer
from .attention import CrystalformerMultiheadAttentionCUDA, gauss_scale_ready
from .cuda_funcs import compile_kernels, register_csr
from .latticeformer_params import LatticeformerParams


# run default-structure layers as one autograd node (fused_layer.py); off = operator by operator
FUSED_LAYER = True


def build_pair_list(sizes: Tensor, counts=None):
    """Dense pair list of a batch of crystals on the GPU, in one call instead of the reference's
    Python loop over crystals.  Returns edges (2,E) int64, e_start (N+1), batch (N),
    crystal_start (B+1).  ``counts = (N, E)`` (atoms, pairs) spares the device-to-host read of
    ``sizes`` when the caller already knows them."""
    if not sizes.is_cuda:
        raise RuntimeError("build_pair_list needs sizes on a CUDA device (there is no CPU path)")
    sizes = sizes.to(torch.int64).contiguous()
    B = sizes.shape[0]
    if counts is None:
        host = sizes.tolist()
        N, E = sum(host), sum(s * s for s in host)
    else:
        N, E = int(counts[0]), int(counts[1])
    dev = sizes.device
    edges = torch.empty((2, E), dtype=torch.int64, device=dev)
    e_start = torch.empty(N + 1, dtype=torch.int64, device=dev)
    batch = torch.empty(N, dtype=torch.int64, device=dev)
    crystal_start = torch.empty(B + 1, dtype=torch.int64, device=dev)
    _lib.invoke("cfb200_edge_index", 2, dev, _lib.iptr(sizes), B, N, E, _lib.iptr(edges), _lib.iptr(e_start),
                _lib.iptr(batch), _lib.iptr(crystal_start))
    register_csr(edges, N, e_start)
    return edges, e_start, batch, crystal_start


def get_edge_index(sizes, device):
    """Same result as the reference's get_edge_index(sizes, device)."""
    if not torch.is_tensor(sizes):
        sizes = torch.tensor(sizes, dtype=torch.int64)
    return build_pair_list(sizes.to(device))[0]


def det_3x3(m):
    return m[:, 0, 0] * m[:, 1, 1] * m[:, 2, 2] + m[:, 0, 1] * m[:, 1, 2] * m[:, 2, 0] \
        + m[:, 0, 2] * m[:, 1, 0] * m[:, 2, 1] - m[:, 0, 2] * m[:, 1, 1] * m[:, 2, 0] \
        - m[:, 0, 0] * m[:, 1, 2] * m[:, 2, 1] - m[:, 0, 1] * m[:, 1, 0] * m[:, 2, 2]


def compute_lattice_distances_for_cuda(pos, batch, trans_vec, sizes, lattice_range, cutoff_radius=0,
                                       output_real=False, output_reci=False, num_pairs=None):
    """Relative positions of all pairs, reciprocal vectors and cell volumes; returns the
    reference's 6-tuple (pos_ij, dist2_min=None, kr_base, rvecs, vcell, edges)."""
    if sizes is None:
        sizes = torch.zeros(trans_vec.shape[0], dtype=torch.long, device=pos.device)
        sizes.scatter_add_(0, batch, torch.ones_like(batch))
    if not torch.is_tensor(sizes):
        sizes = torch.tensor(sizes, dtype=torch.int64)
    counts = (pos.shape[0], num_pairs) if num_pairs is not None else None
    edges = build_pair_list(sizes.to(pos.device), counts)[0]
    vcell = det_3x3(trans_vec).contiguous()
    rvecs = torch.stack([torch.cross(trans_vec[:, 1], trans_vec[:, 2], dim=1),
                         torch.cross(trans_vec[:, 2], trans_vec[:, 0], dim=1),
                         torch.cross(trans_vec[:, 0], trans_vec[:, 1], dim=1)], dim=1) \
        * (2.0 * math.pi / vcell[:, None, None])
    pos_ij = (pos[edges[1]] - pos[edges[0]]).contiguous()
    kr_base = None
    if output_reci:
        kr_base = (rvecs[batch[edges[0]]] @ pos_ij[..., None]).squeeze(2).contiguous()
    return pos_ij, None, kr_base, rvecs.contiguous(), vcell, edges


def _activation(name):
    if callable(name):
        return name
    if name == "relu":
        return F.relu
    if name == "gelu":
        return F.gelu
    raise RuntimeError(f"activation should be relu/gelu, not {name}")


class CrystalformerEncoderLayerCUDA(Module):
    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: Union[str, Callable[[Tensor], Tensor]] = F.relu, layer_norm_eps: float = 1e-5,
                 norm_first: bool = False, no_layer_norm=False, params=LatticeformerParams(), k_dim=0, v_dim=0,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.domain = params.domain
        self.self_attn = CrystalformerMultiheadAttentionCUDA(d_model, nhead, dropout=dropout, kdim=k_dim, vdim=v_dim,
                                                             params=params)
        self.linear1 = Linear(d_model, dim_feedforward)
        self.dropout = Dropout(dropout) if dropout > 0 else Identity()
        self.linear2 = Linear(dim_feedforward, d_model)
        self.norm_first = norm_first
        self.norm1 = LayerNorm(d_model, eps=layer_norm_eps) if not no_layer_norm else Identity()
        self.norm2 = LayerNorm(d_model, eps=layer_norm_eps) if not no_layer_norm else Identity()
        self.dropout1 = Dropout(dropout) if dropout > 0 else Identity()
        self.dropout2 = Dropout(dropout) if dropout > 0 else Identity()
        self.activation = _activation(activation)
        self._fused_meta = None
        xavier_uniform_(self.linear1.weight)
        xavier_uniform_(self.linear2.weight)
        constant_(self.linear1.bias, 0)
        constant_(self.linear2.bias, 0)

    def fixup_initialization(self, num_layers):
        """T-Fixup scaling of the value, output and feed-forward weights (enc.py:814-832)."""
        s = 0.67 * num_layers ** (-1. / 4.)
        with torch.no_grad():
            for w in (self.linear1.weight, self.linear2.weight, self.self_attn.out_proj.weight,
                      self.self_attn.v_proj_weight):
                w.mul_(s)

    def fused_meta(self, x):
        """Scalars for the one-call layer (fused_layer), or None when this layer's configuration or state
        is outside what that path covers."""
        if not (FUSED_LAYER and x.is_cuda and isinstance(self.norm1, Identity) and isinstance(self.norm2, Identity)
                and isinstance(self.dropout, Identity) and self.activation is F.relu):
            return None
        if not gauss_scale_ready(self.self_attn.gauss_scale):
            return None          # the first training forward measures the coefficient statistics
        if self._fused_meta is None:
            self._fused_meta = fused_layer.layer_meta(self) or False
        return self._fused_meta or None

    def fused_apply(self, x, geo, meta):
        return fused_layer.FusedEncoderLayerFunc.apply(x, *fused_layer.layer_parameters(self), geo, meta)

    def _fused_forward(self, x, batch, edges, pos_ij, trans, rvecs):
        """The whole layer as one autograd node for callers that hand over the reference's tensors."""
        meta = self.fused_meta(x)
        if meta is None:
            return None
        geo = getattr(edges, "_cf_geometry", None)
        if geo is None or geo.pos_ij is not pos_ij:
            rvlen = torch.norm(rvecs, 2, dim=-1).contiguous() if meta["cutoff"] != 0.0 else None
            geo = fused_layer.LayerGeometry.from_tensors(pos_ij.contiguous(), trans.contiguous(), batch.contiguous(),
                                                         edges.contiguous(), rvlen, meta["cutoff"])
            edges._cf_geometry = geo
        return self.fused_apply(x, geo, meta)

    def forward(self, src, batch, edges, pos_ij=None, dist2_min=None, trans=None, kr_base=None, rvecs=None,
                vcell=None, onehot=None, this_epoch=None):
        x = src
        if dist2_min is None and pos_ij is not None and rvecs is not None:
            fused = self._fused_forward(x, batch, edges, pos_ij, trans, rvecs)
            if fused is not None:
                return fused
        if self.norm_first:
            x = x + self._sa_block(self.norm1(x), batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot, this_epoch)
            x = x + self._ff_block(self.norm2(x))
        else:
            x = self.norm1(x + self._sa_block(x, batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot, this_epoch))
            x = self.norm2(x + self._ff_block(x))
        return x

    def _sa_block(self, x, batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot, this_epoch):
        x = self.self_attn(x, x, x, batch, batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot,
                           need_weights=False, this_epoch=this_epoch)[0]
        return self.dropout1(x)

    def _ff_block(self, x):
        return self.dropout2(self.linear2(self.dropout(self.activation(self.linear1(x)))))


class CrystalformerEncoderCUDA(Module):
    def __init__(self, d_model: int = 512, nhead: int = 8, num_encoder_layers: int = 6, dim_feedforward: int = 2048,
                 dropout: float = 0.1, activation: Union[str, Callable[[Tensor], Tensor]] = F.relu,
                 layer_norm_eps: float = 1e-5, norm_first: bool = False, t_fixup_init=False, no_layer_norm=False,
                 lattice_params: LatticeformerParams = LatticeformerParams(), k_dim=0, v_dim=0, device=None,
                 dtype=None) -> None:
        super().__init__()
        self.lattice_params = lattice_params
        self.layers = ModuleList([
            CrystalformerEncoderLayerCUDA(d_model, nhead, dim_feedforward, dropout, activation, layer_norm_eps,
                                          norm_first, no_layer_norm, params=lattice_params.getLayerParameters(i),
                                          k_dim=k_dim, v_dim=v_dim)
            for i in range(num_encoder_layers)])
        if t_fixup_init:
            for layer in self.layers:
                layer.fixup_initialization(num_encoder_layers)
        self.num_layers = num_encoder_layers
        self.norm = LayerNorm(d_model, eps=layer_norm_eps) if not no_layer_norm else None
        self.d_model = d_model
        self.nhead = nhead
        P = lattice_params
        angle_dim = P.value_pe_angle_real if P.frame_method != "no" else 0
        compile_kernels(P.lattice_range, nhead, k_dim if k_dim > 0 else d_model // nhead, P.value_pe_dist_real,
                        angle_dim, v_dim if v_dim > 0 else d_model // nhead, P.minimum_range, P.cos_abs,
                        P.value_pe_dist_wscale, P.value_pe_angle_wscale, P.value_pe_dist_coef,
                        P.value_pe_angle_coef, P.symm_break_noise)

    def forward(self, src, pos, batch, trans, sizes, onehot=None, this_epoch=None, num_pairs=None):
        if src.size(-1) != self.d_model:
            raise RuntimeError("the feature number of src must be equal to d_model")
        # Fast path: every layer runs as one library call and the batch is prepared by one
        # (fused_layer.LayerGeometry.from_raw); needs the pair count, which the batch objects of this package carry.
        if num_pairs is not None and torch.is_tensor(sizes) and sizes.is_cuda and sizes.dtype == torch.int64:
            metas = [layer.fused_meta(src) for layer in self.layers]
            if all(m is not None for m in metas) and pos.dtype == torch.float32 and trans.dtype == torch.float32:
                geo = fused_layer.LayerGeometry.from_raw(pos.contiguous(), trans.contiguous(), sizes.contiguous(),
                                                         pos.shape[0], int(num_pairs), metas[0]["cutoff"])
                out = src
                for layer, meta in zip(self.layers, metas):
                    out = layer.fused_apply(out, geo, meta)
                return out if self.norm is None else self.norm(out)
        batch = batch - batch[0]
        pos_ij, dist2_min, kr_base, rvecs, vcell, edges = compute_lattice_distances_for_cuda(
            pos, batch, trans, sizes, self.lattice_params.lattice_range, -1, output_real=True,
            output_reci=any(d in ("reci", "RECI", "multihead") for d in self.lattice_params.domain.split("-")), num_pairs=num_pairs)
        out = src
        for layer in self.layers:
            out = layer(out, batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot, this_epoch)
        if self.norm is not None:
            out = self.norm(out)
        return out
