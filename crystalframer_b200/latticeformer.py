"""Whole-model caller used by the benchmarks: species embedding -> encoder -> mean pooling ->
MLP head (models/latticeformer.py:32-287 of the reference, single-device path).  The reference's
in-forward multi-GPU replication (:211-273) is replaced by one process per GPU."""
import copy

import torch
from torch import nn

from . import pooling
from .encoder import CrystalformerEncoderCUDA
from .latticeformer_params import LatticeformerParams


class ModelParams:
    """Attribute bag holding the keys of the reference's JSON parameter files
    (params/crystalframer/default_jarvis.json)."""
    DEFAULTS = dict(
        num_layers=4, lattice_range=2, adaptive_cutoff_sigma=-3.5, minimum_range=True, model_dim=128, k_dim=0,
        v_dim=0, head_num=8, ff_dim=512, t_fixup_init=True, embedding_dim=[128], t_activation="relu", domain="real",
        gauss_lb_real=0.5, gauss_lb_reci=0.5, gauss_state="q", normalize_gauss=True, positive_func_beta=0.1,
        use_cgcnn_feat=False, scale_real=[1.4], scale_reci=[2.2], value_pe_dist_real=64, value_pe_dist_reci=0,
        value_pe_dist_coef=1.0, value_pe_wave_real=0, value_pe_wave_reci=0, value_pe_dist_max=-10.0,
        value_pe_dist_wscale=1.0, frame_method="max", cos_abs=0, value_pe_angle_real=64, value_pe_angle_wscale=4.0,
        value_pe_angle_coef=1.0, pooling="avr", pre_pooling_op="no", norm_type="no", dropout=0.0, targets="e_form",
        symm_break_noise=1e-5, scale_grad=0.0, use_cuda_code=True)

    def __init__(self, **overrides):
        for k, v in self.DEFAULTS.items():
            setattr(self, k, copy.deepcopy(v))
        for k, v in overrides.items():
            setattr(self, k, v)


class Latticeformer(nn.Module):
    ATOM_FEAT_DIM = 98

    def __init__(self, params):
        super().__init__()
        self.params = params
        model_dim, num_layers = params.model_dim, params.num_layers
        # options of the reference that every parameter file of it leaves off and that are not wired up here
        # (models/latticeformer.py:200-207: CGCNN atom features from a data file, GradientScaler on the embeddings)
        if getattr(params, "use_cgcnn_feat", False):
            raise NotImplementedError("use_cgcnn_feat")
        if getattr(params, "scale_grad", 0.0) > 0:
            raise NotImplementedError("scale_grad > 0")
        lattice_params = LatticeformerParams()
        lattice_params.parseFromArgs(params)
        self.input_embeddings = nn.Linear(self.ATOM_FEAT_DIM, model_dim, bias=False)
        emb_scale = model_dim ** -0.5
        if params.t_fixup_init:
            emb_scale *= (9 * num_layers) ** (-1 / 4)
        nn.init.normal_(self.input_embeddings.weight, mean=0, std=emb_scale)
        self.encoder = CrystalformerEncoderCUDA(
            model_dim, params.head_num, activation=params.t_activation, num_encoder_layers=num_layers,
            dim_feedforward=params.ff_dim, dropout=params.dropout, t_fixup_init=params.t_fixup_init,
            no_layer_norm=params.t_fixup_init, lattice_params=lattice_params, k_dim=params.k_dim, v_dim=params.v_dim)
        # per-atom projection before pooling and normalisation inside the head (models/latticeformer.py:138-190); the
        # reference's parameter files use "no" / "no" throughout
        norms = {"bn": nn.BatchNorm1d, "ln": nn.LayerNorm, "in": nn.InstanceNorm1d, "id": nn.Identity, "no": nn.Identity}
        if params.norm_type not in norms:
            raise NotImplementedError(f"norm_type: {params.norm_type}")
        norm = norms[params.norm_type]
        emb = list(params.embedding_dim)
        pooled_dim = model_dim
        self.proj_before_pooling = None
        if params.pre_pooling_op in ("w+bn+relu", "w+relu"):
            pooled_dim = emb.pop(0)
            if not emb:
                raise ValueError("pre_pooling_op takes the first entry of embedding_dim; the head needs one more")
            mods = [nn.Linear(model_dim, pooled_dim)]
            if params.pre_pooling_op == "w+bn+relu":
                mods.append(norm(pooled_dim))
            self.proj_before_pooling = nn.Sequential(*mods, nn.ReLU(True))
        elif params.pre_pooling_op == "relu":
            self.proj_before_pooling = nn.ReLU(True)
        elif params.pre_pooling_op != "no":
            raise NotImplementedError(f"pre_pooling_op: {params.pre_pooling_op}")
        self.pooling_layer = {"avr": pooling.avr_pool, "max": pooling.max_pool}[params.pooling]
        dims = [pooled_dim] + emb
        layers = []
        for di, do in zip(dims[:-1], dims[1:]):
            layers += [nn.Linear(di, do), norm(do), nn.ReLU(True)]
        final_dim = 1 if isinstance(params.targets, str) else len(params.targets)
        layers.append(nn.Linear(dims[-1], final_dim))
        self.mlp = nn.Sequential(*layers)

    def forward(self, data, this_epoch=None):
        x = self.input_embeddings(data.x)
        x = self.encoder(x, data.pos, data.batch, data.trans_vec, data.sizes, this_epoch=this_epoch,
                         num_pairs=getattr(data, "num_pairs", None))
        if self.proj_before_pooling is not None:
            x = self.proj_before_pooling(x)
        x = self.pooling_layer(x, data.batch, data.sizes)
        return self.mlp(x)
