"""Hyper-parameter bag of the attention layers; field names and defaults follow the reference's
models/latticeformer_params.py:5-87 so that its JSON parameter files can be consumed unchanged."""
import copy
from typing import List


class LatticeformerParams:
    def __init__(self, domain: str = "real", lattice_range: int = 4, minimum_range: bool = True,
                 adaptive_cutoff_sigma: float = -3.5, gauss_lb_real: float = 0.5, gauss_lb_reci: float = 0.5,
                 scale_real: List[float] = [1.4], scale_reci: List[float] = [2.2], normalize_gauss: bool = True,
                 value_pe_dist_real: int = 64, value_pe_dist_coef: float = 1.0, value_pe_dist_max: float = -10.0,
                 value_pe_dist_wscale: float = 1.0, value_pe_wave_real: int = 0, value_pe_dist_reci: int = 0,
                 value_pe_wave_reci: int = 0, value_pe_angle_real: int = 16, value_pe_angle_coef: float = 1.0,
                 value_pe_angle_wscale: float = 4.0, positive_func_beta: float = 0.1, layer_index: int = -1,
                 gauss_state: str = "q", frame_method: str = "max", frame_mode: str = "both", cos_abs: int = 1,
                 symm_break_noise: float = 1e-5) -> None:
        fields = dict(locals())
        fields.pop("self")
        self.__dict__.update(fields)

    def parseFromArgs(self, args):
        for key in list(self.__dict__):
            self.__dict__[key] = getattr(args, key, self.__dict__[key])

    def getLayerParameters(self, layer_index):
        domain = self.domain
        if domain not in ("real", "reci", "multihead"):
            parts = domain.split("-")
            domain = parts[layer_index % len(parts)]
        out = copy.deepcopy(self)
        out.domain = domain
        for name in ("scale_real", "scale_reci"):
            val = getattr(self, name)
            if isinstance(val, (list, tuple)):
                val = val[layer_index % len(val)]
            setattr(out, name, val)
        out.layer_index = layer_index
        return out
