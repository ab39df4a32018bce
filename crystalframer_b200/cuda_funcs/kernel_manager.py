"""Hyper-parameter binding: the counterpart of the reference's kernel registry and JIT step
(models/cuda_funcs/kernel_manager.py:24-167).  The reference substitutes constants into kernel
text and compiles with NVRTC; here the same call binds them in the prebuilt library."""
import ctypes

from .. import _lib


# When True, compile_kernels only records the hyper-parameters; they are bound when the library is first
# loaded.  For processes that build the model classes as parameter containers without ever running them.
DEFER_BINDING = False


class KernelManager:
    """Limits of the reference kept for callers that read them (kernel_manager.py:59-62).
    The kernels of this package have no atom-count limit."""
    MAX_SYSTEM_SIZE: int = 320
    MAX_SYSTEM_SIZE_POW2: int = 512
    RUNNING_SUM_LEN: int = 8
    PE_THREAD_NUM: int = 16
    config = None


def compile_kernels(lattice_range: int, head_num: int, key_head_dim: int, value_pe_dim: int,
                    dim_angle_enc: int, value_head_dim: int, set_minimum_range: bool, cos_abs: int,
                    value_pe_dist_wscale: float, value_pe_angle_wscale: float, value_pe_dist_coef: float,
                    value_pe_angle_coef: float, symm_break_noise: float):
    """Same signature as the reference's compile_kernels (kernel_manager.py:116-123)."""
    if key_head_dim != value_head_dim:
        raise RuntimeError("libcfb200 needs equal key and value head dimensions")
    cfg = _lib.Config(num_heads=head_num, head_dim=key_head_dim, dist_dim=value_pe_dim,
                      angle_dim=dim_angle_enc, lattice_range=lattice_range,
                      minimum_range=lattice_range if set_minimum_range else 0, cos_abs=int(cos_abs),
                      cut_sigma=4, dist_wscale=value_pe_dist_wscale, angle_wscale=value_pe_angle_wscale,
                      dist_coef=value_pe_dist_coef, angle_coef=value_pe_angle_coef,
                      symm_break_noise=symm_break_noise)
    KernelManager.config = cfg
    if DEFER_BINDING and not _lib.loaded():
        _lib.on_load(lambda handle: _lib.check(handle.cfb200_configure(ctypes.byref(cfg)), "cfb200_configure"))
        return cfg
    _lib.check(_lib.lib().cfb200_configure(ctypes.byref(cfg)), "cfb200_configure")
    return cfg


def current_config():
    cfg = _lib.Config()
    _lib.check(_lib.lib().cfb200_get_config(ctypes.byref(cfg)), "cfb200_get_config")
    return cfg
