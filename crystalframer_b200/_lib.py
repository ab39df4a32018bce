"""ctypes binding of libcfb200.so.

There is no fallback: if the shared library is missing or an entry point reports an error,
an exception is raised.  Tensors handed to ``ptr`` must be contiguous CUDA tensors of the
expected dtype; ``None`` becomes a NULL pointer.
"""
import ctypes
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("CFB200_LIB_PATH", os.path.join(HERE, "libcfb200.so"))

_lib = None

i64, f32, vp, u64, i32 = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int32


class Config(ctypes.Structure):
    _fields_ = [("num_heads", i32), ("head_dim", i32), ("dist_dim", i32), ("angle_dim", i32),
                ("lattice_range", i32), ("minimum_range", i32), ("cos_abs", i32), ("cut_sigma", i32),
                ("dist_wscale", f32), ("angle_wscale", f32), ("dist_coef", f32), ("angle_coef", f32),
                ("symm_break_noise", f32)]


class LayerWeights(ctypes.Structure):          # cfb200_layer_weights
    _fields_ = [(n, vp) for n in ("q_proj", "k_proj", "v_proj", "in_bias", "lattice_pos", "gauss_scale", "out_proj",
                                  "out_bias", "pe_dist", "pe_ang1", "pe_ang2", "pe_ang3", "ff1", "ff1_bias", "ff2",
                                  "ff2_bias")]


class LayerGrads(ctypes.Structure):            # cfb200_layer_grads
    _fields_ = [(n, vp) for n in ("q_proj", "k_proj", "v_proj", "in_bias", "lattice_pos", "out_proj", "out_bias",
                                  "pe_dist", "pe_ang1", "pe_ang2", "pe_ang3", "ff1", "ff1_bias", "ff2", "ff2_bias")]


class Geometry(ctypes.Structure):              # cfb200_geometry
    _fields_ = [(n, vp) for n in ("pos_ij", "tvecs", "rvlen", "batch", "edges", "e_start", "order", "counters",
                                  "pair_cache", "pair_list")] + [("N", i64), ("E", i64), ("cache_range", i32), ("split", vp)]


class LayerState(ctypes.Structure):            # cfb200_layer_state
    _fields_ = [(n, vp) for n in ("q", "q_scaled", "k", "v", "a", "frames", "z", "spool", "attn", "lse", "x1", "h", "tasks", "val", "px", "upool")]


class LayerDesc(ctypes.Structure):             # cfb200_layer_desc
    _fields_ = [("d_model", i32), ("ff_dim", i32), ("frame_method", i32), ("gauss_lb", f32), ("beta", f32),
                ("scale_real", f32), ("dist_max", f32), ("cutoff_radius", f32), ("seed1", u64), ("seed2", u64)]


# name -> (restype, argtypes); one entry per declaration of include/cfb200.h
SIGNATURES = {
    "cfb200_configure": (ctypes.c_int, [ctypes.POINTER(Config)]),
    "cfb200_get_config": (ctypes.c_int, [ctypes.POINTER(Config)]),
    "cfb200_version": (ctypes.c_int, []),
    "cfb200_error_string": (ctypes.c_char_p, [ctypes.c_int]),
    "cfb200_status": (ctypes.c_int, [ctypes.POINTER(i32), vp]),
    "cfb200_framed_proj_bwd_workspace_bytes": (i64, [i64, i64]),
    "cfb200_edge_index": (ctypes.c_int, [vp, i64, i64, i64, vp, vp, vp, vp, vp]),
    "cfb200_csr_offsets": (ctypes.c_int, [vp, i64, i64, vp, vp]),
    "cfb200_gauss_coef_fwd": (ctypes.c_int, [vp, vp, vp, i64, f32, f32, f32, vp, vp, vp]),
    "cfb200_gauss_coef_bwd": (ctypes.c_int, [vp, vp, vp, i64, f32, f32, f32, vp, vp, vp, vp, vp]),
    "cfb200_max_frame": (ctypes.c_int, [ctypes.c_int] + [vp] * 9 + [i64, i64, f32, u64] + [vp] * 5),
    "cfb200_max_frame_static": (ctypes.c_int, [ctypes.c_int] + [vp] * 7 + [i64, i64, f32, u64] + [vp] * 5),
    "cfb200_max_frames_static": (ctypes.c_int, [vp] * 7 + [i64, i64, f32, u64, u64] + [vp] * 4 + [ctypes.c_int, vp]),
    "cfb200_lattice_frames": (ctypes.c_int, [vp] * 6 + [i64, i64, f32, u64, u64, u64] + [vp] * 4),
    "cfb200_max_frames": (ctypes.c_int, [vp] * 9 + [i64, i64, f32, u64, u64] + [vp] * 4),
    "cfb200_pair_cache": (ctypes.c_int, [vp] * 4 + [i64, i64, ctypes.c_int, vp, vp, vp]),
    "cfb200_pca_frames": (ctypes.c_int, [vp, vp, i64, i64, u64, vp, vp, vp, vp]),
    "cfb200_max_frame_cached": (ctypes.c_int, [ctypes.c_int] + [vp] * 9 + [i64, i64, f32, u64] + [vp] * 6 + [ctypes.c_int, vp]),
    "cfb200_max_frames_cached": (ctypes.c_int, [vp] * 9 + [i64, i64, f32, u64, u64] + [vp] * 5 + [ctypes.c_int, vp]),
    "cfb200_framed_proj_fwd_cached": (ctypes.c_int, [vp] * 6 + [i64, i64, f32, f32] + [vp] * 11 + [ctypes.c_int, vp]),
    "cfb200_framed_proj_bwd_cached": (ctypes.c_int, [vp] * 7 + [i64, i64, f32, f32] + [vp] * 16 + [i64, vp, ctypes.c_int, vp]),
    "cfb200_sigma_edges": (ctypes.c_int, [vp] * 6 + [i64, i64, f32, u64, vp, vp]),
    "cfb200_max_frame3_workspace_bytes": (i64, [i64, i64]),
    "cfb200_max_frame3": (ctypes.c_int, [vp] * 9 + [i64, i64, f32, u64] + [vp] * 5 + [i64, vp]),
    "cfb200_sigma_edges_cached": (ctypes.c_int, [vp] * 6 + [i64, i64, f32, u64, vp, vp, ctypes.c_int, vp]),
    "cfb200_sigma_frames_cached": (ctypes.c_int, [vp] * 9 + [i64, i64, f32, u64, u64] + [vp] * 4 + [i64, vp, ctypes.c_int, vp]),
    "cfb200_sigma_frames_workspace_bytes": (i64, [i64, i64]),
    "cfb200_sigma_frames": (ctypes.c_int, [vp] * 9 + [i64, i64, f32, u64, u64] + [vp] * 4 + [i64, vp]),
    "cfb200_framed_proj_fwd": (ctypes.c_int, [vp] * 6 + [i64, i64, f32, f32] + [vp] * 10),
    "cfb200_framed_proj_bwd": (ctypes.c_int, [vp] * 7 + [i64, i64, f32, f32] + [vp] * 16 + [i64, vp]),
    "cfb200_deal_by_cost": (ctypes.c_int, [vp, i64, ctypes.c_int32, vp]),
    "cfb200_reci_enc_fwd": (ctypes.c_int, [vp] * 6 + [i64, i64, i64] + [vp] * 3),
    "cfb200_reci_enc_bwd": (ctypes.c_int, [vp] * 7 + [i64, i64, i64] + [vp] * 2),
    "cfb200_proj_fwd": (ctypes.c_int, [vp] * 6 + [i64, i64, f32, f32] + [vp] * 4),
    "cfb200_proj_heads_bwd_workspace_bytes": (i64, [i64, i64, i64]),
    "cfb200_proj_heads_fwd": (ctypes.c_int, [vp] * 6 + [i64, i64, i64, f32, f32] + [vp] * 4),
    "cfb200_proj_heads_bwd": (ctypes.c_int, [vp] * 7 + [i64, i64, i64, f32, f32] + [vp] * 7 + [i64, vp]),
    "cfb200_proj_bwd": (ctypes.c_int, [vp] * 7 + [i64, i64, f32, f32] + [vp] * 7 + [i64, vp]),
    "cfb200_framed_proj_bwd_noalloc": (ctypes.c_int, [vp] * 7 + [i64, i64, f32, f32] + [vp] * 15 + [vp]),
    "cfb200_attn_fused_fwd": (ctypes.c_int, [vp] * 12 + [i64, i64, f32, f32] + [vp] * 8 + [ctypes.c_int] + [vp] * 7
                              + [ctypes.c_int, vp]),
    "cfb200_attn_fused_bwd": (ctypes.c_int, [vp] * 12 + [i64, i64, f32, f32] + [vp] * 8 + [ctypes.c_int] + [vp] * 12
                              + [ctypes.c_int, vp]),
    "cfb200_dpa_fwd": (ctypes.c_int, [vp] * 7 + [i64, i64] + [vp] * 4),
    "cfb200_dpa_bwd": (ctypes.c_int, [vp] * 7 + [i64, i64] + [vp] * 9),
    "cfb200_segment_mean_fwd": (ctypes.c_int, [vp, vp, i64, i64, vp, vp]),
    "cfb200_segment_mean_bwd": (ctypes.c_int, [vp, vp, i64, i64, vp, vp]),
    "cfb200_adamw_clip_step": (ctypes.c_int, [vp] * 4 + [i64, i64] + [f32] * 6 + [ctypes.c_double, ctypes.c_double, vp, vp, vp]),
    "cfb200_adamw_clip_step_avg": (ctypes.c_int, [vp] * 4 + [i64, i64] + [f32] * 6 + [ctypes.c_double, ctypes.c_double, vp, vp,
                                                  vp, f32, vp]),
    "cfb200_batch_geometry_workspace_bytes": (i64, [i64]),
    "cfb200_queue_entries": (i64, [i64]),
    "cfb200_split_ints": (i64, [i64]),
    "cfb200_attn_tasks_bytes": (i64, [i64]),
    "cfb200_batch_geometry": (ctypes.c_int, [vp, vp, vp, i64, i64, i64, ctypes.c_int] + [vp] * 12 + [vp, i64, vp]),
    "cfb200_encoder_layer_workspace_bytes": (i64, [i64, i64, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "cfb200_encoder_layer_fwd": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, vp, i64, vp]),
    "cfb200_encoder_layer_bwd": (ctypes.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, ctypes.c_int, vp, i64, vp]),
    "cfb200_linear": (ctypes.c_int, [vp, vp, vp, vp, i64, i64, i64, ctypes.c_int, ctypes.c_int, vp, vp]),
    "cfb200_timing_begin": (ctypes.c_int, []),
    "cfb200_timing_end": (ctypes.c_int, [vp, vp]),
    "cfb200_probe_throughput": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, vp, vp]),
}


_pending = []


def loaded():
    return _lib is not None


def on_load(fn):
    """Runs ``fn(handle)`` when the shared library is first loaded (only the latest registration is kept)."""
    _pending[:] = [fn]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m crystalframer_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these operators.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
        for fn in _pending:
            fn(handle)
        _pending.clear()
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().cfb200_error_string(rc).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {rc})")


def ptr(t, dtype=torch.float32):
    if t is None:
        return None
    if not (t.is_cuda and t.is_contiguous() and t.dtype == dtype):
        raise ValueError(f"expected a contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}, "
                         f"contiguous={t.is_contiguous()}")
    return t.data_ptr()


def iptr(t):
    return ptr(t, torch.int64)


def stream(device):
    return torch.cuda.current_stream(device).cuda_stream


# ---- launch accounting and optional per-call CUDA-event timing --------------------------------
launch_count = 0          # kernels of this library enqueued since import (all entry points)
_timer = None


class KernelTimer:
    """Brackets every entry-point call with CUDA events on the stream the kernels are enqueued
    on; ``summary()`` synchronises and returns {entry point: (calls, total milliseconds)}."""

    def __init__(self):
        self.records = {}

    def __enter__(self):
        global _timer
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None

    def summary(self):
        torch.cuda.synchronize()
        return {name: (len(ev), sum(a.elapsed_time(b) for a, b in ev)) for name, ev in self.records.items()}


TIMING_STAGES = ("batch_geometry", "linear_fwd", "coef", "frames", "attn_fwd_kernel", "linear_bwd", "attn_bwd_kernel",
                 "attn_bwd_cols_kernel", "wgrad")


class StageTimer:
    """Per-stage CUDA-event times of the one-call entry points (cfb200_timing_begin / _end): ``summary()``
    waits for the events and returns {stage: (brackets, total milliseconds)}."""

    def __enter__(self):
        check(lib().cfb200_timing_begin(), "cfb200_timing_begin")
        return self

    def __exit__(self, *exc):
        pass

    def summary(self):
        ms = (f32 * len(TIMING_STAGES))()
        n = (i32 * len(TIMING_STAGES))()
        check(lib().cfb200_timing_end(ms, n), "cfb200_timing_end")
        return {name: (int(n[i]), float(ms[i])) for i, name in enumerate(TIMING_STAGES) if n[i] > 0}


def _device_index(device):
    if isinstance(device, int):
        return device
    idx = torch.device(device).index
    return torch.cuda.current_device() if idx is None else idx


def invoke(name, n_kernels, device, *args):
    """Calls entry point ``name`` with ``args`` followed by the current stream of ``device``.  The device is
    made current for the call only when it is not already (the usual case costs no device switch)."""
    global launch_count
    fn = getattr(lib(), name)
    idx = _device_index(device)
    if _timer is None and idx == torch.cuda.current_device():
        rc = fn(*args, torch._C._cuda_getCurrentRawStream(idx))
    else:
        with torch.cuda.device(idx):
            st = torch.cuda.current_stream(idx)
            if _timer is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                rc = fn(*args, st.cuda_stream)
                e1.record(st)
                _timer.records.setdefault(name, []).append((e0, e1))
            else:
                rc = fn(*args, st.cuda_stream)
    if rc != 0:
        check(rc, name)
    launch_count += n_kernels


def read_status(device=None):
    """Reads and clears the device status word (synchronises the current stream)."""
    out = i32(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        check(lib().cfb200_status(ctypes.byref(out), stream(device)), "cfb200_status")
    return out.value
