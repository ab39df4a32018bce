"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, the
Python binding covers all of them, and argument checks answer before any CUDA work."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "cfb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cfb200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from crystalframer_b200 import build, _lib
    build.build()
    return _lib


def test_exports_every_declared_symbol(lib):
    names = declared()
    assert len(names) >= 17
    handle = ctypes.CDLL(lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/cfb200.h but not exported"
    assert sorted(lib.SIGNATURES) == names, "Python binding and header disagree"


def test_argument_checks_without_gpu(lib):
    L = lib.lib()
    cfg = lib.Config(num_heads=8, head_dim=16, dist_dim=64, angle_dim=64, lattice_range=2, minimum_range=2, cos_abs=0,
                     cut_sigma=4, dist_wscale=1.0, angle_wscale=4.0, dist_coef=1.0, angle_coef=1.0, symm_break_noise=0.0)
    assert L.cfb200_configure(ctypes.byref(cfg)) == 0
    out = lib.Config()
    assert L.cfb200_get_config(ctypes.byref(out)) == 0 and out.num_heads == 8 and out.angle_dim == 64
    bad = lib.Config.from_buffer_copy(cfg)
    bad.head_dim = 32
    assert L.cfb200_configure(ctypes.byref(bad)) == -3            # unsupported instance
    bad = lib.Config.from_buffer_copy(cfg)
    bad.num_heads = 7
    assert L.cfb200_configure(ctypes.byref(bad)) == -3
    assert L.cfb200_configure(None) == -1
    # shape and NULL checks come before any launch
    assert L.cfb200_framed_proj_fwd(*([None] * 6), -1, 0, 14.0, -3.5, *([None] * 10)) == -2
    assert L.cfb200_framed_proj_fwd(*([None] * 6), 4, 16, 14.0, -3.5, *([None] * 10)) == -1
    assert L.cfb200_dpa_fwd(*([None] * 7), 4, 16, *([None] * 4)) == -1
    assert L.cfb200_max_frame(3, *([None] * 9), 4, 16, -3.5, 0, *([None] * 5)) == -2
    assert L.cfb200_segment_mean_fwd(None, None, 2, 8, None, None) == -1
    assert L.cfb200_framed_proj_bwd_workspace_bytes(100, 1000) > 0
    assert b"pointer" in L.cfb200_error_string(-1)


def test_unconfigured_library_refuses():
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from crystalframer_b200 import _lib\n"
            "L = _lib.lib()\n"
            "print(L.cfb200_dpa_fwd(*([None]*7), 0, 0, *([None]*4)))\n" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True).stdout
    assert out.strip() == "-4"


def test_operators_fail_loudly_without_cuda():
    import torch
    from crystalframer_b200 import cuda_funcs as F
    if torch.cuda.is_available():
        pytest.skip("only meaningful on a machine without a GPU")
    F.compile_kernels(2, 8, 16, 64, 64, 16, True, 0, 1.0, 4.0, 1.0, 1.0, 0.0)
    x = torch.zeros(4, 8, 16)
    with pytest.raises((ValueError, RuntimeError)):
        F.FusedDotProductAttentionCUDA.apply(x, x, x, None, None, torch.zeros(4, dtype=torch.long),
                                             torch.zeros(2, 16, dtype=torch.long))


def test_configuration_is_thread_safe(lib):
    """Several host threads configure and read the bound hyper-parameters at once (the reference runs one Python
    thread per device over process-global kernel state): every read must return one of the written configurations
    whole, never a mixture."""
    import threading
    L = lib.lib()
    base = dict(num_heads=8, head_dim=16, dist_dim=64, lattice_range=2, minimum_range=2, cos_abs=0, cut_sigma=4,
                dist_wscale=1.0, angle_wscale=4.0, dist_coef=1.0, angle_coef=1.0)
    variants = [lib.Config(angle_dim=64, symm_break_noise=1e-5, **base), lib.Config(angle_dim=0, symm_break_noise=0.0, **base)]
    torn, stop = [], threading.Event()

    def writer(i):
        while not stop.is_set():
            assert L.cfb200_configure(ctypes.byref(variants[i])) == 0

    def reader():
        out = lib.Config()
        for _ in range(3000):
            assert L.cfb200_get_config(ctypes.byref(out)) == 0
            pair = (out.angle_dim, round(out.symm_break_noise, 9))
            if pair not in ((64, round(1e-5, 9)), (0, 0.0)):
                torn.append(pair)
            assert L.cfb200_framed_proj_bwd_workspace_bytes(10, 100) > 0
        stop.set()

    threads = [threading.Thread(target=writer, args=(i,)) for i in range(2)] + [threading.Thread(target=reader)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not torn, torn[:3]
    assert L.cfb200_configure(ctypes.byref(variants[0])) == 0
