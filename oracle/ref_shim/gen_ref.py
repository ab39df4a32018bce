"""Compile the reference project's own kernels, from where they lie, into oracle/_ref/.

Test infrastructure only.  Two libraries are produced (both git-ignored; no reference
source text is copied anywhere -- the generated wrappers only ``#include`` the reference
files by path and repeat each kernel's parameter list):

* ``libcfref_cpu.so``: each kernel compiled by g++ against ``cuda_host_shim.h`` and
  driven by a loop over (block, thread), OpenMP-parallel over blocks.  Entry points
  ``cfref_cpu_<kernel>(grid, block, <kernel params>)``.
* ``libcfref_gpu.so``: each kernel compiled by nvcc for sm_100a with a one-line launch
  wrapper ``cfref_gpu_<kernel>(grid, block, stream, <kernel params>)`` -- the reference's
  CUDA kernels as they would run on the same GPU, used as the GPU baseline.

The reference injects its compile-time constants by textual replacement
(models/cuda_funcs/kernel_manager.py:124-159); here the same names are given as -D
macros.  ``check_macro_equivalence`` verifies that no constant name occurs inside a longer
identifier in the kernels used, in which case the two mechanisms give the same program.
"""
import json
import math
import os
import re
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "_ref")

KERNELS = [
    "real_enc_frame_proj_fwd_length", "real_enc_frame_proj_fwd_angle",
    "real_enc_frame_proj_bwd_length", "real_enc_frame_proj_bwd_angle",
    "compute_maximum_frame_each_edge", "compute_second_frame_each_edge",
    "fused_dpa_fwd", "fused_dpa_bwd", "fused_dpa_bwd_q",
    "irregular_transpose", "irregular_mean_fwd",
    "real_enc_proj_fwd", "real_enc_proj_bwd",
    "real_enc_sigma_fwd", "fused_dpa_sigmamat_fwd",
    "compute_second_frame_static_each_edge",
    "compute_lattice_first_frame", "compute_lattice_second_frame", "compute_lattice_third_frame",
    "reci_enc_fwd", "reci_enc_bwd",
    "compute_third_frame_each_edge",
    "real_enc_fwd", "real_enc_bwd",
]


# irregular_mean_fwd calls a helper template that carries no __device__ qualifier; the
# reference's runtime compiler accepts that, nvcc does not, so it has no GPU build here.
GPU_SKIP = {"irregular_mean_fwd"}


def constants(head_num=8, key_head_dim=16, value_pe_dim=64, dim_angle_enc=64, value_head_dim=16,
              lattice_range=2, set_minimum_range=True, cos_abs=0, value_pe_dist_wscale=1.0,
              value_pe_angle_wscale=4.0, value_pe_dist_coef=1.0, value_pe_angle_coef=1.0,
              symm_break_noise=0.0):
    """Same names and values as compile_kernels builds (kernel_manager.py:124-149)."""
    c = {
        "LATTICE_RANGE": lattice_range, "SEARCH_RANGE": 3, "PE_THREAD_NUM": 16, "THREAD_NUM": head_num,
        "HEAD_NUM": head_num, "VPE_DIM": value_pe_dim, "ANGLE_ENC_DIM": dim_angle_enc,
        "V_HEAD_DIM": value_head_dim, "SIGMAMAT_DIM": 6, "K_HEAD_DIM": key_head_dim,
        "SKIP_OUTOF_RADIUS": 0, "MINIMUM_RANGE": lattice_range if set_minimum_range else 0,
        "MAX_SYSTEM_SIZE_POW2": 512, "MAX_SYSTEM_SIZE": 320, "RUNNING_SUM_LEN": 8, "MAXIMUM_RANGE": 10,
        "CUT_SIGMA": 4, "COS_ABS": cos_abs, "AXIS_NUM": 3, "LENGTH_RBF_MUL": value_pe_dist_coef,
        "ANGLE_RBF_MUL": value_pe_angle_coef, "SYMM_BREAK_NOISE": symm_break_noise,
    }
    c["LENGTH_RANGE"] = math.ceil(2 * value_pe_dist_wscale * c["CUT_SIGMA"] + 1)
    c["ANGLE_RANGE"] = math.ceil(2 * value_pe_angle_wscale * c["CUT_SIGMA"] + 1)
    return c


def check_macro_equivalence(text, consts):
    """Replay the reference's ordered textual replacement on every identifier of the
    kernel text and require the outcome a token macro would give: a constant's name turns
    into its value, any other identifier stays untouched."""
    for tok in set(re.findall(r"[A-Za-z_][A-Za-z_0-9]*", text)):
        replaced = tok
        for key, val in consts.items():
            replaced = replaced.replace(key, str(val))
        expect = str(consts[tok]) if tok in consts else tok
        if replaced != expect:
            raise RuntimeError(f"identifier {tok}: textual replacement gives {replaced}, macro gives {expect}")


def parse_params(text, name):
    m = re.search(r"void\s+" + re.escape(name) + r"\s*\(([^)]*)\)", text, re.S)
    if m is None:
        raise RuntimeError(f"kernel {name}: signature not found")
    params = []
    for p in m.group(1).split(","):
        p = re.sub(r"//.*", "", p)
        p = " ".join(p.split())
        if not p:
            continue
        mm = re.match(r"(.*?)([A-Za-z_][A-Za-z_0-9]*)$", p)
        params.append((mm.group(1).strip(), mm.group(2)))
    return params


def _ctype(t):
    t = t.replace("const", "").strip()
    if "*" in t:
        return "ptr"
    t = " ".join(t.split())
    return {"unsigned int": "u32", "unsigned char": "u8", "float": "f32", "long long int": "i64",
            "unsigned long long": "u64", "long long": "i64", "int": "i32", "double": "f64"}[t]


def build(reference_root, force=False, consts=None, tag=""):
    consts = consts or constants()
    os.makedirs(OUT, exist_ok=True)
    kdir = os.path.join(reference_root, "models", "kernels")
    defs = [f"-D{k}={v}" for k, v in consts.items()]
    cpu_objs, gpu_srcs, sigs = [], [], {}
    cpu_lib = os.path.join(OUT, f"libcfref_cpu{tag}.so")
    gpu_lib = os.path.join(OUT, f"libcfref_gpu{tag}.so")
    sig_json = os.path.join(OUT, f"signatures{tag}.json")
    stamp = json.dumps(dict(consts, _kernels=" ".join(KERNELS)), sort_keys=True)
    if (not force and os.path.exists(cpu_lib) and os.path.exists(sig_json)
            and json.load(open(sig_json)).get("_consts") == stamp):
        return
    for name in KERNELS:
        src = os.path.join(kdir, name + ".cu")
        text = open(src).read()
        check_macro_equivalence(text, consts)
        params = parse_params(text, name)
        sigs[name] = [_ctype(t) for t, _ in params]
        plist = ", ".join(f"{t} {n}" for t, n in params)
        args = ", ".join(n for _, n in params)
        inc = f'#include "models/kernels/{name}.cu"\n'
        cpu_src = os.path.join(OUT, f"cpu_{name}{tag}.cpp")
        with open(cpu_src, "w") as f:
            f.write('#include "cuda_host_shim.h"\n' + inc)
            f.write(f'extern "C" void cfref_cpu_{name}(unsigned int grid_, unsigned int block_, {plist}) {{\n'
                    "#pragma omp parallel for schedule(dynamic, 64)\n"
                    "  for (long long b_ = 0; b_ < (long long)grid_; b_++)\n"
                    "    for (unsigned int t_ = 0; t_ < block_; t_++) {\n"
                    "      cfshim_set((unsigned int)b_, t_, grid_, block_);\n"
                    f"      {name}({args});\n"
                    "    }\n}\n")
        obj = cpu_src[:-4] + ".o"
        subprocess.check_call(["g++", "-O2", "-fPIC", "-fopenmp", "-std=c++14", "-w", "-x", "c++",
                               "-ffp-contract=fast", "-I", os.path.join(HERE, "fake_curand"), "-I", HERE,
                               "-I", reference_root, "-I", "/usr/local/cuda/include"] + defs +
                              ["-c", cpu_src, "-o", obj])
        cpu_objs.append(obj)
        gpu_src = os.path.join(OUT, f"gpu_{name}{tag}.cu")
        with open(gpu_src, "w") as f:
            f.write("#include <cuda_runtime.h>\n"
                    "#undef __forceinline__\n"
                    "#define __forceinline__ __device__ __inline__ __attribute__((always_inline))\n" + inc)
            f.write(f'extern "C" int cfref_gpu_{name}(unsigned int grid_, unsigned int block_, void* stream_, {plist}) {{\n'
                    f"  {name}<<<grid_, block_, 0, (cudaStream_t)stream_>>>({args});\n"
                    "  return (int)cudaGetLastError();\n}\n")
        if name not in GPU_SKIP:
            gpu_srcs.append(gpu_src)
    subprocess.check_call(["g++", "-shared", "-fopenmp", "-o", cpu_lib] + cpu_objs)
    sigs["_consts"] = stamp
    json.dump(sigs, open(sig_json, "w"), indent=1)
    # GPU build of the same sources; the noise constant is kept at the CPU build's value.
    try:
        gpu_objs = []
        for s in gpu_srcs:
            o = s[:-3] + ".o"
            subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-w",
                                   "-Xcompiler", "-fPIC", "-std=c++14", "-I", reference_root] + defs +
                                  ["-c", s, "-o", o])
            gpu_objs.append(o)
        subprocess.check_call(["nvcc", "-shared", "-o", gpu_lib] + gpu_objs)
    except (subprocess.CalledProcessError, FileNotFoundError) as exc:
        print("reference GPU build skipped:", exc)


if __name__ == "__main__":
    import sys
    sys.path.insert(0, os.path.dirname(HERE))
    import build_oracle
    root = build_oracle.reference_root()
    if root is None:
        raise SystemExit("reference tree not found: set CF_REFERENCE_ROOT")
    build(root, force="--force" in sys.argv)
