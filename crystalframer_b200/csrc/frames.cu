// Dynamic "max" frames: per (atom, head) the nearest-image axis, the second axis, and the
// Gram-Schmidt completion (replaces compute_maximum_frame_each_edge.cu,
// compute_second_frame_each_edge.cu, the torch_scatter argmax of
// models/cuda_funcs/calc_maximum_frame.py and the torch ops of
// models/indexed_lattice_multi_head_attention_cuda.py:475-481 of the reference).
//
// One warp owns one (atom i, head h); lanes own the atom's pairs (i, j).  All pairs of one
// (atom, head) share the lattice range, so the translation loops are uniform across the warp.
// Per pair a lane finds its candidate image and score; a warp arg-max (lowest pair index on
// ties) picks the atom's axis.  Every float operation that feeds a comparison is written with
// explicit round-to-nearest intrinsics in the reference's evaluation order (no fused
// multiply-add), so that the selected pair and image can be reproduced bit for bit on a CPU.
#include "common.cuh"

namespace cfb {

constexpr int kFrWarps = 4;
constexpr int kFrHd = 16;

struct FrArgs {
    const float* q; const float* k; const float* a_ik; const float* pos_ij; const float* tvecs;
    const float* rvlen; const int64_t* batch; const int64_t* edges; const int64_t* e_start;
    int64_t N, E;
    uint64_t seed1, seed2;
    const float* frame1_in;
    float* frame1; float* frame2; float* frame3;     // mode 1: frame1 out; mode 2: frame2 out (raw); mode 3: all, completed
    int64_t* sel_edge; int32_t* sel_image;
    int mode;
};

struct Cell { float rx, ry, rz, t1x, t1y, t1z, t2x, t2y, t2z, t3x, t3y, t3z; };

__device__ __forceinline__ void separation(const Cell& c, float n1, float n2, float n3, float& dx, float& dy,
                                           float& dz, float& d2)
{
    dx = __fadd_rn(__fadd_rn(__fadd_rn(c.rx, __fmul_rn(c.t1x, n1)), __fmul_rn(c.t2x, n2)), __fmul_rn(c.t3x, n3));
    dy = __fadd_rn(__fadd_rn(__fadd_rn(c.ry, __fmul_rn(c.t1y, n1)), __fmul_rn(c.t2y, n2)), __fmul_rn(c.t3y, n3));
    dz = __fadd_rn(__fadd_rn(__fadd_rn(c.rz, __fmul_rn(c.t1z, n1)), __fmul_rn(c.t2z, n2)), __fmul_rn(c.t3z, n3));
    d2 = __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
}

__device__ __forceinline__ float noise_term(float amp, uint64_t seed, uint64_t tid, uint32_t t)
{
    if (amp == 0.0f) return 0.0f;
    return (float)(((double)hash_uniform(seed, tid, t) - 0.5) * (double)amp);
}

struct Cand { float score; int64_t e; float ux, uy, uz; int img; };

// warp arg-max by (score desc, pair index asc); candidates with e < 0 never win
__device__ __forceinline__ Cand warp_argmax(Cand c)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float s = __shfl_xor_sync(0xffffffffu, c.score, o);
        const long long e = __shfl_xor_sync(0xffffffffu, (long long)c.e, o);
        const float ux = __shfl_xor_sync(0xffffffffu, c.ux, o), uy = __shfl_xor_sync(0xffffffffu, c.uy, o),
                    uz = __shfl_xor_sync(0xffffffffu, c.uz, o);
        const int img = __shfl_xor_sync(0xffffffffu, c.img, o);
        const bool take = e >= 0 && (c.e < 0 || s > c.score || (s == c.score && e < (long long)c.e));
        if (take) { c.score = s; c.e = e; c.ux = ux; c.uy = uy; c.uz = uz; c.img = img; }
    }
    return c;
}

__global__ void __launch_bounds__(kFrWarps * 32) max_frame_kernel(const FrArgs A, const Params P)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t task = (int64_t)blockIdx.x * kFrWarps + warp;
    const int H = P.H;
    if (task >= A.N * H) return;
    const int64_t i = task / H;
    const int h = (int)(task - i * H);
    const int64_t c = A.batch[i];
    const int64_t e0 = A.e_start[i], e1 = A.e_start[i + 1];
    const float a = __ldg(A.a_ik + i * H + h);
    int Rl = 0;
    if (lane < 3) Rl = lattice_range_1d(P, a, P.cutoff_radius != 0.0f ? __ldg(A.rvlen + 3 * c + lane) : 0.0f);
    const int R1 = __shfl_sync(0xffffffffu, Rl, 0), R2 = __shfl_sync(0xffffffffu, Rl, 1), R3 = __shfl_sync(0xffffffffu, Rl, 2);
    Cell cell;
    {
        const float* Tc = A.tvecs + 9 * c;
        cell.t1x = __ldg(Tc); cell.t1y = __ldg(Tc + 1); cell.t1z = __ldg(Tc + 2);
        cell.t2x = __ldg(Tc + 3); cell.t2y = __ldg(Tc + 4); cell.t2z = __ldg(Tc + 5);
        cell.t3x = __ldg(Tc + 6); cell.t3y = __ldg(Tc + 7); cell.t3z = __ldg(Tc + 8);
    }
    float qv[kFrHd];
    {
        const float4* q4 = reinterpret_cast<const float4*>(A.q + (i * H + h) * kFrHd);
#pragma unroll
        for (int d4 = 0; d4 < kFrHd / 4; d4++) {
            const float4 v = __ldg(q4 + d4);
            qv[4 * d4] = v.x; qv[4 * d4 + 1] = v.y; qv[4 * d4 + 2] = v.z; qv[4 * d4 + 3] = v.w;
        }
    }

    float f1x = 0.f, f1y = 0.f, f1z = 0.f;
    if (A.mode == 2) {
        const float* f = A.frame1_in + (i * H + h) * 3;
        f1x = __ldg(f); f1y = __ldg(f + 1); f1z = __ldg(f + 2);
    }

    for (int axis = (A.mode == 2 ? 2 : 1); axis <= (A.mode == 1 ? 1 : 2); axis++) {
        Cand best; best.score = -1e10f; best.e = -1; best.ux = best.uy = best.uz = 0.f; best.img = -1;
        for (int64_t eb = e0; eb < e1; eb += 32) {
            const int64_t e = eb + lane;
            if (e < e1) {
                const int64_t j = A.edges[A.E + e];
                cell.rx = __ldg(A.pos_ij + 3 * e); cell.ry = __ldg(A.pos_ij + 3 * e + 1); cell.rz = __ldg(A.pos_ij + 3 * e + 2);
                float dot = 0.f;
                const float4* k4 = reinterpret_cast<const float4*>(A.k + (j * H + h) * kFrHd);
#pragma unroll
                for (int d4 = 0; d4 < kFrHd / 4; d4++) {
                    const float4 v = __ldg(k4 + d4);
                    dot = __fmaf_rn(qv[4 * d4], v.x, dot); dot = __fmaf_rn(qv[4 * d4 + 1], v.y, dot);
                    dot = __fmaf_rn(qv[4 * d4 + 2], v.z, dot); dot = __fmaf_rn(qv[4 * d4 + 3], v.w, dot);
                }
                const uint64_t tid = (uint64_t)(e * H + h);
                float ux = 0.f, uy = 0.f, uz = 0.f, value;
                int img = -1;
                if (axis == 1) {
                    // nearest image with d^2 > 1e-5 (compute_maximum_frame_each_edge.cu:81-111)
                    float d2_min = 1e10f;
                    int t = 0;
                    for (int n1 = -R1; n1 <= R1; n1++)
                        for (int n2 = -R2; n2 <= R2; n2++)
                            for (int n3 = -R3; n3 <= R3; n3++, t++) {
                                float dx, dy, dz, d2;
                                separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                                if ((double)d2 > 1e-5) {
                                    const float cand = __fadd_rn(d2, noise_term(P.noise, A.seed1, tid, (uint32_t)t));
                                    if (d2_min > cand) {
                                        d2_min = cand;
                                        const float d = __fsqrt_rn(d2);
                                        ux = __fdiv_rn(dx, d); uy = __fdiv_rn(dy, d); uz = __fdiv_rn(dz, d);
                                        img = t;
                                    }
                                }
                            }
                    value = __fmul_rn(a, d2_min);
                } else {
                    // second axis (compute_second_frame_each_edge.cu:81-142)
                    float d2min = 1e10f;
                    for (int n1 = -R1; n1 <= R1; n1++)
                        for (int n2 = -R2; n2 <= R2; n2++)
                            for (int n3 = -R3; n3 <= R3; n3++) {
                                float dx, dy, dz, d2;
                                separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                                if ((double)d2 > 1e-5) d2min = fminf(d2min, d2);
                            }
                    float max_val = -1e15f;
                    value = -1e15f;
                    int t = 0;
                    for (int n1 = -R1; n1 <= R1; n1++)
                        for (int n2 = -R2; n2 <= R2; n2++)
                            for (int n3 = -R3; n3 <= R3; n3++, t++) {
                                float dx, dy, dz, d2;
                                separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                                if ((double)d2 > 1e-5) {
                                    const float d = __fsqrt_rn(d2);
                                    const float vx = __fdiv_rn(dx, d), vy = __fdiv_rn(dy, d), vz = __fdiv_rn(dz, d);
                                    const float cs = __fadd_rn(__fadd_rn(__fmul_rn(vx, f1x), __fmul_rn(vy, f1y)), __fmul_rn(vz, f1z));
                                    const float one_m = __fsub_rn(1.0f, fabsf(cs));
                                    const float clipped = ((double)one_m > 1e-5) ? one_m : 1e-5f;
                                    const float score = __fadd_rn(__fmul_rn(a, __fsub_rn(d2, d2min)), logf(clipped));
                                    const float nz = noise_term(P.noise, A.seed2, tid, (uint32_t)t);
                                    if (score > __fadd_rn(max_val, nz) && (double)fabsf(cs) < 0.9999) {
                                        max_val = __fadd_rn(score, nz);
                                        ux = vx; uy = vy; uz = vz;
                                        value = __fadd_rn(score, __fmul_rn(a, d2min));
                                        img = t;
                                    }
                                }
                            }
                }
                const float s = __fadd_rn(dot, value);
                if (s > best.score) { best.score = s; best.e = e; best.ux = ux; best.uy = uy; best.uz = uz; best.img = img; }
            }
        }
        best = warp_argmax(best);
        if (axis == 1) {
            f1x = best.ux; f1y = best.uy; f1z = best.uz;
            if (A.mode != 2 && lane == 0) {
                float* o = A.frame1 + (i * H + h) * 3;
                o[0] = f1x; o[1] = f1y; o[2] = f1z;
                if (A.mode == 1 && A.sel_edge) A.sel_edge[i * H + h] = best.e;
                if (A.mode == 1 && A.sel_image) A.sel_image[i * H + h] = best.img;
            }
        } else if (lane == 0) {
            float* o2 = A.frame2 + (i * H + h) * 3;
            if (A.mode == 2) {
                o2[0] = best.ux; o2[1] = best.uy; o2[2] = best.uz;
                if (A.sel_edge) A.sel_edge[i * H + h] = best.e;
                if (A.sel_image) A.sel_image[i * H + h] = best.img;
            } else {
                // Gram-Schmidt, normalisation with max(norm, 1e-12), cross product
                const float dot = __fadd_rn(__fadd_rn(__fmul_rn(f1x, best.ux), __fmul_rn(f1y, best.uy)), __fmul_rn(f1z, best.uz));
                const float wx = __fsub_rn(best.ux, __fmul_rn(dot, f1x)), wy = __fsub_rn(best.uy, __fmul_rn(dot, f1y)),
                            wz = __fsub_rn(best.uz, __fmul_rn(dot, f1z));
                float nrm = __fsqrt_rn(__fadd_rn(__fadd_rn(__fmul_rn(wx, wx), __fmul_rn(wy, wy)), __fmul_rn(wz, wz)));
                nrm = fmaxf(nrm, 1e-12f);
                const float gx = __fdiv_rn(wx, nrm), gy = __fdiv_rn(wy, nrm), gz = __fdiv_rn(wz, nrm);
                o2[0] = gx; o2[1] = gy; o2[2] = gz;
                float* o3 = A.frame3 + (i * H + h) * 3;
                o3[0] = __fsub_rn(__fmul_rn(f1y, gz), __fmul_rn(f1z, gy));
                o3[1] = __fsub_rn(__fmul_rn(f1z, gx), __fmul_rn(f1x, gz));
                o3[2] = __fsub_rn(__fmul_rn(f1x, gy), __fmul_rn(f1y, gx));
            }
        }
    }
}

int max_frame(const FrArgs& A, const Params& P, cudaStream_t st)
{
    const int64_t tasks = A.N * P.H;
    if (tasks == 0) return CFB200_OK;
    max_frame_kernel<<<(unsigned)((tasks + kFrWarps - 1) / kFrWarps), kFrWarps * 32, 0, st>>>(A, P);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
