// Shared device helpers of libcfb200 (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/cfb200.h"

#ifndef __CUDA_ARCH__
#define CFB_ARCH_OK 1
#elif __CUDA_ARCH__ >= 1000
#define CFB_ARCH_OK 1
#else
#error "libcfb200 is written for sm_100a only"
#endif

namespace cfb {

constexpr int kWarp = 32;
constexpr float kPiF = 3.141592654f;          // float-rounded pi, as CUDART_PI_F
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kSqrtLog2e = 1.2011224087864498f;

// Derived, launch-time view of cfb200_config (host fills it, kernels take it by value).
struct Params {
    int H, head_dim, dist_dim, angle_dim;
    int lattice_range, minimum_range, cos_abs;
    int win_dist, win_ang;        // LENGTH_RANGE / ANGLE_RANGE; == dim when the full range is computed
    int windowed_dist, windowed_ang;
    float cutoff_radius;
    float c_dist, c_ang, noise;
    float prune;                  // translations with weight below exp(-prune) of the largest skip the bases
    // distance basis: b(dim) = (-d/interval + dim + 1) * step
    float d_interval, d_step, d_cut;      // d_cut = cut_sigma * sigma
    // angle basis: b(dim) = (1 - cos) * sigma_inv - (D - 1 - dim) * step
    float a_interval, a_step, a_sigma_inv, a_cut;   // a_cut = cut_sigma * angle_sigma
};

// Multiprocessors of the current device (asked once per device and host thread: the query costs as much as a launch).
inline int sm_count()
{
    thread_local int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int sms = 148;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        cached[dev] = sms;
    }
    return cached[dev];
}

// Device status word (bits CFB200_ST_*).  The library is built as one translation unit.
__device__ int g_status = 0;

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed FP32: two floats in one 64-bit register, one instruction for two fused multiply-adds (fma.rn.f32x2 and its
// mul twin, sm_100).  Each half is an ordinary IEEE round-to-nearest operation; what is saved is issue slots.
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(const float lo, const float hi)
{
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack2(const f32x2 v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ f32x2 fma2(const f32x2 a, const f32x2 b, const f32x2 c)
{
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ f32x2 mul2(const f32x2 a, const f32x2 b)
{
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_min(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Counter-based uniform in (0,1] for the symmetry-breaking noise of the frame search.
// The reference draws from per-thread curand XORWOW streams whose seed comes from numpy's
// global generator (models/cuda_funcs/calc_maximum_frame.py:43); nothing pins those streams,
// so a stateless hash of (seed, pair*H+head, translation index) is used instead.
__host__ __device__ __forceinline__ float hash_uniform(uint64_t seed, uint64_t tid, uint32_t draw)
{
    uint64_t x = seed ^ (tid * 0x9E3779B97F4A7C15ull) ^ ((uint64_t)draw * 0xD1B54A32D192ED03ull);
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return (float)((uint32_t)(x >> 40) + 1u) * (1.0f / 16777216.0f);
}

// Per-pair translation list (pair_list_kernel): kListPlanes planes of kListLen entries per pair, sorted by
// squared distance -- d^2, x, y, z (fused arithmetic of the lattice-sum kernel) and the packed translation
// (n1 + R) | (n2 + R) << 8 | (n3 + R) << 16 | linear index << 24.  Unused entries hold d^2 = 1e30.
constexpr int kListLen = 128;
constexpr int kListPlanes = 5;
constexpr int kListStride = kListLen * kListPlanes;

// Work estimate of the fused attention kernels, in warp instructions: one pair of an (atom, head) task costs about
// kAtPairCost plus kAtTermCost per translation that survives the pruning.
constexpr float kAtPairCost = 350.0f, kAtTermCost = 70.0f;
// Long tasks are cut into chunks of consecutive pairs whose partial results a small kernel merges afterwards
// (see atom_order_kernel and attn_fused.cu): at most kSplitMaxChunks chunks of at least kSplitMinPairs pairs,
// kSplitSlots partial rows per head, no task below kSplitMinTarget instructions is cut.  kSplitWideSphere: volume of
// the pruning sphere (radius^2 = 16 / |a|) of a Gaussian two standard deviations wider than typical (|a| = 0.051).
constexpr int kSplitSlots = CFB200_SPLIT_SLOTS, kSplitMaxChunks = 8, kSplitMinPairs = 4;
constexpr float kSplitMinTarget = 20000.0f, kSplitWideSphere = 23200.0f, kSplitWideCap = 1500.0f;
constexpr int kSplitPartFwd = 304, kSplitPartBwd = 32;       // floats per partial row and head (289 and 17 used)

// Chunks an (atom, head) task with `pairs` pairs really uses, of the `chunks` its crystal was given: its own
// instruction estimate (translations within the pruning radius of its coefficient a) over the target.  Every warp
// that draws a chunk of the task computes the same number.
__device__ __forceinline__ int split_active_chunks(const float a, const int pairs, const float inv_vol, const float target,
                                                   const int chunks)
{
    const float aa = fmaxf(fabsf(a), 1e-6f);
    const float sphere = 268.08f / (aa * sqrtf(aa)) * inv_vol;          // 4/3 pi (16 / |a|)^(3/2) / volume
    const float terms = fminf(kSplitWideCap, fmaxf(sphere, 1.0f));
    const float est = (float)pairs * (kAtPairCost + kAtTermCost * terms);
    const float want = ceilf(est / target);
    return want >= (float)chunks ? chunks : max((int)want, 1);
}

// Lattice range along one reciprocal axis for Gaussian coefficient a (< 0):
// models/kernels/real_enc_frame_proj_fwd_length.cu:59-86.  (cutoff + 0.01f) * rvl is a float
// product, the division by 2.0 * CUDART_PI_F and the ceil are double, as in the reference.
__device__ __forceinline__ int lattice_range_1d(const Params& P, float a, float rvl)
{
    int R = P.lattice_range;
    float cutoff = P.cutoff_radius;
    if (cutoff != 0.0f) {
        if (cutoff < 0.0f) cutoff = __fmul_rn(__fsqrt_rn(__fdiv_rn(-0.5f, a)), -cutoff);
        float num = __fmul_rn(__fadd_rn(cutoff, 0.01f), rvl);
        // ceil(num / (2.0 * CUDART_PI_F)) in double, without the division: a float estimate, then
        // the smallest integer k with k * 2pi_f >= num, decided by exact double products (both
        // factors have at most 24 + 6 significant bits).  Quotients that the reference's rounded
        // division could push across an integer do not occur for float inputs.
        const double two_pi = 2.0 * (double)kPiF;
        double r = (double)ceilf(num * 0.15915494f);
        if ((double)num > r * two_pi) r += 1.0;
        else if ((double)num <= (r - 1.0) * two_pi) r -= 1.0;
        if (!(num == num)) r = (double)num;          // keep NaN visible to the check below
        // NaN (a >= 0) and runaway ranges are reported through the status word, never looped on
        if (!(r <= (double)CFB200_MAX_RANGE)) {
            atomicOr(&g_status, !(a < 0.0f) ? CFB200_ST_BAD_COEF : CFB200_ST_RANGE_CLAMPED);
            r = !(a < 0.0f) ? (double)P.lattice_range : (double)CFB200_MAX_RANGE;
        }
        R = (int)r;
        if (P.minimum_range > 0) R = max(R, P.minimum_range);
    }
    return R;
}

}  // namespace cfb
