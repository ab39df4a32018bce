// Dynamic "max" frames: per (atom, head) the nearest-image axis, the second axis, and the
// Gram-Schmidt completion (replaces compute_maximum_frame_each_edge.cu,
// compute_second_frame_each_edge.cu, the torch_scatter argmax of
// models/cuda_funcs/calc_maximum_frame.py and the torch ops of
// models/indexed_lattice_multi_head_attention_cuda.py:475-481 of the reference).
//
// grid = (spans of 224 pairs, heads).  A block owns the query atoms whose first pair falls in its
// span and walks all pairs of those atoms, one pair per thread -- about 200 pairs per block
// whatever the crystal sizes, so small crystals do not leave lanes idle.  Each thread sweeps the
// lattice translations of its pair, finds the pair's candidate image and score, and folds
// (score, pair index) into its query atom's slot in shared memory with one 64-bit atomicMax -- an
// order-independent arg-max with "lowest pair index wins" on equal scores.  After the barrier the
// thread that holds an atom's maximum leaves its direction and image index in shared memory.
//
// Every float operation that feeds a comparison is written with explicit round-to-nearest
// intrinsics in the reference's evaluation order (no fused multiply-add), so the selected pair
// and image can be reproduced bit for bit on a CPU.  Both searches are written as order-independent
// arg-min / arg-max with "first translation in the reference's loop order wins" on equal values, which
// is what the reference's sequential loops compute when the symmetry-breaking noise is off; with
// noise on, the winner is the arg-max of score + noise (the reference's running comparison adds
// the noise asymmetrically and therefore depends on the visiting order).
#include "common.cuh"

namespace cfb {

#ifndef CFB_FR_THREADS
#define CFB_FR_THREADS 256
#define CFB_FR_PAIRS 224
#define CFB_FR_BLOCKS 3
#endif
constexpr int kFrPairs = CFB_FR_PAIRS;     // pair-list span whose query atoms one block owns: the block's atoms have up to
                                           // span + (pairs of the last atom - 1) pairs, usually one round of kFrThreads
                                           // threads, sometimes two (measured: 224 beats 192, which always fits one round
                                           // for crystals of up to 64 atoms, by 5 %)
constexpr int kFrThreads = CFB_FR_THREADS;
constexpr int kFrMaxRows = kFrThreads;     // at most one atom starts per pair of the span (kFrPairs <= kFrThreads)
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
    const float4* cache;      // optional per-pair results of pair_cache_kernel, valid for ranges (cache_range)^3
    const float* list;        // optional per-pair sorted translation lists (pair_list_kernel)
    int cache_range;
    int is_static;            // "max_static": queries and keys do not enter the selection and the second axis' score
                              // carries no Gaussian coefficient (compute_second_frame_static_each_edge.cu:126,135)
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
    // (u - 0.5) * amp: u is a multiple of 2^-24 in (0, 1], so u - 0.5 is exact and the single rounding of
    // the float product equals the rounding of the same product formed in double
    return __fmul_rn(__fsub_rn(hash_uniform(seed, tid, t), 0.5f), amp);
}

struct Cand { float value; float ux, uy, uz; int img; float d2raw; };   // d2raw: smallest d^2 > 1e-5 (first axis only)

// The reference compares floats with the double literals 1e-5 and 0.9999.  For a float x these are
// the same decisions as the float comparisons below, because float(1e-5) < 1e-5 and float(0.9999) <
// 0.9999 with no float in between:  x > 1e-5  <=>  x > kTiny,   x < 0.9999  <=>  x <= kCosMax.
constexpr float kTiny = 1e-5f;       // 9.99999974737875e-06
constexpr float kCosMax = 0.9999f;   // 0.99989998340606689453

// centre-out enumeration of one lattice index: k = 0, 1, 2, 3, 4 ... -> n = 0, -1, 1, -2, 2 ...
__device__ __forceinline__ int centre_out(int k) { return (k & 1) ? -((k + 1) >> 1) : (k >> 1); }

// Nearest image with d^2 > 1e-5 (compute_maximum_frame_each_edge.cu:81-111): arg-min over the
// translations of d^2 + noise, the first translation in the reference's loop order on equal values.
// Pass 1 finds the smallest un-perturbed d^2 and, with noise off, the winner itself; with noise on,
// pass 2 draws the noise only for translations within the noise amplitude of that minimum (nothing
// else can win).  The direction is computed once, for the winner.
__device__ __forceinline__ Cand first_axis_candidate(const Cell& cell, float a, int R1, int R2, int R3, float amp,
                                                     uint64_t seed, uint64_t tid, const float4* cached, const int cache_range,
                                                     const float* list = nullptr, const float reach2 = 1e38f)
{
    Cand c; c.ux = c.uy = c.uz = 0.f; c.img = -1;
    float d2raw = 1e10f, d2next = 1e10f;      // smallest and second smallest d^2 > 1e-5 (equal values count twice)
    int t = 0, best_t = -1;
    if (cached != nullptr) {                  // pass 1 is pure geometry: the same for every head and layer
        const float4 g = __ldg(cached);
        d2raw = g.x; d2next = g.y; best_t = __float_as_int(g.z);
        if (best_t >= 0 && (R1 != cache_range || R2 != cache_range || R3 != cache_range)) {
            // the cached index counts the translations of the cached box; here the box is larger
            const int Lc = 2 * cache_range + 1;
            const int q = best_t / Lc, k3 = best_t - q * Lc, k1 = q / Lc, k2 = q - k1 * Lc;
            best_t = ((k1 - cache_range + R1) * (2 * R2 + 1) + (k2 - cache_range + R2)) * (2 * R3 + 1) + (k3 - cache_range + R3);
        }
    } else
    for (int n1 = -R1; n1 <= R1; n1++)
        for (int n2 = -R2; n2 <= R2; n2++)
            for (int n3 = -R3; n3 <= R3; n3++, t++) {
                float dx, dy, dz, d2;
                separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                if (d2 > kTiny) {
                    if (d2 < d2raw) { d2next = d2raw; d2raw = d2; best_t = t; }
                    else if (d2 < d2next) d2next = d2;
                }
            }
    float d2_min = d2raw;
    const float limit = __fadd_rn(d2raw, __fmul_rn(amp, 1.001f));
    if (amp > 0.0f && best_t >= 0 && !(d2next <= limit)) {
        // no other translation is within the noise amplitude of the minimum: the winner stands and
        // only its own noise enters the score
        d2_min = __fadd_rn(d2raw, noise_term(amp, seed, tid, (uint32_t)best_t));
    } else if (amp != 0.0f && best_t >= 0 && list != nullptr && limit < reach2) {
        // The translations within the noise amplitude of the minimum are the first few of the pair's sorted list
        // (the list's distances differ from the ones compared here by a few ulp, hence the margin; everything
        // outside the listed box is farther than reach2).  Same arg-min as the sweep below, written without
        // reference to the visiting order: smallest d^2 + noise, lowest translation index on equal values.
        d2_min = 1e10f; best_t = -1;
        const float stop = limit + fabsf(limit) * 8e-6f + 1e-12f;
        const int L2 = 2 * R2 + 1, L3 = 2 * R3 + 1;
        for (int s = 0; s < kListLen; s++) {
            if (!(__ldg(list + s) <= stop)) break;
            const int code = __float_as_int(__ldg(list + 4 * kListLen + s));
            const int n1 = (code & 255) - cache_range, n2 = ((code >> 8) & 255) - cache_range, n3 = ((code >> 16) & 255) - cache_range;
            float dx, dy, dz, d2;
            separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
            if (d2 > kTiny && d2 <= limit) {
                const int tt = ((n1 + R1) * L2 + (n2 + R2)) * L3 + (n3 + R3);
                const float cand = __fadd_rn(d2, noise_term(amp, seed, tid, (uint32_t)tt));
                if (cand < d2_min || (cand == d2_min && tt < best_t)) { d2_min = cand; best_t = tt; }
            }
        }
    } else if (amp != 0.0f && best_t >= 0) {
        d2_min = 1e10f; best_t = -1;
        t = 0;
        for (int n1 = -R1; n1 <= R1; n1++)
            for (int n2 = -R2; n2 <= R2; n2++)
                for (int n3 = -R3; n3 <= R3; n3++, t++) {
                    float dx, dy, dz, d2;
                    separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                    if (d2 > kTiny && d2 <= limit) {
                        const float cand = __fadd_rn(d2, noise_term(amp, seed, tid, (uint32_t)t));
                        if (d2_min > cand) { d2_min = cand; best_t = t; }
                    }
                }
    }
    if (best_t >= 0) {
        const int L3 = 2 * R3 + 1, L2 = 2 * R2 + 1;
        const int q = best_t / L3, n3 = best_t - q * L3 - R3, n1 = q / L2 - R1, n2 = q - (q / L2) * L2 - R2;
        float dx, dy, dz, d2;
        separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
        const float d = __fsqrt_rn(d2);
        c.ux = __fdiv_rn(dx, d); c.uy = __fdiv_rn(dy, d); c.uz = __fdiv_rn(dz, d);
        c.img = best_t;
    } else {
        d2_min = 1e10f;
    }
    c.value = __fmul_rn(a, d2_min);
    c.d2raw = d2raw;
    return c;
}

// Second axis (compute_second_frame_each_edge.cu:81-142): arg-max over the translations of
// a (d^2 - d^2_min) + log(max(1 - |cos|, 1e-5)) + noise among images with |cos| < 0.9999, the first
// translation in the reference's loop order on equal values.  Translations are visited centre-out so
// that a good candidate is met early; the sqrt, divisions and logarithm are skipped for images whose
// Gaussian part alone cannot reach the running maximum (the logarithm is never positive).
// d2min_known >= 0: the smallest non-zero squared distance, already found by the first-axis sweep
// of the same pair (same operations, same value); otherwise it is searched here.
__device__ __forceinline__ Cand second_axis_candidate(const Cell& cell, float a, int R1, int R2, int R3, float amp,
                                                      uint64_t seed, uint64_t tid, float f1x, float f1y, float f1z,
                                                      float d2min_known, const float* list, const bool is_static = false,
                                                      const int list_range = 0, const float reach2 = 1e38f)
{
    Cand c; c.ux = c.uy = c.uz = 0.f; c.img = -1; c.value = -1e15f; c.d2raw = 0.f;
    float d2min = d2min_known >= 0.f ? d2min_known : 1e10f;
    if (d2min_known < 0.f)
        for (int n1 = -R1; n1 <= R1; n1++)
            for (int n2 = -R2; n2 <= R2; n2++)
                for (int n3 = -R3; n3 <= R3; n3++) {
                    float dx, dy, dz, d2;
                    separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                    if (d2 > kTiny) d2min = fminf(d2min, d2);
                }
    float best = -1e15f;                 // running maximum of score + noise
    const float half = 0.5f * amp;
    const int L2 = 2 * R2 + 1, L3 = 2 * R3 + 1;
    // one candidate: exactly the reference's arithmetic, whatever the visiting order
    auto score_candidate = [&](const int n1, const int n2, const int n3) {
        float dx, dy, dz, d2;
        separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
        if (!(d2 > kTiny)) return;
        // the static variant's score is (d^2 - d^2_min) + log(...): it grows with the distance
        const float gauss = is_static ? __fsub_rn(d2, d2min) : __fmul_rn(a, __fsub_rn(d2, d2min));
        if (__fadd_rn(gauss, half) < best) return;              // score + noise <= gauss + half
        const float d = __fsqrt_rn(d2);
        const float vx = __fdiv_rn(dx, d), vy = __fdiv_rn(dy, d), vz = __fdiv_rn(dz, d);
        const float cs = __fadd_rn(__fadd_rn(__fmul_rn(vx, f1x), __fmul_rn(vy, f1y)), __fmul_rn(vz, f1z));
        if (!(fabsf(cs) <= kCosMax)) return;
        const float one_m = __fsub_rn(1.0f, fabsf(cs));
        const float clipped = one_m > kTiny ? one_m : 1e-5f;
        const float score = __fadd_rn(gauss, logf(clipped));
        const int t = ((n1 + R1) * L2 + (n2 + R2)) * L3 + (n3 + R3);
        const float noisy = amp == 0.0f ? score : __fadd_rn(score, noise_term(amp, seed, tid, (uint32_t)t));
        if (noisy > best || (noisy == best && t < c.img)) {
            best = noisy;
            c.ux = vx; c.uy = vy; c.uz = vz;
            c.value = __fadd_rn(score, is_static ? d2min : __fmul_rn(a, d2min));
            c.img = t;
        }
    };
    bool sweep = list == nullptr;
    if (list != nullptr && is_static) {
        // The static score grows with the distance: candidates farthest-first from the end of the pair's sorted list
        // (only offered where the list holds the task's whole box); the search ends at the first entry whose distance
        // part -- the other part is never positive -- cannot reach the running maximum.
        const int nT = (2 * list_range + 1) * (2 * list_range + 1) * (2 * list_range + 1);
        for (int s = nT - 1; s >= 0; s--) {
            const float d2l = __ldg(list + s);
            const float g_est = d2l - d2min;
            const float slack = d2l * 4e-6f + fabsf(g_est) * 2e-6f + 1e-12f;
            if (g_est + slack + half < best) break;
            const int code = __float_as_int(__ldg(list + 4 * kListLen + s));
            score_candidate((code & 255) - list_range, ((code >> 8) & 255) - list_range, ((code >> 16) & 255) - list_range);
        }
    } else if (list != nullptr) {
        // Candidates nearest-first from the pair's sorted list.  The Gaussian part of the score only falls
        // along the list and the other part is never positive, so the search ends at the first entry whose
        // Gaussian part -- with a margin for the few ulp between the list's fused arithmetic and the
        // arithmetic above -- cannot reach the running maximum: nothing behind it can win or tie.
        // The list holds the translations of the box (list_range)^3.  Where the task's box is larger, every
        // translation outside the listed box is at least sqrt(reach2) away (see box_reach2): the list serves as long
        // as the search ends before that distance, else the whole box is swept.
        // (entries are requested two ahead of their use: the search is a chain of dependent loads otherwise)
        const bool complete = R1 == list_range && R2 == list_range && R3 == list_range;
        float d2_a = __ldg(list), d2_b = __ldg(list + 1);
        int code_a = __float_as_int(__ldg(list + 4 * kListLen)), code_b = __float_as_int(__ldg(list + 4 * kListLen + 1));
        for (int s = 0; s < kListLen; s++) {
            const float d2l = d2_a;
            const int code = code_a;
            d2_a = d2_b; code_a = code_b;
            if (s + 2 < kListLen) { d2_b = __ldg(list + s + 2); code_b = __float_as_int(__ldg(list + 4 * kListLen + s + 2)); }
            if (!(d2l < 1e29f)) { sweep = !complete; break; }           // end of the real entries
            if (!complete && !(d2l < reach2)) { sweep = true; break; }
            const float g_est = a * (d2l - d2min);
            const float slack = fabsf(a) * d2l * 4e-6f + fabsf(g_est) * 2e-6f + 1e-12f;
            if (g_est + slack + half < best) break;
            score_candidate((code & 255) - list_range, ((code >> 8) & 255) - list_range, ((code >> 16) & 255) - list_range);
            if (s == kListLen - 1) sweep = !complete;
        }
    }
    if (sweep) {
        for (int k1 = 0; k1 <= 2 * R1; k1++)
            for (int k2 = 0; k2 <= 2 * R2; k2++)
                for (int k3 = 0; k3 <= 2 * R3; k3++) score_candidate(centre_out(k1), centre_out(k2), centre_out(k3));
    }
    return c;
}

// Squared distance below which every translation of the pair lies inside the box (C)^3: a translation with |n_d| > C on
// axis d is at least (C + 1 - |f_d|) plane spacings of that axis away, f the pair's separation in fractional
// coordinates.  Shrunk by 1e-3 against rounding; 0 if the separation is not within C cells.
__device__ __forceinline__ float box_reach2(const Cell& c, const int C)
{
    const float ax = c.t2y * c.t3z - c.t2z * c.t3y, ay = c.t2z * c.t3x - c.t2x * c.t3z, az = c.t2x * c.t3y - c.t2y * c.t3x;
    const float bx = c.t3y * c.t1z - c.t3z * c.t1y, by = c.t3z * c.t1x - c.t3x * c.t1z, bz = c.t3x * c.t1y - c.t3y * c.t1x;
    const float gx = c.t1y * c.t2z - c.t1z * c.t2y, gy = c.t1z * c.t2x - c.t1x * c.t2z, gz = c.t1x * c.t2y - c.t1y * c.t2x;
    const float vol = c.t1x * ax + c.t1y * ay + c.t1z * az;
    if (!(fabsf(vol) > 1e-12f)) return 0.f;
    const float la = sqrtf(ax * ax + ay * ay + az * az), lb = sqrtf(bx * bx + by * by + bz * bz), lg = sqrtf(gx * gx + gy * gy + gz * gz);
    // (C + 1 - |f_d|) spacing_d = ((C + 1) |vol| - |r . normal_d|) / |normal_d|
    const float r1 = ((float)(C + 1) * fabsf(vol) - fabsf(c.rx * ax + c.ry * ay + c.rz * az)) / la;
    const float r2 = ((float)(C + 1) * fabsf(vol) - fabsf(c.rx * bx + c.ry * by + c.rz * bz)) / lb;
    const float r3 = ((float)(C + 1) * fabsf(vol) - fabsf(c.rx * gx + c.ry * gy + c.rz * gz)) / lg;
    const float r = fminf(r1, fminf(r2, r3));
    return r > 0.f ? r * r * 0.999f : 0.f;
}

// (score, pair) -> 64-bit key whose unsigned order is (score ascending, pair index descending)
__device__ __forceinline__ unsigned long long make_key(float score, unsigned local_pair)
{
    unsigned u = __float_as_uint(score);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - local_pair);
}

// first index i in [0, n] with v[i] >= x (v non-decreasing, v[n] is the total)
__device__ __forceinline__ int64_t lower_bound_i64(const int64_t* v, int64_t n, int64_t x)
{
    int64_t lo = 0, hi = n;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (v[mid] < x) lo = mid + 1; else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(kFrThreads, CFB_FR_BLOCKS) max_frame_kernel(const FrArgs A, const Params P)
{
    __shared__ unsigned long long best[kFrMaxRows];
    __shared__ long long row_start[kFrMaxRows + 1];
    __shared__ float row_a[kFrMaxRows];
    __shared__ int row_R[kFrMaxRows];                 // three ranges, one byte each
    __shared__ float row_f1[kFrMaxRows][3];
    __shared__ float row_dir[kFrMaxRows][3];
    __shared__ int row_img[kFrMaxRows];
    __shared__ long long row_range[2];

    const int H = P.H, h = blockIdx.y, tid = threadIdx.x;
    // The block owns the query atoms whose first pair lies in [kFrPairs*b, kFrPairs*(b+1)) and
    // processes all of their pairs: about kFrPairs pairs per block whatever the crystal sizes.
    if (tid < 2) {
        const int64_t x = ((int64_t)blockIdx.x + tid) * kFrPairs;
        row_range[tid] = x >= A.E ? A.N : lower_bound_i64(A.e_start, A.N, x);
    }
    __syncthreads();
    const int64_t i0 = row_range[0];
    const int rows = (int)(row_range[1] - i0);
    if (rows <= 0) return;
    if (tid <= rows) row_start[tid] = A.e_start[i0 + tid];
    if (tid < rows) {
        const int64_t i = i0 + tid;
        const float a = __ldg(A.a_ik + i * H + h);
        row_a[tid] = a;
        const int64_t c = A.batch[i];
        int pack = 0;
        for (int d = 0; d < 3; d++)
            pack |= lattice_range_1d(P, a, P.cutoff_radius != 0.0f ? __ldg(A.rvlen + 3 * c + d) : 0.0f) << (8 * d);
        row_R[tid] = pack;
        if (A.mode == 2) {
            const float* f = A.frame1_in + (i * H + h) * 3;
            row_f1[tid][0] = __ldg(f); row_f1[tid][1] = __ldg(f + 1); row_f1[tid][2] = __ldg(f + 2);
        }
    }
    __syncthreads();
    const int64_t eb = row_start[0], ee = row_start[rows];
    const unsigned long long none = make_key(-1e10f, 0u);      // a score must exceed -1e10 to be selected
    // a thread meets the same pair in the same round on both axes, so the nearest non-zero distance
    // found on the first axis is kept for the second (for up to three rounds)
    const bool keep_d2 = ee - eb <= 3 * kFrThreads;
    float d2raw0 = -1.f, d2raw1 = -1.f, d2raw2 = -1.f;
    float dot0 = 0.f, dot1 = 0.f, dot2 = 0.f;           // and so is the pair's q.k

    for (int axis = (A.mode == 2 ? 2 : 1); axis <= (A.mode == 1 ? 1 : 2); axis++) {
        if (tid < rows) {
            best[tid] = none;
            row_dir[tid][0] = row_dir[tid][1] = row_dir[tid][2] = 0.f;
            row_img[tid] = -1;
        }
        __syncthreads();
        // ---- every pair of these atoms: candidate image, score, arg-max per query atom ----
        int round = 0;
        for (int64_t base = eb; base < ee; base += kFrThreads, round++) {
            const int64_t e = base + tid;
            int r = 0;
            unsigned long long key = 0ull;
            Cand cd; cd.ux = cd.uy = cd.uz = 0.f; cd.img = -1; cd.value = 0.f;
            if (e < ee) {
#pragma unroll
                for (int s = kFrMaxRows / 2; s > 0; s >>= 1)
                    if (r + s < rows && row_start[r + s] <= e) r += s;
                const int64_t i = i0 + r;
                const int64_t j = A.edges[A.E + e];
                const int64_t c = A.batch[i];
                Cell cell;
                const float* Tc = A.tvecs + 9 * c;
                cell.t1x = __ldg(Tc); cell.t1y = __ldg(Tc + 1); cell.t1z = __ldg(Tc + 2);
                cell.t2x = __ldg(Tc + 3); cell.t2y = __ldg(Tc + 4); cell.t2z = __ldg(Tc + 5);
                cell.t3x = __ldg(Tc + 6); cell.t3y = __ldg(Tc + 7); cell.t3z = __ldg(Tc + 8);
                cell.rx = __ldg(A.pos_ij + 3 * e); cell.ry = __ldg(A.pos_ij + 3 * e + 1); cell.rz = __ldg(A.pos_ij + 3 * e + 2);
                float dot = 0.f;
                const float4* q4 = reinterpret_cast<const float4*>(A.q + (i * H + h) * kFrHd);
                const float4* k4 = reinterpret_cast<const float4*>(A.k + (j * H + h) * kFrHd);
                const bool dot_known = keep_d2 && axis == 2 && A.mode == 3;
                if (dot_known) {
                    dot = round == 0 ? dot0 : (round == 1 ? dot1 : dot2);
                } else if (!A.is_static) {
#pragma unroll
                    for (int d4 = 0; d4 < kFrHd / 4; d4++) {
                        const float4 u = __ldg(q4 + d4), v = __ldg(k4 + d4);
                        dot = __fmaf_rn(u.x, v.x, dot); dot = __fmaf_rn(u.y, v.y, dot);
                        dot = __fmaf_rn(u.z, v.z, dot); dot = __fmaf_rn(u.w, v.w, dot);
                    }
                    if (keep_d2) {
                        if (round == 0) dot0 = dot; else if (round == 1) dot1 = dot; else dot2 = dot;
                    }
                }
                const uint64_t noise_id = (uint64_t)(e * H + h);
                const int pack = row_R[r];
                const int R1 = pack & 255, R2 = (pack >> 8) & 255, R3 = (pack >> 16) & 255;
                // the per-pair cache and list cover the box (cache_range)^3; a task with a larger box can use them where
                // everything outside the cached box is provably farther than what decides the search
                const int C = A.cache_range;
                const bool same_box = R1 == C && R2 == C && R3 == C;
                const bool wider = !same_box && R1 >= C && R2 >= C && R3 >= C && (A.cache != nullptr || A.list != nullptr);
                const float reach2 = wider ? box_reach2(cell, C) : 1e38f;
                if (axis == 1) {
                    // the two nearest images inside the cached box are the two nearest of the larger box
                    const bool hit = A.cache != nullptr && (same_box || (wider && __ldg(&A.cache[e].y) < reach2));
                    cd = first_axis_candidate(cell, row_a[r], R1, R2, R3, P.noise, A.seed1, noise_id,
                                              hit ? A.cache + e : nullptr, C,
                                              hit && A.list != nullptr ? A.list + (size_t)e * kListStride : nullptr, reach2);
                    if (keep_d2) {
                        if (round == 0) d2raw0 = cd.d2raw; else if (round == 1) d2raw1 = cd.d2raw; else d2raw2 = cd.d2raw;
                    }
                } else {
                    float known = round == 0 ? d2raw0 : (round == 1 ? d2raw1 : (round == 2 ? d2raw2 : -1.f));
                    // the smallest non-zero squared distance is cached pair geometry (second axis on its own)
                    if (known < 0.f && A.cache != nullptr && (same_box || (wider && __ldg(&A.cache[e].y) < reach2)))
                        known = __ldg(&A.cache[e].x);
                    // the sorted list serves the search only where the score falls with the distance
                    // (the static search runs farthest-first, so it needs the list of the task's whole box)
                    const bool hit = A.list != nullptr && (same_box || (!A.is_static && wider && reach2 > 0.f));
                    cd = second_axis_candidate(cell, row_a[r], R1, R2, R3, P.noise, A.seed2, noise_id,
                                               row_f1[r][0], row_f1[r][1], row_f1[r][2], known,
                                               hit ? A.list + (size_t)e * kListStride : nullptr, A.is_static != 0, C, reach2);
                }
                const float s = __fadd_rn(dot, cd.value);
                if (s > -1e10f) {
                    key = make_key(s, (unsigned)(e - row_start[r]));
                    atomicMax(&best[r], key);
                }
            }
            __syncthreads();
            // the pair that holds the atom's maximum so far leaves its direction; a better pair
            // of a later round overwrites it after that round's barrier
            if (key != 0ull && best[r] == key) {
                row_dir[r][0] = cd.ux; row_dir[r][1] = cd.uy; row_dir[r][2] = cd.uz;
                row_img[r] = cd.img;
            }
        }
        __syncthreads();
        // ---- one thread per query atom: outputs ----
        if (tid < rows) {
            const int64_t i = i0 + tid;
            const unsigned long long key = best[tid];
            const int64_t e_win = key == none ? -1 : row_start[tid] + (int64_t)(0xFFFFFFFFu - (unsigned)(key & 0xFFFFFFFFull));
            const float ux = row_dir[tid][0], uy = row_dir[tid][1], uz = row_dir[tid][2];
            if (axis == 1) {
                row_f1[tid][0] = ux; row_f1[tid][1] = uy; row_f1[tid][2] = uz;
                if (A.mode != 2) {
                    float* o = A.frame1 + (i * H + h) * 3;
                    o[0] = ux; o[1] = uy; o[2] = uz;
                }
                if (A.mode == 1 && A.sel_edge) A.sel_edge[i * H + h] = e_win;
                if (A.mode == 1 && A.sel_image) A.sel_image[i * H + h] = row_img[tid];
            } else {
                float* o2 = A.frame2 + (i * H + h) * 3;
                if (A.mode == 2) {
                    o2[0] = ux; o2[1] = uy; o2[2] = uz;
                    if (A.sel_edge) A.sel_edge[i * H + h] = e_win;
                    if (A.sel_image) A.sel_image[i * H + h] = row_img[tid];
                } else {
                    // Gram-Schmidt, normalisation with max(norm, 1e-12), cross product
                    const float f1x = row_f1[tid][0], f1y = row_f1[tid][1], f1z = row_f1[tid][2];
                    const float dot = __fadd_rn(__fadd_rn(__fmul_rn(f1x, ux), __fmul_rn(f1y, uy)), __fmul_rn(f1z, uz));
                    const float wx = __fsub_rn(ux, __fmul_rn(dot, f1x)), wy = __fsub_rn(uy, __fmul_rn(dot, f1y)),
                                wz = __fsub_rn(uz, __fmul_rn(dot, f1z));
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
        __syncthreads();
    }
}

// "lattice" frames: thread = (atom, head); the directions of the three shortest lattice vectors of the atom's cell
// within its lattice ranges (replaces compute_lattice_first_frame.cu, compute_lattice_second_frame.cu,
// compute_lattice_third_frame.cu and the host glue of models/cuda_funcs/calc_lattice_frame.py:22-150).  Only an atom's
// self pair takes part in the reference (separation zero), so no pair data is read.  Three greedy searches with a
// running minimum (strict comparison: the first translation in the reference's loop order wins on equal lengths):
// axis 1 the shortest translation; axis 2 the shortest one not collinear with it, on its side; axis 3 the shortest
// one out of their plane, on the side of axis 1; all three negated when axis 3 points against axis 1 x axis 2.
// Outputs are zero where nothing qualifies (the reference leaves them uninitialised).  Unfused IEEE operations in the
// reference's order, so a CPU reproduces the frames bit for bit.  self_pair (N): pair index of (i, i), which names
// the noise stream.
__global__ void __launch_bounds__(128) lattice_frame_kernel(const float* __restrict__ a_ik, const float* __restrict__ tvecs,
                                                            const float* __restrict__ rvlen, const int64_t* __restrict__ batch,
                                                            const int64_t* __restrict__ e_start, const int64_t* __restrict__ edges,
                                                            int64_t N, int64_t E, uint64_t seed1, uint64_t seed2, uint64_t seed3,
                                                            float* __restrict__ f1, float* __restrict__ f2, float* __restrict__ f3,
                                                            const Params P)
{
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int H = P.H;
    if (tid >= N * H) return;
    const int64_t i = tid / H;
    const int h = (int)(tid - i * H);
    const int64_t c = batch[i];
    Cell cell;
    const float* Tc = tvecs + 9 * c;
    cell.t1x = __ldg(Tc); cell.t1y = __ldg(Tc + 1); cell.t1z = __ldg(Tc + 2);
    cell.t2x = __ldg(Tc + 3); cell.t2y = __ldg(Tc + 4); cell.t2z = __ldg(Tc + 5);
    cell.t3x = __ldg(Tc + 6); cell.t3y = __ldg(Tc + 7); cell.t3z = __ldg(Tc + 8);
    cell.rx = cell.ry = cell.rz = 0.f;
    const float a = __ldg(a_ik + i * H + h);
    int R[3];
    for (int d = 0; d < 3; d++) R[d] = lattice_range_1d(P, a, P.cutoff_radius != 0.0f ? __ldg(rvlen + 3 * c + d) : 0.0f);
    uint64_t noise_id = 0;
    if (P.noise != 0.0f) {
        // the atom's pairs run over its crystal's atoms in order: the self pair is at offset (i - first key atom)
        const int64_t e0 = e_start[i];
        noise_id = (uint64_t)((e0 + (i - edges[E + e0])) * H + h);
    }
    float o1[3] = {0.f, 0.f, 0.f}, o2[3] = {0.f, 0.f, 0.f}, o3[3] = {0.f, 0.f, 0.f};
    float cx = 0.f, cy = 0.f, cz = 0.f;
    for (int axis = 0; axis < 3; axis++) {
        if (axis == 2) {
            cx = __fsub_rn(__fmul_rn(o1[1], o2[2]), __fmul_rn(o1[2], o2[1]));
            cy = __fsub_rn(__fmul_rn(o1[2], o2[0]), __fmul_rn(o1[0], o2[2]));
            cz = __fsub_rn(__fmul_rn(o1[0], o2[1]), __fmul_rn(o1[1], o2[0]));
            const float cn = __fsqrt_rn(__fadd_rn(__fadd_rn(__fmul_rn(cx, cx), __fmul_rn(cy, cy)), __fmul_rn(cz, cz)));
            cx = __fdiv_rn(cx, cn); cy = __fdiv_rn(cy, cn); cz = __fdiv_rn(cz, cn);
        }
        const uint64_t seed = axis == 0 ? seed1 : (axis == 1 ? seed2 : seed3);
        float d2_min = 1e10f;
        int t = 0;
        for (int n1 = -R[0]; n1 <= R[0]; n1++)
            for (int n2 = -R[1]; n2 <= R[1]; n2++)
                for (int n3 = -R[2]; n3 <= R[2]; n3++, t++) {
                    float dx, dy, dz, d2;
                    separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                    const float cand = P.noise != 0.0f ? __fadd_rn(d2, noise_term(P.noise, seed, noise_id, (uint32_t)t)) : d2;
                    if (!(d2_min > cand && d2 > kTiny)) continue;
                    const float d = __fsqrt_rn(d2);
                    const float ux = __fdiv_rn(dx, d), uy = __fdiv_rn(dy, d), uz = __fdiv_rn(dz, d);
                    if (axis == 0) {
                        d2_min = cand;
                        o1[0] = ux; o1[1] = uy; o1[2] = uz;
                    } else if (axis == 1) {
                        const float cs = __fadd_rn(__fadd_rn(__fmul_rn(ux, o1[0]), __fmul_rn(uy, o1[1])), __fmul_rn(uz, o1[2]));
                        if (__fsub_rn(1.0f, fabsf(cs)) > kTiny) {
                            const float sg = cs < 0.f ? -1.0f : 1.0f;
                            o2[0] = sg * ux; o2[1] = sg * uy; o2[2] = sg * uz;
                            d2_min = cand;
                        }
                    } else {
                        const float cc = __fadd_rn(__fadd_rn(__fmul_rn(ux, cx), __fmul_rn(uy, cy)), __fmul_rn(uz, cz));
                        const float c1 = __fadd_rn(__fadd_rn(__fmul_rn(ux, o1[0]), __fmul_rn(uy, o1[1])), __fmul_rn(uz, o1[2]));
                        if (fabsf(cc) > kTiny) {
                            const float sg = c1 < 0.f ? -1.0f : 1.0f;
                            o3[0] = sg * ux; o3[1] = sg * uy; o3[2] = sg * uz;
                            d2_min = cand;
                        }
                    }
                }
    }
    const float cc = __fadd_rn(__fadd_rn(__fmul_rn(o3[0], cx), __fmul_rn(o3[1], cy)), __fmul_rn(o3[2], cz));
    const float flip = cc < 0.f ? -1.0f : 1.0f;
    for (int d = 0; d < 3; d++) {
        f1[(i * H + h) * 3 + d] = flip * o1[d];
        f2[(i * H + h) * 3 + d] = flip * o2[d];
        f3[(i * H + h) * 3 + d] = flip * o3[d];
    }
}

// Per-pair geometry that does not depend on the head or the layer, for lattice ranges (R, R, R):
//   x, y: smallest and second smallest d^2 > 1e-5 over the translations (equal values count twice), with
//         the arithmetic of separation() -- what pass 1 of first_axis_candidate() finds;
//   z:    the linear index of the first translation that attains x (-1 if none), as int bits;
//   w:    the smallest d^2 over all translations, with the fused arithmetic of the lattice-sum kernel.
__global__ void __launch_bounds__(256) pair_cache_kernel(const float* __restrict__ pos_ij, const float* __restrict__ tvecs,
                                                         const int64_t* __restrict__ batch, const int64_t* __restrict__ edges,
                                                         int64_t E, int R, float4* __restrict__ out)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const int64_t c = batch[edges[e]];
    Cell cell;
    const float* Tc = tvecs + 9 * c;
    cell.t1x = __ldg(Tc); cell.t1y = __ldg(Tc + 1); cell.t1z = __ldg(Tc + 2);
    cell.t2x = __ldg(Tc + 3); cell.t2y = __ldg(Tc + 4); cell.t2z = __ldg(Tc + 5);
    cell.t3x = __ldg(Tc + 6); cell.t3y = __ldg(Tc + 7); cell.t3z = __ldg(Tc + 8);
    cell.rx = __ldg(pos_ij + 3 * e); cell.ry = __ldg(pos_ij + 3 * e + 1); cell.rz = __ldg(pos_ij + 3 * e + 2);
    float d2raw = 1e10f, d2next = 1e10f, d2all = 1e10f;
    int t = 0, best_t = -1;
    for (int n1 = -R; n1 <= R; n1++)
        for (int n2 = -R; n2 <= R; n2++)
            for (int n3 = -R; n3 <= R; n3++, t++) {
                float dx, dy, dz, d2;
                separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                if (d2 > kTiny) {
                    if (d2 < d2raw) { d2next = d2raw; d2raw = d2; best_t = t; }
                    else if (d2 < d2next) d2next = d2;
                }
                const float f1 = (float)n1, f2 = (float)n2, f3 = (float)n3;
                const float ox = fmaf(cell.t3x, f3, fmaf(cell.t2x, f2, cell.rx)), oy = fmaf(cell.t3y, f3, fmaf(cell.t2y, f2, cell.ry)),
                            oz = fmaf(cell.t3z, f3, fmaf(cell.t2z, f2, cell.rz));
                const float fx = fmaf(cell.t1x, f1, ox), fy = fmaf(cell.t1y, f1, oy), fz = fmaf(cell.t1z, f1, oz);
                d2all = fminf(d2all, fmaf(fz, fz, fmaf(fy, fy, fx * fx)));
            }
    out[e] = make_float4(d2raw, d2next, __int_as_float(best_t), d2all);
}

// Per-pair translation list for lattice ranges (R, R, R) with (2R+1)^3 <= kListLen: all translations of a
// pair sorted by squared distance (equal distances in index order).  Because the weight
// exp(a (d^2 - d^2_min)) falls with the distance, the translations a lattice-sum task has to expand, and the
// candidates a second-axis search has to score, are a prefix of this list, whatever the head or the layer.

// warp = one pair; lane l holds list positions l, l+32, l+64, l+96.  Keys are (bits of d^2) << 32 | index:
// d^2 >= 0, so the unsigned order of the bits is the order of the values, and equal distances fall in
// index order.  A bitonic network sorts the 128 keys: strides below 32 exchange between lanes, strides 32
// and 64 between a lane's own registers.
__global__ void __launch_bounds__(128) pair_list_kernel(const float* __restrict__ pos_ij, const float* __restrict__ tvecs,
                                                        const int64_t* __restrict__ batch, const int64_t* __restrict__ edges,
                                                        int64_t E, int R, float* __restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t e = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (e >= E) return;
    const int L = 2 * R + 1, nT = L * L * L;
    const int64_t c = batch[edges[e]];
    const float* Tc = tvecs + 9 * c;
    const float t1x = __ldg(Tc), t1y = __ldg(Tc + 1), t1z = __ldg(Tc + 2);
    const float t2x = __ldg(Tc + 3), t2y = __ldg(Tc + 4), t2z = __ldg(Tc + 5);
    const float t3x = __ldg(Tc + 6), t3y = __ldg(Tc + 7), t3z = __ldg(Tc + 8);
    const float rx = __ldg(pos_ij + 3 * e), ry = __ldg(pos_ij + 3 * e + 1), rz = __ldg(pos_ij + 3 * e + 2);
    auto separation_fused = [&](const int t, float& dx, float& dy, float& dz, float& d2, int& code) {
        const int q = t / L, k1 = q / L, k2 = q - k1 * L, k3 = t - q * L;
        const float n1 = (float)(k1 - R), n2 = (float)(k2 - R), n3 = (float)(k3 - R);
        const float ox = fmaf(t3x, n3, fmaf(t2x, n2, rx)), oy = fmaf(t3y, n3, fmaf(t2y, n2, ry)), oz = fmaf(t3z, n3, fmaf(t2z, n2, rz));
        dx = fmaf(t1x, n1, ox); dy = fmaf(t1y, n1, oy); dz = fmaf(t1z, n1, oz);
        d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
        code = k1 | (k2 << 8) | (k3 << 16) | (t << 24);
    };
    unsigned long long key[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int t = r * 32 + lane;
        float dx, dy, dz, d2 = 1e30f;
        int code;
        if (t < nT) separation_fused(t, dx, dy, dz, d2, code);
        key[r] = ((unsigned long long)__float_as_uint(d2) << 32) | (unsigned)t;
    }
#pragma unroll
    for (int k = 2; k <= kListLen; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j >= 32) {
                const int dr = j >> 5;
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    if ((r & dr) == 0) {
                        const bool up = (((r * 32 + lane) & k) == 0);
                        const unsigned long long lo = key[r] < key[r | dr] ? key[r] : key[r | dr];
                        const unsigned long long hi = key[r] < key[r | dr] ? key[r | dr] : key[r];
                        key[r] = up ? lo : hi;
                        key[r | dr] = up ? hi : lo;
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key[r], j);
                    const bool up = (((r * 32 + lane) & k) == 0);
                    const bool take_min = ((lane & j) == 0) == up;
                    const bool less = key[r] < other;
                    key[r] = (less == take_min) ? key[r] : other;
                }
            }
        }
    }
    float* o = out + (size_t)e * kListStride + lane;
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int t = (int)(unsigned)(key[r] & 0xffffffffull);
        float dx = 0.f, dy = 0.f, dz = 0.f, d2 = 1e30f;
        int code = -1;
        if (t < nT) separation_fused(t, dx, dy, dz, d2, code);
        o[r * 32] = d2; o[kListLen + r * 32] = dx; o[2 * kListLen + r * 32] = dy; o[3 * kListLen + r * 32] = dz;
        o[4 * kListLen + r * 32] = __int_as_float(code);
    }
}

int pair_cache(const float* pos_ij, const float* tvecs, const int64_t* batch, const int64_t* edges, int64_t E, int R,
               float* out, float* list, cudaStream_t st)
{
    if (E == 0) return CFB200_OK;
    if (out != nullptr)
        pair_cache_kernel<<<(unsigned)((E + 255) / 256), 256, 0, st>>>(pos_ij, tvecs, batch, edges, E, R,
                                                                      reinterpret_cast<float4*>(out));
    if (list != nullptr) {
        if ((2 * R + 1) * (2 * R + 1) * (2 * R + 1) > kListLen) return CFB200_E_UNSUPPORTED;
        pair_list_kernel<<<(unsigned)((E + 3) / 4), 128, 0, st>>>(pos_ij, tvecs, batch, edges, E, R, list);
    }
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int lattice_frames(const float* a_ik, const float* tvecs, const float* rvlen, const int64_t* batch, const int64_t* e_start,
                   const int64_t* edges, int64_t N, int64_t E, uint64_t seed1, uint64_t seed2, uint64_t seed3, float* f1, float* f2,
                   float* f3, const Params& P, cudaStream_t st)
{
    if (N == 0) return CFB200_OK;
    const int64_t n = N * P.H;
    lattice_frame_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(a_ik, tvecs, rvlen, batch, e_start, edges, N, E, seed1, seed2,
                                                                    seed3, f1, f2, f3, P);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int max_frame(const FrArgs& A, const Params& P, cudaStream_t st)
{
    if (A.N == 0 || A.E == 0) return CFB200_OK;
    const unsigned gx = (unsigned)((A.E + kFrPairs - 1) / kFrPairs);
    max_frame_kernel<<<dim3(gx, P.H), kFrThreads, 0, st>>>(A, P);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

// ---- third axis of the frame method "max_wo_orthogonal" (compute_third_frame_each_edge.cu:93-150,
// models/cuda_funcs/calc_maximum_frame.py:173-245): an ablation of the reference that keeps the second axis
// un-orthogonalised and selects a third one like the first two, with log(max(|det(f1, f2, u)|, 1e-5)) in place of the
// collinearity term and |det| > 1e-5 as the condition.  Not on the hot path: thread = (pair, head) sweeps the box with
// the reference's arithmetic (non-fused operations, so a CPU reproduces the selection), warp = (atom, head) takes the
// arg-max of q.k + value over the atom's pairs, lowest pair on equal scores.
struct Fr3Args {
    const float* q; const float* k; const float* a_ik; const float* pos_ij; const float* tvecs; const float* rvlen;
    const int64_t* batch; const int64_t* edges; const int64_t* e_start;
    const float* frame1; const float* frame2;
    int64_t N, E;
    uint64_t seed;
    float* cand;            // scratch (E,H,4): direction, value
    float* frame3; int64_t* sel_edge;
};

__global__ void __launch_bounds__(256) third_axis_edges_kernel(const Fr3Args A, const Params P)
{
    const int H = P.H;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= A.E * H) return;
    const int64_t e = tid / H;
    const int h = (int)(tid - e * H);
    const int64_t i = A.edges[e], c = A.batch[i];
    Cell cell;
    const float* Tc = A.tvecs + 9 * c;
    cell.t1x = __ldg(Tc); cell.t1y = __ldg(Tc + 1); cell.t1z = __ldg(Tc + 2);
    cell.t2x = __ldg(Tc + 3); cell.t2y = __ldg(Tc + 4); cell.t2z = __ldg(Tc + 5);
    cell.t3x = __ldg(Tc + 6); cell.t3y = __ldg(Tc + 7); cell.t3z = __ldg(Tc + 8);
    cell.rx = __ldg(A.pos_ij + 3 * e); cell.ry = __ldg(A.pos_ij + 3 * e + 1); cell.rz = __ldg(A.pos_ij + 3 * e + 2);
    const float a = __ldg(A.a_ik + i * H + h);
    const bool cut = P.cutoff_radius != 0.0f;
    const int R1 = lattice_range_1d(P, a, cut ? __ldg(A.rvlen + 3 * c) : 0.0f);
    const int R2 = lattice_range_1d(P, a, cut ? __ldg(A.rvlen + 3 * c + 1) : 0.0f);
    const int R3 = lattice_range_1d(P, a, cut ? __ldg(A.rvlen + 3 * c + 2) : 0.0f);
    const float* f1 = A.frame1 + (i * H + h) * 3;
    const float* f2 = A.frame2 + (i * H + h) * 3;
    const float f1x = __ldg(f1), f1y = __ldg(f1 + 1), f1z = __ldg(f1 + 2);
    const float f2x = __ldg(f2), f2y = __ldg(f2 + 1), f2z = __ldg(f2 + 2);
    float d2min = 1e10f;
    for (int n1 = -R1; n1 <= R1; n1++)
        for (int n2 = -R2; n2 <= R2; n2++)
            for (int n3 = -R3; n3 <= R3; n3++) {
                float dx, dy, dz, d2;
                separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                if (d2 > kTiny) d2min = fminf(d2min, d2);
            }
    float best = -1e15f, ux = 0.f, uy = 0.f, uz = 0.f, value = -1e15f;
    const float half = 0.5f * P.noise;
    int t = 0;
    for (int n1 = -R1; n1 <= R1; n1++)
        for (int n2 = -R2; n2 <= R2; n2++)
            for (int n3 = -R3; n3 <= R3; n3++, t++) {
                float dx, dy, dz, d2;
                separation(cell, (float)n1, (float)n2, (float)n3, dx, dy, dz, d2);
                if (!(d2 > kTiny)) continue;
                const float gauss = __fmul_rn(a, __fsub_rn(d2, d2min));
                if (gauss + half + 1e-6f < best) continue;              // the logarithm is not positive (|det| <= 1 up to rounding)
                const float d = __fsqrt_rn(d2);
                const float vx = __fdiv_rn(dx, d), vy = __fdiv_rn(dy, d), vz = __fdiv_rn(dz, d);
                float det = __fmul_rn(__fmul_rn(f1x, f2y), vz);
                det = __fadd_rn(det, __fmul_rn(__fmul_rn(f1y, f2z), vx));
                det = __fadd_rn(det, __fmul_rn(__fmul_rn(f1z, f2x), vy));
                det = __fsub_rn(det, __fmul_rn(__fmul_rn(f1z, f2y), vx));
                det = __fsub_rn(det, __fmul_rn(__fmul_rn(f1y, f2x), vz));
                det = __fsub_rn(det, __fmul_rn(__fmul_rn(f1x, f2z), vy));
                const float mag = fabsf(det);
                if (!(mag > kTiny)) continue;
                const float score = __fadd_rn(gauss, logf(mag));
                const float noisy = P.noise == 0.0f ? score : __fadd_rn(score, noise_term(P.noise, A.seed, (uint64_t)tid, (uint32_t)t));
                if (noisy > best) {
                    best = noisy;
                    ux = vx; uy = vy; uz = vz;
                    value = __fadd_rn(score, __fmul_rn(a, d2min));
                }
            }
    reinterpret_cast<float4*>(A.cand)[tid] = make_float4(ux, uy, uz, value);
}

__global__ void __launch_bounds__(256) third_axis_select_kernel(const Fr3Args A, const Params P)
{
    const int H = P.H, lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= A.N * H) return;
    const int64_t i = w / H;
    const int h = (int)(w - i * H);
    const int64_t e0 = A.e_start[i], e1 = A.e_start[i + 1];
    const float4* q4 = reinterpret_cast<const float4*>(A.q + (i * H + h) * kFrHd);
    unsigned long long best = make_key(-1e10f, 0u);          // a score must exceed -1e10 to be selected
    for (int64_t e = e0 + lane; e < e1; e += 32) {
        const int64_t j = A.edges[A.E + e];
        const float4* k4 = reinterpret_cast<const float4*>(A.k + (j * H + h) * kFrHd);
        float dot = 0.f;
#pragma unroll
        for (int d4 = 0; d4 < kFrHd / 4; d4++) {
            const float4 u = __ldg(q4 + d4), v = __ldg(k4 + d4);
            dot = __fmaf_rn(u.x, v.x, dot); dot = __fmaf_rn(u.y, v.y, dot);
            dot = __fmaf_rn(u.z, v.z, dot); dot = __fmaf_rn(u.w, v.w, dot);
        }
        const float s = __fadd_rn(dot, reinterpret_cast<const float4*>(A.cand)[e * H + h].w);
        if (s > -1e10f) {
            const unsigned long long key = make_key(s, (unsigned)(e - e0));
            best = key > best ? key : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if (lane == 0) {
        float* out = A.frame3 + (i * H + h) * 3;
        if (best == make_key(-1e10f, 0u)) {
            out[0] = out[1] = out[2] = 0.f;
            if (A.sel_edge) A.sel_edge[i * H + h] = -1;
        } else {
            const int64_t e = e0 + (int64_t)(0xFFFFFFFFu - (unsigned)(best & 0xffffffffull));
            const float4 c = reinterpret_cast<const float4*>(A.cand)[e * H + h];
            out[0] = c.x; out[1] = c.y; out[2] = c.z;
            if (A.sel_edge) A.sel_edge[i * H + h] = e;
        }
    }
}

int third_axis(const Fr3Args& A, const Params& P, cudaStream_t st)
{
    if (A.N == 0 || A.E == 0) return CFB200_OK;
    const int64_t n1 = A.E * P.H, n2 = A.N * P.H;
    third_axis_edges_kernel<<<(unsigned)((n1 + 255) / 256), 256, 0, st>>>(A, P);
    third_axis_select_kernel<<<(unsigned)((n2 + 7) / 8), 256, 0, st>>>(A, P);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
