// Ragged softmax attention inside each crystal, with an additive logit bias z (E,H) and an
// additive value bias (E,H,16) per pair (replaces fused_dpa_fwd.cu, fused_dpa_bwd.cu,
// fused_dpa_bwd_q.cu and the four irregular_transpose launches of the reference).
//
// These kernels are bound by HBM traffic: every pair contributes 4 B of logit bias and 64 B of
// value bias per head and almost no arithmetic.  A warp owns one atom and Hs of its H heads (the
// heads are split over several warps so that more pairs are in flight per atom: with a handful of
// atoms per crystal the loops are short chains of dependent loads); lane = (jj, h) with
// h = lane % Hs the head within the warp's share and jj = lane / Hs a stride over the atom's pairs,
// so one warp iteration reads 32/Hs consecutive pairs x Hs heads.  The softmax is computed online (running max / sum); the
// log-sum-exp per (atom, head) is kept for the backward pass, which recomputes probabilities
// instead of transposing stored ones:
//   pass 1 (rows, warp = query atom): gz, gvalues, gq
//   pass 2 (columns, warp = key atom): gk, gv from q, lse, gz of the crystal's other atoms.
#include "common.cuh"

namespace cfb {

constexpr int kDpWarps = 4;
constexpr int kDpHd = 16;

struct DpArgs {
    const float* q; const float* k; const float* v; const float* z; const float* b;
    const int64_t* edges; const int64_t* e_start;
    int64_t N, E;
    float* out; float* lse; float* prob;
    const float* gout; float* gq; float* gk; float* gv; float* gz; float* gb;
};

__device__ __forceinline__ void load16(const float* p, float* r)
{
    const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int d4 = 0; d4 < 4; d4++) {
        const float4 t = __ldg(p4 + d4);
        r[4 * d4] = t.x; r[4 * d4 + 1] = t.y; r[4 * d4 + 2] = t.z; r[4 * d4 + 3] = t.w;
    }
}

__device__ __forceinline__ void store16(float* p, const float* r)
{
    float4* p4 = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int d4 = 0; d4 < 4; d4++) p4[d4] = make_float4(r[4 * d4], r[4 * d4 + 1], r[4 * d4 + 2], r[4 * d4 + 3]);
}

__device__ __forceinline__ float dot16(const float* a, const float* b)
{
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < kDpHd; d++) s = fmaf(a[d], b[d], s);
    return s;
}

__global__ void __launch_bounds__(kDpWarps * 32) dpa_fwd_kernel(const DpArgs A, int H, int Hs)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = H / Hs;                                   // warps per atom
    const int64_t gw = (int64_t)blockIdx.x * kDpWarps + warp;
    const int64_t i = gw / S;
    if (i >= A.N) return;
    const int h = (int)(gw - i * S) * Hs + lane % Hs, jj = lane / Hs, G = 32 / Hs;
    const int64_t e0 = A.e_start[i], e1 = A.e_start[i + 1];
    float qv[kDpHd], acc[kDpHd];
    load16(A.q + (i * H + h) * kDpHd, qv);
#pragma unroll
    for (int d = 0; d < kDpHd; d++) acc[d] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int64_t j_first = e1 > e0 ? A.edges[A.E + e0] : 0;
    for (int64_t e = e0 + jj; e < e1; e += G) {
        const int64_t j = A.edges[A.E + e];
        // the backward's column pass locates pairs by the dense layout: report a list that breaks it
        if (j != j_first + (e - e0)) atomicOr(&g_status, CFB200_ST_PAIR_LAYOUT);
        float kv[kDpHd];
        load16(A.k + (j * H + h) * kDpHd, kv);
        float s = dot16(qv, kv);
        if (A.z) s += __ldg(A.z + e * H + h);
        if (A.prob) A.prob[e * H + h] = s;               // raw logit, normalised below
        float vv[kDpHd];
        load16(A.v + (j * H + h) * kDpHd, vv);
        if (A.b) {
            float bb[kDpHd];
            load16(A.b + (e * H + h) * kDpHd, bb);
#pragma unroll
            for (int d = 0; d < kDpHd; d++) vv[d] += bb[d];
        }
        const float mn = fmaxf(m, s);
        const float sc = __expf(m - mn), p = __expf(s - mn);
        l = fmaf(l, sc, p);
#pragma unroll
        for (int d = 0; d < kDpHd; d++) acc[d] = fmaf(acc[d], sc, p * vv[d]);
        m = mn;
    }
    // merge the 32/H partial softmax states of each head
    for (int o = Hs; o < 32; o <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
        const float mn = fmaxf(m, m2);
        const float s1 = (m == -INFINITY) ? 0.f : __expf(m - mn), s2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
        l = l * s1 + l2 * s2;
#pragma unroll
        for (int d = 0; d < kDpHd; d++) acc[d] = acc[d] * s1 + __shfl_xor_sync(0xffffffffu, acc[d], o) * s2;
        m = mn;
    }
    const float lse = m + logf(l);
    if (jj == 0) {
        const float inv = 1.0f / l;
#pragma unroll
        for (int d = 0; d < kDpHd; d++) acc[d] *= inv;
        store16(A.out + (i * H + h) * kDpHd, acc);
        A.lse[i * H + h] = lse;
    }
    if (A.prob)
        for (int64_t e = e0 + jj; e < e1; e += G) A.prob[e * H + h] = __expf(A.prob[e * H + h] - lse);
}

// pass 1: rows.  gvalues_ij = p_ij * gout_i ; gz_ij = p_ij * (gout_i . (v_j + b_ij) - gout_i . out_i)
//         gq_i = sum_j gz_ij * k_j           (fused_dpa_bwd.cu:52-124, fused_dpa_bwd_q.cu:27-52)
__global__ void __launch_bounds__(kDpWarps * 32) dpa_bwd_rows_kernel(const DpArgs A, int H, int Hs)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = H / Hs;                                   // warps per atom
    const int64_t gw = (int64_t)blockIdx.x * kDpWarps + warp;
    const int64_t i = gw / S;
    if (i >= A.N) return;
    const int h = (int)(gw - i * S) * Hs + lane % Hs, jj = lane / Hs, G = 32 / Hs;
    const int64_t e0 = A.e_start[i], e1 = A.e_start[i + 1];
    float qv[kDpHd], go[kDpHd], gq[kDpHd];
    load16(A.q + (i * H + h) * kDpHd, qv);
    load16(A.gout + (i * H + h) * kDpHd, go);
    float D;
    {
        float ov[kDpHd];
        load16(A.out + (i * H + h) * kDpHd, ov);
        D = dot16(go, ov);
    }
    const float lse = __ldg(A.lse + i * H + h);
#pragma unroll
    for (int d = 0; d < kDpHd; d++) gq[d] = 0.f;
    for (int64_t e = e0 + jj; e < e1; e += G) {
        const int64_t j = A.edges[A.E + e];
        float kv[kDpHd], vv[kDpHd];
        load16(A.k + (j * H + h) * kDpHd, kv);
        float s = dot16(qv, kv);
        if (A.z) s += __ldg(A.z + e * H + h);
        const float p = __expf(s - lse);
        load16(A.v + (j * H + h) * kDpHd, vv);
        if (A.b) {
            float bb[kDpHd];
            load16(A.b + (e * H + h) * kDpHd, bb);
#pragma unroll
            for (int d = 0; d < kDpHd; d++) vv[d] += bb[d];
        }
        const float gs = p * (dot16(go, vv) - D);
        A.gz[e * H + h] = gs;
        if (A.gb) {
            float t[kDpHd];
#pragma unroll
            for (int d = 0; d < kDpHd; d++) t[d] = go[d] * p;
            store16(A.gb + (e * H + h) * kDpHd, t);
        }
#pragma unroll
        for (int d = 0; d < kDpHd; d++) gq[d] = fmaf(gs, kv[d], gq[d]);
    }
    for (int o = Hs; o < 32; o <<= 1)
#pragma unroll
        for (int d = 0; d < kDpHd; d++) gq[d] += __shfl_xor_sync(0xffffffffu, gq[d], o);
    if (jj == 0) store16(A.gq + (i * H + h) * kDpHd, gq);
}

// pass 2: columns.  For key atom j of a crystal whose first atom is a0 and size n, the pair
// (i, j) has index e_start[i] + (j - a0).  gk_j = sum_i gz_ij q_i ; gv_j = sum_i p_ij gout_i.
__global__ void __launch_bounds__(kDpWarps * 32) dpa_bwd_cols_kernel(const DpArgs A, int H, int Hs)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = H / Hs;
    const int64_t gw = (int64_t)blockIdx.x * kDpWarps + warp;
    const int64_t j = gw / S;
    if (j >= A.N) return;
    const int h = (int)(gw - j * S) * Hs + lane % Hs, ii = lane / Hs, G = 32 / Hs;
    const int64_t ej0 = A.e_start[j];
    const int64_t n = A.e_start[j + 1] - ej0;
    const int64_t a0 = A.edges[A.E + ej0];
    const int64_t col = j - a0;
    float kv[kDpHd], gk[kDpHd], gv[kDpHd];
    load16(A.k + (j * H + h) * kDpHd, kv);
#pragma unroll
    for (int d = 0; d < kDpHd; d++) gk[d] = gv[d] = 0.f;
    for (int64_t il = ii; il < n; il += G) {
        const int64_t i = a0 + il;
        const int64_t e = A.e_start[i] + col;
        float qv[kDpHd], go[kDpHd];
        load16(A.q + (i * H + h) * kDpHd, qv);
        load16(A.gout + (i * H + h) * kDpHd, go);
        float s = dot16(qv, kv);
        if (A.z) s += __ldg(A.z + e * H + h);
        const float p = __expf(s - __ldg(A.lse + i * H + h));
        const float gs = A.gz[e * H + h];
#pragma unroll
        for (int d = 0; d < kDpHd; d++) {
            gk[d] = fmaf(gs, qv[d], gk[d]);
            gv[d] = fmaf(p, go[d], gv[d]);
        }
    }
    for (int o = Hs; o < 32; o <<= 1)
#pragma unroll
        for (int d = 0; d < kDpHd; d++) {
            gk[d] += __shfl_xor_sync(0xffffffffu, gk[d], o);
            gv[d] += __shfl_xor_sync(0xffffffffu, gv[d], o);
        }
    if (ii == 0) {
        store16(A.gk + (j * H + h) * kDpHd, gk);
        store16(A.gv + (j * H + h) * kDpHd, gv);
    }
}

static bool heads_ok(int H) { return H >= 1 && H <= 32 && (32 % H) == 0; }

// heads per warp: half of them when that still divides a warp evenly (two warps per atom)
static int heads_per_warp(int H)
{
    return (H % 2 == 0 && 32 % (H / 2) == 0) ? H / 2 : H;
}

int dpa_fwd(const DpArgs& A, const Params& P, cudaStream_t st)
{
    if (!heads_ok(P.H)) return CFB200_E_UNSUPPORTED;
    if (A.N == 0) return CFB200_OK;
    const int Hs = heads_per_warp(P.H);
    const int64_t warps = A.N * (P.H / Hs);
    dpa_fwd_kernel<<<(unsigned)((warps + kDpWarps - 1) / kDpWarps), kDpWarps * 32, 0, st>>>(A, P.H, Hs);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int dpa_bwd(const DpArgs& A, const Params& P, cudaStream_t st)
{
    if (!heads_ok(P.H)) return CFB200_E_UNSUPPORTED;
    if (A.N == 0) return CFB200_OK;
    const int Hs = heads_per_warp(P.H);
    const int64_t warps = A.N * (P.H / Hs);
    const unsigned grid = (unsigned)((warps + kDpWarps - 1) / kDpWarps);
    dpa_bwd_rows_kernel<<<grid, kDpWarps * 32, 0, st>>>(A, P.H, Hs);
    dpa_bwd_cols_kernel<<<grid, kDpWarps * 32, 0, st>>>(A, P.H, Hs);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

// the column pass alone, for callers that produced gz themselves
int dpa_bwd_cols(const DpArgs& A, const Params& P, cudaStream_t st)
{
    if (!heads_ok(P.H)) return CFB200_E_UNSUPPORTED;
    if (A.N == 0) return CFB200_OK;
    const int Hs = heads_per_warp(P.H);
    const int64_t warps = A.N * (P.H / Hs);
    dpa_bwd_cols_kernel<<<(unsigned)((warps + kDpWarps - 1) / kDpWarps), kDpWarps * 32, 0, st>>>(A, P.H, Hs);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
