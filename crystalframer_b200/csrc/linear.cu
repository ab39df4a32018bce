// Dense layers of an encoder layer: input projections, output projection and feed-forward block
// (models/indexed_lattice_multi_head_attention_cuda.py:869, :987-988 and
// models/indexed_latticeformer_encoder.py:888-890 of the reference, which calls torch.nn.functional.linear
// for each), their data gradients, and all weight / bias gradients of a layer in one grouped launch.
//
// The problems are small and skinny -- M = atoms of the batch (a few thousand), K and N in {128, 512} -- so a
// single product is a few microseconds of FP32 work and what matters is (i) that the launches come from one
// host call per layer instead of one framework dispatch each, (ii) enough thread blocks to cover the SMs,
// and (iii) epilogues (bias, residual, ReLU and its mask) fused in.  FP32 accumulation on the FMA pipe keeps
// the 1e-4 tolerance of the path without an error-compensated split.
//
// gemm_kernel<B_KN, TM>:  C[M,N] = sum over up to three products A_s[M,K_s] op(B_s) (+ bias) (+ residual),
//   then ReLU or a ReLU mask.  B_KN = false: B is [N,K] (a torch Linear weight; forward), true: B is [K,N]
//   (the same weight used for the data gradient).  Tile 16*TM x 64, BK = 16, 256 threads, TM x 4 outputs per
//   thread, register-prefetched double-buffered shared memory.
// wgrad_kernel:  out[P,Q] = A[M,P]^T B[M,Q] for a table of problems (optionally batched over heads), the
//   M rows split over gridDim.y; every block writes its partial tile and partial column sums of A (the bias
//   gradient) to scratch, and wgrad_reduce_kernel adds the partials in a fixed order (bit-reproducible).
#include <stdlib.h>
#include "common.cuh"

namespace cfb {

constexpr int kGmBN = 64, kGmBK = 16, kGmThreads = 256;
constexpr int kGmLd = 64 + 4;          // shared-memory row length (floats); rows stay 16-byte aligned

struct GemmSeg { const float* A; const float* B; int lda, ldb, K; };
struct GemmArgs {
    GemmSeg seg[3];
    int nseg, M, N;
    float* C; int ldc;
    const float* bias;                  // (N) or NULL
    const float* resid; int ldr;        // (M,N) added to the result, or NULL
    const float* mask; int ldm;         // (M,N): the result is zeroed where mask <= 0 (ReLU backward), or NULL
    int relu;
};

// up to three products of equal shape in one launch (blockIdx.z picks one): the q, k and v projections
struct GemmBatch { GemmArgs g[3]; int n; };

template <bool B_KN, int TM>
__global__ void __launch_bounds__(kGmThreads) gemm_kernel(const GemmBatch Gb)
{
    const GemmArgs& G = Gb.g[blockIdx.z];
    constexpr int BM = 16 * TM;
    __shared__ __align__(16) float As[2][kGmBK][kGmLd];
    __shared__ __align__(16) float Bs[2][kGmBK][kGmLd];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * kGmBN;
    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    const int a_row = tid >> 2, a_k = (tid & 3) * 4;             // A tile: BM rows x 16 k, one float4 per thread
    const int b_row = B_KN ? (tid >> 4) : (tid >> 2);            // B [K,N]: 16 k x 64 n;  B [N,K]: 64 n x 16 k
    const int b_col = B_KN ? (tid & 15) * 4 : (tid & 3) * 4;
    int steps[3], total = 0;
    for (int s = 0; s < G.nseg; s++) { steps[s] = (G.seg[s].K + kGmBK - 1) / kGmBK; total += steps[s]; }

    // Tiles travel global memory -> registers -> shared memory.  Two register sets are in flight, so a tile is
    // requested two steps (about 600 cycles of arithmetic) before it is needed: one step does not cover the latency
    // of L2 at this tile size.
    auto fetch = [&](int step, float4& ra, float4& rb) {
        ra = make_float4(0.f, 0.f, 0.f, 0.f);
        rb = ra;
        if (step >= total) return;
        int s = 0;
        while (step >= steps[s]) { step -= steps[s]; s++; }
        const GemmSeg& S = G.seg[s];
        const int k0 = step * kGmBK;
        if (a_row < BM && m0 + a_row < G.M && k0 + a_k < S.K)
            ra = __ldg(reinterpret_cast<const float4*>(S.A + (size_t)(m0 + a_row) * S.lda + k0 + a_k));
        if (B_KN) {
            if (k0 + b_row < S.K && n0 + b_col < G.N)
                rb = __ldg(reinterpret_cast<const float4*>(S.B + (size_t)(k0 + b_row) * S.ldb + n0 + b_col));
        } else {
            if (n0 + b_row < G.N && k0 + b_col < S.K)
                rb = __ldg(reinterpret_cast<const float4*>(S.B + (size_t)(n0 + b_row) * S.ldb + k0 + b_col));
        }
    };
    auto stash = [&](int buf, const float4& ra, const float4& rb) {
        if (a_row < BM) {
            As[buf][a_k + 0][a_row] = ra.x; As[buf][a_k + 1][a_row] = ra.y;
            As[buf][a_k + 2][a_row] = ra.z; As[buf][a_k + 3][a_row] = ra.w;
        }
        if (B_KN) {
            *reinterpret_cast<float4*>(&Bs[buf][b_row][b_col]) = rb;
        } else {
            Bs[buf][b_col + 0][b_row] = rb.x; Bs[buf][b_col + 1][b_row] = rb.y;
            Bs[buf][b_col + 2][b_row] = rb.z; Bs[buf][b_col + 3][b_row] = rb.w;
        }
    };
    auto compute = [&](int buf) {
#pragma unroll
        for (int kk = 0; kk < kGmBK; kk++) {
            float a[TM];
            if (TM == 4) {
                const float4 u = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
                a[0] = u.x; a[1] = u.y; a[TM - 2] = u.z; a[TM - 1] = u.w;
            } else {
                const float2 u = *reinterpret_cast<const float2*>(&As[buf][kk][ty * 2]);
                a[0] = u.x; a[1] = u.y;
            }
            const float4 b = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
#pragma unroll
            for (int i = 0; i < TM; i++) {
                acc[i][0] = fmaf(a[i], b.x, acc[i][0]); acc[i][1] = fmaf(a[i], b.y, acc[i][1]);
                acc[i][2] = fmaf(a[i], b.z, acc[i][2]); acc[i][3] = fmaf(a[i], b.w, acc[i][3]);
            }
        }
    };

    float4 ra0, rb0, ra1, rb1;
    fetch(0, ra0, rb0);
    stash(0, ra0, rb0);
    fetch(1, ra0, rb0);
    fetch(2, ra1, rb1);
    __syncthreads();
    for (int step = 0; step < total; step += 2) {
        compute(0);
        if (step + 1 < total) { stash(1, ra0, rb0); fetch(step + 3, ra0, rb0); }
        __syncthreads();
        if (step + 1 >= total) break;
        compute(1);
        if (step + 2 < total) { stash(0, ra1, rb1); fetch(step + 4, ra1, rb1); }
        __syncthreads();
    }

    const int n = n0 + tx * 4;
    if (n >= G.N) return;
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (G.bias != nullptr) bv = __ldg(reinterpret_cast<const float4*>(G.bias + n));
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + ty * TM + i;
        if (m >= G.M) continue;
        float4 v = make_float4(acc[i][0] + bv.x, acc[i][1] + bv.y, acc[i][2] + bv.z, acc[i][3] + bv.w);
        if (G.resid != nullptr) {
            const float4 r = __ldg(reinterpret_cast<const float4*>(G.resid + (size_t)m * G.ldr + n));
            v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
        }
        if (G.relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
        if (G.mask != nullptr) {
            const float4 h = __ldg(reinterpret_cast<const float4*>(G.mask + (size_t)m * G.ldm + n));
            v.x = h.x > 0.f ? v.x : 0.f; v.y = h.y > 0.f ? v.y : 0.f; v.z = h.z > 0.f ? v.z : 0.f; v.w = h.w > 0.f ? v.w : 0.f;
        }
        *reinterpret_cast<float4*>(G.C + (size_t)m * G.ldc + n) = v;
    }
}

static inline bool gm_aligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct WgArgs;
static int tc_gemm_batch(const GemmBatch& Gb, bool b_kn, cudaStream_t st);
static bool tc_gemm_covers(const GemmBatch& Gb);
static int tc_wgrad_launch(const WgArgs& W, int tiles, cudaStream_t st);

// CFB200_TC=0 keeps the dense layers on the FP32 pipe (gemm_kernel); default: tensor cores where the shapes allow
static bool use_tensor_cores()
{
    static int v = -1;
    if (v < 0) { const char* e = getenv("CFB200_TC"); v = e ? atoi(e) : 0; }
    return v != 0;
}

static int gemm_check(const GemmArgs& G)
{
    if ((G.N & 3) || (G.ldc & 3) || !gm_aligned(G.C) || !gm_aligned(G.bias) || !gm_aligned(G.resid) || !gm_aligned(G.mask) ||
        (G.resid && (G.ldr & 3)) || (G.mask && (G.ldm & 3)))
        return CFB200_E_SHAPE;
    for (int s = 0; s < G.nseg; s++)
        if ((G.seg[s].K & 3) || (G.seg[s].lda & 3) || (G.seg[s].ldb & 3) || !gm_aligned(G.seg[s].A) || !gm_aligned(G.seg[s].B))
            return CFB200_E_SHAPE;
    return CFB200_OK;
}

// Launches up to three products of the same shape (M, N).  Every leading dimension, K and N must be multiples of
// 4 floats and every pointer 16-byte aligned (float4 accesses).
static int gemm_batch(const GemmBatch& Gb, bool b_kn, cudaStream_t st)
{
    const GemmArgs& G = Gb.g[0];
    if (G.M <= 0 || G.N <= 0 || Gb.n <= 0) return CFB200_OK;
    for (int i = 0; i < Gb.n; i++) {
        if (Gb.g[i].M != G.M || Gb.g[i].N != G.N) return CFB200_E_SHAPE;
        const int rc = gemm_check(Gb.g[i]);
        if (rc != CFB200_OK) return rc;
    }
    if (use_tensor_cores() && tc_gemm_covers(Gb)) return tc_gemm_batch(Gb, b_kn, st);
    const int gy = (G.N + kGmBN - 1) / kGmBN;
    // the 64-row tile when it already gives every SM a block, else the 32-row tile (twice the blocks)
    const bool tall = (int64_t)((G.M + 63) / 64) * gy * Gb.n >= 148;
    if (tall) {
        const dim3 grid((G.M + 63) / 64, gy, Gb.n);
        if (b_kn) gemm_kernel<true, 4><<<grid, kGmThreads, 0, st>>>(Gb);
        else gemm_kernel<false, 4><<<grid, kGmThreads, 0, st>>>(Gb);
    } else {
        const dim3 grid((G.M + 31) / 32, gy, Gb.n);
        if (b_kn) gemm_kernel<true, 2><<<grid, kGmThreads, 0, st>>>(Gb);
        else gemm_kernel<false, 2><<<grid, kGmThreads, 0, st>>>(Gb);
    }
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

static int gemm(const GemmArgs& G, bool b_kn, cudaStream_t st)
{
    GemmBatch Gb;
    Gb.g[0] = G;
    Gb.n = 1;
    return gemm_batch(Gb, b_kn, st);
}

// ---- weight and bias gradients ------------------------------------------------------------------------

constexpr int kWgMaxProb = 12;
constexpr int kWgTile = 64;

struct WgProblem {
    const float* A; const float* B;     // A (M, lda) columns [0,P) ; B (M, ldb) columns [0,Q)
    float* out; float* bias_out;        // out (P, ldo) ; bias_out (P) = column sums of A, or NULL
    int lda, ldb, ldo, P, Q;
    int nb, sA, sB, sO;                 // batches (heads) and their strides in floats
    int tiles_p, tiles_q, tile0;        // tiles of one batch; first tile of this problem in the launch
    int64_t ws_off;                     // floats: partial products [split][nb][P][Q], then partial column sums [split][P]
};
struct WgArgs {
    WgProblem prob[kWgMaxProb];
    int nprob, M, S, rows;              // S splits of `rows` rows each
    float* ws;
    int accumulate;                     // add to out / bias_out instead of overwriting
};

__global__ void __launch_bounds__(kGmThreads) wgrad_kernel(const WgArgs W)
{
    __shared__ __align__(16) float As[2][kGmBK][kGmLd];
    __shared__ __align__(16) float Bs[2][kGmBK][kGmLd];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    int pi = 0;
    while (pi + 1 < W.nprob && (int)blockIdx.x >= W.prob[pi + 1].tile0) pi++;
    const WgProblem& Pb = W.prob[pi];
    int t = blockIdx.x - Pb.tile0;
    const int per = Pb.tiles_p * Pb.tiles_q;
    const int b = t / per;
    t -= b * per;
    const int p0 = (t / Pb.tiles_q) * kWgTile, q0 = (t % Pb.tiles_q) * kWgTile;
    const float* A = Pb.A + (size_t)b * Pb.sA;
    const float* B = Pb.B + (size_t)b * Pb.sB;
    const int split = blockIdx.y;
    const int r0 = split * W.rows, r1 = min(W.M, r0 + W.rows);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    float colsum = 0.f;
    const bool want_bias = Pb.bias_out != nullptr && q0 == 0 && b == 0;
    const int l_row = tid >> 4, l_col = (tid & 15) * 4;          // 16 rows x 64 columns, one float4 per thread and operand
    float4 ra = make_float4(0.f, 0.f, 0.f, 0.f), rb = ra;
    float4 ra1 = make_float4(0.f, 0.f, 0.f, 0.f), rb1 = ra1;
    auto fetch2 = [&](int r, float4& xa, float4& xb) {
        xa = make_float4(0.f, 0.f, 0.f, 0.f);
        xb = xa;
        if (r + l_row < r1) {
            if (p0 + l_col < Pb.P) xa = __ldg(reinterpret_cast<const float4*>(A + (size_t)(r + l_row) * Pb.lda + p0 + l_col));
            if (q0 + l_col < Pb.Q) xb = __ldg(reinterpret_cast<const float4*>(B + (size_t)(r + l_row) * Pb.ldb + q0 + l_col));
        }
    };
    auto stash2 = [&](int buf, const float4& xa, const float4& xb) {
        *reinterpret_cast<float4*>(&As[buf][l_row][l_col]) = xa;
        *reinterpret_cast<float4*>(&Bs[buf][l_row][l_col]) = xb;
    };
    auto compute = [&](int buf) {
#pragma unroll
        for (int kk = 0; kk < kGmBK; kk++) {
            const float4 a = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 bb = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                acc[i][0] = fmaf(av[i], bb.x, acc[i][0]); acc[i][1] = fmaf(av[i], bb.y, acc[i][1]);
                acc[i][2] = fmaf(av[i], bb.z, acc[i][2]); acc[i][3] = fmaf(av[i], bb.w, acc[i][3]);
            }
        }
        if (want_bias && tid < kWgTile) {
#pragma unroll
            for (int kk = 0; kk < kGmBK; kk++) colsum += As[buf][kk][tid];
        }
    };
    // two register sets in flight, as in gemm_kernel: rows beyond r1 read as zeros
    fetch2(r0, ra, rb);
    stash2(0, ra, rb);
    fetch2(r0 + kGmBK, ra, rb);
    fetch2(r0 + 2 * kGmBK, ra1, rb1);
    __syncthreads();
    for (int r = r0; r < r1; r += 2 * kGmBK) {
        compute(0);
        if (r + kGmBK < r1) { stash2(1, ra, rb); fetch2(r + 3 * kGmBK, ra, rb); }
        __syncthreads();
        if (r + kGmBK >= r1) break;
        compute(1);
        if (r + 2 * kGmBK < r1) { stash2(0, ra1, rb1); fetch2(r + 4 * kGmBK, ra1, rb1); }
        __syncthreads();
    }
    // partial tile -> scratch [split][batch][P][Q]
    float* ws = W.ws + Pb.ws_off + ((size_t)split * Pb.nb + b) * Pb.P * Pb.Q;
    const int q = q0 + tx * 4;
    if (q < Pb.Q) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int p = p0 + ty * 4 + i;
            if (p < Pb.P) *reinterpret_cast<float4*>(ws + (size_t)p * Pb.Q + q) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        }
    }
    if (want_bias && tid < kWgTile && p0 + tid < Pb.P)
        W.ws[Pb.ws_off + (size_t)W.S * Pb.nb * Pb.P * Pb.Q + (size_t)split * Pb.P + p0 + tid] = colsum;
}

// grid.x covers the largest problem; grid.y = problem.  Sums the S partials of every output in split order.
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(const WgArgs W)
{
    const WgProblem& Pb = W.prob[blockIdx.y];
    const int64_t nW = (int64_t)Pb.nb * Pb.P * Pb.Q;
    const int64_t nAll = nW + (Pb.bias_out != nullptr ? Pb.P : 0);
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nAll; idx += (int64_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        if (idx < nW) {
            const float* src = W.ws + Pb.ws_off + idx;
            for (int k = 0; k < W.S; k++) s += src[(size_t)k * nW];
            const int64_t b = idx / ((int64_t)Pb.P * Pb.Q), rem = idx - b * Pb.P * Pb.Q;
            const int p = (int)(rem / Pb.Q), q = (int)(rem - (int64_t)p * Pb.Q);
            float* dst = Pb.out + (size_t)b * Pb.sO + (size_t)p * Pb.ldo + q;
            *dst = W.accumulate ? *dst + s : s;
        } else {
            const int p = (int)(idx - nW);
            const float* src = W.ws + Pb.ws_off + (size_t)W.S * nW + p;
            for (int k = 0; k < W.S; k++) s += src[(size_t)k * Pb.P];
            Pb.bias_out[p] = W.accumulate ? Pb.bias_out[p] + s : s;
        }
    }
}

__global__ void axpy_kernel(float* __restrict__ y, const float* __restrict__ x, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] += x[i];
}

// Splits of the M rows: about 16, each a multiple of the 16-row step and at least 64 rows.
static void wgrad_splits(int64_t M, int& S, int& rows)
{
    int64_t r = (M + 15) / 16;
    r = ((r + 15) / 16) * 16;
    if (r < 64) r = 64;
    rows = (int)r;
    S = (int)((M + r - 1) / r);
    if (S < 1) S = 1;
}

// Scratch floats for a layer's weight gradients: S partials of every output.
static int64_t wgrad_workspace_floats(int64_t M, int64_t outputs)
{
    int S, rows;
    wgrad_splits(M, S, rows);
    return (int64_t)S * outputs;
}

// Fills tile counts and scratch offsets, then launches the grouped products and the reduction.  Problems whose
// output is a whole number of 128 x 128 tiles go to the tensor-core kernel (tc_linear.cu), the others (the per-head
// value-encoding weights, 16 rows) to wgrad_kernel; both leave their partials in the same scratch layout.
static int wgrad(WgArgs& W, int64_t ws_floats, cudaStream_t st)
{
    if (W.M <= 0 || W.nprob == 0) return CFB200_OK;
    wgrad_splits(W.M, W.S, W.rows);
    int64_t off = 0, largest = 0;
    for (int i = 0; i < W.nprob; i++) {
        WgProblem& Pb = W.prob[i];
        if ((Pb.lda & 3) || (Pb.ldb & 3) || (Pb.P & 3) || (Pb.Q & 3) || (Pb.sA & 3) || (Pb.sB & 3) || !gm_aligned(Pb.A) ||
            !gm_aligned(Pb.B))
            return CFB200_E_SHAPE;
        Pb.ws_off = off;
        const int64_t n = (int64_t)Pb.nb * Pb.P * Pb.Q + (Pb.bias_out ? Pb.P : 0);
        off += (int64_t)W.S * n;
        off = (off + 3) & ~(int64_t)3;
        if (n > largest) largest = n;
    }
    if (W.ws == nullptr || off > ws_floats) return CFB200_E_WORKSPACE;
    WgArgs tc = W, fp = W;
    tc.nprob = fp.nprob = 0;
    int tc_tiles = 0, fp_tiles = 0;
    for (int i = 0; i < W.nprob; i++) {
        const WgProblem& Pb = W.prob[i];
        const bool on_tc = use_tensor_cores() && Pb.nb == 1 && Pb.P % 128 == 0 && Pb.Q % 128 == 0;
        WgArgs& dst = on_tc ? tc : fp;
        WgProblem& q = dst.prob[dst.nprob++];
        q = Pb;
        const int tile = on_tc ? 128 : kWgTile;
        q.tiles_p = (Pb.P + tile - 1) / tile;
        q.tiles_q = (Pb.Q + tile - 1) / tile;
        int& tiles = on_tc ? tc_tiles : fp_tiles;
        q.tile0 = tiles;
        tiles += Pb.nb * q.tiles_p * q.tiles_q;
    }
    if (tc.nprob > 0) {
        const int rc = tc_wgrad_launch(tc, tc_tiles, st);
        if (rc != CFB200_OK) return rc;
    }
    if (fp.nprob > 0) wgrad_kernel<<<dim3(fp_tiles, W.S), kGmThreads, 0, st>>>(fp);
    int gx = (int)((largest + 255) / 256);
    if (gx > 148) gx = 148;
    wgrad_reduce_kernel<<<dim3(gx, W.nprob), 256, 0, st>>>(W);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
