// The dense layers on the 5th-generation tensor cores: tcgen05.mma (kind::tf32) with FP32 accumulation in
// tensor memory, and an error-compensated three-product split so that the results keep FP32 accuracy
// (the path's tolerance is 1e-4 relative; a single TF32 product has a 10-bit mantissa).
//
//   x = hi + lo,  hi = x with the low 13 mantissa bits cleared (exactly a TF32 number),  lo = x - hi (exact in FP32)
//   A B^T  ~  A_hi B_hi^T + A_hi B_lo^T + A_lo B_hi^T        (the dropped lo x lo term is below 2^-20 relative)
//
// One CTA of 256 threads owns a 128 x 128 output tile.  Per 32-wide slice of the contraction index the threads
// bring both operands from global memory through registers (three register sets: two slices' loads are in flight
// behind the one in work), split them, and store hi and lo parts to one of two shared-memory stages in the
// K-major, 128-byte-swizzled layout the tensor core reads (8-row groups of 1024 bytes, the 16-byte chunk j of row
// r stored at chunk j ^ (r & 7)); operands whose contraction index is not contiguous in global memory (the weight
// in a data gradient, both operands of a weight gradient) are transposed by that staging.  One thread then issues
// 4 (k-steps of 8) x 3 (products) tcgen05.mma instructions and commits them to the stage's mbarrier, which is
// waited on before the stage is written again two slices later.  The epilogue reads the accumulator with
// tcgen05.ld (a warp reads the TMEM lanes of its quarter: rows; warps w and w + 4 take half of the columns each),
// applies bias / residual / ReLU / ReLU mask and stores.  Every wait on the mbarrier is bounded: on expiry the kernel sets CFB200_ST_TC_TIMEOUT, frees its
// tensor memory and returns.
//
// No TMA: the operands need the hi / lo split on the way to shared memory, so they pass through registers anyway.
#include <atomic>
#include "common.cuh"

namespace cfb {

constexpr int kTcThreads = 256;
constexpr int kTcTile = 128;                 // rows of either operand per tile
constexpr int kTcKc = 32;                    // contraction slice: 32 floats = one 128-byte swizzle row
constexpr int kTcOperandBytes = kTcTile * kTcKc * 4;            // 16 KB
constexpr int kTcStageBytes = 4 * kTcOperandBytes;              // A hi, A lo, B hi, B lo
constexpr int kTcSmemBytes = 2 * kTcStageBytes + 1024;          // two stages + alignment slack
constexpr uint32_t kTcSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of the 16-byte chunk j (0..7) of row r (0..127) in a K-major 128-byte-swizzled operand tile
__device__ __forceinline__ uint32_t tc_chunk_offset(int r, int j)
{
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4));
}

__device__ __forceinline__ void tc_split(const float x, float& hi, float& lo)
{
    hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    lo = x - hi;
}

// shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row groups 1024 bytes apart, descriptor version 1
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr)
{
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}

// instruction descriptor: D = F32, A = B = TF32, both K-major, M = 128, N = 128
constexpr uint32_t kTcIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTcTile >> 3) << 17) | ((uint32_t)(kTcTile >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kTcIdesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ bool tc_wait(uint32_t mbar, uint32_t parity)
{
    for (uint32_t it = 0; it < kTcSpinLimit; it++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// One operand of a product: element (r, k) of the (rows x K) operand is src[r * ld + k] (k contiguous), or, when
// `transposed`, src[k * ld + r].
struct TcOperand { const float* src; int ld; int rows; int transposed; };

// registers holding one 128 x 32 slice of both operands: 4 float4 per thread and operand
struct TcSlice { float4 a[4], b[4]; };

__device__ __forceinline__ void tc_fetch1(float4* v, const TcOperand& Op, const int r0, const int k0, const int K, const int tid)
{
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!Op.transposed) {
            const int q = tid + kTcThreads * i, r = q >> 3, j = q & 7;           // row r, 16-byte chunk j
            if (r0 + r < Op.rows && k0 + 4 * j < K) x = __ldg(reinterpret_cast<const float4*>(Op.src + (size_t)(r0 + r) * Op.ld + k0 + 4 * j));
        } else {
            const int r = 4 * (warp + 8 * i), k = lane;                          // rows r..r+3 of contraction index k
            if (r0 + r < Op.rows && k0 + k < K) x = __ldg(reinterpret_cast<const float4*>(Op.src + (size_t)(k0 + k) * Op.ld + r0 + r));
        }
        v[i] = x;
    }
}

__device__ __forceinline__ void tc_stash1(const float4* v, const TcOperand& Op, uint8_t* hi_base, uint8_t* lo_base, const int tid)
{
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float x[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        float h[4], l[4];
#pragma unroll
        for (int c = 0; c < 4; c++) tc_split(x[c], h[c], l[c]);
        if (!Op.transposed) {
            const int q = tid + kTcThreads * i, r = q >> 3, j = q & 7;
            const uint32_t off = tc_chunk_offset(r, j);
            *reinterpret_cast<float4*>(hi_base + off) = make_float4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<float4*>(lo_base + off) = make_float4(l[0], l[1], l[2], l[3]);
        } else {
            const int r = 4 * (warp + 8 * i), k = lane;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t off = tc_chunk_offset(r + c, k >> 2) + (uint32_t)((k & 3) << 2);
                *reinterpret_cast<float*>(hi_base + off) = h[c];
                *reinterpret_cast<float*>(lo_base + off) = l[c];
            }
        }
    }
}

// CTA-wide state of one tile computation: two shared-memory stages, each with the mbarrier its instructions commit to
struct TcCta {
    uint8_t* stage[2];
    uint32_t mbar[2], tmem;
    uint32_t slices_done;
    bool failed;
};

__device__ __forceinline__ void tc_begin(TcCta& T, uint8_t* smem_raw, uint64_t* mbar_slots, uint32_t* tmem_slot)
{
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    T.stage[0] = aligned; T.stage[1] = aligned + kTcStageBytes;
    T.mbar[0] = smem_u32(mbar_slots); T.mbar[1] = smem_u32(mbar_slots + 1);
    T.slices_done = 0;
    T.failed = false;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(T.mbar[0]) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(T.mbar[1]) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if ((threadIdx.x >> 5) == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTcTile) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    T.tmem = *tmem_slot;
}

// Adds one 32-wide slice held in registers to the accumulator: splits it into the stage slices_done & 1 of shared
// memory (once the instructions that read that stage two slices ago have finished) and issues its instructions.
__device__ __forceinline__ void tc_slice(TcCta& T, const TcSlice& S, const TcOperand& OpA, const TcOperand& OpB)
{
    const int tid = threadIdx.x;
    const uint32_t s = T.slices_done, st = s & 1;
    if (s >= 2 && !T.failed) {
        const bool ok = tc_wait(T.mbar[0] + 8 * st, ((s >> 1) - 1) & 1);
        T.failed = __syncthreads_or(ok ? 0 : 1) != 0;
    }
    if (T.failed) return;
    uint8_t* base = T.stage[0] + st * kTcStageBytes;
    tc_stash1(S.a, OpA, base, base + kTcOperandBytes, tid);
    tc_stash1(S.b, OpB, base + 2 * kTcOperandBytes, base + 3 * kTcOperandBytes, tid);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy stores -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t ah = tc_smem_desc(smem_u32(base)), al = tc_smem_desc(smem_u32(base + kTcOperandBytes));
        const uint64_t bh = tc_smem_desc(smem_u32(base + 2 * kTcOperandBytes)), bl = tc_smem_desc(smem_u32(base + 3 * kTcOperandBytes));
#pragma unroll
        for (int k = 0; k < kTcKc / 8; k++) {                         // 8 TF32 values = 32 bytes per instruction: 2 descriptor units
            const uint64_t adv = (uint64_t)(2 * k);
            tc_mma(T.tmem, ah + adv, bh + adv, (s > 0 || k > 0) ? 1u : 0u);
            tc_mma(T.tmem, ah + adv, bl + adv, 1u);
            tc_mma(T.tmem, al + adv, bh + adv, 1u);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(T.mbar[0] + 8 * st) : "memory");
    }
    T.slices_done++;
}

// Waits for the last slice (its commit covers every instruction issued before it); true if the accumulator is complete.
__device__ __forceinline__ bool tc_finish(TcCta& T)
{
    if (T.slices_done > 0 && !T.failed) {
        const uint32_t s = T.slices_done - 1;
        const bool ok = tc_wait(T.mbar[0] + 8 * (s & 1), (s >> 1) & 1);
        T.failed = __syncthreads_or(ok ? 0 : 1) != 0;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (T.failed && threadIdx.x == 0) atomicOr(&g_status, CFB200_ST_TC_TIMEOUT);
    return !T.failed && T.slices_done > 0;
}

__device__ __forceinline__ void tc_end(TcCta& T)
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if ((threadIdx.x >> 5) == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(T.tmem), "r"((uint32_t)kTcTile) : "memory");
}

// Output row and column range of this thread in the epilogue: a warp may read the TMEM lanes 32 (w & 3) .. + 31
// only, so warps w and w + 4 share 32 rows and take 64 columns each.
__device__ __forceinline__ int tc_row() { return ((threadIdx.x >> 5) & 3) * 32 + (threadIdx.x & 31); }
__device__ __forceinline__ int tc_col0() { return (threadIdx.x >> 7) * (kTcTile / 2); }

// 16 consecutive accumulator columns of this thread's row
__device__ __forceinline__ void tc_load16(uint32_t tmem, int col, float* v)
{
    const uint32_t addr = tmem + ((uint32_t)(((threadIdx.x >> 5) & 3) * 32) << 16) + (uint32_t)col;
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr) : "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// ---- C = sum_s A_s op(B_s) (+ bias) (+ residual), ReLU / mask: same contract as gemm_kernel (linear.cu) ----------
template <bool B_KN>
__global__ void __launch_bounds__(kTcThreads, 1) tc_gemm_kernel(const GemmBatch Gb)
{
    extern __shared__ uint8_t tc_smem[];
    __shared__ uint64_t mbar_slots[2];
    __shared__ uint32_t tmem_slot;
    const GemmArgs& G = Gb.g[blockIdx.z];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * kTcTile, n0 = blockIdx.y * kTcTile;
    TcCta T;
    tc_begin(T, tc_smem, mbar_slots, &tmem_slot);
    int total = 0;
    for (int s = 0; s < G.nseg; s++) total += G.seg[s].K / kTcKc;
    TcOperand OA, OB;
    OA.rows = G.M; OA.transposed = 0; OB.rows = G.N; OB.transposed = B_KN ? 1 : 0;
    // slice index -> (segment, offset): three register sets keep two slices' loads in flight behind the one in work
    auto fetch = [&](TcSlice& R, int slice) {
        if (slice >= total) return;
        int s = 0;
        while (slice >= G.seg[s].K / kTcKc) { slice -= G.seg[s].K / kTcKc; s++; }
        OA.src = G.seg[s].A; OA.ld = G.seg[s].lda; OB.src = G.seg[s].B; OB.ld = G.seg[s].ldb;
        tc_fetch1(R.a, OA, m0, slice * kTcKc, G.seg[s].K, tid);
        tc_fetch1(R.b, OB, n0, slice * kTcKc, G.seg[s].K, tid);
    };
    TcSlice R0, R1, R2;
    fetch(R0, 0); fetch(R1, 1); fetch(R2, 2);
    for (int s = 0; s < total; s += 3) {
        tc_slice(T, R0, OA, OB); fetch(R0, s + 3);
        if (s + 1 < total) { tc_slice(T, R1, OA, OB); fetch(R1, s + 4); }
        if (s + 2 < total) { tc_slice(T, R2, OA, OB); fetch(R2, s + 5); }
    }
    if (tc_finish(T)) {
        const int m = m0 + tc_row();
        for (int c0 = tc_col0(); c0 < tc_col0() + kTcTile / 2; c0 += 16) {
            float v[16];
            tc_load16(T.tmem, c0, v);
            const int n = n0 + c0;
            if (m < G.M && n < G.N) {
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {
                    float4 o = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
                    const int nn = n + 4 * q4;
                    if (G.bias != nullptr) { const float4 b = __ldg(reinterpret_cast<const float4*>(G.bias + nn)); o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w; }
                    if (G.resid != nullptr) {
                        const float4 r = __ldg(reinterpret_cast<const float4*>(G.resid + (size_t)m * G.ldr + nn));
                        o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
                    }
                    if (G.relu) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
                    if (G.mask != nullptr) {
                        const float4 hm = __ldg(reinterpret_cast<const float4*>(G.mask + (size_t)m * G.ldm + nn));
                        o.x = hm.x > 0.f ? o.x : 0.f; o.y = hm.y > 0.f ? o.y : 0.f; o.z = hm.z > 0.f ? o.z : 0.f; o.w = hm.w > 0.f ? o.w : 0.f;
                    }
                    *reinterpret_cast<float4*>(G.C + (size_t)m * G.ldc + nn) = o;
                }
            }
        }
    }
    tc_end(T);
}

// whether tc_gemm_kernel covers a batch: every N a multiple of the 128-wide tile, every K a multiple of 32
static bool tc_gemm_covers(const GemmBatch& Gb)
{
    for (int i = 0; i < Gb.n; i++) {
        if (Gb.g[i].N % kTcTile) return false;
        for (int s = 0; s < Gb.g[i].nseg; s++)
            if (Gb.g[i].seg[s].K % kTcKc) return false;
    }
    return true;
}

static int tc_gemm_batch(const GemmBatch& Gb, bool b_kn, cudaStream_t st)
{
    const GemmArgs& G = Gb.g[0];
    static std::atomic<bool> attr_done[2][64];
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = b_kn ? tc_gemm_kernel<true> : tc_gemm_kernel<false>;
    if (!attr_done[b_kn ? 1 : 0][dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) != cudaSuccess) return CFB200_E_CUDA;
        attr_done[b_kn ? 1 : 0][dev & 63] = true;
    }
    const dim3 grid((G.M + kTcTile - 1) / kTcTile, G.N / kTcTile, Gb.n);
    kern<<<grid, kTcThreads, kTcSmemBytes, st>>>(Gb);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

// ---- weight gradients: out[P,Q] = A[M,P]^T B[M,Q], rows split over gridDim.y, partial tiles to scratch -------
// Same problem table, scratch layout and reduction as wgrad_kernel (linear.cu); tiles are 128 x 128 and both
// operands are staged transposed (the contraction index, the atom, is the slow index of A and B in memory).
__global__ void __launch_bounds__(kTcThreads, 1) tc_wgrad_kernel(const WgArgs W)
{
    extern __shared__ uint8_t tc_smem[];
    __shared__ uint64_t mbar_slots[2];
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x;
    int pi = 0;
    while (pi + 1 < W.nprob && (int)blockIdx.x >= W.prob[pi + 1].tile0) pi++;
    const WgProblem& Pb = W.prob[pi];
    const int t = blockIdx.x - Pb.tile0;
    const int p0 = (t / Pb.tiles_q) * kTcTile, q0 = (t % Pb.tiles_q) * kTcTile;
    const int split = blockIdx.y;
    const int r0 = split * W.rows, r1 = min(W.M, r0 + W.rows);
    TcCta T;
    tc_begin(T, tc_smem, mbar_slots, &tmem_slot);
    TcOperand OA, OB;
    OA.src = Pb.A; OA.ld = Pb.lda; OA.rows = Pb.P; OA.transposed = 1;
    OB.src = Pb.B; OB.ld = Pb.ldb; OB.rows = Pb.Q; OB.transposed = 1;
    const int total = r1 > r0 ? (r1 - r0 + kTcKc - 1) / kTcKc : 0;
    auto fetch = [&](TcSlice& R, int slice) {
        if (slice >= total) return;
        tc_fetch1(R.a, OA, p0, r0 + slice * kTcKc, r1, tid);
        tc_fetch1(R.b, OB, q0, r0 + slice * kTcKc, r1, tid);
    };
    TcSlice R0, R1, R2;
    fetch(R0, 0); fetch(R1, 1); fetch(R2, 2);
    for (int s = 0; s < total; s += 3) {
        tc_slice(T, R0, OA, OB); fetch(R0, s + 3);
        if (s + 1 < total) { tc_slice(T, R1, OA, OB); fetch(R1, s + 4); }
        if (s + 2 < total) { tc_slice(T, R2, OA, OB); fetch(R2, s + 5); }
    }
    const bool have = tc_finish(T);
    float* ws = W.ws + Pb.ws_off + (size_t)split * Pb.P * Pb.Q;
    const int p = p0 + tc_row();
    for (int c0 = tc_col0(); c0 < tc_col0() + kTcTile / 2; c0 += 16) {
        float v[16];
        if (have) tc_load16(T.tmem, c0, v);
        else {
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = 0.f;          // an empty row range contributes zeros
        }
        const int q = q0 + c0;
        if ((have || total == 0) && p < Pb.P && q < Pb.Q) {
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++)
                *reinterpret_cast<float4*>(ws + (size_t)p * Pb.Q + q + 4 * q4) = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
        }
    }
    tc_end(T);
}

// Partial column sums of A (the bias gradients) for the problems that ask for them: grid (problem, split),
// thread = column.  Same scratch slots as wgrad_kernel's.
__global__ void __launch_bounds__(256) wgrad_colsum_kernel(const WgArgs W)
{
    const WgProblem& Pb = W.prob[blockIdx.x];
    if (Pb.bias_out == nullptr) return;
    const int split = blockIdx.y;
    const int r0 = split * W.rows, r1 = min(W.M, r0 + W.rows);
    for (int p = threadIdx.x; p < Pb.P; p += blockDim.x) {
        float s = 0.f;
        for (int r = r0; r < r1; r++) s += __ldg(Pb.A + (size_t)r * Pb.lda + p);
        W.ws[Pb.ws_off + (size_t)W.S * Pb.nb * Pb.P * Pb.Q + (size_t)split * Pb.P + p] = s;
    }
}

static int tc_wgrad_launch(const WgArgs& W, int tiles, cudaStream_t st)
{
    static std::atomic<bool> attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        if (cudaFuncSetAttribute(tc_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes) != cudaSuccess) return CFB200_E_CUDA;
        attr_done[dev & 63] = true;
    }
    tc_wgrad_kernel<<<dim3(tiles, W.S), kTcThreads, kTcSmemBytes, st>>>(W);
    wgrad_colsum_kernel<<<dim3(W.nprob, W.S), 256, 0, st>>>(W);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
