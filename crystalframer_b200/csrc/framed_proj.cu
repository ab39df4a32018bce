// Lattice-sum attention bias and frame-projected value position encoding, forward and
// backward (replaces real_enc_frame_proj_{fwd,bwd}_{length,angle}.cu of the reference).
//
// Work decomposition
//   grid  = (resident blocks, heads); a block owns one head and a strided subset of the pairs,
//           which it stages 32 at a time.
//   warp  = one (pair, head) task at a time (LatticeLane, lattice_lane.cuh).  Lanes first evaluate 32
//           lattice translations in parallel -- from the pair's sorted list where one exists, else by
//           slab sweeps -- (weight w = exp(a (d^2 - d^2_min)), window positions), drop translations
//           whose weight is below exp(-P.prune) of the largest, and leave one record per surviving
//           translation in shared memory.  Then the warp walks the survivors: lane l owns basis
//           indices l and l+32 of each of the four 64-wide Gaussian bases (distance, three frame
//           axes) and keeps their running sums in registers, so the data-dependent window offset
//           becomes a per-lane predicate instead of an indexed shared-memory update.
//   forward: after 4 tasks a warp multiplies its own 4 basis vectors (4 x 256) with the head's
//           16 x 256 projection from shared memory; warps never wait for one another.
//   backward: after 8 tasks per warp the block's 64 basis vectors (64 x 256) sit in shared memory
//           and the block accumulates their outer product with the upstream gradient in registers
//           -- one weight-gradient partial per block, not per pair.
//
// Numerics follow the reference's float expressions for every integer decision (lattice range,
// window start / end); Gaussians use ex2.approx on pre-scaled arguments.
#include <atomic>
#include "lattice_lane.cuh"

namespace cfb {

constexpr int kFpWarps = 8;
constexpr int kFpThreads = kFpWarps * 32;
// pairs a warp handles between two projections (forward) or between two block barriers (backward:
// more pairs per barrier shorten the wait for the slowest warp; shared memory has the room at 2 blocks/SM)
__host__ __device__ constexpr int fp_tasks_per_warp(bool bwd) { return bwd ? 8 : 4; }
__host__ __device__ constexpr int fp_slots(bool bwd) { return kFpWarps * fp_tasks_per_warp(bwd); }   // staged pairs
constexpr int kFpK = 256;                              // 4 bases x 64
// staging row stride: the backward reads a row per lane with 128-bit loads (padded, conflict-free); the
// forward reads rows as half-warp broadcasts and needs no padding
__host__ __device__ constexpr int fp_stage_stride(bool bwd) { return bwd ? 260 : 256; }
constexpr int kHd = 16;                                // head dimension of this instance
// resident blocks per SM the kernels are compiled for (register budget): forward 3, backward 2
__host__ __device__ constexpr int fp_blocks_per_sm(bool bwd) { return bwd ? 2 : 3; }


struct FpArgs {
    const float* a_ik; const float* pos_ij; const float* tvecs; const float* rvlen;
    const int64_t* batch; const int64_t* edges;
    int64_t N, E;
    const float* W[4];        // distance (H,16,64), axis 1..3 (H,16,angle_dim)
    const float* frame[3];    // each (N,H,3)
    float* z; float* values;                     // forward outputs
    const float* z_in; const float* gz; const float* gv;   // backward inputs
    const float4* cache;      // optional per-pair geometry (pair_cache_kernel), valid for ranges (cache_range)^3
    const float* list;        // optional per-pair translation lists (pair_list_kernel): (E, kListPlanes, kListLen)
    int cache_range;
    float* ga_e;              // (E,H) per-pair coefficient gradient (scratch)
    float* gW_part;           // (gridDim.x, H, 16, 256) per-block weight gradient (scratch)
};

constexpr int kWfStride = 260;                         // forward: W stored [o][k] with padded rows (conflict-free 128-bit reads by 16 rows)
constexpr int kWtStride = 20;                          // backward: W stored [k][o] with padded rows (conflict-free 128-bit reads)
// shared memory: projection weights | staged basis vectors | per-warp translation records (forward 6 floats
// per record, backward 8) | backward only: upstream gradients of the staged pairs [32][16]
__host__ __device__ constexpr int fp_w_floats(bool bwd) { return bwd ? kFpK * kWtStride : kHd * kWfStride; }
__host__ __device__ constexpr int fp_rec_floats(bool bwd) { return bwd ? 8 * 32 : 6 * 32; }
__host__ __device__ constexpr size_t fp_smem_bytes(bool bwd)
{
    return sizeof(float) * ((size_t)fp_w_floats(bwd) + (size_t)fp_slots(bwd) * fp_stage_stride(bwd) +
                            (size_t)kFpWarps * fp_rec_floats(bwd) + (bwd ? fp_slots(bwd) * kHd : 0));
}

// two fp32 multiply-adds in one instruction (packed fp32 arithmetic of sm_100): the projection loops are
// bound by instruction issue, not by the FMA pipe
__device__ __forceinline__ float2 fma2(float a0, float a1, float b0, float b1, float2 c)
{
    return __ffma2_rn(make_float2(a0, a1), make_float2(b0, b1), c);
}

template <bool BWD, bool ANG>
__global__ void __launch_bounds__(kFpThreads, fp_blocks_per_sm(BWD)) framed_proj_kernel(const FpArgs A, const Params P)
{
    extern __shared__ __align__(16) float smem[];
    constexpr int kFpStageStride = fp_stage_stride(BWD);
    constexpr int kFpSlots = fp_slots(BWD), kFpTasksPerWarp = fp_tasks_per_warp(BWD);
    float* W_s = smem;                                          // fwd: [16][260]; bwd: [256][20] (transposed)
    float* stage = W_s + fp_w_floats(BWD);                      // [32][stride]
    float* tbuf = stage + kFpSlots * kFpStageStride;            // per warp: float4[32] then float4[32] (bwd) / float2[32] (fwd)
    float* side = tbuf + kFpWarps * fp_rec_floats(BWD);         // bwd: gv [32][16]

    const int h = blockIdx.y, H = P.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // projection weights of this head: W_s[o][basis*64 + dim]
    for (int idx = threadIdx.x; idx < kHd * kFpK / 4; idx += kFpThreads) {
        const int o = idx >> 6, k4 = idx & 63, b = k4 >> 4, d4 = k4 & 15;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const int width = b == 0 ? 64 : P.angle_dim;          // columns this basis' weights hold (zero beyond)
        if (A.W[b] != nullptr && 4 * d4 < width)
            v = __ldg(reinterpret_cast<const float4*>(A.W[b] + ((size_t)h * kHd + o) * width) + d4);
        if (!BWD) {
            reinterpret_cast<float4*>(W_s)[o * (kWfStride / 4) + k4] = v;
        } else {
            const int k = k4 * 4;
            W_s[(k + 0) * kWtStride + o] = v.x; W_s[(k + 1) * kWtStride + o] = v.y;
            W_s[(k + 2) * kWtStride + o] = v.z; W_s[(k + 3) * kWtStride + o] = v.w;
        }
    }

    float2 gacc[2][4];
    if (BWD) {
#pragma unroll
        for (int j = 0; j < 4; j++) gacc[0][j] = gacc[1][j] = make_float2(0.f, 0.f);
    }
    LatticeLane<BWD, ANG> L;
    L.init(P, lane, tbuf + warp * fp_rec_floats(BWD));
    __syncthreads();

    // Pair assignment: block b takes pairs b, b + G, b + 2G, ... (G = gridDim.x) and stages them 32
    // at a time.  Every block therefore samples the whole batch evenly, which balances the very
    // uneven per-pair cost (small cells keep hundreds of translations, large cells a dozen)
    // without any dynamic scheduling -- the assignment, and with it every sum, stays deterministic.
    const int64_t G = gridDim.x;
    const int64_t myPairs = A.E > (int64_t)blockIdx.x ? (A.E - blockIdx.x + G - 1) / G : 0;
    const int64_t nChunks = (myPairs + kFpSlots - 1) / kFpSlots;
    auto slot_of = [&](int tsk) { return BWD ? tsk * kFpWarps + warp : warp * kFpTasksPerWarp + tsk; };
    // The chain pair -> query atom -> crystal -> cell is three dependent loads; the first two are
    // issued one task ahead so that a task starts with its atom and crystal already in registers.
    int i_next = 0, c_next = 0;
    if (nChunks > 0) {
        const int64_t e0 = (int64_t)slot_of(0) * G + blockIdx.x;
        if (e0 < A.E) { i_next = (int)A.edges[e0]; c_next = (int)A.batch[i_next]; }
    }
    for (int64_t chunk = 0; chunk < nChunks; chunk++) {
        for (int tsk = 0; tsk < kFpTasksPerWarp; tsk++) {
            const int slot = slot_of(tsk);
            const int64_t e = (chunk * kFpSlots + slot) * G + blockIdx.x;
            float* srow = stage + slot * kFpStageStride;
            if (e >= A.E) {      // a warp's pairs come in increasing order: nothing left to prefetch either
#pragma unroll
                for (int j = 0; j < 8; j++) srow[j * 32 + lane] = 0.f;
                if (BWD && lane < kHd) side[slot * kHd + lane] = 0.f;
                continue;
            }
            const int64_t i = i_next, c = c_next;
            const bool last_tsk = tsk + 1 == kFpTasksPerWarp;
            const int64_t e_next = ((chunk + (last_tsk ? 1 : 0)) * kFpSlots + slot_of(last_tsk ? 0 : tsk + 1)) * G + blockIdx.x;
            if (e_next < A.E) i_next = (int)A.edges[e_next];
            // per-pair lattice arithmetic: LatticeLane (lattice_lane.cuh)
            L.a = __ldg(A.a_ik + i * H + h);
            if (ANG) {
#pragma unroll
                for (int x = 0; x < 3; x++) {
                    const float* f = A.frame[x] + (i * H + h) * 3;
                    L.fx[x] = __ldg(f); L.fy[x] = __ldg(f + 1); L.fz[x] = __ldg(f + 2);
                }
            }
            // backward: the pair's upstream gradients are requested now and first used after the lattice
            // loops (lanes 0..15 hold gv, lane 16 holds gz), so their latency is off the critical path
            float g_up = 0.f;
            if (BWD) {
                L.ref = __ldg(A.z_in + e * H + h);
                if (lane < kHd) g_up = __ldg(A.gv + (e * H + h) * kHd + lane);
                else if (lane == kHd) g_up = __ldg(A.gz + e * H + h);
            }
            int Rl = 0;
            if (lane < 3) Rl = lattice_range_1d(P, L.a, P.cutoff_radius != 0.0f ? __ldg(A.rvlen + 3 * c + lane) : 0.0f);
            const int R1 = __shfl_sync(0xffffffffu, Rl, 0), R2 = __shfl_sync(0xffffffffu, Rl, 1), R3 = __shfl_sync(0xffffffffu, Rl, 2);
            L.reset();
            if (A.list != nullptr && R1 == A.cache_range && R2 == A.cache_range && R3 == A.cache_range) {
                // the pair's translations sorted by distance, prepared once per batch: a prefix is expanded
                L.run_list(P, A.list + (size_t)e * kListStride);
            } else {
                // slab sweeps over (n1; n2, n3) for lattice ranges the lists do not cover
                L.run_slabs(P, R1, R2, R3, __ldg(A.pos_ij + 3 * e), __ldg(A.pos_ij + 3 * e + 1), __ldg(A.pos_ij + 3 * e + 2),
                            A.tvecs + 9 * c);
            }
            const float a = L.a, d2min = L.ref;
            const float sum_l = L.sum_l, px_l = L.px_l;
            const float (&sd)[2] = L.sd;
            const float (&sa)[3][2] = L.sa;
            const float (&qd)[2] = L.qd;
            const float (&qa)[3][2] = L.qa;

            if (e_next < A.E) c_next = (int)A.batch[i_next];

            if (!BWD) {
                const float sum = warp_sum(sum_l);
                if (lane == 0) A.z[e * H + h] = logf(sum) + d2min * a;
                const float inv = 1.0f / sum;
                const float kd = P.c_dist * inv, ka = P.c_ang * inv;
                srow[lane] = sd[0] * kd; srow[32 + lane] = sd[1] * kd;
#pragma unroll
                for (int x = 0; x < 3; x++) {
                    srow[64 + 64 * x + lane] = sa[x][0] * ka;
                    srow[96 + 64 * x + lane] = sa[x][1] * ka;
                }
            } else {
                const float px = warp_sum(px_l);
                // G = W^T gv restricted to this lane's eight basis indices
                float gvr[kHd];
                if (lane < kHd) side[slot * kHd + lane] = g_up;
                const float gz_e = __shfl_sync(0xffffffffu, g_up, kHd);
                __syncwarp();
                const float4* gv4 = reinterpret_cast<const float4*>(side + slot * kHd);
#pragma unroll
                for (int o4 = 0; o4 < kHd / 4; o4++) {
                    const float4 v = gv4[o4];
                    gvr[4 * o4] = v.x; gvr[4 * o4 + 1] = v.y; gvr[4 * o4 + 2] = v.z; gvr[4 * o4 + 3] = v.w;
                }
                float G[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float4* wrow = reinterpret_cast<const float4*>(W_s + (j * 32 + lane) * kWtStride);
                    float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                    for (int o4 = 0; o4 < kHd / 4; o4++) {
                        const float4 u = wrow[o4];
                        acc = fma2(u.x, u.y, gvr[4 * o4], gvr[4 * o4 + 1], acc);
                        acc = fma2(u.z, u.w, gvr[4 * o4 + 2], gvr[4 * o4 + 3], acc);
                    }
                    G[j] = acc.x + acc.y;
                }
                float Ad = fmaf(G[0], qd[0], G[1] * qd[1]), Bd = fmaf(G[0], sd[0], G[1] * sd[1]);
                float Aa = 0.f, Ba = 0.f;
#pragma unroll
                for (int x = 0; x < 3; x++) {
                    Aa = fmaf(G[2 + 2 * x], qa[x][0], fmaf(G[3 + 2 * x], qa[x][1], Aa));
                    Ba = fmaf(G[2 + 2 * x], sa[x][0], fmaf(G[3 + 2 * x], sa[x][1], Ba));
                }
                Ad = warp_sum(Ad); Bd = warp_sum(Bd); Aa = warp_sum(Aa); Ba = warp_sum(Ba);
                if (lane == 0) {
                    // the reference scales the whole length-kernel result, gz term included, by the
                    // distance coefficient (models/cuda_funcs/real_space_framed_proj.py:183)
                    const float g_len = fmaf(px, gz_e, Ad - px * Bd);
                    const float g_ang = Aa - px * Ba;
                    A.ga_e[e * H + h] = P.c_dist * g_len + P.c_ang * g_ang;
                }
                // stage the averaged bases for the weight-gradient outer product; the reference
                // leaves the distance weights' gradient unscaled and scales the angle ones
                srow[lane] = sd[0]; srow[32 + lane] = sd[1];
#pragma unroll
                for (int x = 0; x < 3; x++) {
                    srow[64 + 64 * x + lane] = sa[x][0] * P.c_ang;
                    srow[96 + 64 * x + lane] = sa[x][1] * P.c_ang;
                }
            }
        }
        if (!BWD) {
            // warp-level projection of the warp's own four pairs: lane = (output o, pair half)
            __syncwarp();
            if (A.values != nullptr) {
                const int o = lane & 15, half = lane >> 4;
                const int slot0 = warp * kFpTasksPerWarp + 2 * half;
                const float4* wr = reinterpret_cast<const float4*>(W_s + o * kWfStride);
                const float4* s0 = reinterpret_cast<const float4*>(stage + slot0 * kFpStageStride);
                const float4* s1 = s0 + kFpStageStride / 4;
                float2 a01 = make_float2(0.f, 0.f), a23 = a01, b01 = a01, b23 = a01;
#pragma unroll 8
                for (int k4 = 0; k4 < kFpK / 4; k4++) {
                    const float4 u = wr[k4], s = s0[k4], t = s1[k4];
                    a01 = fma2(s.x, s.y, u.x, u.y, a01); a23 = fma2(s.z, s.w, u.z, u.w, a23);
                    b01 = fma2(t.x, t.y, u.x, u.y, b01); b23 = fma2(t.z, t.w, u.z, u.w, b23);
                }
                const float acc0 = (a01.x + a01.y) + (a23.x + a23.y), acc1 = (b01.x + b01.y) + (b23.x + b23.y);
                const int64_t e0 = (chunk * kFpSlots + slot0) * G + blockIdx.x, e1 = e0 + G;
                if (e0 < A.E) A.values[(e0 * H + h) * kHd + o] = acc0;
                if (e1 < A.E) A.values[(e1 * H + h) * kHd + o] = acc1;
            }
            __syncwarp();
            continue;
        }
        __syncthreads();
        {
            // in this phase lane l owns basis indices 4l..4l+3 and 128+4l..128+4l+3 (128-bit reads)
            for (int slot = 0; slot < kFpSlots; slot++) {
                const float2 g = *reinterpret_cast<const float2*>(side + slot * kHd + 2 * warp);
                const float4* srow = reinterpret_cast<const float4*>(stage + slot * kFpStageStride) + lane;
                const float4 s0 = srow[0], s1 = srow[32];
                gacc[0][0] = fma2(s0.x, s0.y, g.x, g.x, gacc[0][0]); gacc[0][1] = fma2(s0.z, s0.w, g.x, g.x, gacc[0][1]);
                gacc[0][2] = fma2(s1.x, s1.y, g.x, g.x, gacc[0][2]); gacc[0][3] = fma2(s1.z, s1.w, g.x, g.x, gacc[0][3]);
                gacc[1][0] = fma2(s0.x, s0.y, g.y, g.y, gacc[1][0]); gacc[1][1] = fma2(s0.z, s0.w, g.y, g.y, gacc[1][1]);
                gacc[1][2] = fma2(s1.x, s1.y, g.y, g.y, gacc[1][2]); gacc[1][3] = fma2(s1.z, s1.w, g.y, g.y, gacc[1][3]);
            }
        }
        __syncthreads();
    }

    if (BWD) {
        float* dst = A.gW_part + (((size_t)blockIdx.x * H + h) * kHd + 2 * warp) * kFpK + 4 * lane;
        *reinterpret_cast<float4*>(dst) = make_float4(gacc[0][0].x, gacc[0][0].y, gacc[0][1].x, gacc[0][1].y);
        *reinterpret_cast<float4*>(dst + 128) = make_float4(gacc[0][2].x, gacc[0][2].y, gacc[0][3].x, gacc[0][3].y);
        *reinterpret_cast<float4*>(dst + kFpK) = make_float4(gacc[1][0].x, gacc[1][0].y, gacc[1][1].x, gacc[1][1].y);
        *reinterpret_cast<float4*>(dst + kFpK + 128) = make_float4(gacc[1][2].x, gacc[1][2].y, gacc[1][3].x, gacc[1][3].y);
    }
}

// ga (N,H): ordered sum of the per-pair gradients of each atom's pairs
__global__ void reduce_ga_kernel(const float* __restrict__ ga_e, const int64_t* __restrict__ e_start,
                                 int64_t N, int H, float* __restrict__ ga)
{
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= N * H) return;
    const int64_t i = tid / H;
    const int h = (int)(tid - i * H);
    float s = 0.f;
    for (int64_t e = e_start[i]; e < e_start[i + 1]; e++) s += ga_e[e * H + h];
    ga[tid] = s;
}

// weight gradients: ordered sum over the per-block partials, split into the four tensors
__global__ void reduce_gw_kernel(const float* __restrict__ part, int nPart, int H, int angle_dim, float* gWd, float* gW1,
                                 float* gW2, float* gW3)
{
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;   // (h, o, k)
    if (tid >= H * kHd * kFpK) return;
    float s = 0.f;
    for (int x = 0; x < nPart; x++) s += part[(size_t)x * H * kHd * kFpK + tid];
    const int k = tid & (kFpK - 1), ho = tid >> 8, b = k >> 6, dim = k & 63;
    float* dst = b == 0 ? gWd : (b == 1 ? gW1 : (b == 2 ? gW2 : gW3));
    const int width = b == 0 ? 64 : angle_dim;                 // the angle weights are (H,16,angle_dim)
    if (dst != nullptr && dim < width) dst[ho * width + dim] = s;
}

// Resident blocks along x: the kernel is persistent (each block strides over the chunks), so the
// grid is one wave of fp_blocks_per_sm() blocks per SM, split evenly between the heads.

static int grid_x_for(int64_t E, int H, bool bwd)
{
    const int sms = sm_count();
    const int64_t chunks = (E + fp_slots(bwd) - 1) / fp_slots(bwd);
    int64_t want = ((int64_t)sms * fp_blocks_per_sm(bwd)) / H;
    if (want < 1) want = 1;
    if (chunks < want) want = chunks < 1 ? 1 : chunks;
    return (int)want;
}

int64_t framed_proj_bwd_workspace_bytes(int64_t N, int64_t E, int H)
{
    (void)N;
    const int gx = grid_x_for(E, H, true);
    size_t ga_e = ((size_t)E * H * sizeof(float) + 255) / 256 * 256;
    return (int64_t)(ga_e + (size_t)gx * H * kHd * kFpK * sizeof(float));
}

template <bool BWD, bool ANG>
static int launch_fp(const FpArgs& A, const Params& P, int gx, cudaStream_t st)
{
    auto kern = framed_proj_kernel<BWD, ANG>;
    static std::atomic<bool> attr_done[64];   // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp_smem_bytes(BWD)) != cudaSuccess)
            return CFB200_E_CUDA;
        attr_done[dev & 63] = true;
    }
    kern<<<dim3(gx, P.H), kFpThreads, fp_smem_bytes(BWD), st>>>(A, P);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int framed_proj_fwd(const FpArgs& A, const Params& P, cudaStream_t st)
{
    if (A.E == 0) return CFB200_OK;
    const int gx = grid_x_for(A.E, P.H, false);
    return A.W[1] != nullptr ? launch_fp<false, true>(A, P, gx, st) : launch_fp<false, false>(A, P, gx, st);
}

int framed_proj_bwd(FpArgs A, const Params& P, const int64_t* e_start, float* ga, float* gW[4], void* ws,
                    int64_t ws_bytes, cudaStream_t st)
{
    if (ws_bytes < framed_proj_bwd_workspace_bytes(A.N, A.E, P.H) || ws == nullptr) return CFB200_E_WORKSPACE;
    const int gx = grid_x_for(A.E, P.H, true);
    size_t ga_e_bytes = ((size_t)A.E * P.H * sizeof(float) + 255) / 256 * 256;
    A.ga_e = reinterpret_cast<float*>(ws);
    A.gW_part = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + ga_e_bytes);
    int nPart = gx;
    if (A.E > 0) {
        int rc = A.W[1] != nullptr ? launch_fp<true, true>(A, P, gx, st) : launch_fp<true, false>(A, P, gx, st);
        if (rc != CFB200_OK) return rc;
    } else {
        nPart = 0;
    }
    if (A.N > 0) {
        const int64_t nt = A.N * P.H;
        reduce_ga_kernel<<<(unsigned)((nt + 255) / 256), 256, 0, st>>>(A.ga_e, e_start, A.N, P.H, ga);
    }
    const int nw = P.H * kHd * kFpK;
    reduce_gw_kernel<<<(nw + 255) / 256, 256, 0, st>>>(A.gW_part, nPart, P.H, P.angle_dim, gW[0], gW[1], gW[2], gW[3]);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
