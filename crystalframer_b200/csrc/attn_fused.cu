// Periodic attention of one encoder layer as two kernels: lattice-sum bias, frame-projected value
// encoding and ragged softmax attention together, forward and backward (what
// RealEncodingWithFramedProjFuncCUDA followed by FusedDotProductAttentionCUDA compute in the reference,
// models/indexed_lattice_multi_head_attention_cuda.py:944-985).
//
// The value encoding is linear in the 256 basis sums of a pair, values_ij = W s_ij, so the attention
// output  out_i = sum_j p_ij (v_j + W s_ij) = sum_j p_ij v_j + W (sum_j p_ij s_ij)  needs the 16 x 256
// projection once per (atom, head) instead of once per (pair, head), and the (E,H,16) value encoding and
// its gradient never exist in memory.  Backward likewise: W^T gout_i is formed once per (atom, head), the
// weight gradient is  sum_i gout_i (x) S_i  with the pooled basis S_i = sum_j p_ij s_ij saved by the
// forward (a small GEMM left to the caller), and the coefficient gradient of an atom is accumulated by
// the warp that walks its pairs -- no scratch, no second-stage reductions.
//
// Work decomposition: grid = (resident blocks, heads); warp = one (atom, head) at a time, walking the
// atom's pairs with an online softmax.  The cost of an atom varies a hundredfold (1 to 64+ pairs, a few
// to a hundred surviving translations each), so warps draw atoms from a per-head queue in the order given
// by ``order`` (most expensive first).  Which warp computes an atom does not affect any result: nothing is
// accumulated across atoms, so every sum stays deterministic.  The per-pair lattice arithmetic is LatticeLane
// (lattice_lane.cuh).  Outputs of the forward: out (N,H,16), z (E,H), lse (N,H), spool (N,H,256) with the
// distance part unscaled and the angle parts times the angle coefficient (the scaling the reference's
// weight gradients carry).  The backward leaves gz (E,H) for the column pass that forms gk and gv
// (dpa_bwd_cols_kernel), gq (N,H,16) with respect to the scaled query, and ga (N,H).
//
// Chunked queue (kernels instantiated with TASKS): one warp walks the pairs of an (atom, head) one after the other, so an
// atom of a dense 64-atom cell with a wide Gaussian can take several times a warp's average load and the launch
// would end with that warp alone.  attn_plan_kernel turns the batch's work queue (atom_order_kernel) and the layer's
// coefficients into a table of tasks per head: an atom whole, or one chunk of its pairs.  A chunk is computed exactly
// like an atom with fewer pairs and leaves its result in a partial row; attn_merge_fwd / _bwd_kernel combine the
// rows of an atom in chunk order (softmax-weighted by the chunks' log-sum-exp; plain sums backward), so results do
// not depend on which warp ran what.
#include <atomic>
#include "lattice_lane.cuh"

namespace cfb {

// warps per block (two blocks per SM either way): the forward runs best with 10 (96 registers), the backward,
// which holds more state per lane, with 8 (no spills)
__host__ __device__ constexpr int at_warps(bool bwd) { return bwd ? 8 : 10; }
constexpr int kAtHd = 16;
constexpr int kAtK = 256;
constexpr int kAtWfStride = 260;      // forward: W [16][260], conflict-free 128-bit reads by 16 rows
constexpr int kAtWtStride = 20;       // backward: W transposed [256][20]
constexpr int kAtFwdBlocks = 2, kAtBwdBlocks = 2;   // resident blocks per SM the kernels are compiled for

struct AtArgs {
    const float* qs; const float* k; const float* v; const float* a_ik;
    const float* pos_ij; const float* tvecs; const float* rvlen;
    const int64_t* batch; const int64_t* edges; const int64_t* e_start; const int32_t* order;
    int* counters;            // (H) work-queue heads, zeroed before the launch
    // task table of the chunked queue (attn_plan_kernel), or NULL: then ``order`` (or the atom index) is the queue
    const int4* tasks; int64_t n_entries;
    int* chunk_count;         // (H) chunk entries in use per head: they sit at the end of the chunk region
    float* part_out; float* part_lse; float* part_spool;               // forward results of chunks (kSplitSlots rows)
    float* part_gq; float* part_ga;                                    // backward results of chunks
    int64_t N, E;
    const float* W[4]; const float* frame[3];
    const float* list; int cache_range;
    float* z; float* out; float* lse; float* spool;                    // forward outputs
    const float* gout; const float* z_in;                             // backward inputs (plus out, lse above)
    float* gz; float* gq; float* ga;                                   // backward outputs
    // what a training forward leaves for a backward pass without a second lattice sum: per pair its value encoding
    // (E,H,16) and sum p d^2 (E,H); per atom the projection of the attention-pooled d^2-weighted basis sums (N,H,16)
    float* val; float* px; float* upool;
    float* part_upool;                                                  // its chunk results (kSplitSlots rows)
};

__host__ __device__ constexpr size_t at_smem_bytes(bool bwd)
{
    // projection weights | per-warp translation records | per-warp row (forward: pooled basis, backward: gout)
    return sizeof(float) * ((bwd ? kAtK * kAtWtStride : kAtHd * kAtWfStride) + at_warps(bwd) * (bwd ? 8 * 32 : 6 * 32) +
                            at_warps(bwd) * (bwd ? 32 : kAtK));
}

// per-(atom, head) inputs shared by both directions
struct AtomTask {
    int64_t i, c, e0, e1;
    int R1, R2, R3;
    bool use_list;
};

template <int MODE, bool ANG>
__device__ __forceinline__ AtomTask load_atom(const AtArgs& A, const Params& P, LatticeLane<MODE, ANG>& L, const int64_t i,
                                              const int h, const int lane)
{
    AtomTask T;
    const int H = P.H;
    T.i = i; T.c = A.batch[i];
    T.e0 = A.e_start[i]; T.e1 = A.e_start[i + 1];
    L.a = __ldg(A.a_ik + i * H + h);
    if (ANG) {
#pragma unroll
        for (int x = 0; x < 3; x++) {
            const float* f = A.frame[x] + (i * H + h) * 3;
            L.fx[x] = __ldg(f); L.fy[x] = __ldg(f + 1); L.fz[x] = __ldg(f + 2);
        }
    }
    int Rl = 0;
    if (lane < 3) Rl = lattice_range_1d(P, L.a, P.cutoff_radius != 0.0f ? __ldg(A.rvlen + 3 * T.c + lane) : 0.0f);
    T.R1 = __shfl_sync(0xffffffffu, Rl, 0); T.R2 = __shfl_sync(0xffffffffu, Rl, 1); T.R3 = __shfl_sync(0xffffffffu, Rl, 2);
    T.use_list = A.list != nullptr && T.R1 == A.cache_range && T.R2 == A.cache_range && T.R3 == A.cache_range;
    return T;
}

template <int MODE, bool ANG>
__device__ __forceinline__ void run_pair(const AtArgs& A, const Params& P, LatticeLane<MODE, ANG>& L, const AtomTask& T,
                                         const int64_t e)
{
    L.reset();
    if (T.use_list) {
        L.run_list(P, A.list + (size_t)e * kListStride);
    } else {
        L.run_slabs(P, T.R1, T.R2, T.R3, __ldg(A.pos_ij + 3 * e), __ldg(A.pos_ij + 3 * e + 1), __ldg(A.pos_ij + 3 * e + 2),
                    A.tvecs + 9 * T.c);
    }
}

// next atom of this head's work queue (one atomic per task; the whole warp gets the same answer)
__device__ __forceinline__ int64_t next_task(int* counter, const int lane)
{
    int t = 0;
    if (lane == 0) t = atomicAdd(counter, 1);
    return (int64_t)__shfl_sync(0xffffffffu, t, 0);
}

template <bool ANG, bool TASKS>
__global__ void __launch_bounds__(at_warps(false) * 32, kAtFwdBlocks) attn_fwd_kernel(const AtArgs A, const Params P)
{
    extern __shared__ __align__(16) float smem[];
    float* W_s = smem;                                      // [16][260]
    float* tbuf = W_s + kAtHd * kAtWfStride;                // per warp 6 x 32
    float* rows = tbuf + at_warps(false) * 6 * 32;          // per warp 256: pooled basis, forward scaling
    const int h = blockIdx.y, H = P.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int idx = threadIdx.x; idx < kAtHd * kAtK / 4; idx += at_warps(false) * 32) {
        const int o = idx >> 6, k4 = idx & 63, b = k4 >> 4, d4 = k4 & 15;
        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
        const int width = b == 0 ? 64 : P.angle_dim;          // columns this basis' weights hold (zero beyond)
        if (A.W[b] != nullptr && 4 * d4 < width) w = __ldg(reinterpret_cast<const float4*>(A.W[b] + ((size_t)h * kAtHd + o) * width) + d4);
        reinterpret_cast<float4*>(W_s)[o * (kAtWfStride / 4) + k4] = w;
    }
    LatticeLane<0, ANG> L;
    L.init(P, lane, tbuf + warp * 6 * 32);
    float* srow = rows + warp * kAtK;
    __syncthreads();
    // the queue of this head begins where its chunk entries begin
    const int first = TASKS ? kSplitSlots - __ldg(A.chunk_count + h) : 0;

    for (;;) {
        const int64_t t = next_task(A.counters + h, lane) + first;
        if (t >= (TASKS ? A.n_entries : A.N)) break;
        int64_t i, row;
        AtomTask T;
        if (TASKS) {
            const int4 d = __ldg(A.tasks + (size_t)h * A.n_entries + t);
            const int cnt = d.w & 0xFFFFFF;
            if (cnt == 0) continue;                         // an entry this head does not use
            i = d.x; row = d.y;
            T = load_atom<0, ANG>(A, P, L, i, h, lane);
            T.e0 += d.z; T.e1 = T.e0 + cnt;
        } else {
            i = A.order != nullptr ? (int64_t)A.order[t] : t;
            row = i;
            T = load_atom<0, ANG>(A, P, L, i, h, lane);
        }
        const float qd = lane < kAtHd ? __ldg(A.qs + (i * H + h) * kAtHd + lane) : 0.f;
        float m = -INFINITY, l = 0.f, V = 0.f;
        float S[8];
#pragma unroll
        for (int r = 0; r < 8; r++) S[r] = 0.f;
        // the pairs of an atom run over the atoms of its crystal in order: key atom = first atom + offset
        const int64_t j0 = A.edges[A.E + T.e0];
        for (int64_t e = T.e0; e < T.e1; e++) {
            const int64_t j = j0 + (e - T.e0);
            if (lane == 0 && __ldg(A.edges + A.E + e) != j) atomicOr(&g_status, CFB200_ST_PAIR_LAYOUT);   // not the dense layout
            float kd = 0.f, vd = 0.f;
            if (lane < kAtHd) { kd = __ldg(A.k + (j * H + h) * kAtHd + lane); vd = __ldg(A.v + (j * H + h) * kAtHd + lane); }
            run_pair<0, ANG>(A, P, L, T, e);
            const float sum = warp_sum(L.sum_l);
            const float qk = warp_sum(qd * kd);
            const float zv = logf(sum) + L.ref * L.a;
            if (lane == 0) A.z[e * H + h] = zv;
            const float s = qk + zv;
            const float mn = fmaxf(m, s);
            const float sc = __expf(m - mn), p = __expf(s - mn);
            const float f = p / sum;
            l = fmaf(l, sc, p);
            V = fmaf(V, sc, p * vd);
            S[0] = fmaf(S[0], sc, f * L.sd[0]); S[1] = fmaf(S[1], sc, f * L.sd[1]);
#pragma unroll
            for (int x = 0; x < 3; x++) {
                S[2 + 2 * x] = fmaf(S[2 + 2 * x], sc, f * L.sa[x][0]);
                S[3 + 2 * x] = fmaf(S[3 + 2 * x], sc, f * L.sa[x][1]);
            }
            m = mn;
        }
        const float inv_l = T.e1 > T.e0 ? 1.0f / l : 0.f;
        // an atom's results go to its row, a chunk's to a partial row (numbered from N)
        const bool partial = TASKS && row >= A.N;
        if (partial) row -= A.N;
        if (lane == 0) (partial ? A.part_lse : A.lse)[row * H + h] = m + logf(l);
        // pooled basis: to memory with the scaling of the weight gradients, to shared memory with the
        // scaling of the values
        float* sp = (partial ? A.part_spool : A.spool) + (row * H + h) * kAtK;
        {
            const float d0 = S[0] * inv_l, d1 = S[1] * inv_l;
            sp[lane] = d0; sp[32 + lane] = d1;
            srow[lane] = d0 * P.c_dist; srow[32 + lane] = d1 * P.c_dist;
#pragma unroll
            for (int x = 0; x < 3; x++) {
                const float a0 = S[2 + 2 * x] * inv_l * P.c_ang, a1 = S[3 + 2 * x] * inv_l * P.c_ang;
                sp[64 + 64 * x + lane] = a0; sp[96 + 64 * x + lane] = a1;
                srow[64 + 64 * x + lane] = a0; srow[96 + 64 * x + lane] = a1;
            }
        }
        __syncwarp();
        // out_d = sum_j p_ij v_jd + W_d . S: lane = (output d, half of the 256 basis indices)
        {
            const int d = lane & 15, half = lane >> 4;
            const float4* wr = reinterpret_cast<const float4*>(W_s + d * kAtWfStride) + half * 32;
            const float4* sr = reinterpret_cast<const float4*>(srow) + half * 32;
            float acc = 0.f;
#pragma unroll 8
            for (int k4 = 0; k4 < 32; k4++) {
                const float4 u = wr[k4], s4 = sr[k4];
                acc = fmaf(s4.x, u.x, fmaf(s4.y, u.y, fmaf(s4.z, u.z, fmaf(s4.w, u.w, acc))));
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (lane < kAtHd) (partial ? A.part_out : A.out)[(row * H + h) * kAtHd + lane] = fmaf(V, inv_l, acc);
        }
        __syncwarp();
    }
}

// ---- training forward: also leaves what the backward pass needs of every pair ------------------------------
// With s_ij the basis sums of a pair, t_ij the same sums weighted with d^2 and x_ij = sum p d^2, the backward pass is
//   gz_ij = p_ij (gout_i . (v_j + W s_ij) - gout_i . out_i)
//   ga_i  = sum_j c_dist x_ij gz_ij + p_ij gout_i . W (t_ij - x_ij s_ij)
//         = gout_i . W (sum_j p_ij t_ij) + sum_j (c_dist x_ij gz_ij - p_ij x_ij gout_i . W s_ij)
// so it needs the lattice sums only through the pair's value encoding W s_ij (16 numbers), x_ij, and the projection
// of the attention-pooled t of the atom (16 numbers per atom).  None of these depends on gout: the training forward
// projects W s_ij per pair (one 16 x 256 product), pools t beside s, and stores 68 bytes per (pair, head); the
// backward pass (attn_bwd_saved_kernel) is then a plain ragged attention backward: no second lattice sum.  The
// attention output sums the stored value encodings directly; the pooled s is still kept for the weight gradients.
constexpr int kAtTrainWarps = 12;
constexpr size_t kAtTrainSmem = sizeof(float) * (kAtHd * kAtWfStride + kAtTrainWarps * 8 * 32 + kAtTrainWarps * 3 * kAtK);

// out_d = W_d . row: lane = (output d, half of the 256 basis indices); every lane returns the full sum of its d.
// Packed FP32: two products per instruction, two partial sums.
__device__ __forceinline__ float project_row(const float* W_s, const float* row, const int lane)
{
    const int d = lane & 15, half = lane >> 4;
    const ulonglong2* wr = reinterpret_cast<const ulonglong2*>(W_s + d * kAtWfStride) + half * 32;
    const ulonglong2* sr = reinterpret_cast<const ulonglong2*>(row) + half * 32;
    f32x2 acc = pack2(0.f, 0.f);
#pragma unroll 8
    for (int k4 = 0; k4 < 32; k4++) {
        const ulonglong2 w4 = wr[k4], s4 = sr[k4];
        acc = fma2(s4.x, w4.x, acc);
        acc = fma2(s4.y, w4.y, acc);
    }
    float a0, a1;
    unpack2(acc, a0, a1);
    const float sum = a0 + a1;
    return sum + __shfl_xor_sync(0xffffffffu, sum, 16);
}

template <bool ANG, bool TASKS>
__global__ void __launch_bounds__(kAtTrainWarps * 32, 2) attn_fwd_train_kernel(const AtArgs A, const Params P)
{
    extern __shared__ __align__(16) float smem[];
    float* W_s = smem;                                      // [16][260]
    float* tbuf = W_s + kAtHd * kAtWfStride;                // per warp 8 x 32
    float* rows = tbuf + kAtTrainWarps * 8 * 32;            // per warp 256: the basis vector being projected
    const int H = P.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    LatticeLane<2, ANG> L;
    L.init(P, lane, tbuf + warp * 8 * 32);
    float* srow = rows + warp * 3 * kAtK;
    // pooled basis sums of this lane as four packed pairs (indices l, l + 32 of each basis): Sp[32 x], x < 4; then the
    // d^2-weighted ones
    f32x2* Sp = reinterpret_cast<f32x2*>(srow + kAtK) + lane;
    f32x2* Tq = Sp + kAtK / 2;
    __shared__ int head_open;

    // A block serves its own head first and then, turn by turn, the head with the most entries left: the heads' Gaussian
    // widths differ, so their queues hold up to a fifth more or less work than the average, and the blocks of the light
    // heads would otherwise sit idle while the heaviest head finishes.  Switching heads costs a reload of the 16 KB of
    // projection weights.
    for (int turn = 0; turn < 2 * H; turn++) {
    int h = blockIdx.y;
    if (turn > 0) {
        __syncthreads();                                    // every warp is done with the previous head's weights
        if (threadIdx.x == 0) {
            // the head with the most entries left in its queue (a stale count costs a wasted or a missed turn at most)
            int best = -1, most = 0;
            for (int hh = 0; hh < H; hh++) {
                const int limit = TASKS ? (int)(A.n_entries - kSplitSlots) + __ldg(A.chunk_count + hh) : (int)A.N;
                const int left = limit - atomicAdd(A.counters + hh, 0);
                if (left > most) { most = left; best = hh; }
            }
            head_open = best;
        }
        __syncthreads();
        h = head_open;
        if (h < 0) break;                                   // every queue is drained
    }
    const int first = TASKS ? kSplitSlots - __ldg(A.chunk_count + h) : 0;
    for (int idx = threadIdx.x; idx < kAtHd * kAtK / 4; idx += kAtTrainWarps * 32) {
        const int o = idx >> 6, k4 = idx & 63, b = k4 >> 4, d4 = k4 & 15;
        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
        const int width = b == 0 ? 64 : P.angle_dim;          // columns this basis' weights hold (zero beyond)
        if (A.W[b] != nullptr && 4 * d4 < width) w = __ldg(reinterpret_cast<const float4*>(A.W[b] + ((size_t)h * kAtHd + o) * width) + d4);
        reinterpret_cast<float4*>(W_s)[o * (kAtWfStride / 4) + k4] = w;
    }
    __syncthreads();

    for (;;) {
        const int64_t t = next_task(A.counters + h, lane) + first;
        if (t >= (TASKS ? A.n_entries : A.N)) break;
        int64_t i, row;
        AtomTask T;
        if (TASKS) {
            const int4 d = __ldg(A.tasks + (size_t)h * A.n_entries + t);
            const int cnt = d.w & 0xFFFFFF;
            if (cnt == 0) continue;
            i = d.x; row = d.y;
            T = load_atom<2, ANG>(A, P, L, i, h, lane);
            T.e0 += d.z; T.e1 = T.e0 + cnt;
        } else {
            i = A.order != nullptr ? (int64_t)A.order[t] : t;
            row = i;
            T = load_atom<2, ANG>(A, P, L, i, h, lane);
        }
        const float qd = lane < kAtHd ? __ldg(A.qs + (i * H + h) * kAtHd + lane) : 0.f;
        float m = -INFINITY, l = 0.f, V = 0.f;
#pragma unroll
        for (int x = 0; x < 4; x++) Sp[32 * x] = Tq[32 * x] = pack2(0.f, 0.f);        // attention-pooled sums, plain and d^2-weighted
        const int64_t j0 = A.edges[A.E + T.e0];
        for (int64_t e = T.e0; e < T.e1; e++) {
            const int64_t j = j0 + (e - T.e0);
            if (lane == 0 && __ldg(A.edges + A.E + e) != j) atomicOr(&g_status, CFB200_ST_PAIR_LAYOUT);   // not the dense layout
            float kd = 0.f, vd = 0.f;
            if (lane < kAtHd) { kd = __ldg(A.k + (j * H + h) * kAtHd + lane); vd = __ldg(A.v + (j * H + h) * kAtHd + lane); }
            run_pair<2, ANG>(A, P, L, T, e);
            float r0 = L.sum_l, r1 = L.px_l, r2 = qd * kd;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                r0 += __shfl_xor_sync(0xffffffffu, r0, o); r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                r2 += __shfl_xor_sync(0xffffffffu, r2, o);
            }
            const float sum = r0, qk = r2;
            const float inv = 1.0f / sum;
            const float zv = logf(sum) + L.ref * L.a;
            if (lane == 0) { A.z[e * H + h] = zv; A.px[e * H + h] = r1 * inv; }
            // the pair's value encoding: its normalised basis sums, with the scaling of the values, times W
            {
                const float cd = inv * P.c_dist, ca = inv * P.c_ang;
                srow[lane] = L.sd[0] * cd; srow[32 + lane] = L.sd[1] * cd;
#pragma unroll
                for (int x = 0; x < 3; x++) { srow[64 + 64 * x + lane] = L.sa[x][0] * ca; srow[96 + 64 * x + lane] = L.sa[x][1] * ca; }
            }
            __syncwarp();
            const float val_d = project_row(W_s, srow, lane);
            if (lane < kAtHd) A.val[(e * H + h) * kAtHd + lane] = val_d;
            __syncwarp();
            const float s = qk + zv;
            const float mn = fmaxf(m, s);
            const float sc = __expf(m - mn), p = __expf(s - mn);
            const float f = p * inv;
            l = fmaf(l, sc, p);
            V = fmaf(V, sc, p * (vd + val_d));
            {
                const f32x2 sc2 = pack2(sc, sc), f2 = pack2(f, f);
                Sp[0] = fma2(Sp[0], sc2, mul2(f2, pack2(L.sd[0], L.sd[1])));
                Tq[0] = fma2(Tq[0], sc2, mul2(f2, pack2(L.qd[0], L.qd[1])));
#pragma unroll
                for (int x = 0; x < 3; x++) {
                    Sp[32 + 32 * x] = fma2(Sp[32 + 32 * x], sc2, mul2(f2, pack2(L.sa[x][0], L.sa[x][1])));
                    Tq[32 + 32 * x] = fma2(Tq[32 + 32 * x], sc2, mul2(f2, pack2(L.qa[x][0], L.qa[x][1])));
                }
            }
            m = mn;
        }
        const float inv_l = T.e1 > T.e0 ? 1.0f / l : 0.f;
        const bool partial = TASKS && row >= A.N;
        if (partial) row -= A.N;
        if (lane == 0) (partial ? A.part_lse : A.lse)[row * H + h] = m + logf(l);
        float* sp = (partial ? A.part_spool : A.spool) + (row * H + h) * kAtK;
        {
            float s0, s1, t0, t1;
            unpack2(Sp[0], s0, s1); unpack2(Tq[0], t0, t1);
            sp[lane] = s0 * inv_l; sp[32 + lane] = s1 * inv_l;
            srow[lane] = t0 * inv_l * P.c_dist; srow[32 + lane] = t1 * inv_l * P.c_dist;
#pragma unroll
            for (int x = 0; x < 3; x++) {
                unpack2(Sp[32 + 32 * x], s0, s1); unpack2(Tq[32 + 32 * x], t0, t1);
                sp[64 + 64 * x + lane] = s0 * inv_l * P.c_ang; sp[96 + 64 * x + lane] = s1 * inv_l * P.c_ang;
                srow[64 + 64 * x + lane] = t0 * inv_l * P.c_ang; srow[96 + 64 * x + lane] = t1 * inv_l * P.c_ang;
            }
        }
        __syncwarp();
        const float up_d = project_row(W_s, srow, lane);     // W (pooled d^2-weighted sums)
        if (lane < kAtHd) {
            (partial ? A.part_out : A.out)[(row * H + h) * kAtHd + lane] = V * inv_l;
            (partial ? A.part_upool : A.upool)[(row * H + h) * kAtHd + lane] = up_d;
        }
        __syncwarp();
    }
    }   // heads in turn
}

// Backward pass from the results of the training forward: warp = (atom, head), lane = pair (32 at a time).  Per pair
//   p = exp(q.k + z - lse),  gz = p (gout . (v_j + values_ij) - gout . out_i),
//   ga += c_dist x gz - p x gout . values_ij,  gq += gz k_j;   and ga += gout . upool once per atom
// (the coefficient gradient of attn_bwd_kernel, reference quirk included).  The 16-component dot products run inside
// the lanes; the 17 per-atom sums are reduced over the lanes once at the end, in a fixed order.
__global__ void __launch_bounds__(256) attn_bwd_saved_kernel(const AtArgs A, const Params P)
{
    const int lane = threadIdx.x & 31, H = P.H;
    const int64_t task = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (task >= A.N * H) return;
    const int64_t i = task / H;
    const int h = (int)(task - i * H);
    float q[kAtHd], g[kAtHd], gq[kAtHd];
    float D = 0.f, gup = 0.f;
    {
        const float4* q4 = reinterpret_cast<const float4*>(A.qs + (i * H + h) * kAtHd);
        const float4* g4 = reinterpret_cast<const float4*>(A.gout + (i * H + h) * kAtHd);
        const float4* o4 = reinterpret_cast<const float4*>(A.out + (i * H + h) * kAtHd);
        const float4* u4 = reinterpret_cast<const float4*>(A.upool + (i * H + h) * kAtHd);
#pragma unroll
        for (int c = 0; c < kAtHd / 4; c++) {
            const float4 a = __ldg(q4 + c), b = __ldg(g4 + c), o = __ldg(o4 + c), u = __ldg(u4 + c);
            q[4 * c] = a.x; q[4 * c + 1] = a.y; q[4 * c + 2] = a.z; q[4 * c + 3] = a.w;
            g[4 * c] = b.x; g[4 * c + 1] = b.y; g[4 * c + 2] = b.z; g[4 * c + 3] = b.w;
            D = fmaf(b.x, o.x, fmaf(b.y, o.y, fmaf(b.z, o.z, fmaf(b.w, o.w, D))));
            gup = fmaf(b.x, u.x, fmaf(b.y, u.y, fmaf(b.z, u.z, fmaf(b.w, u.w, gup))));
        }
#pragma unroll
        for (int c = 0; c < kAtHd; c++) gq[c] = 0.f;
    }
    const float lse = __ldg(A.lse + i * H + h);
    const int64_t e0 = A.e_start[i], e1 = A.e_start[i + 1];
    const int64_t j0 = e1 > e0 ? A.edges[A.E + e0] : 0;
    float ga = 0.f;
    for (int64_t e = e0 + lane; e < e1; e += 32) {
        const int64_t j = j0 + (e - e0);
        const float4* k4 = reinterpret_cast<const float4*>(A.k + (j * H + h) * kAtHd);
        const float4* v4 = reinterpret_cast<const float4*>(A.v + (j * H + h) * kAtHd);
        const float4* x4 = reinterpret_cast<const float4*>(A.val + (e * H + h) * kAtHd);
        const float zin = __ldg(A.z_in + e * H + h), px = __ldg(A.px + e * H + h);
        float kk[kAtHd];
        float qk = 0.f, gov = 0.f, cB = 0.f;
#pragma unroll
        for (int c = 0; c < kAtHd / 4; c++) {
            const float4 a = __ldg(k4 + c), b = __ldg(v4 + c), x = __ldg(x4 + c);
            kk[4 * c] = a.x; kk[4 * c + 1] = a.y; kk[4 * c + 2] = a.z; kk[4 * c + 3] = a.w;
            qk = fmaf(q[4 * c], a.x, fmaf(q[4 * c + 1], a.y, fmaf(q[4 * c + 2], a.z, fmaf(q[4 * c + 3], a.w, qk))));
            gov = fmaf(g[4 * c], b.x, fmaf(g[4 * c + 1], b.y, fmaf(g[4 * c + 2], b.z, fmaf(g[4 * c + 3], b.w, gov))));
            cB = fmaf(g[4 * c], x.x, fmaf(g[4 * c + 1], x.y, fmaf(g[4 * c + 2], x.z, fmaf(g[4 * c + 3], x.w, cB))));
        }
        const float p_att = __expf(qk + zin - lse);
        const float gzv = p_att * (gov + cB - D);
        A.gz[e * H + h] = gzv;
        ga += px * fmaf(P.c_dist, gzv, -p_att * cB);
#pragma unroll
        for (int c = 0; c < kAtHd; c++) gq[c] = fmaf(gzv, kk[c], gq[c]);
    }
    // the lanes' sums, one butterfly per value (fixed order)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ga += __shfl_xor_sync(0xffffffffu, ga, o);
#pragma unroll
        for (int c = 0; c < kAtHd; c++) gq[c] += __shfl_xor_sync(0xffffffffu, gq[c], o);
    }
    if (lane == 0) A.ga[i * H + h] = ga + gup;
    if (lane == 0) {
        float4* o4 = reinterpret_cast<float4*>(A.gq + (i * H + h) * kAtHd);
#pragma unroll
        for (int c = 0; c < kAtHd / 4; c++) o4[c] = make_float4(gq[4 * c], gq[4 * c + 1], gq[4 * c + 2], gq[4 * c + 3]);
    }
}

template <bool ANG, bool TASKS>
__global__ void __launch_bounds__(at_warps(true) * 32, kAtBwdBlocks) attn_bwd_kernel(const AtArgs A, const Params P)
{
    extern __shared__ __align__(16) float smem[];
    float* W_s = smem;                                      // [256][20]: W transposed
    float* tbuf = W_s + kAtK * kAtWtStride;                 // per warp 8 x 32
    float* rows = tbuf + at_warps(true) * 8 * 32;           // per warp 32: gout of the atom
    const int h = blockIdx.y, H = P.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int idx = threadIdx.x; idx < kAtHd * kAtK / 4; idx += at_warps(true) * 32) {
        const int o = idx >> 6, k4 = idx & 63, b = k4 >> 4, d4 = k4 & 15;
        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
        const int width = b == 0 ? 64 : P.angle_dim;          // columns this basis' weights hold (zero beyond)
        if (A.W[b] != nullptr && 4 * d4 < width) w = __ldg(reinterpret_cast<const float4*>(A.W[b] + ((size_t)h * kAtHd + o) * width) + d4);
        const int k = k4 * 4;
        W_s[(k + 0) * kAtWtStride + o] = w.x; W_s[(k + 1) * kAtWtStride + o] = w.y;
        W_s[(k + 2) * kAtWtStride + o] = w.z; W_s[(k + 3) * kAtWtStride + o] = w.w;
    }
    LatticeLane<1, ANG> L;
    L.init(P, lane, tbuf + warp * 8 * 32);
    float* grow = rows + warp * 32;
    __syncthreads();
    const int first = TASKS ? kSplitSlots - __ldg(A.chunk_count + h) : 0;

    for (;;) {
        const int64_t t = next_task(A.counters + h, lane) + first;
        if (t >= (TASKS ? A.n_entries : A.N)) break;
        int64_t i, row;
        AtomTask T;
        if (TASKS) {
            const int4 d = __ldg(A.tasks + (size_t)h * A.n_entries + t);
            const int cnt = d.w & 0xFFFFFF;
            if (cnt == 0) continue;
            i = d.x; row = d.y;
            T = load_atom<1, ANG>(A, P, L, i, h, lane);
            T.e0 += d.z; T.e1 = T.e0 + cnt;
        } else {
            i = A.order != nullptr ? (int64_t)A.order[t] : t;
            row = i;
            T = load_atom<1, ANG>(A, P, L, i, h, lane);
        }
        float qd = 0.f, god = 0.f, od = 0.f;
        if (lane < kAtHd) {
            qd = __ldg(A.qs + (i * H + h) * kAtHd + lane);
            god = __ldg(A.gout + (i * H + h) * kAtHd + lane);
            od = __ldg(A.out + (i * H + h) * kAtHd + lane);
        }
        const float D = warp_sum(god * od);
        const float lse = __ldg(A.lse + i * H + h);
        // G = W^T gout restricted to this lane's eight basis indices
        grow[lane] = god;
        __syncwarp();
        float G[8];
        {
            float gvr[kAtHd];
            const float4* g4 = reinterpret_cast<const float4*>(grow);
#pragma unroll
            for (int o4 = 0; o4 < kAtHd / 4; o4++) {
                const float4 u = g4[o4];
                gvr[4 * o4] = u.x; gvr[4 * o4 + 1] = u.y; gvr[4 * o4 + 2] = u.z; gvr[4 * o4 + 3] = u.w;
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float4* wrow = reinterpret_cast<const float4*>(W_s + (j * 32 + lane) * kAtWtStride);
                float acc = 0.f;
#pragma unroll
                for (int o4 = 0; o4 < kAtHd / 4; o4++) {
                    const float4 u = wrow[o4];
                    acc = fmaf(u.x, gvr[4 * o4], fmaf(u.y, gvr[4 * o4 + 1], fmaf(u.z, gvr[4 * o4 + 2], fmaf(u.w, gvr[4 * o4 + 3], acc))));
                }
                G[j] = acc;
            }
        }
        __syncwarp();
        float gq = 0.f, ga_acc = 0.f;
        const int64_t j0 = A.edges[A.E + T.e0];
        float z_next = __ldg(A.z_in + T.e0 * H + h);
        for (int64_t e = T.e0; e < T.e1; e++) {
            const int64_t j = j0 + (e - T.e0);
            float kd = 0.f, vd = 0.f;
            if (lane < kAtHd) { kd = __ldg(A.k + (j * H + h) * kAtHd + lane); vd = __ldg(A.v + (j * H + h) * kAtHd + lane); }
            const float zin = z_next;
            if (e + 1 < T.e1) z_next = __ldg(A.z_in + (e + 1) * H + h);      // requested one pair ahead
            L.ref = zin;
            run_pair<1, ANG>(A, P, L, T, e);
            // one butterfly for the five warp-wide sums of this pair; the four dot products of G with the
            // basis sums enter the results only through two combinations
            float r0 = qd * kd, r1 = god * vd, r2 = L.px_l;
            float Ad = fmaf(G[0], L.qd[0], G[1] * L.qd[1]), Bd = fmaf(G[0], L.sd[0], G[1] * L.sd[1]);
            float Aa = 0.f, Ba = 0.f;
#pragma unroll
            for (int x = 0; x < 3; x++) {
                Aa = fmaf(G[2 + 2 * x], L.qa[x][0], fmaf(G[3 + 2 * x], L.qa[x][1], Aa));
                Ba = fmaf(G[2 + 2 * x], L.sa[x][0], fmaf(G[3 + 2 * x], L.sa[x][1], Ba));
            }
            float r3 = fmaf(P.c_dist, Ad, P.c_ang * Aa), r4 = fmaf(P.c_dist, Bd, P.c_ang * Ba);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                r0 += __shfl_xor_sync(0xffffffffu, r0, o); r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                r2 += __shfl_xor_sync(0xffffffffu, r2, o); r3 += __shfl_xor_sync(0xffffffffu, r3, o);
                r4 += __shfl_xor_sync(0xffffffffu, r4, o);
            }
            const float qk = r0, gov = r1, px = r2, cA = r3, cB = r4;
            const float p_att = __expf(qk + zin - lse);
            // gradient with respect to the logit bias: p (gout . (v_j + values_ij) - gout . out_i), where
            // gout . values_ij = c_dist G_d . s_d + c_ang G_a . s_a = cB
            const float gzv = p_att * (gov + cB - D);
            if (lane == 0) A.gz[e * H + h] = gzv;
            // coefficient gradient; the upstream gradient of the pair's values is p gout, so its W^T image is p G:
            //   c_dist [px gz + p (Ad - px Bd)] + c_ang [p (Aa - px Ba)] = c_dist px gz + p (cA - px cB).
            // The reference scales the whole length-kernel result, gz term included, by the distance coefficient
            // (models/cuda_funcs/real_space_framed_proj.py:183).
            ga_acc += fmaf(P.c_dist * px, gzv, p_att * (cA - px * cB));
            gq = fmaf(gzv, kd, gq);
        }
        const bool partial = TASKS && row >= A.N;
        if (partial) row -= A.N;
        if (lane == 0) (partial ? A.part_ga : A.ga)[row * H + h] = ga_acc;
        if (lane < kAtHd) (partial ? A.part_gq : A.gq)[(row * H + h) * kAtHd + lane] = gq;
    }
}

static int at_grid_x(int64_t N, int H, bool bwd)
{
    const int sms = sm_count();
    int64_t want = ((int64_t)sms * (bwd ? kAtBwdBlocks : kAtFwdBlocks)) / H;
    if (want < 1) want = 1;
    const int64_t need = (N + at_warps(bwd) - 1) / at_warps(bwd);
    if (need < want) want = need < 1 ? 1 : need;
    return (int)want;
}

// thread = (queue entry, head): the task table.  Entry (x, y, z, w) = atom, result row (the atom, or N + partial row of
// a chunk), offset of the first pair within the atom's pairs, pairs | chunks in use << 24 | (chunk == 1) << 28;
// w = 0: nothing to do.  split: the chunked queue of atom_order_kernel (chunks 1.. in the first kSplitSlots entries,
// then the atoms).
__global__ void __launch_bounds__(256) attn_plan_kernel(const int32_t* __restrict__ order, const int32_t* __restrict__ split,
                                                        const float* __restrict__ a_ik, const int64_t* __restrict__ e_start,
                                                        int64_t N, int64_t n_entries, int H, int* __restrict__ chunk_count,
                                                        int4* __restrict__ tasks)
{
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y;
    if (t >= n_entries) return;
    int4 d = make_int4(0, 0, 0, 0);
    const int info = __ldg(split + 4 + 2 * t);
    if (info != 0) {
        const int i = __ldg(order + t);
        const int chunks = (info >> 4) & 15, index = info & 15;
        const int pairs = (int)(e_start[i + 1] - e_start[i]);
        int active = 1;
        if (chunks > 1)
            active = split_active_chunks(__ldg(a_ik + (int64_t)i * H + h), pairs, __int_as_float(__ldg(split + 4 + 2 * t + 1)),
                                         __int_as_float(__ldg(split + 1)), chunks);
        if (index < active && pairs > 0) {
            const int lo = pairs * index / active, hi = pairs * (index + 1) / active;
            d.x = i;
            d.y = active > 1 ? (int)N + (info >> 8) + index : i;
            d.z = lo;
            d.w = (hi - lo) | (active << 24) | ((index == 1 ? 1 : 0) << 28);
        }
    }
    if (t >= kSplitSlots) {
        tasks[(size_t)h * n_entries + t] = d;                    // an atom's entry keeps its place
    } else if (d.w != 0) {
        // chunk entries in use gather at the end of the chunk region, in any order (they are all about one target long)
        const int pos = atomicAdd(chunk_count + h, 1);
        tasks[(size_t)h * n_entries + (kSplitSlots - 1 - pos)] = d;
    }
}

// warp = (entry of the queue's chunk region, head): where the entry is chunk 1 of a task (so the task was cut), the
// chunks' results are combined in chunk order.  Forward: chunk c holds the attention output, pooled basis and
// log-sum-exp over its own pairs; the whole is their average weighted by exp(lse_c - lse).
__global__ void __launch_bounds__(256) attn_merge_fwd_kernel(const AtArgs A, const int H)
{
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int h = blockIdx.y;
    if (t >= kSplitSlots || t < kSplitSlots - __ldg(A.chunk_count + h)) return;
    const int4 d = __ldg(A.tasks + (size_t)h * A.n_entries + t);
    const int active = (d.w >> 24) & 15;
    if (!((d.w >> 28) & 1)) return;
    const int64_t i = d.x, r0 = d.y - A.N - 1;
    float m = -INFINITY;
    for (int c = 0; c < active; c++) m = fmaxf(m, __ldg(A.part_lse + (r0 + c) * H + h));
    float wsum = 0.f;
    for (int c = 0; c < active; c++) wsum += __expf(__ldg(A.part_lse + (r0 + c) * H + h) - m);
    float o = 0.f, s[8];
#pragma unroll
    for (int r = 0; r < 8; r++) s[r] = 0.f;
    for (int c = 0; c < active; c++) {
        const float w = __expf(__ldg(A.part_lse + (r0 + c) * H + h) - m) / wsum;
        if (lane < kAtHd) o = fmaf(w, __ldg(A.part_out + ((r0 + c) * H + h) * kAtHd + lane), o);
        const float* sp = A.part_spool + ((r0 + c) * H + h) * kAtK;
#pragma unroll
        for (int r = 0; r < 8; r++) s[r] = fmaf(w, __ldg(sp + r * 32 + lane), s[r]);
    }
    if (lane == 0) A.lse[i * H + h] = m + logf(wsum);
    if (lane < kAtHd) A.out[(i * H + h) * kAtHd + lane] = o;
    if (A.upool != nullptr && lane < kAtHd) {
        float u = 0.f;
        for (int c = 0; c < active; c++)
            u = fmaf(__expf(__ldg(A.part_lse + (r0 + c) * H + h) - m) / wsum, __ldg(A.part_upool + ((r0 + c) * H + h) * kAtHd + lane), u);
        A.upool[(i * H + h) * kAtHd + lane] = u;
    }
#pragma unroll
    for (int r = 0; r < 8; r++) A.spool[(i * H + h) * kAtK + r * 32 + lane] = s[r];
}

// Backward: the chunks' parts of the query gradient and of the coefficient gradient are summed in chunk order.
__global__ void __launch_bounds__(256) attn_merge_bwd_kernel(const AtArgs A, const int H)
{
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int h = blockIdx.y;
    if (t >= kSplitSlots || t < kSplitSlots - __ldg(A.chunk_count + h)) return;
    const int4 d = __ldg(A.tasks + (size_t)h * A.n_entries + t);
    const int active = (d.w >> 24) & 15;
    if (!((d.w >> 28) & 1)) return;
    const int64_t i = d.x, r0 = d.y - A.N - 1;
    float gq = 0.f, ga = 0.f;
    for (int c = 0; c < active; c++) {
        if (lane < kAtHd) gq += __ldg(A.part_gq + ((r0 + c) * H + h) * kAtHd + lane);
        ga += __ldg(A.part_ga + (r0 + c) * H + h);
    }
    if (lane == 0) A.ga[i * H + h] = ga;
    if (lane < kAtHd) A.gq[(i * H + h) * kAtHd + lane] = gq;
}

template <bool BWD, bool ANG, bool TASKS>
static int launch_at(const AtArgs& A, const Params& P, cudaStream_t st)
{
    auto kern = BWD ? (void (*)(const AtArgs, const Params))attn_bwd_kernel<ANG, TASKS>
                    : (void (*)(const AtArgs, const Params))attn_fwd_kernel<ANG, TASKS>;
    static std::atomic<bool> attr_done[64];   // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)at_smem_bytes(BWD)) != cudaSuccess)
            return CFB200_E_CUDA;
        attr_done[dev & 63] = true;
    }
    kern<<<dim3(at_grid_x(A.N, P.H, BWD), P.H), at_warps(BWD) * 32, at_smem_bytes(BWD), st>>>(A, P);
    if (TASKS) {
        const dim3 grid(kSplitSlots / 8, P.H);
        if (BWD) attn_merge_bwd_kernel<<<grid, 256, 0, st>>>(A, P.H);
        else attn_merge_fwd_kernel<<<grid, 256, 0, st>>>(A, P.H);
    }
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

// the task table of one layer (both directions use it)
int attn_plan(const int32_t* order, const int32_t* split, const float* a_ik, const int64_t* e_start, int64_t N,
              int64_t n_entries, int H, int* chunk_count, int4* tasks, cudaStream_t st)
{
    if (n_entries <= 0) return CFB200_OK;
    if (cudaMemsetAsync(chunk_count, 0, sizeof(int) * H, st) != cudaSuccess) return CFB200_E_CUDA;
    attn_plan_kernel<<<dim3((unsigned)((n_entries + 255) / 256), H), 256, 0, st>>>(order, split, a_ik, e_start, N, n_entries, H,
                                                                                  chunk_count, tasks);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

template <bool ANG, bool TASKS>
static int launch_train(const AtArgs& A, const Params& P, cudaStream_t st)
{
    auto kern = attn_fwd_train_kernel<ANG, TASKS>;
    static std::atomic<bool> attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAtTrainSmem) != cudaSuccess) return CFB200_E_CUDA;
        attr_done[dev & 63] = true;
    }
    kern<<<dim3(at_grid_x(A.N, P.H, true), P.H), kAtTrainWarps * 32, kAtTrainSmem, st>>>(A, P);
    if (TASKS) attn_merge_fwd_kernel<<<dim3(kSplitSlots / 8, P.H), 256, 0, st>>>(A, P.H);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

// A.val set: the training forward (per-pair results for attn_fused_bwd).
int attn_fused_fwd(const AtArgs& A, const Params& P, cudaStream_t st)
{
    if (A.N == 0) return CFB200_OK;
    if (cudaMemsetAsync(A.counters, 0, sizeof(int) * P.H, st) != cudaSuccess) return CFB200_E_CUDA;
    const bool ang = A.W[1] != nullptr;
    if (A.val != nullptr) {
        if (A.tasks != nullptr) return ang ? launch_train<true, true>(A, P, st) : launch_train<false, true>(A, P, st);
        return ang ? launch_train<true, false>(A, P, st) : launch_train<false, false>(A, P, st);
    }
    if (A.tasks != nullptr) return ang ? launch_at<false, true, true>(A, P, st) : launch_at<false, false, true>(A, P, st);
    return ang ? launch_at<false, true, false>(A, P, st) : launch_at<false, false, false>(A, P, st);
}

// A.val set: from the per-pair results of the training forward; else by recomputing the lattice sums.
int attn_fused_bwd(const AtArgs& A, const Params& P, cudaStream_t st)
{
    if (A.N == 0) return CFB200_OK;
    if (A.val != nullptr) {
        const int64_t tasks = A.N * P.H;
        attn_bwd_saved_kernel<<<(unsigned)((tasks + 7) / 8), 256, 0, st>>>(A, P);
        return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
    }
    if (cudaMemsetAsync(A.counters, 0, sizeof(int) * P.H, st) != cudaSuccess) return CFB200_E_CUDA;
    const bool ang = A.W[1] != nullptr;
    if (A.tasks != nullptr) return ang ? launch_at<true, true, true>(A, P, st) : launch_at<true, false, true>(A, P, st);
    return ang ? launch_at<true, true, false>(A, P, st) : launch_at<true, false, false>(A, P, st);
}

}  // namespace cfb
