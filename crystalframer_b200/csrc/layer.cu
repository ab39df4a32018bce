// Whole-batch preparation and whole-layer entry points: every kernel of an encoder layer's forward
// (or backward) pass is enqueued by ONE host call.
//
// The reference runs a layer as ~35 framework operations plus its CuPy Functions
// (models/indexed_latticeformer_encoder.py:848-890, models/indexed_lattice_multi_head_attention_cuda.py:737-996)
// and prepares a batch with ~60 more (models/indexed_latticeformer_encoder.py:15-32, :175-245).  At a few
// thousand atoms per batch each of those operations is microseconds of GPU work, so the step time was set by
// the host's dispatch cost.  Here the host makes one call per layer and direction and one per batch.
//
// This file is included at the end of api.cu (it uses make_params and the kernel files above it).

namespace cfb {

// ---- per-crystal cell quantities ------------------------------------------------------------------------
// thread = crystal: reciprocal vectors 2 pi (b x c, c x a, a x b) / det, their lengths, the cell volume, and
// the work-queue key of the crystal's atoms, an instruction estimate of one (atom, head) task of the attention
// kernels: size x (cost of a pair + cost of a translation x translations in reach of a Gaussian of typical width,
// about a sphere of radius 8 A over the cell volume, between 1 and 125).
// (models/indexed_latticeformer_encoder.py:205-222, models/indexed_lattice_multi_head_attention_cuda.py:539.)
__global__ void __launch_bounds__(128) cell_kernel(const float* __restrict__ tvecs, const int64_t* __restrict__ sizes, int64_t B,
                                                   float* __restrict__ rvecs, float* __restrict__ rvlen,
                                                   float* __restrict__ vcell, float* __restrict__ key,
                                                   float* __restrict__ inv_vol)
{
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= B) return;
    float m[9];
#pragma unroll
    for (int i = 0; i < 9; i++) m[i] = __ldg(tvecs + 9 * c + i);
    // determinant, term by term with separate roundings (the reference forms it with elementwise tensor operations)
    float det = __fmul_rn(__fmul_rn(m[0], m[4]), m[8]);
    det = __fadd_rn(det, __fmul_rn(__fmul_rn(m[1], m[5]), m[6]));
    det = __fadd_rn(det, __fmul_rn(__fmul_rn(m[2], m[3]), m[7]));
    det = __fsub_rn(det, __fmul_rn(__fmul_rn(m[2], m[4]), m[6]));
    det = __fsub_rn(det, __fmul_rn(__fmul_rn(m[0], m[5]), m[7]));
    det = __fsub_rn(det, __fmul_rn(__fmul_rn(m[1], m[3]), m[8]));
    const float s = __fdiv_rn(2.0f * kPiF, det);
    const float* r[3] = {m, m + 3, m + 6};
#pragma unroll
    for (int d = 0; d < 3; d++) {
        const float* u = r[(d + 1) % 3];
        const float* w = r[(d + 2) % 3];
        const float x = __fmul_rn(__fsub_rn(__fmul_rn(u[1], w[2]), __fmul_rn(u[2], w[1])), s);
        const float y = __fmul_rn(__fsub_rn(__fmul_rn(u[2], w[0]), __fmul_rn(u[0], w[2])), s);
        const float z = __fmul_rn(__fsub_rn(__fmul_rn(u[0], w[1]), __fmul_rn(u[1], w[0])), s);
        if (rvecs != nullptr) { rvecs[9 * c + 3 * d] = x; rvecs[9 * c + 3 * d + 1] = y; rvecs[9 * c + 3 * d + 2] = z; }
        rvlen[3 * c + d] = __fsqrt_rn(__fadd_rn(__fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)), __fmul_rn(z, z)));
    }
    if (vcell != nullptr) vcell[c] = det;
    const float vol = fmaxf(fabsf(det), 1e-6f);
    const float survivors = fminf(fmaxf(2145.0f / vol, 1.0f), 125.0f);
    key[c] = (float)sizes[c] * (kAtPairCost + kAtTermCost * survivors);
    if (inv_vol != nullptr) inv_vol[c] = 1.0f / vol;
}

// thread = pair: separation of the pair's atoms in the home cell
__global__ void __launch_bounds__(256) pos_ij_kernel(const float* __restrict__ pos, const int64_t* __restrict__ edges, int64_t E,
                                                     float* __restrict__ pos_ij)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const int64_t i = edges[e], j = edges[E + e];
#pragma unroll
    for (int d = 0; d < 3; d++) pos_ij[3 * e + d] = __fsub_rn(__ldg(pos + 3 * j + d), __ldg(pos + 3 * i + d));
}

// exclusive scan of v over the block's threads (blockDim.x a multiple of 32, at most 1024); returns the value
// before this thread's and leaves the block's total in *total (shared).  tmp: 32 shared ints.
__device__ __forceinline__ int block_scan_exclusive(const int v, int* tmp, int* total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, s, o); if (lane >= o) s += t; }
    if (lane == 31) tmp[warp] = s;
    __syncthreads();
    if (warp == 0) {
        int w = lane < (int)(blockDim.x >> 5) ? tmp[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += t; }
        tmp[lane] = w;
    }
    __syncthreads();
    const int out = (warp ? tmp[warp - 1] : 0) + s - v;
    if (threadIdx.x == blockDim.x - 1) *total = out + v;
    __syncthreads();
    return out;
}

// One block: the work queue of the attention kernels -- crystals by decreasing key (equal keys in index
// order, ranked by counting), the atoms of a crystal in their own order.
//
// Without ``split``, ``order`` holds the N atoms.  With it the queue also cuts long tasks into chunks (see
// attn_fused.cu): a crystal whose atoms may be expensive (cost of an atom for a Gaussian two standard deviations
// wider than typical, against ``target`` = half the average load per warp at typical width) gets ``want`` chunks
// per atom and want partial rows per atom.  Queue layout: kSplitSlots entries for the chunks 1 .. want-1 (heaviest
// crystal first; the unused rest empty), then the N atoms, whose entries stand for chunk 0 or for the whole task.
// How many chunks an (atom, head) really uses is decided per layer from its own coefficient (attn_plan_kernel).
// split (int32): [0] chunk entries in use, [1] bits of target, [2] partial rows in use, [3] 0; then
// (info, bits of 1/volume) per queue entry, info = chunk | chunks << 4 | first partial row << 8 (0: empty entry).
__global__ void __launch_bounds__(1024) atom_order_kernel(const float* __restrict__ key, const float* __restrict__ inv_vol,
                                                          const int64_t* __restrict__ sizes,
                                                          const int64_t* __restrict__ crystal_start, int64_t B, int64_t N,
                                                          int workers, int32_t* __restrict__ by_rank,
                                                          int32_t* __restrict__ start_of, int32_t* __restrict__ want_of,
                                                          int32_t* __restrict__ slot_of, int32_t* __restrict__ order,
                                                          int32_t* __restrict__ split)
{
    __shared__ int tmp[32];
    __shared__ int total;
    __shared__ float red[32];
    __shared__ float target_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float load = 0.f;                                           // sum over atoms of their key
    for (int64_t c = threadIdx.x; c < B; c += blockDim.x) {
        const float kc = key[c];
        int rank = 0;
        for (int64_t o = 0; o < B; o++) {
            const float ko = __ldg(key + o);
            rank += (ko > kc || (ko == kc && o < c)) ? 1 : 0;
        }
        by_rank[rank] = (int32_t)c;
        load += kc * (float)sizes[c];
    }
    load = warp_sum(load);
    if (lane == 0) red[warp] = load;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];          // fixed order
        target_s = fmaxf(0.5f * t / (float)max(workers, 1), kSplitMinTarget);
    }
    __syncthreads();
    const float target = target_s;
    const int base_atoms = split != nullptr ? kSplitSlots : 0;  // where the atoms' entries begin
    // chunks wanted per crystal and its partial rows, in rank order; crystals that find no rows left stay whole
    int carry = 0, used = 0;
    for (int64_t base = 0; base < B; base += blockDim.x) {
        const int64_t r = base + threadIdx.x;
        int want = 1, n = 0;
        if (r < B && split != nullptr) {
            const int c = by_rank[r];
            n = (int)sizes[c];
            const float wide = fminf(kSplitWideSphere * __ldg(inv_vol + c), kSplitWideCap);
            const float heavy = (float)n * (kAtPairCost + kAtTermCost * fmaxf(wide, 1.0f));
            want = (int)ceilf(heavy / target);
            want = max(1, min(want, min(kSplitMaxChunks, n / kSplitMinPairs)));
        }
        const int cnt = want > 1 ? n * want : 0;
        const int off = carry + block_scan_exclusive(cnt, tmp, &total);
        if (r < B) {
            const bool fits = off + cnt <= kSplitSlots;
            want_of[r] = fits ? want : 1;
            slot_of[r] = fits ? off : 0;
            if (fits && cnt > 0) used = max(used, off + cnt);
        }
        carry += total;
        __syncthreads();
    }
    if (split != nullptr) {                                     // partial rows in use: the largest end
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) used = max(used, __shfl_xor_sync(0xffffffffu, used, o));
        if (lane == 0) tmp[warp] = used;
        __syncthreads();
        if (threadIdx.x == 0) {
            int u = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) u = max(u, tmp[w]);
            split[1] = __float_as_int(target); split[2] = u; split[3] = 0;
        }
        __syncthreads();
    }
    // queue positions: every crystal's atoms once, and size x (chunks - 1) entries in the chunk region
    int carry_atoms = 0, carry_chunks = 0;
    for (int64_t base = 0; base < B; base += blockDim.x) {
        const int64_t r = base + threadIdx.x;
        const int n = r < B ? (int)sizes[by_rank[r]] : 0;
        const int extra = r < B ? n * (want_of[r] - 1) : 0;
        const int off = carry_atoms + block_scan_exclusive(n, tmp, &total);
        carry_atoms += total;
        __syncthreads();
        const int off2 = carry_chunks + block_scan_exclusive(extra, tmp, &total);
        carry_chunks += total;
        __syncthreads();
        if (r < B) { start_of[r] = off; want_of[r] |= off2 << 4; }      // chunk-region offset above the count
    }
    if (split != nullptr) {
        if (threadIdx.x == 0) split[0] = carry_chunks;
        for (int x = carry_chunks + threadIdx.x; x < kSplitSlots; x += blockDim.x) {     // the unused chunk entries
            order[x] = 0; split[4 + 2 * x] = 0; split[4 + 2 * x + 1] = 0;
        }
    }
    for (int64_t r = warp; r < B; r += blockDim.x >> 5) {          // warp = crystal, lanes = its entries
        const int c = by_rank[r];
        const int n = (int)sizes[c], a0 = (int)crystal_start[c], o0 = base_atoms + start_of[r];
        const int want = want_of[r] & 15, c0 = want_of[r] >> 4, s0 = slot_of[r];
        const int vbits = split != nullptr ? __float_as_int(__ldg(inv_vol + c)) : 0;
        for (int t = lane; t < n; t += 32) {
            order[o0 + t] = a0 + t;
            if (split != nullptr) {
                split[4 + 2 * (o0 + t)] = (want << 4) | ((want > 1 ? s0 + t * want : 0) << 8);
                split[4 + 2 * (o0 + t) + 1] = vbits;
            }
        }
        for (int x = lane; x < n * (want - 1); x += 32) {          // chunks 1 .. want-1, chunk-major
            const int k = 1 + x / n, t = x - (k - 1) * n;
            order[c0 + x] = a0 + t;
            split[4 + 2 * (c0 + x)] = k | (want << 4) | ((s0 + t * want) << 8);
            split[4 + 2 * (c0 + x) + 1] = vbits;
        }
    }
}

}  // namespace cfb

namespace {

// ---- optional per-stage timing of the one-call entry points (a measurement aid) ----------------------------
// Between cfb200_timing_begin() and cfb200_timing_end() every stage of cfb200_batch_geometry and
// cfb200_encoder_layer_fwd / _bwd is bracketed by CUDA events on the stream it is enqueued on.  Meant for one
// host thread; off by default, and then the entry points create no events.
constexpr int kTmMax = 16384;
bool g_tm_on = false;
int g_tm_n = 0;
cudaEvent_t g_tm_ev[kTmMax][2];
int g_tm_id[kTmMax];

struct TmScope {
    cudaStream_t st; int slot = -1;
    TmScope(int id, cudaStream_t s) : st(s)
    {
        if (!g_tm_on || g_tm_n >= kTmMax) return;
        if (cudaEventCreate(&g_tm_ev[g_tm_n][0]) != cudaSuccess || cudaEventCreate(&g_tm_ev[g_tm_n][1]) != cudaSuccess) return;
        slot = g_tm_n++;
        g_tm_id[slot] = id;
        cudaEventRecord(g_tm_ev[slot][0], st);
    }
    ~TmScope() { if (slot >= 0) cudaEventRecord(g_tm_ev[slot][1], st); }
};

// carves consecutive 256-byte aligned regions out of a scratch buffer
struct Carver {
    char* base; int64_t bytes; int64_t used = 0; bool ok = true;
    Carver(void* p, int64_t n) : base(reinterpret_cast<char*>(p)), bytes(n) {}
    template <typename T> T* take(int64_t count)
    {
        const int64_t need = (count * (int64_t)sizeof(T) + 255) & ~(int64_t)255;
        if (base == nullptr || used + need > bytes) { ok = false; used += need; return nullptr; }
        T* out = reinterpret_cast<T*>(base + used);
        used += need;
        return out;
    }
};

inline int64_t pad256(int64_t b) { return (b + 255) & ~(int64_t)255; }

// A second stream per host thread and device, on which the layer backward runs the weight gradients that are ready
// early beside the attention backward (fork and join by events, so the caller's stream sees one ordered call).
// Created on first use; CFB200_SIDE_STREAM=0 keeps everything on the caller's stream.
struct SideLane { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; bool failed = false; };
thread_local SideLane g_side[64];

SideLane* side_lane()
{
    static const bool enabled = [] { const char* e = getenv("CFB200_SIDE_STREAM"); return !(e && e[0] == '0'); }();
    if (!enabled) return nullptr;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    SideLane& L = g_side[dev];
    if (L.failed) return nullptr;
    if (L.stream == nullptr) {
        if (cudaStreamCreateWithFlags(&L.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&L.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&L.join, cudaEventDisableTiming) != cudaSuccess) {
            L.failed = true;
            L.stream = nullptr;
            return nullptr;
        }
    }
    return &L;
}

// outputs of all weight / bias gradients of one layer (floats), for the partial-sum scratch
int64_t layer_grad_outputs(int D, int F, int H, bool angles)
{
    int64_t n = 0;
    n += (int64_t)D * F + D + 3;          // ff2 + bias (each problem's scratch is rounded to 4 floats)
    n += (int64_t)F * D + F + 3;          // ff1 + bias
    n += (int64_t)D * D + D + 3;          // out projection
    n += 3 * ((int64_t)D * D + D + 3);    // q, k, v
    n += (angles ? 4 : 1) * ((int64_t)H * 16 * 64 + 3);
    return n;
}

int64_t layer_bwd_workspace_bytes(int64_t N, int64_t E, int D, int F, int H, bool angles)
{
    int64_t b = 0;
    b += pad256(N * F * 4);                       // gh
    b += 6 * pad256(N * D * 4);                   // gx1, go, gqs, gk, gv, gq
    b += pad256(N * H * 4) + pad256(E * H * 4);   // ga, gz
    b += pad256(cfb::wgrad_workspace_floats(N, layer_grad_outputs(D, F, H, angles)) * 4);
    b += pad256(D * 4);                           // gradient of lattice_pos before it is added to its destination
    b += pad256((int64_t)cfb::kCoSplits * D * 4);  // its partial sums over slices of the atoms
    b += pad256((int64_t)cfb::kSplitSlots * H * cfb::kSplitPartBwd * 4);   // partial results of chunked attention tasks
    return b;
}

}  // namespace

extern "C" {

int64_t cfb200_batch_geometry_workspace_bytes(int64_t B) { return B < 0 ? -1 : pad256(B * 4) * 6; }

int64_t cfb200_queue_entries(int64_t N) { return N < 0 ? -1 : N + cfb::kSplitSlots; }

int64_t cfb200_split_ints(int64_t N) { return N < 0 ? -1 : 4 + 2 * (N + cfb::kSplitSlots); }

int64_t cfb200_attn_tasks_bytes(int64_t N)
{
    if (!g_configured || N < 0) return -1;
    return (N + cfb::kSplitSlots) * 16 * (int64_t)g_cfg.num_heads + 256;
}

int cfb200_batch_geometry(const float* pos, const float* tvecs, const int64_t* sizes, int64_t B, int64_t N, int64_t E,
                          int range, int64_t* edges, int64_t* e_start, int64_t* batch, int64_t* crystal_start,
                          float* pos_ij, float* rvecs, float* rvlen, float* vcell, float* pair_cache, float* pair_list,
                          int32_t* order, int32_t* split, void* workspace, int64_t workspace_bytes, void* stream)
{
    if (B < 0 || N < 0 || E < 0 || range < 0 || range > CFB200_MAX_RANGE) return CFB200_E_SHAPE;
    if (N > 0x7fffffff) return CFB200_E_TOO_LARGE;
    if (B == 0) return CFB200_OK;
    if (!pos || !tvecs || !sizes || !edges || !e_start || !batch || !crystal_start || !pos_ij || !rvlen || !order)
        return CFB200_E_NULL;
    if (pair_cache != nullptr && (reinterpret_cast<uintptr_t>(pair_cache) & 15u) != 0) return CFB200_E_SHAPE;
    Carver ws(workspace, workspace_bytes);
    float* key = ws.take<float>(B);
    int32_t* by_rank = ws.take<int32_t>(B);
    int32_t* start_of = ws.take<int32_t>(B);
    int32_t* want_of = ws.take<int32_t>(B);
    int32_t* slot_of = ws.take<int32_t>(B);
    float* inv_vol = ws.take<float>(B);
    if (!ws.ok) return CFB200_E_WORKSPACE;
    if (split != nullptr && !g_configured) return CFB200_E_NOT_CONFIGURED;
    if (split != nullptr && B > 0x7ffffff) return CFB200_E_TOO_LARGE;
    cudaStream_t st = S(stream);
    TmScope tm(CFB200_TM_GEOMETRY, st);
    int rc = cfb::edge_index(sizes, B, N, E, edges, e_start, batch, crystal_start, st);
    if (rc != CFB200_OK) return rc;
    cfb::cell_kernel<<<(unsigned)((B + 127) / 128), 128, 0, st>>>(tvecs, sizes, B, rvecs, rvlen, vcell, key, inv_vol);
    if (E > 0) cfb::pos_ij_kernel<<<(unsigned)((E + 255) / 256), 256, 0, st>>>(pos, edges, E, pos_ij);
    // warps that serve one head's queue in the training forward, the launch the chunks are cut for
    const int heads = split != nullptr ? g_cfg.num_heads : 1;
    const int workers = cfb::at_grid_x(N, heads, true) * cfb::kAtTrainWarps;
    cfb::atom_order_kernel<<<1, 1024, 0, st>>>(key, inv_vol, sizes, crystal_start, B, N, workers, by_rank, start_of, want_of,
                                               slot_of, order, split);
    if (cudaGetLastError() != cudaSuccess) return CFB200_E_CUDA;
    if (E > 0 && range > 0 && (pair_cache != nullptr || pair_list != nullptr)) {
        float* list = pair_list;
        if ((2 * range + 1) * (2 * range + 1) * (2 * range + 1) > cfb::kListLen) list = nullptr;
        rc = cfb::pair_cache(pos_ij, tvecs, batch, edges, E, range, pair_cache, list, st);
    }
    return rc;
}

int64_t cfb200_encoder_layer_workspace_bytes(int64_t N, int64_t E, int d_model, int ff_dim, int frame_method)
{
    if (!g_configured || N < 0 || E < 0 || d_model <= 0 || ff_dim <= 0) return -1;
    const int H = g_cfg.num_heads;
    int64_t fwd = frame_method == 2 ? pad256(cfb200_sigma_frames_workspace_bytes(N, E)) : 0;
    // partial results of chunked attention tasks (the frames' scratch is free again by then)
    const int64_t parts = pad256((int64_t)cfb::kSplitSlots * H * cfb::kSplitPartFwd * 4);
    if (parts > fwd) fwd = parts;
    int64_t bwd = layer_bwd_workspace_bytes(N, E, d_model, ff_dim, H, frame_method != 0);
    return fwd > bwd ? fwd : bwd;
}

static int layer_check(const cfb200_layer_desc* L, const cfb200_layer_weights* W, const cfb200_geometry* G)
{
    if (!g_configured) return CFB200_E_NOT_CONFIGURED;
    if (!L || !W || !G) return CFB200_E_NULL;
    const int H = g_cfg.num_heads;
    if (L->d_model != H * g_cfg.head_dim || g_cfg.head_dim != 16 || g_cfg.dist_dim != 64 || L->ff_dim <= 0 || (L->ff_dim & 3))
        return CFB200_E_UNSUPPORTED;
    if (L->frame_method < 0 || L->frame_method > 5) return CFB200_E_UNSUPPORTED;
    if (L->frame_method != 0 && g_cfg.angle_dim == 0) return CFB200_E_UNSUPPORTED;
    if (G->N < 0 || G->E < 0) return CFB200_E_SHAPE;
    if (G->N > 0x7fffffff) return CFB200_E_TOO_LARGE;
    if (!W->q_proj || !W->k_proj || !W->v_proj || !W->in_bias || !W->lattice_pos || !W->out_proj || !W->out_bias ||
        !W->pe_dist || !W->ff1 || !W->ff1_bias || !W->ff2 || !W->ff2_bias)
        return CFB200_E_NULL;
    if (L->frame_method != 0 && !(W->pe_ang1 && W->pe_ang2 && W->pe_ang3)) return CFB200_E_NULL;
    if (G->N > 0 && (!G->pos_ij || !G->tvecs || !G->batch || !G->edges || !G->e_start || !G->counters)) return CFB200_E_NULL;
    if (L->cutoff_radius != 0.0f && G->N > 0 && !G->rvlen) return CFB200_E_NULL;
    return CFB200_OK;
}

static void layer_attn_args(cfb::AtArgs& A, const cfb200_layer_desc* L, const cfb200_layer_weights* W,
                            const cfb200_geometry* G, const cfb200_layer_state* St)
{
    memset(&A, 0, sizeof(A));
    const bool ang = L->frame_method != 0;
    const int64_t fr = G->N * g_cfg.num_heads * 3;
    A.qs = St->q_scaled; A.k = St->k; A.v = St->v; A.a_ik = St->a; A.pos_ij = G->pos_ij; A.tvecs = G->tvecs; A.rvlen = G->rvlen;
    A.batch = G->batch; A.edges = G->edges; A.e_start = G->e_start; A.order = G->order; A.counters = G->counters;
    if (G->split != nullptr && St->tasks == nullptr) {
        A.order = G->order + cfb::kSplitSlots;         // the plain queue: the atoms' entries follow the chunk region
    }
    if (G->split != nullptr && St->tasks != nullptr) {
        // the table's last 256 bytes hold the per-head counts of chunk entries in use
        A.tasks = reinterpret_cast<const int4*>(St->tasks);
        A.n_entries = G->N + cfb::kSplitSlots;
        A.chunk_count = reinterpret_cast<int*>(reinterpret_cast<char*>(St->tasks) + A.n_entries * 16 * g_cfg.num_heads);
    }
    A.N = G->N; A.E = G->E;
    A.W[0] = W->pe_dist;
    if (ang) {
        A.W[1] = W->pe_ang1; A.W[2] = W->pe_ang2; A.W[3] = W->pe_ang3;
        A.frame[0] = St->frames; A.frame[1] = St->frames + fr; A.frame[2] = St->frames + 2 * fr;
    }
    A.list = G->pair_list; A.cache_range = G->cache_range;
    A.val = St->val; A.px = St->px; A.upool = St->upool;
}

int cfb200_encoder_layer_fwd(const cfb200_layer_desc* L, const cfb200_layer_weights* W, const cfb200_geometry* G,
                             const float* x, cfb200_layer_state* St, float* x_out, void* workspace,
                             int64_t workspace_bytes, void* stream)
{
    int rc = layer_check(L, W, G);
    if (rc != CFB200_OK) return rc;
    const int64_t N = G->N, E = G->E;
    if (N == 0) return CFB200_OK;
    if (!x || !x_out || !St) return CFB200_E_NULL;
    if (!St->q || !St->q_scaled || !St->k || !St->v || !St->a || !St->z || !St->spool || !St->attn || !St->lse || !St->x1 || !St->h)
        return CFB200_E_NULL;
    const int H = g_cfg.num_heads, D = L->d_model, F = L->ff_dim;
    const bool ang = L->frame_method != 0;
    if (ang && !St->frames) return CFB200_E_NULL;
    cfb::Params P;
    rc = make_params(L->dist_max, L->cutoff_radius, P, !ang);
    if (rc != CFB200_OK) return rc;
    cudaStream_t st = S(stream);

    // input projections: q, k, v = x W^T + b, one launch
    {
        TmScope tm(CFB200_TM_LINEAR_FWD, st);
        const float* Wqkv[3] = {W->q_proj, W->k_proj, W->v_proj};
        float* qkv[3] = {St->q, St->k, St->v};
        cfb::GemmBatch gb;
        memset(&gb, 0, sizeof(gb));
        gb.n = 3;
        for (int i = 0; i < 3; i++) {
            cfb::GemmArgs& g = gb.g[i];
            g.seg[0] = {x, Wqkv[i], D, D, D}; g.nseg = 1; g.M = (int)N; g.N = D; g.C = qkv[i]; g.ldc = D; g.bias = W->in_bias + i * D;
        }
        if ((rc = cfb::gemm_batch(gb, false, st)) != CFB200_OK) return rc;
    }
    // Gaussian coefficients and the scaled query
    {
        TmScope tm(CFB200_TM_COEF, st);
        cfb::CoefArgs C;
        if ((rc = coef_args(C, St->q, W->lattice_pos, W->gauss_scale, N, L->gauss_lb, L->beta, L->scale_real)) != CFB200_OK) return rc;
        C.a = St->a; C.qs = St->q_scaled;
        if ((rc = cfb::coef_fwd(C, st)) != CFB200_OK) return rc;
    }
    // frames
    const int64_t fr = N * H * 3;
    if (L->frame_method == 1) {
        TmScope tm(CFB200_TM_FRAMES, st);
        rc = frames_common(3, St->q_scaled, St->k, St->a, G->pos_ij, G->tvecs, G->rvlen, G->batch, G->edges, G->e_start, N, E,
                           L->cutoff_radius, L->seed1, L->seed2, nullptr, St->frames, St->frames + fr, St->frames + 2 * fr,
                           nullptr, nullptr, stream, G->pair_cache, G->pair_list, G->cache_range);
    } else if (L->frame_method == 3) {
        TmScope tm(CFB200_TM_FRAMES, st);
        rc = frames_common(3, St->q_scaled, St->k, St->a, G->pos_ij, G->tvecs, G->rvlen, G->batch, G->edges, G->e_start, N, E,
                           L->cutoff_radius, L->seed1, L->seed2, nullptr, St->frames, St->frames + fr, St->frames + 2 * fr,
                           nullptr, nullptr, stream, G->pair_cache, G->pair_list, G->cache_range, 1);
    } else if (L->frame_method == 4) {
        TmScope tm(CFB200_TM_FRAMES, st);
        rc = cfb200_lattice_frames(St->a, G->tvecs, G->rvlen, G->batch, G->edges, G->e_start, N, E, L->cutoff_radius, L->seed1,
                                   L->seed2, L->seed1 ^ L->seed2, St->frames, St->frames + fr, St->frames + 2 * fr, stream);
    } else if (L->frame_method == 5) {
        TmScope tm(CFB200_TM_FRAMES, st);
        rc = cfb200_pca_frames(G->pos_ij, G->e_start, N, E, L->seed1, St->frames, St->frames + fr, St->frames + 2 * fr, stream);
    } else if (L->frame_method == 2) {
        TmScope tm(CFB200_TM_FRAMES, st);
        rc = cfb200_sigma_frames_cached(St->q_scaled, St->k, St->a, G->pos_ij, G->tvecs, G->rvlen, G->batch, G->edges,
                                        G->e_start, N, E, L->cutoff_radius, L->seed1, L->seed2, St->frames, St->frames + fr,
                                        St->frames + 2 * fr, workspace, workspace_bytes, G->pair_list, G->cache_range, stream);
    }
    if (rc != CFB200_OK) return rc;
    // lattice sums, value encoding and attention
    {
        TmScope tm(CFB200_TM_ATTN_FWD, st);
        cfb::AtArgs A;
        layer_attn_args(A, L, W, G, St);
        A.out = St->attn; A.z = St->z; A.lse = St->lse; A.spool = St->spool;
        if (A.tasks != nullptr) {
            const int64_t rows = (int64_t)cfb::kSplitSlots * H;
            if (workspace == nullptr || workspace_bytes < rows * cfb::kSplitPartFwd * 4) return CFB200_E_WORKSPACE;
            if ((reinterpret_cast<uintptr_t>(St->tasks) & 15u) != 0) return CFB200_E_SHAPE;
            A.part_spool = reinterpret_cast<float*>(workspace);
            A.part_out = A.part_spool + rows * 256;
            A.part_lse = A.part_out + rows * 16;
            A.part_upool = A.part_lse + rows;
            // this layer's task table: which entries of the queue this layer's coefficients leave whole, cut or unused
            if ((rc = cfb::attn_plan(G->order, G->split, St->a, G->e_start, N, A.n_entries, H, A.chunk_count,
                                     reinterpret_cast<int4*>(St->tasks), st)) != CFB200_OK)
                return rc;
        }
        if ((rc = cfb::attn_fused_fwd(A, P, st)) != CFB200_OK) return rc;
    }
    // x1 = attn Wo^T + bo + x ; h = relu(x1 Wf1^T + bf1) ; x_out = h Wf2^T + bf2 + x1
    TmScope tm(CFB200_TM_LINEAR_FWD, st);
    cfb::GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.seg[0] = {St->attn, W->out_proj, D, D, D}; g.nseg = 1; g.M = (int)N; g.N = D; g.C = St->x1; g.ldc = D;
    g.bias = W->out_bias; g.resid = x; g.ldr = D;
    if ((rc = cfb::gemm(g, false, st)) != CFB200_OK) return rc;
    memset(&g, 0, sizeof(g));
    g.seg[0] = {St->x1, W->ff1, D, D, D}; g.nseg = 1; g.M = (int)N; g.N = F; g.C = St->h; g.ldc = F; g.bias = W->ff1_bias; g.relu = 1;
    if ((rc = cfb::gemm(g, false, st)) != CFB200_OK) return rc;
    memset(&g, 0, sizeof(g));
    g.seg[0] = {St->h, W->ff2, F, F, F}; g.nseg = 1; g.M = (int)N; g.N = D; g.C = x_out; g.ldc = D;
    g.bias = W->ff2_bias; g.resid = St->x1; g.ldr = D;
    return cfb::gemm(g, false, st);
}

int cfb200_encoder_layer_bwd(const cfb200_layer_desc* L, const cfb200_layer_weights* W, const cfb200_geometry* G,
                             const float* x, const cfb200_layer_state* St, const float* g_out, float* g_x,
                             const cfb200_layer_grads* Gr, int accumulate, void* workspace, int64_t workspace_bytes,
                             void* stream)
{
    int rc = layer_check(L, W, G);
    if (rc != CFB200_OK) return rc;
    const int64_t N = G->N, E = G->E;
    if (!Gr) return CFB200_E_NULL;
    if (N == 0) return CFB200_OK;
    if (!x || !g_out || !g_x || !St) return CFB200_E_NULL;
    const int H = g_cfg.num_heads, D = L->d_model, F = L->ff_dim;
    const bool ang = L->frame_method != 0;
    if (!Gr->q_proj || !Gr->k_proj || !Gr->v_proj || !Gr->in_bias || !Gr->lattice_pos || !Gr->out_proj || !Gr->out_bias ||
        !Gr->pe_dist || !Gr->ff1 || !Gr->ff1_bias || !Gr->ff2 || !Gr->ff2_bias || (ang && !(Gr->pe_ang1 && Gr->pe_ang2 && Gr->pe_ang3)))
        return CFB200_E_NULL;
    cfb::Params P;
    rc = make_params(L->dist_max, L->cutoff_radius, P, !ang);
    if (rc != CFB200_OK) return rc;
    cudaStream_t st = S(stream);
    Carver ws(workspace, workspace_bytes);
    float* gh = ws.take<float>(N * F);
    float* gx1 = ws.take<float>(N * D);
    float* go = ws.take<float>(N * D);
    float* gqs = ws.take<float>(N * D);
    float* gk = ws.take<float>(N * D);
    float* gv = ws.take<float>(N * D);
    float* gq = ws.take<float>(N * D);
    float* ga = ws.take<float>(N * H);
    float* gz = ws.take<float>(E * H);
    const int64_t wg_floats = cfb::wgrad_workspace_floats(N, layer_grad_outputs(D, F, H, ang));
    float* wg = ws.take<float>(wg_floats);
    float* gw_tmp = ws.take<float>(D);
    float* coef_part = ws.take<float>((int64_t)cfb::kCoSplits * D);
    float* split_part = ws.take<float>((int64_t)cfb::kSplitSlots * H * cfb::kSplitPartBwd);
    if (!ws.ok) return CFB200_E_WORKSPACE;

    cfb::GemmArgs g;
    {
    TmScope tm(CFB200_TM_LINEAR_BWD, st);
    // gh = (g_out Wf2) masked by h > 0
    memset(&g, 0, sizeof(g));
    g.seg[0] = {g_out, W->ff2, D, F, D}; g.nseg = 1; g.M = (int)N; g.N = F; g.C = gh; g.ldc = F; g.mask = St->h; g.ldm = F;
    if ((rc = cfb::gemm(g, true, st)) != CFB200_OK) return rc;
    // gx1 = g_out + gh Wf1
    memset(&g, 0, sizeof(g));
    g.seg[0] = {gh, W->ff1, F, D, F}; g.nseg = 1; g.M = (int)N; g.N = D; g.C = gx1; g.ldc = D; g.resid = g_out; g.ldr = D;
    if ((rc = cfb::gemm(g, true, st)) != CFB200_OK) return rc;
    // go = gx1 Wo
    memset(&g, 0, sizeof(g));
    g.seg[0] = {gx1, W->out_proj, D, D, D}; g.nseg = 1; g.M = (int)N; g.N = D; g.C = go; g.ldc = D;
    if ((rc = cfb::gemm(g, true, st)) != CFB200_OK) return rc;
    }
    // Weight and bias gradients whose inputs exist by now (feed-forward, output projection, value-encoding weights:
    // out[P,Q] = A^T B over the atoms) run on the side stream beside the attention backward below.
    const int64_t early_out = ((int64_t)D * F + D + 3) + ((int64_t)F * D + F + 3) + ((int64_t)D * D + D + 3) +
                              (ang ? 4 : 1) * ((int64_t)H * 16 * 64 + 3);
    const int64_t early_floats = (cfb::wgrad_workspace_floats(N, early_out) + 3) & ~(int64_t)3;
    SideLane* lane = side_lane();
    {
        cudaStream_t sw = st;
        if (lane != nullptr) {
            if (cudaEventRecord(lane->fork, st) != cudaSuccess || cudaStreamWaitEvent(lane->stream, lane->fork, 0) != cudaSuccess)
                return CFB200_E_CUDA;
            sw = lane->stream;
        }
        TmScope tm_w(CFB200_TM_WGRAD, sw);
        cfb::WgArgs Wg;
        memset(&Wg, 0, sizeof(Wg));
        Wg.M = (int)N; Wg.ws = wg; Wg.accumulate = accumulate;
        auto add = [&](const float* A, int lda, int Pn, const float* B, int ldb, int Qn, float* out, int ldo, float* bias) {
            cfb::WgProblem& p = Wg.prob[Wg.nprob++];
            p.A = A; p.B = B; p.out = out; p.bias_out = bias; p.lda = lda; p.ldb = ldb; p.ldo = ldo; p.P = Pn; p.Q = Qn; p.nb = 1;
        };
        add(g_out, D, D, St->h, F, F, Gr->ff2, F, Gr->ff2_bias);
        add(gh, F, F, St->x1, D, D, Gr->ff1, D, Gr->ff1_bias);
        add(gx1, D, D, St->attn, D, D, Gr->out_proj, D, Gr->out_bias);
        // value-encoding weights: gW_b[h] (16 x 64) = sum_i go[i,h,:]^T spool[i,h,64b:64b+64]
        float* gpe[4] = {Gr->pe_dist, Gr->pe_ang1, Gr->pe_ang2, Gr->pe_ang3};
        for (int b = 0; b < (ang ? 4 : 1); b++) {
            cfb::WgProblem& p = Wg.prob[Wg.nprob++];
            p.A = go; p.lda = D; p.P = 16; p.sA = 16;
            const int width = b == 0 ? 64 : g_cfg.angle_dim;          // the angle weights are (H,16,angle_dim)
            p.B = St->spool + 64 * b; p.ldb = H * 256; p.Q = width; p.sB = 256;
            p.out = gpe[b]; p.ldo = width; p.sO = 16 * width; p.nb = H; p.bias_out = nullptr;
        }
        if ((rc = cfb::wgrad(Wg, early_floats, sw)) != CFB200_OK) return rc;
        if (lane != nullptr && cudaEventRecord(lane->join, sw) != cudaSuccess) return CFB200_E_CUDA;
    }
    // attention, lattice sums
    {
        cfb::AtArgs A;
        layer_attn_args(A, L, W, G, const_cast<cfb200_layer_state*>(St));
        A.out = St->attn; A.lse = St->lse; A.z_in = St->z; A.gout = go; A.gq = gqs; A.ga = ga; A.gz = gz;
        A.part_gq = split_part; A.part_ga = split_part + (int64_t)cfb::kSplitSlots * H * 16;
        {
            TmScope tm(CFB200_TM_ATTN_BWD, st);
            if ((rc = cfb::attn_fused_bwd(A, P, st)) != CFB200_OK) return rc;
        }
        TmScope tm(CFB200_TM_ATTN_BWD_COLS, st);
        cfb::DpArgs Dp;
        memset(&Dp, 0, sizeof(Dp));
        Dp.q = St->q_scaled; Dp.k = St->k; Dp.v = St->v; Dp.z = St->z; Dp.edges = G->edges; Dp.e_start = G->e_start; Dp.N = N; Dp.E = E;
        Dp.lse = St->lse; Dp.gout = go; Dp.gz = gz; Dp.gk = gk; Dp.gv = gv;
        if ((rc = cfb::dpa_bwd_cols(Dp, P, st)) != CFB200_OK) return rc;
    }
    // Gaussian coefficients: gq = gqs / sqrt(hd) + ga da/dq ; g lattice_pos
    float* gw_lat = accumulate ? gw_tmp : Gr->lattice_pos;
    {
        TmScope tm(CFB200_TM_COEF, st);
        cfb::CoefArgs C;
        if ((rc = coef_args(C, St->q, W->lattice_pos, W->gauss_scale, N, L->gauss_lb, L->beta, L->scale_real)) != CFB200_OK) return rc;
        C.ga = ga; C.gqs = gqs; C.gq = gq; C.gw = gw_lat; C.partial = coef_part;
        if ((rc = cfb::coef_bwd(C, st)) != CFB200_OK) return rc;
    }
    // Weight and bias gradients of the in-projections (their inputs are the last results of the chain above) on the
    // side stream, behind the early group, beside the data-gradient product below.
    {
        cudaStream_t sw = st;
        if (lane != nullptr) {
            if (cudaEventRecord(lane->fork, st) != cudaSuccess || cudaStreamWaitEvent(lane->stream, lane->fork, 0) != cudaSuccess)
                return CFB200_E_CUDA;
            sw = lane->stream;
        }
        TmScope tm_w(CFB200_TM_WGRAD, sw);
        cfb::WgArgs Wg;
        memset(&Wg, 0, sizeof(Wg));
        Wg.M = (int)N; Wg.ws = wg + early_floats; Wg.accumulate = accumulate;
        auto add = [&](const float* A, int lda, int Pn, const float* B, int ldb, int Qn, float* out, int ldo, float* bias) {
            cfb::WgProblem& p = Wg.prob[Wg.nprob++];
            p.A = A; p.B = B; p.out = out; p.bias_out = bias; p.lda = lda; p.ldb = ldb; p.ldo = ldo; p.P = Pn; p.Q = Qn; p.nb = 1;
        };
        add(gq, D, D, x, D, D, Gr->q_proj, D, Gr->in_bias);
        add(gk, D, D, x, D, D, Gr->k_proj, D, Gr->in_bias + D);
        add(gv, D, D, x, D, D, Gr->v_proj, D, Gr->in_bias + 2 * D);
        if ((rc = cfb::wgrad(Wg, wg_floats - early_floats, sw)) != CFB200_OK) return rc;
        // the side stream works in order: this record also stands for the early group
        if (lane != nullptr && cudaEventRecord(lane->join, sw) != cudaSuccess) return CFB200_E_CUDA;
    }
    // g_x = gx1 + gq Wq + gk Wk + gv Wv
    {
        TmScope tm(CFB200_TM_LINEAR_BWD, st);
        memset(&g, 0, sizeof(g));
        g.seg[0] = {gq, W->q_proj, D, D, D}; g.seg[1] = {gk, W->k_proj, D, D, D}; g.seg[2] = {gv, W->v_proj, D, D, D};
        g.nseg = 3; g.M = (int)N; g.N = D; g.C = g_x; g.ldc = D; g.resid = gx1; g.ldr = D;
        if ((rc = cfb::gemm(g, true, st)) != CFB200_OK) return rc;
    }
    // the weight gradients must be complete when this call's work is (the next call reuses the workspace)
    if (lane != nullptr && cudaStreamWaitEvent(st, lane->join, 0) != cudaSuccess) return CFB200_E_CUDA;
    if (accumulate) {
        cfb::axpy_kernel<<<(D + 127) / 128, 128, 0, st>>>(Gr->lattice_pos, gw_tmp, D);
        if (cudaGetLastError() != cudaSuccess) return CFB200_E_CUDA;
    }
    return CFB200_OK;
}

int cfb200_linear(const float* x, const float* weight, const float* bias, const float* residual, int64_t M, int64_t N,
                  int64_t K, int relu, int weight_is_kn, float* y, void* stream)
{
    if (M < 0 || N <= 0 || K <= 0 || M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return CFB200_E_SHAPE;
    if (M == 0) return CFB200_OK;
    if (!x || !weight || !y) return CFB200_E_NULL;
    cfb::GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.seg[0] = {x, weight, (int)K, weight_is_kn ? (int)N : (int)K, (int)K};
    g.nseg = 1; g.M = (int)M; g.N = (int)N; g.C = y; g.ldc = (int)N; g.bias = bias; g.resid = residual; g.ldr = (int)N; g.relu = relu;
    return cfb::gemm(g, weight_is_kn != 0, S(stream));
}

int cfb200_timing_begin(void)
{
    for (int i = 0; i < g_tm_n; i++) { cudaEventDestroy(g_tm_ev[i][0]); cudaEventDestroy(g_tm_ev[i][1]); }
    g_tm_n = 0;
    g_tm_on = true;
    return CFB200_OK;
}

int cfb200_timing_end(float* ms_by_stage, int32_t* calls_by_stage)
{
    g_tm_on = false;
    if (!ms_by_stage || !calls_by_stage) return CFB200_E_NULL;
    for (int i = 0; i < CFB200_TM_STAGES; i++) { ms_by_stage[i] = 0.f; calls_by_stage[i] = 0; }
    int rc = CFB200_OK;
    for (int i = 0; i < g_tm_n; i++) {
        float ms = 0.f;
        if (cudaEventSynchronize(g_tm_ev[i][1]) != cudaSuccess || cudaEventElapsedTime(&ms, g_tm_ev[i][0], g_tm_ev[i][1]) != cudaSuccess)
            rc = CFB200_E_CUDA;
        else { ms_by_stage[g_tm_id[i]] += ms; calls_by_stage[g_tm_id[i]]++; }
        cudaEventDestroy(g_tm_ev[i][0]);
        cudaEventDestroy(g_tm_ev[i][1]);
    }
    g_tm_n = 0;
    return rc;
}

}  // extern "C"
