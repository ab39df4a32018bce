// Pair-list construction, CSR offsets and per-crystal mean pooling (replaces the Python loop of
// get_edge_index, models/indexed_latticeformer_encoder.py:15-32, the scatter_add + cumsum of
// models/cuda_funcs/fused_dpa.py:24-26 and irregular_mean_fwd.cu of the reference).
// All of it is index or streaming work bound by HBM traffic.
#include "common.cuh"

namespace cfb {

// Exclusive scans of sizes and sizes^2 by one block: crystal_start[c] = atoms before crystal c,
// e_start[crystal_start[c]] = pairs before crystal c.
__global__ void __launch_bounds__(1024) crystal_scan_kernel(const int64_t* __restrict__ sizes, int64_t B, int64_t N,
                                                            int64_t E, int64_t* __restrict__ crystal_start,
                                                            int64_t* __restrict__ e_start)
{
    __shared__ long long warp_a[32], warp_p[32];
    __shared__ long long carry_a, carry_p;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { carry_a = 0; carry_p = 0; }
    __syncthreads();
    for (int64_t base = 0; base < B; base += 1024) {
        const int64_t c = base + threadIdx.x;
        const long long n = c < B ? (long long)sizes[c] : 0;
        long long sa = n, sp = n * n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long ta = __shfl_up_sync(0xffffffffu, sa, o), tp = __shfl_up_sync(0xffffffffu, sp, o);
            if (lane >= o) { sa += ta; sp += tp; }
        }
        if (lane == 31) { warp_a[warp] = sa; warp_p[warp] = sp; }
        __syncthreads();
        if (warp == 0) {
            long long wa = warp_a[lane], wp = warp_p[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long ta = __shfl_up_sync(0xffffffffu, wa, o), tp = __shfl_up_sync(0xffffffffu, wp, o);
                if (lane >= o) { wa += ta; wp += tp; }
            }
            warp_a[lane] = wa; warp_p[lane] = wp;
        }
        __syncthreads();
        const long long off_a = carry_a + (warp ? warp_a[warp - 1] : 0);
        const long long off_p = carry_p + (warp ? warp_p[warp - 1] : 0);
        const long long excl_a = off_a + sa - n, excl_p = off_p + sp - n * n;
        if (c < B) {
            crystal_start[c] = excl_a;
            if (n > 0 && excl_a < N) e_start[excl_a] = excl_p;
        }
        __syncthreads();
        if (threadIdx.x == 1023) { carry_a = off_a + sa; carry_p = off_p + sp; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        crystal_start[B] = carry_a;
        e_start[N] = E;
        if (carry_a != N || carry_p != E) atomicOr(&g_status, CFB200_ST_SIZE_MISMATCH);
    }
}

// One block per crystal: atoms' CSR offsets, crystal index, and the dense n x n pair block.
__global__ void __launch_bounds__(256) edge_fill_kernel(const int64_t* __restrict__ sizes,
                                                        const int64_t* __restrict__ crystal_start, int64_t B,
                                                        int64_t N, int64_t E, int64_t* __restrict__ edges,
                                                        int64_t* __restrict__ e_start, int64_t* __restrict__ batch)
{
    for (int64_t c = blockIdx.x; c < B; c += gridDim.x) {
        const int64_t n = sizes[c], a0 = crystal_start[c];
        if (n <= 0 || a0 + n > N) continue;
        const int64_t p0 = e_start[a0];          // written by the scan kernel
        __syncthreads();                          // everyone has read e_start[a0] before it is rewritten below
        if (p0 + n * n > E) continue;
        for (int64_t il = threadIdx.x; il < n; il += blockDim.x) {
            e_start[a0 + il] = p0 + il * n;
            if (batch) batch[a0 + il] = c;
        }
        for (int64_t t = threadIdx.x; t < n * n; t += blockDim.x) {
            const int64_t il = t / n, jl = t - il * n;
            edges[p0 + t] = a0 + il;
            edges[E + p0 + t] = a0 + jl;
        }
    }
}

// e_start from a pair list sorted by query atom: e_start[i] = first pair whose query atom is >= i
__global__ void csr_offsets_kernel(const int64_t* __restrict__ edge_i, int64_t E, int64_t N, int64_t* __restrict__ e_start)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e > E) return;
    const int64_t prev = e == 0 ? -1 : edge_i[e - 1];
    const int64_t cur = e == E ? N : edge_i[e];
    for (int64_t i = prev + 1; i <= cur && i <= N; i++) e_start[i] = e;
}

// One warp per (crystal, 32-channel group): lanes own consecutive channels, the warp walks the
// crystal's atoms in order, so each step reads one 128-byte line and the sum order is fixed.
__global__ void __launch_bounds__(128) segment_mean_fwd_kernel(const float* __restrict__ x, const int64_t* __restrict__ start,
                                                               int64_t B, int64_t D, float* __restrict__ out)
{
    const int64_t groups = (D + 31) / 32;
    const int64_t task = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (task >= B * groups) return;
    const int64_t c = task / groups, d = (task - c * groups) * 32 + (threadIdx.x & 31);
    if (d >= D) return;
    const int64_t s = start[c], t = start[c + 1];
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int64_t i = s;
    for (; i + 3 < t; i += 4) {
        a0 += x[i * D + d]; a1 += x[(i + 1) * D + d]; a2 += x[(i + 2) * D + d]; a3 += x[(i + 3) * D + d];
    }
    for (; i < t; i++) a0 += x[i * D + d];
    out[c * D + d] = ((a0 + a1) + (a2 + a3)) / (float)(t - s);
}

__global__ void __launch_bounds__(128) segment_mean_bwd_kernel(const float* __restrict__ gout, const int64_t* __restrict__ start,
                                                               int64_t B, int64_t D, float* __restrict__ gx)
{
    const int64_t groups = (D + 31) / 32;
    const int64_t task = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (task >= B * groups) return;
    const int64_t c = task / groups, d = (task - c * groups) * 32 + (threadIdx.x & 31);
    if (d >= D) return;
    const int64_t s = start[c], t = start[c + 1];
    const float g = gout[c * D + d] / (float)(t - s);
    for (int64_t i = s; i < t; i++) gx[i * D + d] = g;
}

int edge_index(const int64_t* sizes, int64_t B, int64_t N, int64_t E, int64_t* edges, int64_t* e_start, int64_t* batch,
               int64_t* crystal_start, cudaStream_t st)
{
    crystal_scan_kernel<<<1, 1024, 0, st>>>(sizes, B, N, E, crystal_start, e_start);
    if (B > 0) {
        const unsigned grid = (unsigned)(B < 65535 ? B : 65535);
        edge_fill_kernel<<<grid, 256, 0, st>>>(sizes, crystal_start, B, N, E, edges, e_start, batch);
    }
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int csr_offsets(const int64_t* edge_i, int64_t E, int64_t N, int64_t* e_start, cudaStream_t st)
{
    csr_offsets_kernel<<<(unsigned)((E + 1 + 255) / 256), 256, 0, st>>>(edge_i, E, N, e_start);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int segment_mean(bool bwd, const float* in, const int64_t* start, int64_t B, int64_t D, float* out, cudaStream_t st)
{
    const int64_t tasks = B * ((D + 31) / 32);
    if (tasks == 0) return CFB200_OK;
    const unsigned grid = (unsigned)((tasks + 3) / 4);
    if (bwd) segment_mean_bwd_kernel<<<grid, 128, 0, st>>>(in, start, B, D, out);
    else segment_mean_fwd_kernel<<<grid, 128, 0, st>>>(in, start, B, D, out);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
