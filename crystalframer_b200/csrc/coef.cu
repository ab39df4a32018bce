// Gaussian coefficient of every (atom, head): a = [(1-lb) elu((q.w + shift) scale beta/(1-lb)) + 1] * c,
// c = -1/(2 r0^2) < 0, together with the scaled query q / sqrt(head_dim) the attention kernels take
// (replaces the chain of torch operations of
// models/indexed_lattice_multi_head_attention_cuda.py:896-940 and :179, :447 of the reference).
// Elementwise work over N*H*16 floats: bound by HBM traffic (128 B read + 68 B written per (atom, head)).
#include "common.cuh"

namespace cfb {

constexpr int kCoHd = 16;

struct CoefArgs {
    const float* q; const float* w; const float* gauss_scale;   // gauss_scale: [scale, shift] on the device, or NULL
    int64_t N; int H;
    float lb, beta, cmul, qscale;
    float* a; float* qs;
    const float* ga; const float* gqs; float* gq; float* gw;
    float* partial;          // optional scratch of kCoSplits * H * 16 floats: the backward then runs kCoSplits blocks per head
};

constexpr int kCoSplits = 32;

__device__ __forceinline__ float coef_from_dot(const CoefArgs& A, float dot, float scale, float shift, float& dadot)
{
    const float alpha = (dot + shift) * scale;
    const float x = alpha * (A.beta / (1.0f - A.lb));
    const float ex = expf(fminf(x, 0.0f));
    const float elu = x > 0.0f ? x : ex - 1.0f;
    dadot = A.cmul * A.beta * (x > 0.0f ? 1.0f : ex) * scale;
    return ((1.0f - A.lb) * elu + 1.0f) * A.cmul;
}

__global__ void __launch_bounds__(256) coef_fwd_kernel(const CoefArgs A)
{
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= A.N * A.H) return;
    const int h = (int)(t % A.H);
    const float scale = A.gauss_scale ? __ldg(A.gauss_scale) : 1.0f, shift = A.gauss_scale ? __ldg(A.gauss_scale + 1) : 0.0f;
    const float4* q4 = reinterpret_cast<const float4*>(A.q + t * kCoHd);
    const float4* w4 = reinterpret_cast<const float4*>(A.w + h * kCoHd);
    float4* o4 = reinterpret_cast<float4*>(A.qs + t * kCoHd);
    float dot = 0.f;
#pragma unroll
    for (int d = 0; d < kCoHd / 4; d++) {
        const float4 u = __ldg(q4 + d), v = __ldg(w4 + d);
        dot = fmaf(u.x, v.x, fmaf(u.y, v.y, fmaf(u.z, v.z, fmaf(u.w, v.w, dot))));
        o4[d] = make_float4(u.x * A.qscale, u.y * A.qscale, u.z * A.qscale, u.w * A.qscale);
    }
    float dadot;
    A.a[t] = coef_from_dot(A, dot, scale, shift, dadot);
}

// One block per head (and per slice of the atoms when scratch is given): gq = gqs * qscale + (ga da/ddot) w ;
// gw[h] = sum_i (ga da/ddot) q_i, summed in a fixed order (thread-strided partials, a tree over the block, then the
// slices in order by coef_bwd_reduce_kernel).
__global__ void __launch_bounds__(256) coef_bwd_kernel(const CoefArgs A)
{
    __shared__ float part[256][kCoHd + 1];
    const int h = blockIdx.x, tid = threadIdx.x;
    const int64_t chunk = (A.N + gridDim.y - 1) / gridDim.y;
    const int64_t i_begin = (int64_t)blockIdx.y * chunk, i_end = min(A.N, i_begin + chunk);
    const float scale = A.gauss_scale ? __ldg(A.gauss_scale) : 1.0f, shift = A.gauss_scale ? __ldg(A.gauss_scale + 1) : 0.0f;
    float wv[kCoHd], acc[kCoHd];
#pragma unroll
    for (int d = 0; d < kCoHd; d++) { wv[d] = __ldg(A.w + h * kCoHd + d); acc[d] = 0.f; }
    for (int64_t i = i_begin + tid; i < i_end; i += 256) {
        const int64_t t = i * A.H + h;
        const float4* q4 = reinterpret_cast<const float4*>(A.q + t * kCoHd);
        const float4* g4 = reinterpret_cast<const float4*>(A.gqs + t * kCoHd);
        float4* o4 = reinterpret_cast<float4*>(A.gq + t * kCoHd);
        float qv[kCoHd];
        float dot = 0.f;
#pragma unroll
        for (int d = 0; d < kCoHd / 4; d++) {
            const float4 u = __ldg(q4 + d);
            qv[4 * d] = u.x; qv[4 * d + 1] = u.y; qv[4 * d + 2] = u.z; qv[4 * d + 3] = u.w;
            dot = fmaf(u.x, wv[4 * d], fmaf(u.y, wv[4 * d + 1], fmaf(u.z, wv[4 * d + 2], fmaf(u.w, wv[4 * d + 3], dot))));
        }
        float dadot;
        coef_from_dot(A, dot, scale, shift, dadot);
        const float gdot = __ldg(A.ga + t) * dadot;
#pragma unroll
        for (int d = 0; d < kCoHd / 4; d++) {
            const float4 g = __ldg(g4 + d);
            o4[d] = make_float4(fmaf(g.x, A.qscale, gdot * wv[4 * d]), fmaf(g.y, A.qscale, gdot * wv[4 * d + 1]),
                                fmaf(g.z, A.qscale, gdot * wv[4 * d + 2]), fmaf(g.w, A.qscale, gdot * wv[4 * d + 3]));
        }
#pragma unroll
        for (int d = 0; d < kCoHd; d++) acc[d] = fmaf(gdot, qv[d], acc[d]);
    }
#pragma unroll
    for (int d = 0; d < kCoHd; d++) part[tid][d] = acc[d];
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (tid < s)
#pragma unroll
            for (int d = 0; d < kCoHd; d++) part[tid][d] += part[tid + s][d];
        __syncthreads();
    }
    if (tid < kCoHd) {
        if (gridDim.y == 1) A.gw[h * kCoHd + tid] = part[0][tid];
        else A.partial[((size_t)blockIdx.y * A.H + h) * kCoHd + tid] = part[0][tid];
    }
}

__global__ void coef_bwd_reduce_kernel(const CoefArgs A, int splits)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= A.H * kCoHd) return;
    float s = 0.f;
    for (int y = 0; y < splits; y++) s += A.partial[(size_t)y * A.H * kCoHd + t];
    A.gw[t] = s;
}

int coef_fwd(const CoefArgs& A, cudaStream_t st)
{
    const int64_t n = A.N * A.H;
    if (n == 0) return CFB200_OK;
    coef_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(A);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int coef_bwd(const CoefArgs& A, cudaStream_t st)
{
    if (A.partial != nullptr && A.N > 1024) {
        coef_bwd_kernel<<<dim3(A.H, kCoSplits), 256, 0, st>>>(A);
        coef_bwd_reduce_kernel<<<(A.H * kCoHd + 127) / 128, 128, 0, st>>>(A, kCoSplits);
    } else {
        coef_bwd_kernel<<<dim3(A.H, 1), 256, 0, st>>>(A);
    }
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
