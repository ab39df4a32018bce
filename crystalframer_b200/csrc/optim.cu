// Gradient clipping by global norm and the AdamW update on flat buffers, two launches per training step
// (replaces torch.nn.utils.clip_grad_norm_ followed by torch.optim.AdamW.step as the reference's
// Lightning module configures them, models/regression.py / params "clip_norm" and "adamw": tens of
// launches and about a millisecond of host work per step for the 60 tensors of the 4-layer model).
//
//   launch 1: per-block partial sums of squares of the gradient (fixed grid, fixed order)
//   launch 2: every block adds the partials in the same order, forms clip = min(1, max_norm / (norm + 1e-6))
//             and updates its slice:
//                 g  = clip * grad
//                 p *= 1 - lr * weight_decay                (elements before decay_end only)
//                 m  = m + (1 - beta1) (g - m)              v = beta2 v + (1 - beta2) g^2
//                 p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps)
//             with bc1 = 1 - beta1^t, bc2 = 1 - beta2^t formed by the caller in double;
//             optionally the running average of the weights that the reference keeps over its last epochs
//             (torch.optim.swa_utils.AveragedModel.update_parameters after opt.step, models/regression.py:150-152):
//                 avg += (p - avg) * avg_weight,  avg_weight = 1 / (models averaged so far + 1).
// Sums run in a fixed order, so the step is reproducible bit for bit.
#include "common.cuh"

namespace cfb {

constexpr int kOptBlocks = 256;
constexpr int kOptThreads = 256;

__global__ void __launch_bounds__(kOptThreads) grad_sumsq_kernel(const float* __restrict__ g, int64_t n, float* __restrict__ partial)
{
    __shared__ float red[kOptThreads];
    float s = 0.f;
    for (int64_t i = (int64_t)blockIdx.x * kOptThreads + threadIdx.x; i < n; i += (int64_t)kOptBlocks * kOptThreads) {
        const float v = g[i];
        s = fmaf(v, v, s);
    }
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = kOptThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}

struct AdamArgs {
    float* p; const float* g; float* m; float* v;
    int64_t n, decay_end;
    float lr, beta1, beta2, eps, weight_decay, max_norm, inv_bc1, inv_sqrt_bc2;
    const float* partial; float* norm_out;
    float* avg; float avg_weight;          // running average of the parameters (NULL: none)
};

__global__ void __launch_bounds__(kOptThreads) adamw_clip_kernel(const AdamArgs A)
{
    __shared__ float red[kOptThreads];
    red[threadIdx.x] = threadIdx.x < kOptBlocks ? A.partial[threadIdx.x] : 0.f;
    __syncthreads();
    for (int o = kOptThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    const float norm = sqrtf(red[0]);
    if (blockIdx.x == 0 && threadIdx.x == 0 && A.norm_out != nullptr) *A.norm_out = norm;
    float clip = 1.0f;
    if (A.max_norm > 0.0f) clip = fminf(A.max_norm / (norm + 1e-6f), 1.0f);
    const float keep = 1.0f - A.lr * A.weight_decay, step = A.lr * A.inv_bc1;
    for (int64_t i = (int64_t)blockIdx.x * kOptThreads + threadIdx.x; i < A.n; i += (int64_t)gridDim.x * kOptThreads) {
        const float g = A.g[i] * clip;
        float p = A.p[i];
        if (i < A.decay_end) p *= keep;
        const float m = fmaf(1.0f - A.beta1, g - A.m[i], A.m[i]);
        const float v = fmaf(A.beta2, A.v[i], (1.0f - A.beta2) * g * g);
        A.m[i] = m; A.v[i] = v;
        p -= step * m / (sqrtf(v) * A.inv_sqrt_bc2 + A.eps);
        A.p[i] = p;
        if (A.avg != nullptr) { const float s = A.avg[i]; A.avg[i] = fmaf(p - s, A.avg_weight, s); }
    }
}

int adamw_clip_step(const AdamArgs& A, float* partial, cudaStream_t st)
{
    if (A.n == 0) return CFB200_OK;
    grad_sumsq_kernel<<<kOptBlocks, kOptThreads, 0, st>>>(A.g, A.n, partial);
    int blocks = (int)((A.n + kOptThreads - 1) / kOptThreads);
    if (blocks > 1184) blocks = 1184;                       // 8 blocks per SM on 148 SMs
    adamw_clip_kernel<<<blocks, kOptThreads, 0, st>>>(A);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
