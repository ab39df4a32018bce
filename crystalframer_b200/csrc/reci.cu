// Reciprocal-space lattice sum of the plain Crystalformer ("reci" and "multihead" domains) and its gradient
// (replaces models/kernels/reci_enc_fwd.cu:17-67 and reci_enc_bwd.cu:19-70, launched by
// models/cuda_funcs/reci_space_enc.py:46,80):
//     sum_ek = sum_n w(n1) exp(a_ik |n G|^2) cos(n . kr_e)      n1 in [0,R] (w = 1 at 0, else 2), n2, n3 in [-R,R]
//     z_ek   = log(max(sum, 1e-6)) + 1.5 log(-4 pi a_ik) - log(vcell)
//     ga_ik  = sum_e gz_ek (sum_ek < 1e-6 ? 0 : 1 / sum_ek) sum_n w |nG|^2 exp(a_ik |nG|^2) cos(n . kr_e)
// The reference gives a thread to every (pair, head) and lets it evaluate one exponential and one cosine per
// term.  The exponential depends on (atom, head, n) only and the cosine on (pair, n) only, so here a warp owns an
// atom: it first fills a table of the (R+1)(2R+1)^2 x 8 exponentials of 8 heads in shared memory, then every lane
// takes a pair, forms each cosine once and feeds 8 accumulators from the table (shared-memory broadcasts).
// Per pair that is 75 cosines instead of 600 cosines and 600 exponentials at R = 2, H = 8.
#include "common.cuh"

namespace cfb {

constexpr int kReciWarps = 4;       // warps (atoms) per block
constexpr int kReciHeads = 8;       // heads per pass over an atom's pairs
constexpr int kReciMaxRange = 3;    // table: (R+1)(2R+1)^2 x 8 floats per warp (6.3 KB at R = 3)

struct ReciArgs {
    const float* a; const float* kr; const float* rvecs; const float* vcell;
    const int64_t* batch; const int64_t* e_start;
    const float* gz; const float* sumexp_in;
    float* z; float* sumexp; float* ga;
    int N, H, R;
};

template <bool BWD>
__global__ void __launch_bounds__(kReciWarps * 32) reci_enc_kernel(const ReciArgs A)
{
    extern __shared__ __align__(16) float reci_table[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * kReciWarps + warp;
    if (i >= A.N) return;                                   // no block barrier below: warps are independent
    const int R = A.R, w = 2 * R + 1, terms = (R + 1) * w * w;
    float* tbl = reci_table + (size_t)warp * terms * kReciHeads;
    const int64_t c = A.batch[i];
    float g[9];
#pragma unroll
    for (int t = 0; t < 9; t++) g[t] = A.rvecs[c * 9 + t];
    const int64_t e0 = A.e_start[i], e1 = A.e_start[i + 1];
    const float log_vcell = BWD ? 0.0f : logf(A.vcell[c]);

    for (int h0 = 0; h0 < A.H; h0 += kReciHeads) {
        __syncwarp();
        // table of this head group: weight * exp(a |nG|^2), times |nG|^2 for the gradient
        for (int idx = lane; idx < terms * kReciHeads; idx += 32) {
            const int n = idx / kReciHeads, hh = idx % kReciHeads;
            const float n1 = (float)(n / (w * w)), n2 = (float)((n / w) % w - R), n3 = (float)(n % w - R);
            const float k1 = g[0] * n1 + g[3] * n2 + g[6] * n3;
            const float k2 = g[1] * n1 + g[4] * n2 + g[7] * n3;
            const float k3 = g[2] * n1 + g[5] * n2 + g[8] * n3;
            const float kk = k1 * k1 + k2 * k2 + k3 * k3;
            float v = 0.0f;
            if (h0 + hh < A.H) {
                v = expf(A.a[(int64_t)i * A.H + h0 + hh] * kk) * (n1 == 0.0f ? 1.0f : 2.0f);
                if (BWD) v *= kk;
            }
            tbl[idx] = v;
        }
        __syncwarp();
        float total[kReciHeads];
#pragma unroll
        for (int hh = 0; hh < kReciHeads; hh++) total[hh] = 0.0f;
        for (int64_t e = e0 + lane; e < e1; e += 32) {
            const float p1 = A.kr[e * 3], p2 = A.kr[e * 3 + 1], p3 = A.kr[e * 3 + 2];
            float acc[kReciHeads];
#pragma unroll
            for (int hh = 0; hh < kReciHeads; hh++) acc[hh] = 0.0f;
            const float4* row = reinterpret_cast<const float4*>(tbl);
            for (int n1 = 0; n1 <= R; n1++)
                for (int n2 = -R; n2 <= R; n2++)
                    for (int n3 = -R; n3 <= R; n3++, row += 2) {
                        const float cs = cosf(p1 * (float)n1 + p2 * (float)n2 + p3 * (float)n3);
                        const float4 lo = row[0], hi = row[1];
                        acc[0] = fmaf(lo.x, cs, acc[0]); acc[1] = fmaf(lo.y, cs, acc[1]);
                        acc[2] = fmaf(lo.z, cs, acc[2]); acc[3] = fmaf(lo.w, cs, acc[3]);
                        acc[4] = fmaf(hi.x, cs, acc[4]); acc[5] = fmaf(hi.y, cs, acc[5]);
                        acc[6] = fmaf(hi.z, cs, acc[6]); acc[7] = fmaf(hi.w, cs, acc[7]);
                    }
#pragma unroll
            for (int hh = 0; hh < kReciHeads; hh++) {
                if (h0 + hh >= A.H) break;
                const int64_t eh = e * A.H + h0 + hh;
                if (!BWD) {
                    const float a = A.a[(int64_t)i * A.H + h0 + hh];
                    A.z[eh] = logf(fmaxf(acc[hh], 1e-6f)) + 1.5f * logf(-12.5663706144f * a) - log_vcell;
                    A.sumexp[eh] = acc[hh];
                } else {
                    const float se = A.sumexp_in[eh];
                    total[hh] += acc[hh] * A.gz[eh] * (se < 1e-6f ? 0.0f : 1.0f / se);
                }
            }
        }
        if (BWD) {
#pragma unroll
            for (int hh = 0; hh < kReciHeads; hh++) {
                float t = total[hh];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                if (lane == 0 && h0 + hh < A.H) A.ga[(int64_t)i * A.H + h0 + hh] = t;
            }
        }
    }
}

int reci_enc(const ReciArgs& A, bool bwd, cudaStream_t st)
{
    if (A.N == 0) return CFB200_OK;
    if (A.R < 0 || A.R > kReciMaxRange) return CFB200_E_UNSUPPORTED;
    const int w = 2 * A.R + 1;
    const size_t smem = (size_t)kReciWarps * (A.R + 1) * w * w * kReciHeads * sizeof(float);
    const int blocks = (A.N + kReciWarps - 1) / kReciWarps;
    if (bwd) reci_enc_kernel<true><<<blocks, kReciWarps * 32, smem, st>>>(A);
    else reci_enc_kernel<false><<<blocks, kReciWarps * 32, smem, st>>>(A);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
