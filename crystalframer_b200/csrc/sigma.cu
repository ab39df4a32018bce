// Weighted-PCA frames: per (pair, head) the softmax-weighted second moments of the separation
// vector over the lattice translations, pooled per (atom, head) with the attention weights, then a
// symmetric 3x3 eigen-decomposition (replaces real_enc_sigma_fwd.cu, select_edges.cu,
// fused_dpa_sigmamat_fwd.cu and the torch.linalg.det / eigh / randint block of
// models/indexed_lattice_multi_head_attention_cuda.py:656-725 of the reference).
//
// Where the reference is ill-defined this file takes the evident intent and says so:
//  * the pooling attention is biased with the lattice-sum log-weights z (the reference passes an
//    uninitialised buffer, models/cuda_funcs/real_space_enc_proj.py:54,97-125);
//  * the per-atom tie-breaking matrix is d d^T / d^2 of the nearest non-zero image among ALL of
//    the atom's pairs (the reference lets every pair's thread write the same slot, last writer wins);
//  * eigenvectors are signed so that their largest component is positive (LAPACK leaves the sign
//    open), the random row signs come from the library's counter-based hash.
#include "common.cuh"

namespace cfb {

constexpr int kSgHd = 16;

struct SgArgs {
    const float* q; const float* k; const float* a_ik; const float* pos_ij; const float* tvecs; const float* rvlen;
    const int64_t* batch; const int64_t* edges; const int64_t* e_start;
    int64_t N, E;
    uint64_t seed_noise, seed_sign;
    float* ws;                       // (E,H,11): z, six moments, nearest d^2, nearest direction
    float* frame1; float* frame2; float* frame3;
    const float* list;               // optional per-pair sorted translation lists (pair_list_kernel), box (cache_range)^3
    int cache_range;
};

// One (pair, head) by a sweep over its whole box of translations: two passes (nearest distance, then weights and
// moments), the nearest non-zero image on the way.  The mapping of the reference's real_enc_sigma_fwd.cu; here it
// serves the pairs whose box the sorted list does not cover.
__device__ void sigma_pair_sweep(const SgArgs& A, const Params& P, const int64_t e, const int h, const int64_t c,
                                 const float a, const int R1, const int R2, const int R3)
{
    const int H = P.H;
    const int64_t tid = e * H + h;
    const float rx = __ldg(A.pos_ij + 3 * e), ry = __ldg(A.pos_ij + 3 * e + 1), rz = __ldg(A.pos_ij + 3 * e + 2);
    const float* Tc = A.tvecs + 9 * c;
    const float t1x = __ldg(Tc), t1y = __ldg(Tc + 1), t1z = __ldg(Tc + 2);
    const float t2x = __ldg(Tc + 3), t2y = __ldg(Tc + 4), t2z = __ldg(Tc + 5);
    const float t3x = __ldg(Tc + 6), t3y = __ldg(Tc + 7), t3z = __ldg(Tc + 8);
    float d2min = 1e10f;
    for (int n1 = -R1; n1 <= R1; n1++)
        for (int n2 = -R2; n2 <= R2; n2++)
            for (int n3 = -R3; n3 <= R3; n3++) {
                const float dx = fmaf(t3x, (float)n3, fmaf(t2x, (float)n2, fmaf(t1x, (float)n1, rx)));
                const float dy = fmaf(t3y, (float)n3, fmaf(t2y, (float)n2, fmaf(t1y, (float)n1, ry)));
                const float dz = fmaf(t3z, (float)n3, fmaf(t2z, (float)n2, fmaf(t1z, (float)n1, rz)));
                d2min = fminf(d2min, fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
            }
    float sum = 0.f, m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f, m4 = 0.f, m5 = 0.f;
    float best = 1e8f, bx = 0.f, by = 0.f, bz = 0.f;
    int t = 0;
    for (int n1 = -R1; n1 <= R1; n1++)
        for (int n2 = -R2; n2 <= R2; n2++)
            for (int n3 = -R3; n3 <= R3; n3++, t++) {
                const float dx = fmaf(t3x, (float)n3, fmaf(t2x, (float)n2, fmaf(t1x, (float)n1, rx)));
                const float dy = fmaf(t3y, (float)n3, fmaf(t2y, (float)n2, fmaf(t1y, (float)n1, ry)));
                const float dz = fmaf(t3z, (float)n3, fmaf(t2z, (float)n2, fmaf(t1z, (float)n1, rz)));
                const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                const float w = ex2_approx(a * (d2 - d2min) * kLog2e);
                sum += w;
                const float wx = dx * w, wy = dy * w, wz = dz * w;
                m0 = fmaf(dx, wx, m0); m1 = fmaf(dx, wy, m1); m2 = fmaf(dx, wz, m2);
                m3 = fmaf(dy, wy, m3); m4 = fmaf(dy, wz, m4); m5 = fmaf(dz, wz, m5);
                if (d2 > 1e-5f && d2 - 0.5f * P.noise < best) {
                    float cand = d2;
                    if (P.noise != 0.0f)
                        cand = d2 + (float)(((double)hash_uniform(A.seed_noise, (uint64_t)tid, (uint32_t)t) - 0.5) * (double)P.noise);
                    if (best > cand) { best = cand; bx = dx; by = dy; bz = dz; }
                }
            }
    const float inv = 1.0f / sum;
    float* o = A.ws + tid * 11;
    o[0] = logf(sum) + d2min * a;
    o[1] = m0 * inv; o[2] = m1 * inv; o[3] = m2 * inv; o[4] = m3 * inv; o[5] = m4 * inv; o[6] = m5 * inv;
    o[7] = best;
    const float rn = rsqrtf(fmaxf(bx * bx + by * by + bz * bz, 1e-30f));
    o[8] = bx * rn; o[9] = by * rn; o[10] = bz * rn;
}

// thread = (pair, head): every pair by the sweep (no sorted lists at hand, or a head count that does not divide 32)
__global__ void __launch_bounds__(256) sigma_edges_kernel(const SgArgs A, const Params P)
{
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int H = P.H;
    if (tid >= A.E * H) return;
    const int64_t e = tid / H;
    const int h = (int)(tid - e * H);
    const int64_t i = A.edges[e], c = A.batch[i];
    const float a = __ldg(A.a_ik + i * H + h);
    int R[3];
#pragma unroll
    for (int d = 0; d < 3; d++) R[d] = lattice_range_1d(P, a, P.cutoff_radius != 0.0f ? __ldg(A.rvlen + 3 * c + d) : 0.0f);
    sigma_pair_sweep(A, P, e, h, c, a, R[0], R[1], R[2]);
}

// warp = pair, lane = (slot, head) with 32 / H slots per head.  The weight exp(a (d^2 - d^2_min)) falls with the
// distance, so the translations that matter to a (pair, head) -- those above the pruning threshold of the lattice-sum
// kernels, and the nearest non-zero image with whatever lies within the noise amplitude of it -- are a prefix of the
// pair's sorted list, which all heads share: the slots of a head walk that prefix in turns (typically 3-4 entries
// each instead of two sweeps over 125 translations), their partial sums meet by shuffles.  A (pair, head) whose box
// is larger than the listed one and whose prefix could reach outside it sweeps that box, its slots sharing the planes.
constexpr int kSgListWarps = 8;

__global__ void __launch_bounds__(kSgListWarps * 32) sigma_edges_list_kernel(const SgArgs A, const Params P)
{
    const int H = P.H, lane = threadIdx.x & 31;
    const int64_t e = (int64_t)blockIdx.x * kSgListWarps + (threadIdx.x >> 5);
    if (e >= A.E) return;
    const int h = lane % H, slot = lane / H, slots = 32 / H;
    const int64_t i = A.edges[e], c = A.batch[i];
    const float a = __ldg(A.a_ik + i * H + h);
    int R1, R2, R3;
    {
        const bool cut = P.cutoff_radius != 0.0f;
        R1 = lattice_range_1d(P, a, cut ? __ldg(A.rvlen + 3 * c) : 0.0f);
        R2 = lattice_range_1d(P, a, cut ? __ldg(A.rvlen + 3 * c + 1) : 0.0f);
        R3 = lattice_range_1d(P, a, cut ? __ldg(A.rvlen + 3 * c + 2) : 0.0f);
    }
    const float* list = A.list + (size_t)e * kListStride;
    // the pair's first 32 distances: the smallest, and the smallest that counts as non-zero
    const float dl = __ldg(list + lane);
    const float d2min = __shfl_sync(0xffffffffu, dl, 0);
    const unsigned nz = __ballot_sync(0xffffffffu, dl > 1.0001e-5f && dl < 1e29f);
    const unsigned unclear = __ballot_sync(0xffffffffu, dl > 0.9999e-5f && dl <= 1.0001e-5f);
    const float d2nz = nz != 0u ? __shfl_sync(0xffffffffu, dl, __ffs(nz) - 1) : -1.f;
    Cell cell;
    {
        const float* Tc = A.tvecs + 9 * c;
        cell.t1x = __ldg(Tc); cell.t1y = __ldg(Tc + 1); cell.t1z = __ldg(Tc + 2);
        cell.t2x = __ldg(Tc + 3); cell.t2y = __ldg(Tc + 4); cell.t2z = __ldg(Tc + 5);
        cell.t3x = __ldg(Tc + 6); cell.t3y = __ldg(Tc + 7); cell.t3z = __ldg(Tc + 8);
        cell.rx = __ldg(A.pos_ij + 3 * e); cell.ry = __ldg(A.pos_ij + 3 * e + 1); cell.rz = __ldg(A.pos_ij + 3 * e + 2);
    }
    const int C = A.cache_range;
    const bool same_box = R1 == C && R2 == C && R3 == C;
    const bool wider = !same_box && R1 >= C && R2 >= C && R3 >= C;
    const float reach2 = wider ? box_reach2(cell, C) : 1e38f;
    // list distances and the sweep's differ in the last bits (another order of the fused operations): margins
    const float w_limit = a < 0.f ? d2min + P.prune / (-a) : 1e38f;
    const float nz_limit = d2nz + fabsf(P.noise) + fabsf(d2nz) * 8e-6f + 1e-12f;
    const float far = fmaxf(w_limit, nz_limit);
    const bool usable = a < 0.f && d2nz >= 0.f && unclear == 0u && (same_box || (wider && far < reach2));
    // A head whose list does not serve sweeps its whole box, the slots taking the planes n1 in turns: first the
    // smallest distance (the slots' minima meet by shuffles, which every lane of the warp executes), then weights,
    // moments and the nearest non-zero image with the sweep's own arithmetic.
    float d2ref = d2min;
    {
        float dmin = 1e10f;
        if (!usable)
            for (int n1 = -R1 + slot; n1 <= R1; n1 += slots)
                for (int n2 = -R2; n2 <= R2; n2++)
                    for (int n3 = -R3; n3 <= R3; n3++) {
                        const float dx = fmaf(cell.t3x, (float)n3, fmaf(cell.t2x, (float)n2, fmaf(cell.t1x, (float)n1, cell.rx)));
                        const float dy = fmaf(cell.t3y, (float)n3, fmaf(cell.t2y, (float)n2, fmaf(cell.t1y, (float)n1, cell.ry)));
                        const float dz = fmaf(cell.t3z, (float)n3, fmaf(cell.t2z, (float)n2, fmaf(cell.t1z, (float)n1, cell.rz)));
                        dmin = fminf(dmin, fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
                    }
        for (int o = H; o < 32; o <<= 1) dmin = fminf(dmin, __shfl_xor_sync(0xffffffffu, dmin, o));
        if (!usable) d2ref = dmin;
    }
    float sum = 0.f, m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f, m4 = 0.f, m5 = 0.f;
    float best = 1e8f, bx = 0.f, by = 0.f, bz = 0.f;
    int best_t = 0x7fffffff;
    const int64_t tid = e * H + h;
    const int L2 = 2 * R2 + 1, L3 = 2 * R3 + 1;
    if (!usable) {
        for (int n1 = -R1 + slot; n1 <= R1; n1 += slots)
            for (int n2 = -R2; n2 <= R2; n2++)
                for (int n3 = -R3; n3 <= R3; n3++) {
                    const float dx = fmaf(cell.t3x, (float)n3, fmaf(cell.t2x, (float)n2, fmaf(cell.t1x, (float)n1, cell.rx)));
                    const float dy = fmaf(cell.t3y, (float)n3, fmaf(cell.t2y, (float)n2, fmaf(cell.t1y, (float)n1, cell.ry)));
                    const float dz = fmaf(cell.t3z, (float)n3, fmaf(cell.t2z, (float)n2, fmaf(cell.t1z, (float)n1, cell.rz)));
                    const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                    const float w = ex2_approx(a * (d2 - d2ref) * kLog2e);
                    sum += w;
                    const float wx = dx * w, wy = dy * w, wz = dz * w;
                    m0 = fmaf(dx, wx, m0); m1 = fmaf(dx, wy, m1); m2 = fmaf(dx, wz, m2);
                    m3 = fmaf(dy, wy, m3); m4 = fmaf(dy, wz, m4); m5 = fmaf(dz, wz, m5);
                    if (d2 > 1e-5f && d2 - 0.5f * fabsf(P.noise) <= best) {
                        const int t = ((n1 + R1) * L2 + (n2 + R2)) * L3 + (n3 + R3);
                        float cand = d2;
                        if (P.noise != 0.0f)
                            cand = d2 + (float)(((double)hash_uniform(A.seed_noise, (uint64_t)tid, (uint32_t)t) - 0.5) * (double)P.noise);
                        if (cand < best || (cand == best && t < best_t)) { best = cand; best_t = t; bx = dx; by = dy; bz = dz; }
                    }
                }
    }
    if (usable) {
        for (int s = slot; s < kListLen; s += slots) {
            const float d2l = __ldg(list + s);
            if (!(d2l <= far)) break;                       // sorted: nothing behind it matters either
            if (d2l <= w_limit) {
                const float dx = __ldg(list + kListLen + s), dy = __ldg(list + 2 * kListLen + s), dz = __ldg(list + 3 * kListLen + s);
                const float w = ex2_approx(a * (d2l - d2min) * kLog2e);
                sum += w;
                const float wx = dx * w, wy = dy * w, wz = dz * w;
                m0 = fmaf(dx, wx, m0); m1 = fmaf(dx, wy, m1); m2 = fmaf(dx, wz, m2);
                m3 = fmaf(dy, wy, m3); m4 = fmaf(dy, wz, m4); m5 = fmaf(dz, wz, m5);
            }
            if (d2l > 0.9999e-5f && d2l <= nz_limit) {
                // a candidate for the nearest non-zero image: the sweep's own arithmetic decides
                const int code = __float_as_int(__ldg(list + 4 * kListLen + s));
                const int n1 = (code & 255) - C, n2 = ((code >> 8) & 255) - C, n3 = ((code >> 16) & 255) - C;
                const float dx = fmaf(cell.t3x, (float)n3, fmaf(cell.t2x, (float)n2, fmaf(cell.t1x, (float)n1, cell.rx)));
                const float dy = fmaf(cell.t3y, (float)n3, fmaf(cell.t2y, (float)n2, fmaf(cell.t1y, (float)n1, cell.ry)));
                const float dz = fmaf(cell.t3z, (float)n3, fmaf(cell.t2z, (float)n2, fmaf(cell.t1z, (float)n1, cell.rz)));
                const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                if (d2 > 1e-5f) {
                    const int t = ((n1 + R1) * L2 + (n2 + R2)) * L3 + (n3 + R3);
                    float cand = d2;
                    if (P.noise != 0.0f)
                        cand = d2 + (float)(((double)hash_uniform(A.seed_noise, (uint64_t)tid, (uint32_t)t) - 0.5) * (double)P.noise);
                    if (cand < best || (cand == best && t < best_t)) { best = cand; best_t = t; bx = dx; by = dy; bz = dz; }
                }
            }
        }
    }
    // the slots of a head meet: lanes h, h + H, h + 2H, ...
    for (int o = H; o < 32; o <<= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        m0 += __shfl_xor_sync(0xffffffffu, m0, o); m1 += __shfl_xor_sync(0xffffffffu, m1, o);
        m2 += __shfl_xor_sync(0xffffffffu, m2, o); m3 += __shfl_xor_sync(0xffffffffu, m3, o);
        m4 += __shfl_xor_sync(0xffffffffu, m4, o); m5 += __shfl_xor_sync(0xffffffffu, m5, o);
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int ot = __shfl_xor_sync(0xffffffffu, best_t, o);
        const float ox = __shfl_xor_sync(0xffffffffu, bx, o), oy = __shfl_xor_sync(0xffffffffu, by, o),
                    oz = __shfl_xor_sync(0xffffffffu, bz, o);
        if (ob < best || (ob == best && ot < best_t)) { best = ob; best_t = ot; bx = ox; by = oy; bz = oz; }
    }
    if (slot == 0) {
        const float inv = 1.0f / sum;
        float* o = A.ws + (e * H + h) * 11;
        o[0] = logf(sum) + d2ref * a;
        o[1] = m0 * inv; o[2] = m1 * inv; o[3] = m2 * inv; o[4] = m3 * inv; o[5] = m4 * inv; o[6] = m5 * inv;
        o[7] = best;
        const float rn = rsqrtf(fmaxf(bx * bx + by * by + bz * bz, 1e-30f));
        o[8] = bx * rn; o[9] = by * rn; o[10] = bz * rn;
    }
}

// eigen-decomposition of a symmetric 3x3 matrix by cyclic Jacobi rotations; eigenvalues ascending,
// eigenvectors in the columns of V, each signed so that its largest component is positive
__device__ void eigh3(float M[3][3], float w[3], float V[3][3])
{
    for (int r = 0; r < 3; r++) for (int c = 0; c < 3; c++) V[r][c] = r == c ? 1.0f : 0.0f;
    for (int sweep = 0; sweep < 8; sweep++) {
        const float off = fabsf(M[0][1]) + fabsf(M[0][2]) + fabsf(M[1][2]);
        if (off < 1e-12f * (fabsf(M[0][0]) + fabsf(M[1][1]) + fabsf(M[2][2])) || off == 0.0f) break;
        for (int p = 0; p < 2; p++)
            for (int q = p + 1; q < 3; q++) {
                if (M[p][q] == 0.0f) continue;
                const float theta = (M[q][q] - M[p][p]) / (2.0f * M[p][q]);
                const float tt = copysignf(1.0f, theta) / (fabsf(theta) + sqrtf(fmaf(theta, theta, 1.0f)));
                const float cs = rsqrtf(fmaf(tt, tt, 1.0f)), sn = tt * cs;
                for (int r = 0; r < 3; r++) {          // M <- M J
                    const float mp = M[r][p], mq = M[r][q];
                    M[r][p] = cs * mp - sn * mq; M[r][q] = sn * mp + cs * mq;
                }
                for (int c = 0; c < 3; c++) {          // M <- J^T M
                    const float mp = M[p][c], mq = M[q][c];
                    M[p][c] = cs * mp - sn * mq; M[q][c] = sn * mp + cs * mq;
                }
                for (int r = 0; r < 3; r++) {
                    const float vp = V[r][p], vq = V[r][q];
                    V[r][p] = cs * vp - sn * vq; V[r][q] = sn * vp + cs * vq;
                }
            }
    }
    for (int c = 0; c < 3; c++) w[c] = M[c][c];
    for (int a = 0; a < 2; a++)                        // sort ascending
        for (int b = 0; b < 2 - a; b++)
            if (w[b] > w[b + 1]) {
                const float tw = w[b]; w[b] = w[b + 1]; w[b + 1] = tw;
                for (int r = 0; r < 3; r++) { const float tv = V[r][b]; V[r][b] = V[r][b + 1]; V[r][b + 1] = tv; }
            }
    for (int c = 0; c < 3; c++) {
        int big = 0;
        if (fabsf(V[1][c]) > fabsf(V[big][c])) big = 1;
        if (fabsf(V[2][c]) > fabsf(V[big][c])) big = 2;
        if (V[big][c] < 0.0f) for (int r = 0; r < 3; r++) V[r][c] = -V[r][c];
    }
}

// warp = (atom, head): attention pooling of the pairs' moments, then the frame
__global__ void __launch_bounds__(128) sigma_frames_kernel(const SgArgs A, const Params P)
{
    const int lane = threadIdx.x & 31;
    const int64_t task = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int H = P.H;
    if (task >= A.N * H) return;
    const int64_t i = task / H;
    const int h = (int)(task - i * H);
    const int64_t e0 = A.e_start[i], e1 = A.e_start[i + 1];
    float qv[kSgHd];
    {
        const float4* q4 = reinterpret_cast<const float4*>(A.q + (i * H + h) * kSgHd);
#pragma unroll
        for (int d = 0; d < 4; d++) { const float4 u = __ldg(q4 + d); qv[4 * d] = u.x; qv[4 * d + 1] = u.y; qv[4 * d + 2] = u.z; qv[4 * d + 3] = u.w; }
    }
    // pass 1: maximum logit
    float mx = -INFINITY;
    for (int64_t e = e0 + lane; e < e1; e += 32) {
        const int64_t j = A.edges[A.E + e];
        const float4* k4 = reinterpret_cast<const float4*>(A.k + (j * H + h) * kSgHd);
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < 4; d++) { const float4 u = __ldg(k4 + d); s = fmaf(qv[4 * d], u.x, fmaf(qv[4 * d + 1], u.y, fmaf(qv[4 * d + 2], u.z, fmaf(qv[4 * d + 3], u.w, s)))); }
        mx = fmaxf(mx, s + A.ws[(e * H + h) * 11]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    // pass 2: weighted sums, nearest image of the atom
    float acc[7] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float nd2 = 1e9f, nx = 0.f, ny = 0.f, nz = 0.f;
    long long ne = 0x7fffffffffffffffLL;
    for (int64_t e = e0 + lane; e < e1; e += 32) {
        const int64_t j = A.edges[A.E + e];
        const float4* k4 = reinterpret_cast<const float4*>(A.k + (j * H + h) * kSgHd);
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < 4; d++) { const float4 u = __ldg(k4 + d); s = fmaf(qv[4 * d], u.x, fmaf(qv[4 * d + 1], u.y, fmaf(qv[4 * d + 2], u.z, fmaf(qv[4 * d + 3], u.w, s)))); }
        const float* r = A.ws + (e * H + h) * 11;
        const float p = __expf(s + r[0] - mx);
        acc[6] += p;
#pragma unroll
        for (int m = 0; m < 6; m++) acc[m] = fmaf(p, r[1 + m], acc[m]);
        if (r[7] < nd2) { nd2 = r[7]; nx = r[8]; ny = r[9]; nz = r[10]; ne = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int m = 0; m < 7; m++) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
        const float d2o = __shfl_xor_sync(0xffffffffu, nd2, o);
        const long long eo = __shfl_xor_sync(0xffffffffu, ne, o);
        const float xo = __shfl_xor_sync(0xffffffffu, nx, o), yo = __shfl_xor_sync(0xffffffffu, ny, o), zo = __shfl_xor_sync(0xffffffffu, nz, o);
        if (d2o < nd2 || (d2o == nd2 && eo < ne)) { nd2 = d2o; ne = eo; nx = xo; ny = yo; nz = zo; }
    }
    if (lane != 0) return;
    const float inv = 1.0f / acc[6];
    float M[3][3];
    M[0][0] = acc[0] * inv; M[0][1] = M[1][0] = acc[1] * inv; M[0][2] = M[2][0] = acc[2] * inv;
    M[1][1] = acc[3] * inv; M[1][2] = M[2][1] = acc[4] * inv; M[2][2] = acc[5] * inv;
    const float det = M[0][0] * (M[1][1] * M[2][2] - M[1][2] * M[2][1]) - M[0][1] * (M[1][0] * M[2][2] - M[1][2] * M[2][0])
                      + M[0][2] * (M[1][0] * M[2][1] - M[1][1] * M[2][0]);
    float V[3][3] = {{1.f, 0.f, 0.f}, {0.f, 1.f, 0.f}, {0.f, 0.f, 1.f}}, w[3];
    if (det > 1e-5f) {
        if (P.noise > 0.0f) {
            const float s = cbrtf(det) * P.noise;
            const float u[3] = {nx, ny, nz};
            for (int r = 0; r < 3; r++) for (int c = 0; c < 3; c++) M[r][c] = fmaf(u[r] * u[c], s, M[r][c]);
        }
        eigh3(M, w, V);
    }
    // frame r = row r of V, with a hash-drawn sign; then all three times the determinant
    float Fm[3][3];
    for (int r = 0; r < 3; r++) {
        const float sgn = hash_uniform(A.seed_sign, (uint64_t)(i * H + h), (uint32_t)r) > 0.5f ? 1.0f : -1.0f;
        for (int c = 0; c < 3; c++) Fm[r][c] = V[r][c] * sgn;
    }
    const float dF = Fm[0][0] * (Fm[1][1] * Fm[2][2] - Fm[1][2] * Fm[2][1]) - Fm[0][1] * (Fm[1][0] * Fm[2][2] - Fm[1][2] * Fm[2][0])
                     + Fm[0][2] * (Fm[1][0] * Fm[2][1] - Fm[1][1] * Fm[2][0]);
    const float flip = dF < 0.0f ? -1.0f : 1.0f;
    float* o1 = A.frame1 + (i * H + h) * 3; float* o2 = A.frame2 + (i * H + h) * 3; float* o3 = A.frame3 + (i * H + h) * 3;
    for (int c = 0; c < 3; c++) { o1[c] = Fm[0][c] * flip; o2[c] = Fm[1][c] * flip; o3[c] = Fm[2][c] * flip; }
}

// "pca" frames (replaces ComputePCAFrame, models/cuda_funcs/calc_pca_frame.py:22-76 of the reference, which is
// torch_scatter + torch.linalg.eigh + torch.randint): warp = atom.  The scatter matrix of the atom's pair
// separations in the home cell about their mean, sum_j (r_ij - mean)(r_ij - mean)^T, its eigenvectors by ascending
// eigenvalue as the three axes -- the same for every head -- then per (atom, head) a hash-drawn sign per axis and all
// three times the determinant of the signed triple (the reference draws the signs with torch.randint, and its
// eigenvectors' own signs are LAPACK's: neither is pinned; here an eigenvector's largest component is positive before
// the drawn sign).  No lattice translations enter.
__global__ void __launch_bounds__(128) pca_frames_kernel(const float* __restrict__ pos_ij, const int64_t* __restrict__ e_start,
                                                         int64_t N, int H, uint64_t seed, float* __restrict__ f1,
                                                         float* __restrict__ f2, float* __restrict__ f3)
{
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (i >= N) return;
    const int64_t e0 = e_start[i], e1 = e_start[i + 1];
    float sx = 0.f, sy = 0.f, sz = 0.f;
    for (int64_t e = e0 + lane; e < e1; e += 32) { sx += __ldg(pos_ij + 3 * e); sy += __ldg(pos_ij + 3 * e + 1); sz += __ldg(pos_ij + 3 * e + 2); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sx += __shfl_xor_sync(0xffffffffu, sx, o); sy += __shfl_xor_sync(0xffffffffu, sy, o); sz += __shfl_xor_sync(0xffffffffu, sz, o);
    }
    const float inv_n = e1 > e0 ? 1.0f / (float)(e1 - e0) : 0.f;
    const float mx = sx * inv_n, my = sy * inv_n, mz = sz * inv_n;
    float c[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int64_t e = e0 + lane; e < e1; e += 32) {
        const float x = __ldg(pos_ij + 3 * e) - mx, y = __ldg(pos_ij + 3 * e + 1) - my, z = __ldg(pos_ij + 3 * e + 2) - mz;
        c[0] = fmaf(x, x, c[0]); c[1] = fmaf(x, y, c[1]); c[2] = fmaf(x, z, c[2]);
        c[3] = fmaf(y, y, c[3]); c[4] = fmaf(y, z, c[4]); c[5] = fmaf(z, z, c[5]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int m = 0; m < 6; m++) c[m] += __shfl_xor_sync(0xffffffffu, c[m], o);
    float M[3][3], w[3], V[3][3];
    M[0][0] = c[0]; M[0][1] = M[1][0] = c[1]; M[0][2] = M[2][0] = c[2]; M[1][1] = c[3]; M[1][2] = M[2][1] = c[4]; M[2][2] = c[5];
    eigh3(M, w, V);                                      // every lane: the same small computation
    for (int h = lane; h < H; h += 32) {
        float Fm[3][3];                                  // Fm[r] = axis r = column r of V with its drawn sign
        for (int r = 0; r < 3; r++) {
            const float sgn = hash_uniform(seed, (uint64_t)(i * H + h), (uint32_t)r) > 0.5f ? 1.0f : -1.0f;
            for (int k = 0; k < 3; k++) Fm[r][k] = V[k][r] * sgn;
        }
        const float det = Fm[0][0] * (Fm[1][1] * Fm[2][2] - Fm[1][2] * Fm[2][1]) - Fm[0][1] * (Fm[1][0] * Fm[2][2] - Fm[1][2] * Fm[2][0])
                          + Fm[0][2] * (Fm[1][0] * Fm[2][1] - Fm[1][1] * Fm[2][0]);
        float* o1 = f1 + (i * H + h) * 3; float* o2 = f2 + (i * H + h) * 3; float* o3 = f3 + (i * H + h) * 3;
        for (int k = 0; k < 3; k++) { o1[k] = Fm[0][k] * det; o2[k] = Fm[1][k] * det; o3[k] = Fm[2][k] * det; }
    }
}

int pca_frames(const float* pos_ij, const int64_t* e_start, int64_t N, int H, uint64_t seed, float* f1, float* f2, float* f3,
               cudaStream_t st)
{
    if (N == 0) return CFB200_OK;
    pca_frames_kernel<<<(unsigned)((N + 3) / 4), 128, 0, st>>>(pos_ij, e_start, N, H, seed, f1, f2, f3);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

static void launch_sigma_edges(const SgArgs& A, const Params& P, cudaStream_t st)
{
    if (A.list != nullptr && P.H <= 32 && 32 % P.H == 0) {
        sigma_edges_list_kernel<<<(unsigned)((A.E + kSgListWarps - 1) / kSgListWarps), kSgListWarps * 32, 0, st>>>(A, P);
    } else {
        const int64_t n1 = A.E * P.H;
        sigma_edges_kernel<<<(unsigned)((n1 + 255) / 256), 256, 0, st>>>(A, P);
    }
}

// the per-pair records alone (what the reference's real_enc_sigma_fwd.cu leaves, plus the logit it omits)
int sigma_edges(const SgArgs& A, const Params& P, cudaStream_t st)
{
    if (A.N == 0 || A.E == 0) return CFB200_OK;
    launch_sigma_edges(A, P, st);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

int sigma_frames(const SgArgs& A, const Params& P, cudaStream_t st)
{
    if (A.N == 0 || A.E == 0) return CFB200_OK;
    launch_sigma_edges(A, P, st);
    const int64_t n2 = A.N * P.H;
    sigma_frames_kernel<<<(unsigned)((n2 + 3) / 4), 128, 0, st>>>(A, P);
    return cudaGetLastError() == cudaSuccess ? CFB200_OK : CFB200_E_CUDA;
}

}  // namespace cfb
