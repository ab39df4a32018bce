// The per-pair part of the lattice sum as a reusable device object: one warp evaluates one
// (pair, head); lane l owns basis indices l and l+32 of the four 64-wide Gaussian bases (distance,
// three frame axes) and keeps their sums in registers.  See framed_proj.cu for the method; this is the
// same arithmetic, packaged for kernels that walk the pairs of an atom one after the other.
#pragma once
#include "common.cuh"

namespace cfb {

constexpr float kLlLog2e = 1.4426950408889634f;
constexpr float kLlSqrtLog2e = 1.2011224087864498f;

// exact float value of a small integer (|n| < 2^22) without a conversion instruction
__device__ __forceinline__ float ll_int_to_float(int n)
{
    return __int_as_float(0x4B400000 + n) - 12582912.0f;
}

// MODE 0: forward, basis sums only.  MODE 1: backward by recomputation: weights relative to the pair's z, plus the
// sums weighted with d^2 that the coefficient gradient needs.  MODE 2: forward that also forms those d^2-weighted sums
// (weights relative to d^2_min, as in mode 0), so that the backward pass needs no second lattice sum.
template <int MODE, bool ANG>
struct LatticeLane {
    static constexpr bool BWD = MODE != 0;        // d^2-weighted sums and sum p d^2 are formed
    static constexpr bool REFZ = MODE == 1;       // ref is the pair's z (else d^2_min, found here)
    // per-lane basis constants, pre-scaled so that a Gaussian is ex2(-b*b)
    float cd_lo, cd_hi, ca_lo, ca_hi;
    float inv_d_interval, d_cut_scaled, xd_scale, inv_a_interval, xa_scale;
    unsigned win_d, win_a;
    bool wide_d;
    int lane;
    float4* tb;       // per-warp records: [32] first halves, then [32] second halves (float4 backward, float2 forward)
    // per-pair state
    float sd[2], sa[3][2];      // basis sums
    float qd[2], qa[3][2];      // modes 1, 2: sums of g * p * d^2
    float sum_l, px_l;          // per-lane parts of sum w and (backward) sum w d^2
    float a, ref;               // Gaussian coefficient; forward: d^2_min, backward: z of the pair
    float fx[3], fy[3], fz[3];  // frame axes of the query atom

    __device__ __forceinline__ void init(const Params& P, int lane_, float* records)
    {
        lane = lane_;
        const float dstep = P.d_step * kLlSqrtLog2e, astep = P.a_step * kLlSqrtLog2e;
        cd_lo = (float)(lane + 1) * dstep; cd_hi = (float)(lane + 33) * dstep;
        // angle Gaussian k sits at (angle_dim - 1 - k) steps; this lane owns k = lane and k = lane + 32
        ca_lo = (float)(P.angle_dim - 1 - lane) * astep; ca_hi = (float)(P.angle_dim - 33 - lane) * astep;
        win_d = (unsigned)P.win_dist; win_a = (unsigned)P.win_ang;
        inv_d_interval = 1.0f / P.d_interval; d_cut_scaled = P.d_cut / P.d_interval;
        xd_scale = dstep / P.d_interval;
        inv_a_interval = P.angle_dim > 1 ? 1.0f / P.a_interval : 0.0f;
        xa_scale = P.a_sigma_inv * kLlSqrtLog2e;
        wide_d = P.win_dist > 32;
        tb = reinterpret_cast<float4*>(records);
    }

    __device__ __forceinline__ void reset()
    {
        sd[0] = sd[1] = qd[0] = qd[1] = 0.f;
#pragma unroll
        for (int x = 0; x < 3; x++) sa[x][0] = sa[x][1] = qa[x][0] = qa[x][1] = 0.f;
        sum_l = px_l = 0.f;
    }

    // log of a translation's weight; adds its contribution to the normaliser (and, backward, to sum p d^2)
    __device__ __forceinline__ float weigh(const float d2)
    {
        const float arg = REFZ ? fmaf(a, d2, -ref) : a * (d2 - ref);
        const float w = ex2_approx(arg * kLlLog2e);
        sum_l += w;
        if (BWD) px_l = fmaf(w, d2, px_l);
        return arg;
    }

    // One group of up to 32 translations, one per lane: window records of the lanes that keep theirs, then
    // the walk over these survivors.  (dx, dy, dz) is read only where keep is set.
    __device__ __forceinline__ void expand(const Params& P, const bool keep, const float arg, const float d2,
                                           const float dx, const float dy, const float dz)
    {
        float2* tb2 = reinterpret_cast<float2*>(tb + 32);
        if (keep) {
            // d and 1/d from one reciprocal square root plus a Newton step; quotients by the basis spacings
            // become products with their reciprocals (last-bit differences from IEEE sqrt / division)
            float rinv = rsqrtf(fmaxf(d2, 1e-30f));
            rinv = rinv * fmaf(-0.5f * d2 * rinv, rinv, 1.5f);
            const float d = d2 * rinv;
            int lo_d = 0;
            if (P.windowed_dist) {
                lo_d = (int)(fmaf(d, inv_d_interval, -d_cut_scaled) - 1.0f);
                lo_d = min(max(lo_d, 0), 64 - P.win_dist);
            }
            const float xd = -d * xd_scale;
            float xa[3] = {0.f, 0.f, 0.f};
            int lo_pack = lo_d;
            if (ANG) {
#pragma unroll
                for (int x = 0; x < 3; x++) {
                    float cosv = 1e3f;
                    if (d2 > 1e-5f) cosv = fmaf(dz, fz[x], fmaf(dy, fy[x], dx * fx[x])) * rinv;
                    if (P.cos_abs) cosv = fabsf(cosv);
                    int lo = 0;
                    if (P.windowed_ang) {
                        const float en = fmaf(cosv + 1.0f + P.a_cut, inv_a_interval, 1.0f);
                        int end = (int)fminf(en, (float)P.angle_dim);
                        end = max(end, P.win_ang);
                        lo = end - P.win_ang;
                    }
                    xa[x] = (1.0f - cosv) * xa_scale;
                    lo_pack |= lo << (8 * (x + 1));
                }
            }
            tb[lane] = make_float4(arg * kLlLog2e, xd, xa[0], xa[1]);     // log2 of the weight
            if (BWD) tb[32 + lane] = make_float4(xa[2], __int_as_float(lo_pack), d2, 0.f);
            else tb2[lane] = make_float2(xa[2], __int_as_float(lo_pack));
        }
        unsigned mask = __ballot_sync(0xffffffffu, keep);
        __syncwarp();
        while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const float4 r0 = tb[src];
            float4 r1;
            if (BWD) { r1 = tb[32 + src]; } else { const float2 t = tb2[src]; r1 = make_float4(t.x, t.y, 0.f, 0.f); }
            const float lw = r0.x, d2s = r1.z;          // Gaussian times weight = ex2(lw - b*b)
            const int lo_pack = __float_as_int(r1.y);
            {   // distance basis
                const int lo = (int)__byte_perm((unsigned)lo_pack, 0u, 0x4440);
                const bool in0 = (unsigned)(lane - lo) < win_d, in1 = (unsigned)(lane + 32 - lo) < win_d;
                if (!wide_d) {
                    const float b = r0.y + (in1 ? cd_hi : cd_lo);
                    const float g = ex2_approx(fmaf(-b, b, lw));
                    if (in0) { sd[0] += g; if (BWD) qd[0] = fmaf(g, d2s, qd[0]); }
                    if (in1) { sd[1] += g; if (BWD) qd[1] = fmaf(g, d2s, qd[1]); }
                } else {
                    const float b0 = r0.y + cd_lo, b1 = r0.y + cd_hi;
                    const float g0 = ex2_approx(fmaf(-b0, b0, lw)), g1 = ex2_approx(fmaf(-b1, b1, lw));
                    if (in0) { sd[0] += g0; if (BWD) qd[0] = fmaf(g0, d2s, qd[0]); }
                    if (in1) { sd[1] += g1; if (BWD) qd[1] = fmaf(g1, d2s, qd[1]); }
                }
            }
            if (ANG) {
                const float xa[3] = {r0.z, r0.w, r1.x};
#pragma unroll
                for (int x = 0; x < 3; x++) {
                    const int lo = (int)__byte_perm((unsigned)lo_pack, 0u, 0x4441 + x);
                    const float b0 = xa[x] - ca_lo, b1 = xa[x] - ca_hi;
                    const float g0 = ex2_approx(fmaf(-b0, b0, lw)), g1 = ex2_approx(fmaf(-b1, b1, lw));
                    if ((unsigned)(lane - lo) < win_a) { sa[x][0] += g0; if (BWD) qa[x][0] = fmaf(g0, d2s, qa[x][0]); }
                    if ((unsigned)(lane + 32 - lo) < win_a) { sa[x][1] += g1; if (BWD) qa[x][1] = fmaf(g1, d2s, qa[x][1]); }
                }
            }
        }
        __syncwarp();
    }

    // The pair's translations from its sorted list (list = the pair's kListStride floats).  Forward: sets
    // ref = d^2_min first.  All listed translations enter the normaliser; the groups that hold survivors
    // come first and the loop stops at the first group without any.
    __device__ __forceinline__ void run_list(const Params& P, const float* __restrict__ list)
    {
        const float* Ll = list + lane;
        const float dl0 = __ldg(Ll), dl1 = __ldg(Ll + 32), dl2 = __ldg(Ll + 64), dl3 = __ldg(Ll + 96);
        const float lx0 = __ldg(Ll + kListLen), ly0 = __ldg(Ll + 2 * kListLen), lz0 = __ldg(Ll + 3 * kListLen);
        if (!REFZ) ref = __shfl_sync(0xffffffffu, dl0, 0);
        const float a0 = weigh(dl0), a1 = weigh(dl1), a2 = weigh(dl2), a3 = weigh(dl3);
        for (int g = 0; g < kListLen / 32; g++) {
            const float d2 = g == 0 ? dl0 : (g == 1 ? dl1 : (g == 2 ? dl2 : dl3));
            const float arg = g == 0 ? a0 : (g == 1 ? a1 : (g == 2 ? a2 : a3));
            const bool keep = arg > -P.prune;
            if (!__any_sync(0xffffffffu, keep)) break;
            float dx = lx0, dy = ly0, dz = lz0;
            if (g > 0 && keep) {
                const float* Lg = Ll + g * 32;
                dx = __ldg(Lg + kListLen); dy = __ldg(Lg + 2 * kListLen); dz = __ldg(Lg + 3 * kListLen);
            }
            expand(P, keep, arg, d2, dx, dy, dz);
        }
    }

    // The pair's translations by slab sweeps over (n1; n2, n3), for lattice ranges without a list.
    // r = separation of the pair, t1..t3 = cell vectors.  Forward: finds d^2_min first.
    __device__ __forceinline__ void run_slabs(const Params& P, const int R1, const int R2, const int R3,
                                              const float rx, const float ry, const float rz, const float* __restrict__ Tc)
    {
        const float t1x = __ldg(Tc), t1y = __ldg(Tc + 1), t1z = __ldg(Tc + 2);
        const float t2x = __ldg(Tc + 3), t2y = __ldg(Tc + 4), t2z = __ldg(Tc + 5);
        const float t3x = __ldg(Tc + 6), t3y = __ldg(Tc + 7), t3z = __ldg(Tc + 8);
        const int L1 = 2 * R1 + 1, L3 = 2 * R3 + 1, L23 = (2 * R2 + 1) * L3;
        const int nSub = (L23 + 31) >> 5;
        const float invL3 = 1.0f / (float)L3;
        for (int pass = REFZ ? 1 : 0; pass < 2; pass++) {
            float d2min = 1e10f;
            for (int sub = 0; sub < nSub; sub++) {
                const int idx = sub * 32 + lane;
                int q2 = (int)(((float)idx + 0.5f) * invL3), r3 = idx - q2 * L3;
                if (r3 < 0) { q2--; r3 += L3; } else if (r3 >= L3) { q2++; r3 -= L3; }
                const float n2 = ll_int_to_float(q2 - R2), n3 = ll_int_to_float(r3 - R3);
                const float ox = fmaf(t3x, n3, fmaf(t2x, n2, rx)), oy = fmaf(t3y, n3, fmaf(t2y, n2, ry)),
                            oz = fmaf(t3z, n3, fmaf(t2z, n2, rz));
                const bool valid = idx < L23;
                for (int k1 = 0; k1 < L1; k1++) {
                    const float n1 = ll_int_to_float(k1 - R1);
                    const float dx = fmaf(t1x, n1, ox), dy = fmaf(t1y, n1, oy), dz = fmaf(t1z, n1, oz);
                    const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                    if (pass == 0) {
                        if (valid) d2min = fminf(d2min, d2);
                    } else {
                        float arg = -1e30f;
                        if (valid) arg = weigh(d2);
                        expand(P, arg > -P.prune, arg, d2, dx, dy, dz);
                    }
                }
            }
            if (pass == 0) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) d2min = fminf(d2min, __shfl_xor_sync(0xffffffffu, d2min, o));
                ref = d2min;
            }
        }
    }
};

}  // namespace cfb
