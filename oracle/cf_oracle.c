/*
 * CPU oracle for the periodic lattice-sum attention path of CrystalFramer.
 *
 * THIS IS TEST INFRASTRUCTURE.  It is a plain-C restatement of the reference's
 * algorithm, used only by tests, by the smoke check and by the CPU baseline leg
 * of the benchmark.  The product (the CUDA library) never links or calls it.
 *
 * Every routine names the reference file and lines whose arithmetic it restates
 * (paths are relative to the reference project root).  The restatement follows
 * the reference's float expressions literally where an integer decision hangs on
 * them (lattice range, window start/end, image selection); compile with
 * -ffp-contract=off so that the C compiler does not fuse what is written here.
 *
 * The file is compiled twice: REAL=float (symbols cfo_*_f32, the parity oracle)
 * and REAL=double (symbols cfo_*_f64, used to judge which side of a float
 * disagreement is closer to the exact value).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL float
#endif

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#ifdef REAL_IS_DOUBLE
#define FN(name) CAT(name, _f64)
#define R_SQRT sqrt
#define R_EXP exp
#define R_LOG log
#define R_FABS fabs
#define R_FMIN fmin
#define R_FMAX fmax
#else
#define FN(name) CAT(name, _f32)
#define R_SQRT sqrtf
#define R_EXP expf
#define R_LOG logf
#define R_FABS fabsf
#define R_FMIN fminf
#define R_FMAX fmaxf
#endif

typedef REAL real;

/* float-rounded pi, as CUDART_PI_F in math_constants.h */
#define PI_F 3.141592654f

typedef struct {
    int32_t H;             /* heads                                             */
    int32_t head_dim;      /* q/k/v head dimension (K_HEAD_DIM == V_HEAD_DIM)    */
    int32_t D_dist;        /* VPE_DIM: number of distance Gaussians              */
    int32_t D_ang;         /* ANGLE_ENC_DIM: number of angle Gaussians per axis  */
    int32_t lattice_range; /* LATTICE_RANGE                                      */
    int32_t minimum_range; /* MINIMUM_RANGE (0 = off)                            */
    int32_t cos_abs;       /* COS_ABS                                            */
    int32_t win_dist;      /* LENGTH_RANGE                                       */
    int32_t win_ang;       /* ANGLE_RANGE                                        */
    int32_t cut_sigma;     /* CUT_SIGMA                                          */
    float dist_max;
    float wscale_dist;
    float angle_sigma;
    float c_dist;          /* length_rbf_mul                                     */
    float c_ang;           /* angle_rbf_mul                                      */
    float cutoff_radius;   /* <0: adaptive, multiple of sigma; 0: fixed range    */
    float symm_break_noise;
} cfo_config;

/* --------------------------------------------------------------------------
 * Counter-based uniform in (0,1] for the symmetry-breaking noise.  The
 * reference draws from curand XORWOW streams seeded from numpy's global RNG
 * (models/cuda_funcs/calc_maximum_frame.py:43); nothing pins those streams, so
 * this restatement and the CUDA library share this hash instead.
 * -------------------------------------------------------------------------- */
static inline float cfo_uniform(uint64_t seed, uint64_t tid, uint32_t draw)
{
    uint64_t x = seed ^ (tid * 0x9E3779B97F4A7C15ull) ^ ((uint64_t)draw * 0xD1B54A32D192ED03ull);
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return (float)((uint32_t)(x >> 40) + 1u) * (1.0f / 16777216.0f);
}

/* --------------------------------------------------------------------------
 * Pair list: models/indexed_latticeformer_encoder.py:15-32 (get_edge_index)
 * and the CSR offsets of models/cuda_funcs/fused_dpa.py:24-26.
 * -------------------------------------------------------------------------- */
void FN(cfo_edge_index)(const int64_t* sizes, int64_t B, int64_t* edges /* (2,E) */,
                        int64_t* e_start /* (N+1) */, int64_t E)
{
    int64_t atom0 = 0, e = 0;
    for (int64_t c = 0; c < B; c++) {
        int64_t n = sizes[c];
        for (int64_t i = 0; i < n; i++) {
            e_start[atom0 + i] = e;
            for (int64_t j = 0; j < n; j++, e++) {
                edges[e] = atom0 + i;
                edges[E + e] = atom0 + j;
            }
        }
        atom0 += n;
    }
    e_start[atom0] = e;
}

/* --------------------------------------------------------------------------
 * Lattice range per (atom, head):
 * models/kernels/real_enc_frame_proj_fwd_length.cu:59-86 (the same block opens
 * every lattice kernel).  cutoff and (cutoff+0.01f)*rvl are float, the division
 * by 2.0*CUDART_PI_F is double, ceil is double, the result is cast to int.
 * -------------------------------------------------------------------------- */
static inline void lattice_range(const cfo_config* cfg, float a, const float* rvlen3, int R[3])
{
    R[0] = R[1] = R[2] = cfg->lattice_range;
    float cutoff = cfg->cutoff_radius;
    if (cutoff != 0.0f) {
        if (cutoff < 0) cutoff = sqrtf(-0.5f / a) * (-cutoff);
        for (int d = 0; d < 3; d++) {
            float num = (cutoff + 0.01f) * rvlen3[d];
            R[d] = (int)ceil((double)num / (2.0 * (double)PI_F));
            if (cfg->minimum_range > 0 && R[d] < cfg->minimum_range) R[d] = cfg->minimum_range;
        }
    }
}

void FN(cfo_lattice_range)(const cfo_config* cfg, const float* a_ik, const float* rvlen /* (B,3) */,
                           const int64_t* batch_i, int64_t N, int32_t* R_out /* (N,H,3) */)
{
    for (int64_t i = 0; i < N; i++)
        for (int k = 0; k < cfg->H; k++) {
            int R[3];
            lattice_range(cfg, a_ik[i * cfg->H + k], rvlen + 3 * batch_i[i], R);
            for (int d = 0; d < 3; d++) R_out[(i * cfg->H + k) * 3 + d] = R[d];
        }
}

/* Translated separation: the reference writes r + t1*n1 + t2*n2 + t3*n3 with
 * float loop counters (real_enc_frame_proj_fwd_length.cu:91-98). */
#define FOR_TRANSLATIONS(R)                                    \
    for (real n1 = -(real)(R)[0]; n1 <= (real)(R)[0]; n1++)    \
    for (real n2 = -(real)(R)[1]; n2 <= (real)(R)[1]; n2++)    \
    for (real n3 = -(real)(R)[2]; n3 <= (real)(R)[2]; n3++)

#define SEPARATION(r, T)                                               \
    real dx = (r)[0] + (T)[0] * n1 + (T)[3] * n2 + (T)[6] * n3;        \
    real dy = (r)[1] + (T)[1] * n1 + (T)[4] * n2 + (T)[7] * n3;        \
    real dz = (r)[2] + (T)[2] * n1 + (T)[5] * n2 + (T)[8] * n3;        \
    real d2 = dx * dx + dy * dy + dz * dz;

/* --------------------------------------------------------------------------
 * Distance window: real_enc_frame_proj_fwd_length.cu:130-161.  Returns the first
 * basis index and fills g[0..count).
 * -------------------------------------------------------------------------- */
static inline int dist_window(const cfo_config* cfg, real d, real* g, int* count)
{
    const real step = (real)1.0 / ((real)cfg->wscale_dist * R_SQRT((real)2.0));
    const real interval = (real)cfg->dist_max / cfg->D_dist;
    const real sig = interval * (real)cfg->wscale_dist;
    if (cfg->D_dist - cfg->win_dist > 8) {
        int start = (int)((d - cfg->cut_sigma * sig) / interval - 1);
        if (start < 0) start = 0;
        if (start > cfg->D_dist - cfg->win_dist) start = cfg->D_dist - cfg->win_dist;
        real b = -d / interval * step + step * start;
        for (int m = 0; m < cfg->win_dist; m++) {
            b += step;
            g[m] = R_EXP(-b * b);
        }
        *count = cfg->win_dist;
        return start;
    }
    real b = -d / interval * step;
    for (int m = 0; m < cfg->D_dist; m++) {
        b += step;
        g[m] = R_EXP(-b * b);
    }
    *count = cfg->D_dist;
    return 0;
}

/* --------------------------------------------------------------------------
 * Angle window: real_enc_frame_proj_fwd_angle.cu:136-175.  g[m] belongs to basis
 * index first+m (the reference walks the window downwards from end_dim-1).
 * -------------------------------------------------------------------------- */
static inline int angle_window(const cfo_config* cfg, real dx, real dy, real dz, real d2,
                               const real* f, real* g, int* count)
{
    const int D = cfg->D_ang;
    const real span = cfg->cos_abs ? (real)1.0 : (real)2.0;
    const real asig = (real)cfg->angle_sigma;
    const real step = span / ((D - 1) * asig * R_SQRT((real)2));
    const real interval = span / (D - 1);
    const real sigma_inv = (real)1.0 / (asig * R_SQRT((real)2));
    real c = (real)1e3;
    if ((double)d2 > 1e-5) c = (dx * f[0] + dy * f[1] + dz * f[2]) / R_SQRT(d2);
    if (cfg->cos_abs) c = R_FABS(c);
    if (D - cfg->win_ang > 8) {
        real e = (c + (real)1.0 + cfg->cut_sigma * asig) / interval + (real)1.0;
        if (e > (real)D) e = (real)D;
        int end = (int)e;
        if (end < cfg->win_ang) end = cfg->win_ang;
        real ang = (-c + (real)1.0) * sigma_inv - (D - end) * step;
        for (int m = 0; m < cfg->win_ang; m++) {
            g[cfg->win_ang - 1 - m] = R_EXP(-ang * ang);
            ang -= step;
        }
        *count = cfg->win_ang;
        return end - cfg->win_ang;
    }
    real ang = (-c + (real)1.0) * sigma_inv - (D - 1) * step;
    for (int m = 0; m < D; m++) {
        g[m] = R_EXP(-ang * ang);
        ang += step;
    }
    *count = D;
    return 0;
}

/* --------------------------------------------------------------------------
 * Forward: log-sum-exp bias and frame-projected value encoding.
 *   real_enc_frame_proj_fwd_length.cu:88-194, real_enc_frame_proj_fwd_angle.cu:84-208,
 *   host scaling models/cuda_funcs/real_space_framed_proj.py:84,105.
 * W_d: (H,hd,D_dist); W_a: (3,H,hd,D_ang) or NULL; frames: (3,N,H,3).
 * Optional debug outputs: R_eh (E,H,3) is not produced here, see cfo_lattice_range.
 * -------------------------------------------------------------------------- */
void FN(cfo_framed_proj_fwd)(const cfo_config* cfg, const real* a_ik, const real* rpos /* (E,3) */,
                             const real* tvecs /* (B,3,3) */, const float* rvlen /* (B,3) */,
                             const int64_t* batch_i, const int64_t* edges, int64_t N, int64_t E,
                             const real* W_d, const real* W_a, const real* frames,
                             real* z_ek, real* v_ekd)
{
    const int H = cfg->H, hd = cfg->head_dim, Dd = cfg->D_dist, Da = cfg->D_ang;
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t e = 0; e < E; e++) {
        const int64_t i = edges[e];
        const int64_t c = batch_i[i];
        const real* r = rpos + 3 * e;
        const real* T = tvecs + 9 * c;
        real sd[512], sa[3][512], g[512];
        for (int k = 0; k < H; k++) {
            const real a = a_ik[i * H + k];
            int R[3];
            lattice_range(cfg, (float)a, rvlen + 3 * c, R);
            real d2min = (real)1e10;
            FOR_TRANSLATIONS(R) { SEPARATION(r, T); (void)dx; (void)dy; (void)dz; d2min = R_FMIN(d2min, d2); }
            for (int m = 0; m < Dd; m++) sd[m] = 0;
            for (int ax = 0; ax < 3; ax++) for (int m = 0; m < Da; m++) sa[ax][m] = 0;
            real sum = 0;
            FOR_TRANSLATIONS(R) {
                SEPARATION(r, T);
                real w = R_EXP(a * (d2 - d2min));
                sum += w;
                if (Dd > 0 && v_ekd) {
                    int cnt, first = dist_window(cfg, R_SQRT(d2), g, &cnt);
                    for (int m = 0; m < cnt; m++) sd[first + m] += g[m] * w;
                }
                if (W_a && v_ekd) {
                    for (int ax = 0; ax < 3; ax++) {
                        const real* f = frames + ((ax * N + i) * H + k) * 3;
                        int cnt, first = angle_window(cfg, dx, dy, dz, d2, f, g, &cnt);
                        for (int m = 0; m < cnt; m++) sa[ax][first + m] += g[m] * w;
                    }
                }
            }
            z_ek[e * H + k] = R_LOG(sum) + d2min * a;
            if (!v_ekd) continue;
            real* v = v_ekd + (e * H + k) * hd;
            for (int o = 0; o < hd; o++) {
                real acc = 0;
                const real* W = W_d + ((int64_t)k * hd + o) * Dd;
                for (int m = 0; m < Dd; m++) acc += W[m] * sd[m];
                real out = acc / sum * (real)cfg->c_dist;
                if (W_a) {
                    real outa = 0;
                    for (int ax = 0; ax < 3; ax++) {
                        const real* Wx = W_a + (((int64_t)ax * H + k) * hd + o) * Da;
                        real accx = 0;
                        for (int m = 0; m < Da; m++) accx += Wx[m] * sa[ax][m];
                        outa += accx / sum;
                    }
                    out += outa * (real)cfg->c_ang;
                }
                v[o] = out;
            }
        }
    }
}

/* --------------------------------------------------------------------------
 * Backward by recomputation with p = exp(a d^2 - z):
 *   real_enc_frame_proj_bwd_length.cu:100-237, real_enc_frame_proj_bwd_angle.cu:104-275,
 *   host scalings models/cuda_funcs/real_space_framed_proj.py:183,209-212.
 * As in the reference, the whole length-kernel result (including the gz term) is
 * multiplied by c_dist, the angle parts by c_ang, gW_d is left unscaled and gW_a
 * is scaled by c_ang.  Weight gradients are returned summed over atoms, which is
 * what autograd's sum_to_size makes of the reference's per-atom (N,H,hd,D) output.
 * -------------------------------------------------------------------------- */
void FN(cfo_framed_proj_bwd)(const cfo_config* cfg, const real* a_ik, const real* rpos,
                             const real* tvecs, const float* rvlen, const int64_t* batch_i,
                             const int64_t* edges, const int64_t* e_start, int64_t N, int64_t E,
                             const real* W_d, const real* W_a, const real* frames,
                             const real* z_ek, const real* gz_ek, const real* gv_ekd,
                             real* ga_ik /* (N,H) */, real* gW_d /* (H,hd,Dd) */,
                             real* gW_a /* (3,H,hd,Da) */)
{
    const int H = cfg->H, hd = cfg->head_dim, Dd = cfg->D_dist, Da = cfg->D_ang;
    const int64_t nWd = (int64_t)H * hd * Dd, nWa = (int64_t)3 * H * hd * Da;
    memset(gW_d, 0, sizeof(real) * nWd);
    if (W_a) memset(gW_a, 0, sizeof(real) * nWa);
    int nthreads = 1;
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    extern int omp_get_thread_num(void);
    nthreads = omp_get_max_threads();
#endif
    real* part_d = (real*)calloc((size_t)nthreads * nWd, sizeof(real));
    real* part_a = W_a ? (real*)calloc((size_t)nthreads * nWa, sizeof(real)) : NULL;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < N; i++) {
        int th = 0;
#ifdef _OPENMP
        th = omp_get_thread_num();
#endif
        real* pd = part_d + (size_t)th * nWd;
        real* pa = part_a ? part_a + (size_t)th * nWa : NULL;
        const int64_t c = batch_i[i];
        const real* T = tvecs + 9 * c;
        real g[512], sv[512], Gv[512];
        for (int k = 0; k < H; k++) {
            const real a = a_ik[i * H + k];
            int R[3];
            lattice_range(cfg, (float)a, rvlen + 3 * c, R);
            real ga_len = 0, ga_ang = 0;
            for (int64_t e = e_start[i]; e < e_start[i + 1]; e++) {
                const real* r = rpos + 3 * e;
                const real z = z_ek[e * H + k];
                const real* gv = gv_ekd + (e * H + k) * hd;
                /* ---- length part ---- */
                {
                    for (int m = 0; m < Dd; m++) { Gv[m] = 0; sv[m] = 0; }
                    for (int o = 0; o < hd; o++) {
                        const real* W = W_d + ((int64_t)k * hd + o) * Dd;
                        for (int m = 0; m < Dd; m++) Gv[m] += W[m] * gv[o];
                    }
                    real px_avr = 0, pbg_avr = 0, sum_v = 0;
                    FOR_TRANSLATIONS(R) {
                        SEPARATION(r, T); (void)dx; (void)dy; (void)dz;
                        real p = R_EXP(a * d2 - z);
                        real px = d2 * p;
                        px_avr += px;
                        int cnt, first = dist_window(cfg, R_SQRT(d2), g, &cnt);
                        real bg = 0;
                        for (int m = 0; m < cnt; m++) {
                            bg += g[m] * Gv[first + m];
                            sv[first + m] += g[m] * p;
                        }
                        sum_v += px * bg;
                        pbg_avr += p * bg;
                    }
                    ga_len += px_avr * gz_ek[e * H + k];
                    ga_len += sum_v - px_avr * pbg_avr;
                    for (int o = 0; o < hd; o++)
                        for (int m = 0; m < Dd; m++) pd[((int64_t)k * hd + o) * Dd + m] += sv[m] * gv[o];
                }
                /* ---- angle parts ---- */
                if (W_a) for (int ax = 0; ax < 3; ax++) {
                    const real* f = frames + ((ax * N + i) * H + k) * 3;
                    for (int m = 0; m < Da; m++) { Gv[m] = 0; sv[m] = 0; }
                    for (int o = 0; o < hd; o++) {
                        const real* W = W_a + (((int64_t)ax * H + k) * hd + o) * Da;
                        for (int m = 0; m < Da; m++) Gv[m] += W[m] * gv[o];
                    }
                    real px_avr = 0, pbg_avr = 0, sum_v = 0;
                    FOR_TRANSLATIONS(R) {
                        SEPARATION(r, T);
                        real p = R_EXP(a * d2 - z);
                        real px = d2 * p;
                        px_avr += px;
                        int cnt, first = angle_window(cfg, dx, dy, dz, d2, f, g, &cnt);
                        real bg = 0;
                        for (int m = 0; m < cnt; m++) {
                            bg += g[m] * Gv[first + m];
                            sv[first + m] += g[m] * p;
                        }
                        sum_v += px * bg;
                        pbg_avr += p * bg;
                    }
                    ga_ang += sum_v - px_avr * pbg_avr;
                    for (int o = 0; o < hd; o++)
                        for (int m = 0; m < Da; m++)
                            pa[(((int64_t)ax * H + k) * hd + o) * Da + m] += sv[m] * gv[o];
                }
            }
            ga_ik[i * H + k] = ga_len * (real)cfg->c_dist + ga_ang * (real)cfg->c_ang;
        }
    }
    for (int t = 0; t < nthreads; t++) {
        for (int64_t m = 0; m < nWd; m++) gW_d[m] += part_d[(size_t)t * nWd + m];
        if (W_a) for (int64_t m = 0; m < nWa; m++) gW_a[m] += part_a[(size_t)t * nWa + m] * (real)cfg->c_ang;
    }
    free(part_d);
    free(part_a);
}

/* --------------------------------------------------------------------------
 * Frame construction, per (pair, head) candidates.
 *   first axis : models/kernels/compute_maximum_frame_each_edge.cu:81-111
 *   second axis: models/kernels/compute_second_frame_each_edge.cu:81-142
 * When no image qualifies the reference leaves its outputs uninitialised; here
 * the direction is zero and the score keeps its starting value.
 * sel_image is the linear translation index ((n1+R1)*(2R2+1)+(n2+R2))*(2R3+1)+(n3+R3).
 * -------------------------------------------------------------------------- */
void FN(cfo_frame1_edges)(const cfo_config* cfg, const real* a_ik, const real* rpos, const real* tvecs,
                          const float* rvlen, const int64_t* batch_i, const int64_t* edges,
                          int64_t N, int64_t E, uint64_t seed,
                          real* dir /* (E,H,3) */, real* value /* (E,H) */, int32_t* sel_image /* (E,H) */)
{
    const int H = cfg->H;
    (void)N;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t e = 0; e < E; e++) {
        const int64_t i = edges[e], c = batch_i[i];
        const real* r = rpos + 3 * e;
        const real* T = tvecs + 9 * c;
        for (int k = 0; k < H; k++) {
            const real a = a_ik[i * H + k];
            int R[3];
            lattice_range(cfg, (float)a, rvlen + 3 * c, R);
            real d2_min = (real)1e10, bx = 0, by = 0, bz = 0;
            int32_t t = 0, best = -1;
            FOR_TRANSLATIONS(R) {
                SEPARATION(r, T);
                real d = R_SQRT(d2);
                if ((double)d2 > 1e-5) {
                    real noise = 0;
                    if (cfg->symm_break_noise != 0.0f)
                        noise = (real)(float)(((double)cfo_uniform(seed, (uint64_t)(e * H + k), (uint32_t)t) - 0.5) *
                                              (double)cfg->symm_break_noise);
                    if (d2_min > d2 + noise) {
                        d2_min = d2 + noise;
                        bx = dx / d; by = dy / d; bz = dz / d;
                        best = t;
                    }
                }
                t++;
            }
            real* o = dir + (e * H + k) * 3;
            o[0] = bx; o[1] = by; o[2] = bz;
            value[e * H + k] = a * d2_min;
            sel_image[e * H + k] = best;
        }
    }
}

/* is_static: the "max_static" variant (models/kernels/compute_second_frame_static_each_edge.cu:126,135), whose
 * score is (d^2 - d^2_min) + log(...) and whose value is score + d^2_min -- the Gaussian coefficient does not
 * enter, so the score GROWS with the distance. */
static void FN(frame2_edges_impl)(const cfo_config* cfg, int is_static, const real* a_ik, const real* rpos, const real* tvecs,
                                  const float* rvlen, const int64_t* batch_i, const int64_t* edges,
                                  int64_t N, int64_t E, uint64_t seed, const real* frame1 /* (N,H,3) */,
                                  real* dir, real* value, int32_t* sel_image)
{
    const int H = cfg->H;
    (void)N;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t e = 0; e < E; e++) {
        const int64_t i = edges[e], c = batch_i[i];
        const real* r = rpos + 3 * e;
        const real* T = tvecs + 9 * c;
        for (int k = 0; k < H; k++) {
            const real a = a_ik[i * H + k];
            const real* f1 = frame1 + (i * H + k) * 3;
            int R[3];
            lattice_range(cfg, (float)a, rvlen + 3 * c, R);
            real d2min = (real)1e10;
            FOR_TRANSLATIONS(R) {
                SEPARATION(r, T); (void)dx; (void)dy; (void)dz;
                if ((double)d2 > 1e-5) d2min = R_FMIN(d2min, d2);
            }
            /* arg-max of score + noise, first translation on equal values.  With the noise off this
             * is what the reference's running comparison (score > max_val + rand, :130) selects;
             * with noise on the reference adds the noise asymmetrically (to the running maximum of
             * the earlier winner and again to the challenger's threshold), which makes its result
             * depend on the loop order -- that case is unpinned and the symmetric rule is used. */
            real max_val = (real)-1e15, bx = 0, by = 0, bz = 0, bval = (real)-1e15;
            int32_t t = 0, best = -1;
            FOR_TRANSLATIONS(R) {
                SEPARATION(r, T);
                real d = R_SQRT(d2);
                if ((double)d2 > 1e-5) {
                    real ux = dx / d, uy = dy / d, uz = dz / d;
                    real cs = ux * f1[0] + uy * f1[1] + uz * f1[2];
                    real one_m = (real)1 - R_FABS(cs);
                    real clipped = ((double)one_m > 1e-5) ? one_m : (real)1e-5;
                    real score = (is_static ? (d2 - d2min) : a * (d2 - d2min)) + R_LOG(clipped);
                    real noisy = score;
                    if (cfg->symm_break_noise != 0.0f)
                        noisy = score + (real)(float)(((double)cfo_uniform(seed, (uint64_t)(e * H + k), (uint32_t)t) - 0.5) *
                                                      (double)cfg->symm_break_noise);
                    if (noisy > max_val && (double)R_FABS(cs) < 0.9999) {
                        max_val = noisy;
                        bx = ux; by = uy; bz = uz;
                        bval = score + (is_static ? d2min : a * d2min);
                        best = t;
                    }
                }
                t++;
            }
            real* o = dir + (e * H + k) * 3;
            o[0] = bx; o[1] = by; o[2] = bz;
            value[e * H + k] = bval;
            sel_image[e * H + k] = best;
        }
    }
}

void FN(cfo_frame2_edges)(const cfo_config* cfg, const real* a_ik, const real* rpos, const real* tvecs,
                          const float* rvlen, const int64_t* batch_i, const int64_t* edges,
                          int64_t N, int64_t E, uint64_t seed, const real* frame1, real* dir, real* value, int32_t* sel_image)
{
    FN(frame2_edges_impl)(cfg, 0, a_ik, rpos, tvecs, rvlen, batch_i, edges, N, E, seed, frame1, dir, value, sel_image);
}

void FN(cfo_frame2_static_edges)(const cfo_config* cfg, const real* a_ik, const real* rpos, const real* tvecs,
                                 const float* rvlen, const int64_t* batch_i, const int64_t* edges,
                                 int64_t N, int64_t E, uint64_t seed, const real* frame1, real* dir, real* value,
                                 int32_t* sel_image)
{
    FN(frame2_edges_impl)(cfg, 1, a_ik, rpos, tvecs, rvlen, batch_i, edges, N, E, seed, frame1, dir, value, sel_image);
}

/* Third axis of the frame method "max_wo_orthogonal" (models/kernels/compute_third_frame_each_edge.cu:93-150,
 * models/cuda_funcs/calc_maximum_frame.py:173-245): per (pair, head) the image maximising
 * a (d^2 - d^2_min) + log(max(|det(f1, f2, u)|, 1e-5)) among the images with |det| > 1e-5, u the unit vector to the
 * image; value = score + a d^2_min.  Where no image qualifies the reference leaves its outputs unwritten; here the
 * direction is zero and the value -1e15, which no selection picks.  Noise: the symmetric rule of the second axis. */
void FN(cfo_frame3_edges)(const cfo_config* cfg, const real* a_ik, const real* rpos, const real* tvecs,
                          const float* rvlen, const int64_t* batch_i, const int64_t* edges, int64_t N, int64_t E,
                          uint64_t seed, const real* frame1 /* (N,H,3) */, const real* frame2 /* (N,H,3) */,
                          real* dir, real* value, int32_t* sel_image)
{
    const int H = cfg->H;
    (void)N;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t e = 0; e < E; e++) {
        const int64_t i = edges[e], c = batch_i[i];
        const real* r = rpos + 3 * e;
        const real* T = tvecs + 9 * c;
        for (int k = 0; k < H; k++) {
            const real a = a_ik[i * H + k];
            const real* f1 = frame1 + (i * H + k) * 3;
            const real* f2 = frame2 + (i * H + k) * 3;
            int R[3];
            lattice_range(cfg, (float)a, rvlen + 3 * c, R);
            real d2min = (real)1e10;
            FOR_TRANSLATIONS(R) {
                SEPARATION(r, T); (void)dx; (void)dy; (void)dz;
                if ((double)d2 > 1e-5) d2min = R_FMIN(d2min, d2);
            }
            real max_val = (real)-1e15, bx = 0, by = 0, bz = 0, bval = (real)-1e15;
            int32_t t = 0, best = -1;
            FOR_TRANSLATIONS(R) {
                SEPARATION(r, T);
                real d = R_SQRT(d2);
                if ((double)d2 > 1e-5) {
                    real ux = dx / d, uy = dy / d, uz = dz / d;
                    real det = f1[0] * f2[1] * uz + f1[1] * f2[2] * ux + f1[2] * f2[0] * uy - f1[2] * f2[1] * ux -
                               f1[1] * f2[0] * uz - f1[0] * f2[2] * uy;
                    real mag = R_FABS(det);
                    real clipped = ((double)mag > 1e-5) ? mag : (real)1e-5;
                    real score = a * (d2 - d2min) + R_LOG(clipped);
                    real noisy = score;
                    if (cfg->symm_break_noise != 0.0f)
                        noisy = score + (real)(float)(((double)cfo_uniform(seed, (uint64_t)(e * H + k), (uint32_t)t) - 0.5) *
                                                      (double)cfg->symm_break_noise);
                    if (noisy > max_val && (double)mag > 1e-5) {
                        max_val = noisy;
                        bx = ux; by = uy; bz = uz;
                        bval = score + a * d2min;
                        best = t;
                    }
                }
                t++;
            }
            real* o = dir + (e * H + k) * 3;
            o[0] = bx; o[1] = by; o[2] = bz;
            value[e * H + k] = bval;
            sel_image[e * H + k] = best;
        }
    }
}

/* --------------------------------------------------------------------------
 * Lattice frames: the three shortest lattice vectors of the atom's cell, per (atom, head)
 * (models/kernels/compute_lattice_first_frame.cu:86-110, compute_lattice_second_frame.cu:95-130,
 * compute_lattice_third_frame.cu:96-170; host glue models/cuda_funcs/calc_lattice_frame.py:22-150).
 * Only the self pair (i == j, separation 0) takes part, so the frames depend on the cell and, through
 * the lattice ranges, on the Gaussian coefficient.  Axis 1: the shortest translation; axis 2: the shortest
 * translation not collinear with axis 1 (1 - |cos| > 1e-5), flipped to the side of axis 1; axis 3: the
 * shortest translation out of their plane (|cos to the normalised cross product| > 1e-5), flipped to the side
 * of axis 1; finally all three are negated when axis 3 points against the cross product.  Running minimum with
 * strict comparison: the first translation in loop order wins on equal lengths.  Outputs are zero where no
 * translation qualifies (the reference leaves them uninitialised).  seeds: one per axis.
 * -------------------------------------------------------------------------- */
void FN(cfo_lattice_frames)(const cfo_config* cfg, const real* a_ik, const real* tvecs, const float* rvlen,
                            const int64_t* batch_i, int64_t N, const uint64_t* seeds, const int64_t* self_pair /* (N) */,
                            real* f1 /* (N,H,3) */, real* f2, real* f3)
{
    const int H = cfg->H;
    const real zero3[3] = {0, 0, 0};
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t i = 0; i < N; i++) {
        const int64_t c = batch_i[i];
        const real* T = tvecs + 9 * c;
        const real* r = zero3;
        for (int k = 0; k < H; k++) {
            const real a = a_ik[i * H + k];
            int R[3];
            lattice_range(cfg, (float)a, rvlen + 3 * c, R);
            const uint64_t tid = (uint64_t)(self_pair[i] * H + k);
            real* o1 = f1 + (i * H + k) * 3; real* o2 = f2 + (i * H + k) * 3; real* o3 = f3 + (i * H + k) * 3;
            for (int d = 0; d < 3; d++) o1[d] = o2[d] = o3[d] = 0;
            for (int axis = 0; axis < 3; axis++) {
                real d2_min = (real)1e10;
                real cx = 0, cy = 0, cz = 0;
                if (axis == 2) {
                    cx = o1[1] * o2[2] - o1[2] * o2[1];
                    cy = o1[2] * o2[0] - o1[0] * o2[2];
                    cz = o1[0] * o2[1] - o1[1] * o2[0];
                    real cn = R_SQRT(cx * cx + cy * cy + cz * cz);
                    cx = cx / cn; cy = cy / cn; cz = cz / cn;
                }
                int32_t t = 0;
                FOR_TRANSLATIONS(R) {
                    SEPARATION(r, T);
                    real d = R_SQRT(d2);
                    real noise = 0;
                    if (cfg->symm_break_noise != 0.0f)
                        noise = (real)(float)(((double)cfo_uniform(seeds[axis], tid, (uint32_t)t) - 0.5) * (double)cfg->symm_break_noise);
                    if (d2_min > d2 + noise && (double)d2 > 1e-5) {
                        real ux = dx / d, uy = dy / d, uz = dz / d;
                        if (axis == 0) {
                            d2_min = d2 + noise;
                            o1[0] = ux; o1[1] = uy; o1[2] = uz;
                        } else if (axis == 1) {
                            real cs = ux * o1[0] + uy * o1[1] + uz * o1[2];
                            if ((double)((real)1 - R_FABS(cs)) > 1e-5) {
                                real sg = cs < 0 ? (real)-1 : (real)1;
                                o2[0] = sg * ux; o2[1] = sg * uy; o2[2] = sg * uz;
                                d2_min = d2 + noise;
                            }
                        } else {
                            real cc = ux * cx + uy * cy + uz * cz;
                            real c1 = ux * o1[0] + uy * o1[1] + uz * o1[2];
                            if ((double)R_FABS(cc) > 1e-5) {
                                real sg = c1 < 0 ? (real)-1 : (real)1;
                                o3[0] = sg * ux; o3[1] = sg * uy; o3[2] = sg * uz;
                                d2_min = d2 + noise;
                            }
                        }
                    }
                    t++;
                }
                if (axis == 2) {
                    real cc = o3[0] * cx + o3[1] * cy + o3[2] * cz;
                    if (cc < 0) for (int d = 0; d < 3; d++) { o1[d] = -o1[d]; o2[d] = -o2[d]; o3[d] = -o3[d]; }
                }
            }
        }
    }
}

/* --------------------------------------------------------------------------
 * Weighted-PCA frames, per (pair, head) part: softmax-weighted second moments of the
 * separation vector over the translations, sigma = sum_n w_n d d^T / sum_n w_n (xx, xy, xz, yy,
 * yz, zz), models/kernels/real_enc_sigma_fwd.cu:92-165, plus the lattice-sum bias
 * z = log sum_n exp(a d^2) that the reference's pooling attention is meant to receive (the
 * reference hands it an uninitialised buffer, models/cuda_funcs/real_space_enc_proj.py:54,97-125).
 * near_d2 / near_dir: the nearest image with d^2 > 1e-5 (arg-min of d^2 + noise), from which the
 * per-atom tie-breaking matrix of real_enc_sigma_fwd.cu:150-159 is built.
 * -------------------------------------------------------------------------- */
void FN(cfo_sigma_edges)(const cfo_config* cfg, const real* a_ik, const real* rpos, const real* tvecs,
                         const float* rvlen, const int64_t* batch_i, const int64_t* edges,
                         int64_t N, int64_t E, uint64_t seed, real* z_ek, real* sigma /* (E,H,6) */,
                         real* near_d2 /* (E,H) */, real* near_dir /* (E,H,3) */)
{
    const int H = cfg->H;
    (void)N;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t e = 0; e < E; e++) {
        const int64_t i = edges[e], c = batch_i[i];
        const real* r = rpos + 3 * e;
        const real* T = tvecs + 9 * c;
        for (int k = 0; k < H; k++) {
            const real a = a_ik[i * H + k];
            int R[3];
            lattice_range(cfg, (float)a, rvlen + 3 * c, R);
            real d2min = (real)1e10;
            FOR_TRANSLATIONS(R) { SEPARATION(r, T); (void)dx; (void)dy; (void)dz; d2min = R_FMIN(d2min, d2); }
            real sum = 0, m[6] = {0, 0, 0, 0, 0, 0}, best = (real)1e8, bd[3] = {0, 0, 0};
            int32_t t = 0;
            FOR_TRANSLATIONS(R) {
                SEPARATION(r, T);
                real w = R_EXP(a * (d2 - d2min));
                sum += w;
                m[0] += dx * dx * w; m[1] += dx * dy * w; m[2] += dx * dz * w;
                m[3] += dy * dy * w; m[4] += dy * dz * w; m[5] += dz * dz * w;
                if ((double)d2 > 1e-5) {
                    real noise = 0;
                    if (cfg->symm_break_noise != 0.0f)
                        noise = (real)(float)(((double)cfo_uniform(seed, (uint64_t)(e * H + k), (uint32_t)t) - 0.5) *
                                              (double)cfg->symm_break_noise);
                    if (best > d2 + noise) {
                        best = d2 + noise;
                        real d = R_SQRT(d2);
                        bd[0] = dx / d; bd[1] = dy / d; bd[2] = dz / d;
                    }
                }
                t++;
            }
            for (int q = 0; q < 6; q++) sigma[(e * H + k) * 6 + q] = m[q] / sum;
            z_ek[e * H + k] = R_LOG(sum) + d2min * a;
            near_d2[e * H + k] = best;
            for (int q = 0; q < 3; q++) near_dir[(e * H + k) * 3 + q] = bd[q];
        }
    }
}

/* Per-(atom, head) selection: q_i.k_j + value, argmax over the atom's pairs
 * (models/cuda_funcs/calc_maximum_frame.py:72-84,146-163).  The reference leaves
 * ties to torch_scatter; here the lowest pair index wins.  The dot product is a
 * left-to-right fused-multiply-add chain so that it can be reproduced bit for bit. */
void FN(cfo_frame_select)(const cfo_config* cfg, const real* q /* (N,H,hd) */, const real* k,
                          const int64_t* edges, const int64_t* e_start, int64_t N, int64_t E,
                          const real* dir, const real* value, real* frame /* (N,H,3) */,
                          int64_t* sel_edge /* (N,H) */)
{
    const int H = cfg->H, hd = cfg->head_dim;
    for (int64_t i = 0; i < N; i++)
        for (int h = 0; h < H; h++) {
            real best = (real)-1e10;
            int64_t arg = -1;
            for (int64_t e = e_start[i]; e < e_start[i + 1]; e++) {
                const int64_t j = edges[E + e];
                real dot = 0;
                for (int d = 0; d < hd; d++)
#ifdef REAL_IS_DOUBLE
                    dot = fma(q[(i * H + h) * hd + d], k[(j * H + h) * hd + d], dot);
#else
                    dot = fmaf(q[(i * H + h) * hd + d], k[(j * H + h) * hd + d], dot);
#endif
                real s = dot + value[e * H + h];
                if (s > best) { best = s; arg = e; }
            }
            sel_edge[i * H + h] = arg;
            for (int d = 0; d < 3; d++) frame[(i * H + h) * 3 + d] = arg >= 0 ? dir[(arg * H + h) * 3 + d] : 0;
        }
}

/* Gram-Schmidt completion: models/indexed_lattice_multi_head_attention_cuda.py:475-481
 * (F.normalize divides by max(norm, 1e-12)). */
void FN(cfo_frame_complete)(const real* f1, const real* f2max, int64_t NH, real* f2, real* f3)
{
    for (int64_t t = 0; t < NH; t++) {
        const real* a = f1 + 3 * t; const real* b = f2max + 3 * t;
        real dot = a[0] * b[0] + a[1] * b[1] + a[2] * b[2];
        real u[3] = { b[0] - dot * a[0], b[1] - dot * a[1], b[2] - dot * a[2] };
        real nrm = R_SQRT(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]);
        if (nrm < (real)1e-12) nrm = (real)1e-12;
        for (int d = 0; d < 3; d++) f2[3 * t + d] = u[d] / nrm;
        const real* v = f2 + 3 * t;
        f3[3 * t + 0] = a[1] * v[2] - a[2] * v[1];
        f3[3 * t + 1] = a[2] * v[0] - a[0] * v[2];
        f3[3 * t + 2] = a[0] * v[1] - a[1] * v[0];
    }
}

/* --------------------------------------------------------------------------
 * Ragged softmax attention with additive logit bias and additive value bias.
 *   forward : models/kernels/fused_dpa_fwd.cu:44-125
 *   backward: models/kernels/fused_dpa_bwd.cu:52-124, fused_dpa_bwd_q.cu:27-52
 * q arrives already divided by sqrt(head_dim)
 * (models/indexed_lattice_multi_head_attention_cuda.py:179).
 * -------------------------------------------------------------------------- */
void FN(cfo_dpa_fwd)(const cfo_config* cfg, const real* q, const real* k, const real* v,
                     const real* aij /* (E,H) or NULL */, const real* bij /* (E,H,hd) or NULL */,
                     const int64_t* edges, const int64_t* e_start, int64_t N, int64_t E,
                     real* prob /* (E,H) */, real* out /* (N,H,hd) */)
{
    const int H = cfg->H, hd = cfg->head_dim;
#pragma omp parallel for schedule(dynamic, 8)
    for (int64_t i = 0; i < N; i++)
        for (int h = 0; h < H; h++) {
            const int64_t e0 = e_start[i], e1 = e_start[i + 1];
            real mx = (real)-1e20;
            for (int64_t e = e0; e < e1; e++) {
                const int64_t j = edges[E + e];
                real s = 0;
                for (int d = 0; d < hd; d++) s += q[(i * H + h) * hd + d] * k[(j * H + h) * hd + d];
                if (aij) s += aij[e * H + h];
                prob[e * H + h] = s;
                mx = R_FMAX(mx, s);
            }
            real sum = 0;
            for (int64_t e = e0; e < e1; e++) {
                real w = R_EXP(prob[e * H + h] - mx);
                prob[e * H + h] = w;
                sum += w;
            }
            real* o = out + (i * H + h) * hd;
            for (int d = 0; d < hd; d++) o[d] = 0;
            for (int64_t e = e0; e < e1; e++) {
                const int64_t j = edges[E + e];
                real p = prob[e * H + h] / sum;
                prob[e * H + h] = p;
                for (int d = 0; d < hd; d++) {
                    real val = v[(j * H + h) * hd + d];
                    if (bij) val += bij[(e * H + h) * hd + d];
                    o[d] += val * p;
                }
            }
        }
}

void FN(cfo_dpa_bwd)(const cfo_config* cfg, const real* q, const real* k, const real* v,
                     const real* bij, const int64_t* edges, const int64_t* e_start, int64_t N,
                     int64_t E, const real* prob, const real* out, const real* gout,
                     real* gq, real* gk, real* gv, real* gaij, real* gbij /* may be NULL */)
{
    const int H = cfg->H, hd = cfg->head_dim;
    memset(gq, 0, sizeof(real) * N * H * hd);
    memset(gk, 0, sizeof(real) * N * H * hd);
    memset(gv, 0, sizeof(real) * N * H * hd);
    /* serial over atoms: gk/gv scatter into key rows */
    for (int64_t i = 0; i < N; i++)
        for (int h = 0; h < H; h++)
            for (int64_t e = e_start[i]; e < e_start[i + 1]; e++) {
                const int64_t j = edges[E + e];
                const real p = prob[e * H + h];
                real gs = 0;
                for (int d = 0; d < hd; d++) {
                    real t = gout[(i * H + h) * hd + d] * p;
                    gv[(j * H + h) * hd + d] += t;
                    if (gbij) gbij[(e * H + h) * hd + d] = t;
                    real val = v[(j * H + h) * hd + d] - out[(i * H + h) * hd + d];
                    if (bij) val += bij[(e * H + h) * hd + d];
                    gs += val * t;
                }
                gaij[e * H + h] = gs;
                for (int d = 0; d < hd; d++) {
                    gk[(j * H + h) * hd + d] += gs * q[(i * H + h) * hd + d];
                    gq[(i * H + h) * hd + d] += gs * k[(j * H + h) * hd + d];
                }
            }
}

/* --------------------------------------------------------------------------
 * Per-crystal mean over atoms and its gradient:
 *   models/kernels/irregular_mean_fwd.cu:49-90 (tree-ordered sum, then /len),
 *   models/cuda_funcs/irregular_mean.py:59-69.
 * The summation order here is plain left to right.
 * -------------------------------------------------------------------------- */
void FN(cfo_mean_fwd)(const real* x /* (N,D) */, const int64_t* start /* (B+1) */, int64_t B, int64_t D, real* out)
{
    for (int64_t c = 0; c < B; c++)
        for (int64_t d = 0; d < D; d++) {
            real s = 0;
            for (int64_t i = start[c]; i < start[c + 1]; i++) s += x[i * D + d];
            out[c * D + d] = s / (real)(start[c + 1] - start[c]);
        }
}

void FN(cfo_mean_bwd)(const real* gout /* (B,D) */, const int64_t* start, int64_t B, int64_t D, real* gx)
{
    for (int64_t c = 0; c < B; c++)
        for (int64_t i = start[c]; i < start[c + 1]; i++)
            for (int64_t d = 0; d < D; d++) gx[i * D + d] = gout[c * D + d] / (real)(start[c + 1] - start[c]);
}

/* --------------------------------------------------------------------------
 * Reciprocal-space lattice sum and its gradient:
 *   models/kernels/reci_enc_fwd.cu:17-67, models/kernels/reci_enc_bwd.cu:19-70,
 *   models/cuda_funcs/reci_space_enc.py:19-62 (forward), :64-97 (backward).
 *   sum_ek = sum_n w(n1) exp(a_ik |n G|^2) cos(n . kr_e),  n1 in [0,R] (w = 1 at 0, else 2: the
 *            summand is even in n), n2, n3 in [-R,R], G the rows of rvecs (reciprocal vectors);
 *   z_ek   = log(max(sum, 1e-6)) + 1.5 log(-4 pi a) - log(vcell);
 *   ga_ik  = sum_e gz_ek (sum < 1e-6 ? 0 : 1/sum) sum_n w |nG|^2 exp(a |nG|^2) cos(n . kr)
 * (the reference's gradient leaves out the term of the normaliser, which is the same for every pair of
 * an (atom, head) and cancels in the softmax that consumes z).
 * -------------------------------------------------------------------------- */
#ifdef REAL_IS_DOUBLE
#define R_COS cos
#else
#define R_COS cosf
#endif

void FN(cfo_reci_enc_fwd)(const real* a_ik, const real* kr /* (E,3) */, const real* rvecs /* (B,3,3) */,
                          const real* vcell /* (B) */, const int64_t* batch, const int64_t* edges, int64_t N,
                          int64_t H, int64_t E, int R, real* z /* (E,H) */, real* sumexp /* (E,H) */)
{
    (void)N;
    for (int64_t e = 0; e < E; e++) {
        const int64_t i = edges[e], c = batch[i];
        const real* g = rvecs + c * 9;
        for (int64_t h = 0; h < H; h++) {
            const real a = a_ik[i * H + h];
            real sum = 0;
            for (int n1 = 0; n1 <= R; n1++) {
                const real w = n1 == 0 ? (real)1 : (real)2;
                for (int n2 = -R; n2 <= R; n2++)
                    for (int n3 = -R; n3 <= R; n3++) {
                        const real k1 = g[0] * n1 + g[3] * n2 + g[6] * n3;
                        const real k2 = g[1] * n1 + g[4] * n2 + g[7] * n3;
                        const real k3 = g[2] * n1 + g[5] * n2 + g[8] * n3;
                        const real ex = R_EXP(a * (k1 * k1 + k2 * k2 + k3 * k3));
                        sum += ex * R_COS(kr[e * 3] * n1 + kr[e * 3 + 1] * n2 + kr[e * 3 + 2] * n3) * w;
                    }
            }
            const real four_pi = (real)12.5663706144;
            z[e * H + h] = R_LOG(R_FMAX(sum, (real)1e-6)) + (real)1.5 * R_LOG(-four_pi * a) - R_LOG(vcell[c]);
            sumexp[e * H + h] = sum;
        }
    }
}

void FN(cfo_reci_enc_bwd)(const real* a_ik, const real* kr, const real* rvecs, const int64_t* batch,
                          const int64_t* e_start /* (N+1) */, const real* gz, const real* sumexp, int64_t N,
                          int64_t H, int R, real* ga /* (N,H) */)
{
    for (int64_t i = 0; i < N; i++) {
        const real* g = rvecs + batch[i] * 9;
        for (int64_t h = 0; h < H; h++) {
            const real a = a_ik[i * H + h];
            real total = 0;
            for (int64_t e = e_start[i]; e < e_start[i + 1]; e++) {
                real s = 0;
                for (int n1 = 0; n1 <= R; n1++) {
                    const real w = n1 == 0 ? (real)1 : (real)2;
                    for (int n2 = -R; n2 <= R; n2++)
                        for (int n3 = -R; n3 <= R; n3++) {
                            const real k1 = g[0] * n1 + g[3] * n2 + g[6] * n3;
                            const real k2 = g[1] * n1 + g[4] * n2 + g[7] * n3;
                            const real k3 = g[2] * n1 + g[5] * n2 + g[8] * n3;
                            const real kk = k1 * k1 + k2 * k2 + k3 * k3;
                            s += kk * R_EXP(a * kk) * R_COS(kr[e * 3] * n1 + kr[e * 3 + 1] * n2 + kr[e * 3 + 2] * n3) * w;
                        }
                }
                const real se = sumexp[e * H + h];
                total += s * gz[e * H + h] * (se < (real)1e-6 ? (real)0 : (real)1 / se);
            }
            ga[i * H + h] = total;
        }
    }
}
