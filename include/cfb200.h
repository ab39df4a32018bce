/*
 * libcfb200 -- C ABI of the B200 (sm_100a) implementation of CrystalFramer's periodic
 * lattice-sum attention path.
 *
 * Conventions (they replace those of the reference's CuPy RawKernel layer,
 * models/cuda_funcs/kernel_manager.py:14-167 and the _to_cupy helpers of each Function):
 *   - every pointer is a device pointer on the current device unless it says "host";
 *     all reals are contiguous float32, all indices contiguous int64 (as the reference);
 *   - the library allocates no device memory and never synchronises: work is enqueued on `stream`
 *     (a cudaStream_t passed as void*), scratch memory is passed in by the caller
 *     (cfb200_encoder_layer_bwd creates one more stream and two events per host thread and
 *     device on first use, for work it forks from and joins back into `stream`;
 *     CFB200_SIDE_STREAM=0 in the environment keeps it on `stream`);
 *   - a call returns 0 on success or a negative CFB200_E_* code; kernels never trap -- a
 *     condition found on the device (non-negative Gaussian coefficient, clamped lattice
 *     range) sets a bit in a status word read with cfb200_status();
 *   - hyper-parameters the reference bakes into its kernel text (compile_kernels,
 *     kernel_manager.py:116-167) are bound once per process with cfb200_configure().
 *
 * Pair lists: every entry point that takes `edges` together with `e_start` expects the reference's
 * dense layout (get_edge_index, models/indexed_latticeformer_encoder.py:15-32): pairs sorted by query
 * atom, and the pairs of an atom running over the atoms of its crystal in order, so that the key atom of
 * pair e of atom i is edges[1][e_start[i]] + (e - e_start[i]).  The attention kernels use that identity in
 * their backward passes; a list that breaks it sets CFB200_ST_PAIR_LAYOUT in the status word.
 *
 * Each entry point names the reference interface it replaces by file:line (paths relative
 * to the reference project root).
 */
#ifndef CFB200_H
#define CFB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CFB200_OK 0
#define CFB200_E_NULL (-1)         /* a required pointer is NULL                               */
#define CFB200_E_SHAPE (-2)        /* negative or inconsistent extent                          */
#define CFB200_E_UNSUPPORTED (-3)  /* no kernel instance for the configured hyper-parameters   */
#define CFB200_E_NOT_CONFIGURED (-4)
#define CFB200_E_WORKSPACE (-5)    /* scratch buffer missing or too small                      */
#define CFB200_E_CUDA (-6)         /* launch failed; see cudaGetLastError                      */
#define CFB200_E_TOO_LARGE (-7)    /* problem exceeds the fixed scratch of a *_noalloc entry   */

/* bits of the device status word */
#define CFB200_ST_BAD_COEF 1       /* a Gaussian coefficient a_ik was not negative             */
#define CFB200_ST_RANGE_CLAMPED 2  /* a lattice range exceeded CFB200_MAX_RANGE and was clamped */
#define CFB200_ST_SIZE_MISMATCH 4 /* sizes do not sum to the N and E passed to cfb200_edge_index */
#define CFB200_ST_TC_TIMEOUT 8    /* a tensor-core kernel gave up waiting for its own instructions   */
#define CFB200_ST_PAIR_LAYOUT 16  /* the pair list is not the dense n x n block of every crystal       */
#define CFB200_MAX_RANGE 48
#define CFB200_SPLIT_SLOTS 4096    /* partial results of chunked attention tasks a batch may hold per head */

typedef struct cfb200_config {
    int32_t num_heads;        /* HEAD_NUM / THREAD_NUM                                  */
    int32_t head_dim;         /* K_HEAD_DIM == V_HEAD_DIM                               */
    int32_t dist_dim;         /* VPE_DIM: distance Gaussians                            */
    int32_t angle_dim;        /* ANGLE_ENC_DIM: angle Gaussians per frame axis, 0 = off */
    int32_t lattice_range;    /* LATTICE_RANGE                                          */
    int32_t minimum_range;    /* MINIMUM_RANGE (0 = off)                                */
    int32_t cos_abs;          /* COS_ABS                                                */
    int32_t cut_sigma;        /* CUT_SIGMA (the reference fixes 4)                      */
    float dist_wscale;        /* value_pe_dist_wscale  -> LENGTH_RANGE                  */
    float angle_wscale;       /* value_pe_angle_wscale -> ANGLE_RANGE and angle sigma   */
    float dist_coef;          /* value_pe_dist_coef  (length_rbf_mul)                   */
    float angle_coef;         /* value_pe_angle_coef (angle_rbf_mul)                    */
    float symm_break_noise;   /* SYMM_BREAK_NOISE                                       */
} cfb200_config;

/* Replaces compile_kernels(...) (models/cuda_funcs/kernel_manager.py:116-167): binds the
 * hyper-parameters for all later calls of this process.  Returns CFB200_E_UNSUPPORTED when no
 * kernel instance exists for them. */
int cfb200_configure(const cfb200_config* cfg /* host */);
int cfb200_get_config(cfb200_config* out /* host */);
int cfb200_version(void);
const char* cfb200_error_string(int code);

/* Reads and clears the device status word (synchronises `stream`). */
int cfb200_status(int32_t* status_out /* host */, void* stream);

/* Number of resident thread blocks the lattice-sum kernels launch along x; the size of the
 * backward scratch buffer depends on it. */
int64_t cfb200_framed_proj_bwd_workspace_bytes(int64_t N, int64_t E);

/* Replaces get_edge_index (models/indexed_latticeformer_encoder.py:15-32), the CSR offsets
 * each Function rebuilds (models/cuda_funcs/fused_dpa.py:24-26) and the per-atom crystal
 * index.  sizes (B); edges (2,E) row 0 = query atom, row 1 = key atom; e_start (N+1);
 * batch (N); crystal_start (B+1) atom offsets.  N and E must equal sum(sizes), sum(sizes^2). */
int cfb200_edge_index(const int64_t* sizes, int64_t B, int64_t N, int64_t E, int64_t* edges,
                      int64_t* e_start, int64_t* batch, int64_t* crystal_start, void* stream);

/* CSR offsets from a pair list sorted by query atom (models/cuda_funcs/fused_dpa.py:24-26). */
int cfb200_csr_offsets(const int64_t* edge_i, int64_t E, int64_t N, int64_t* e_start, void* stream);

/* Replaces the torch operations that turn queries into Gaussian coefficients
 * (models/indexed_lattice_multi_head_attention_cuda.py:896-940, gauss_state "q") and the two
 * divisions of q by sqrt(head_dim) (:179, :447): a (N,H) = [(1-lb) elu(((q.w) + shift) scale
 * beta/(1-lb)) + 1] * (-1/(2 scale_real^2)) and q_scaled (N,H,head_dim).  w is lattice_pos_weights
 * (H*head_dim); gauss_scale points to [scale, shift] on the device (the module's gauss_scale
 * parameter) or is NULL for no normalisation.  The backward takes the gradients w.r.t. a and
 * q_scaled and returns those w.r.t. q (N,H,head_dim) and w (H*head_dim, summed in a fixed order). */
int cfb200_gauss_coef_fwd(const float* q, const float* w, const float* gauss_scale, int64_t N, float lb,
                          float beta, float scale_real, float* a, float* q_scaled, void* stream);
int cfb200_gauss_coef_bwd(const float* q, const float* w, const float* gauss_scale, int64_t N, float lb,
                          float beta, float scale_real, const float* ga, const float* gq_scaled,
                          float* gq, float* gw, void* stream);

/* Replaces ComputeFrame1MaximumMethodCUDA.forward / ComputeFrame2MaximumMethodCUDA.forward
 * (models/cuda_funcs/calc_maximum_frame.py:24-170) with kernels
 * compute_maximum_frame_each_edge.cu / compute_second_frame_each_edge.cu and the per-atom
 * argmax.  axis = 1: nearest-image axis; axis = 2: second axis given frame1 (N,H,3).
 * q_scaled is q / sqrt(head_dim).  Outputs: frame (N,H,3); optional sel_edge (N,H) int64 and
 * sel_image (N,H) int32 (linear translation index) name the selected pair and image. */
int cfb200_max_frame(int axis, const float* q_scaled, const float* k, const float* a_ik,
                     const float* pos_ij, const float* tvecs, const float* rvlen,
                     const int64_t* batch, const int64_t* edges, const int64_t* e_start,
                     int64_t N, int64_t E, float cutoff_radius, uint64_t seed,
                     const float* frame1, float* frame, int64_t* sel_edge, int32_t* sel_image,
                     void* stream);

/* The "max_static" frame method: replaces ComputeFrame1MaximumStaticMethodCUDA / ComputeFrame2MaximumStaticMethodCUDA
 * (models/cuda_funcs/calc_maximum_static_frame.py:24-170; kernels compute_maximum_frame_each_edge.cu,
 * compute_second_frame_static_each_edge.cu).  As cfb200_max_frame, but queries and keys do not enter the per-atom
 * arg-max and the second axis' score is (d^2 - d^2_min) + log(max(1 - |cos|, 1e-5)) without the Gaussian
 * coefficient.  cfb200_max_frames_static: both axes and the Gram-Schmidt completion in one launch (pair_cache
 * optional, as in cfb200_max_frames_cached). */
/* The "pca" frame method: replaces ComputePCAFrame (models/cuda_funcs/calc_pca_frame.py:22-76).  Per atom the
 * eigenvectors, by ascending eigenvalue, of the scatter matrix of its pair separations in the home cell (pos_ij
 * about their mean; no lattice translations); per (atom, head) a drawn sign per axis, then all three axes times the
 * determinant of the signed triple.  The signs come from a hash of (seed, atom, head, axis) where the reference uses
 * torch.randint, and an eigenvector's own sign is fixed by "largest component positive" where the reference has
 * LAPACK's: the axes agree with the reference's up to sign. */
int cfb200_pca_frames(const float* pos_ij, const int64_t* e_start, int64_t N, int64_t E, uint64_t seed,
                      float* frame1, float* frame2, float* frame3, void* stream);

int cfb200_max_frame_static(int axis, const float* a_ik, const float* pos_ij, const float* tvecs,
                            const float* rvlen, const int64_t* batch, const int64_t* edges,
                            const int64_t* e_start, int64_t N, int64_t E, float cutoff_radius, uint64_t seed,
                            const float* frame1, float* frame, int64_t* sel_edge, int32_t* sel_image,
                            void* stream);
int cfb200_max_frames_static(const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen,
                             const int64_t* batch, const int64_t* edges, const int64_t* e_start, int64_t N,
                             int64_t E, float cutoff_radius, uint64_t seed1, uint64_t seed2, float* frame1,
                             float* frame2, float* frame3, const float* pair_cache, int cache_range,
                             void* stream);

/* The "lattice" frame method: replaces ComputeLatticeFrameCUDA (models/cuda_funcs/calc_lattice_frame.py:22-150;
 * kernels compute_lattice_first_frame.cu, compute_lattice_second_frame.cu, compute_lattice_third_frame.cu).
 * Per (atom, head) the directions of the three shortest lattice vectors of the atom's cell within its lattice
 * ranges: shortest; shortest not collinear with it; shortest out of their plane; signs fixed as in the reference.
 * frame1..3 (N,H,3); zero where nothing qualifies.  seed1..3: noise seeds of the three searches. */
int cfb200_lattice_frames(const float* a_ik, const float* tvecs, const float* rvlen, const int64_t* batch,
                          const int64_t* edges, const int64_t* e_start, int64_t N, int64_t E,
                          float cutoff_radius, uint64_t seed1, uint64_t seed2, uint64_t seed3, float* frame1,
                          float* frame2, float* frame3, void* stream);

/* Both axes plus the Gram-Schmidt completion
 * (models/indexed_lattice_multi_head_attention_cuda.py:435-493) in one launch. */
int cfb200_max_frames(const float* q_scaled, const float* k, const float* a_ik,
                      const float* pos_ij, const float* tvecs, const float* rvlen,
                      const int64_t* batch, const int64_t* edges, const int64_t* e_start,
                      int64_t N, int64_t E, float cutoff_radius, uint64_t seed1, uint64_t seed2,
                      float* frame1, float* frame2, float* frame3, void* stream);

/* The per-pair part of the weighted-PCA frames alone: replaces the weighted_pca branch of
 * RealPeriodicEncodingWithProjFuncCUDA.forward (models/cuda_funcs/real_space_enc_proj.py:80-125; kernels
 * select_edges.cu, real_enc_sigma_fwd.cu).  records (E,H,11) per (pair, head): [0] the lattice-sum logit
 * z = log sum_n exp(a d_n^2) (the reference returns an uninitialised buffer in its place), [1..6] the
 * weight-averaged second moments xx, xy, xz, yy, yz, zz of the pair's images (the reference's sigma_mat),
 * [7] the smallest d^2 > 1e-5 (plus tie-breaking noise), [8..10] the unit vector to that image. */
int cfb200_sigma_edges(const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen,
                       const int64_t* batch, const int64_t* edges, int64_t N, int64_t E, float cutoff_radius,
                       uint64_t seed_noise, float* records, void* stream);

/* Weighted-PCA frames.  Replaces RealPeriodicEncodingWithProjFuncCUDA with
 * frame_method "weighted_pca" (models/cuda_funcs/real_space_enc_proj.py:80-125; kernels
 * select_edges.cu, real_enc_sigma_fwd.cu), FusedDotProductAttentionSigmaMatCUDA
 * (models/cuda_funcs/fused_dpa_sigmamat.py; kernel fused_dpa_sigmamat_fwd.cu) and the
 * determinant / eigen-decomposition / sign block of
 * models/indexed_lattice_multi_head_attention_cuda.py:656-725.  Outputs frame1..3 (N,H,3), a
 * right-handed orthonormal triad per (atom, head).  The pooling attention uses the lattice-sum
 * log-weights as its bias (the reference hands it an uninitialised buffer); eigenvector signs are
 * fixed by "largest component positive", row signs come from seed_sign.  workspace: at least
 * cfb200_sigma_frames_workspace_bytes(N,E) bytes. */
int64_t cfb200_sigma_frames_workspace_bytes(int64_t N, int64_t E);
int cfb200_sigma_frames(const float* q_scaled, const float* k, const float* a_ik, const float* pos_ij,
                        const float* tvecs, const float* rvlen, const int64_t* batch,
                        const int64_t* edges, const int64_t* e_start, int64_t N, int64_t E,
                        float cutoff_radius, uint64_t seed_noise, uint64_t seed_sign, float* frame1,
                        float* frame2, float* frame3, void* workspace, int64_t workspace_bytes,
                        void* stream);

/* Replaces ComputeFrame3MaximumMethodCUDA (models/cuda_funcs/calc_maximum_frame.py:173-245; kernel
 * compute_third_frame_each_edge.cu), the third axis of the frame method "max_wo_orthogonal": per (pair, head) the
 * image maximising a (d^2 - d^2_min) + log|det(frame1, frame2, u)| among the images with |det| > 1e-5, then per
 * (atom, head) the pair maximising q.k + that value (lowest pair on equal scores).  frame1, frame2 (N,H,3): the first
 * axis and the UN-orthogonalised second axis (cfb200_max_frame with axis 1 and 2).  frame3 (N,H,3) out; sel_edge
 * (N,H) optional.  Where no image of any pair qualifies the frame is zero and sel_edge -1 (the reference leaves its
 * outputs unwritten there).  workspace: cfb200_max_frame3_workspace_bytes(N,E) bytes, 16-byte aligned. */
int64_t cfb200_max_frame3_workspace_bytes(int64_t N, int64_t E);
int cfb200_max_frame3(const float* q_scaled, const float* k, const float* a_ik, const float* pos_ij,
                      const float* tvecs, const float* rvlen, const int64_t* batch, const int64_t* edges,
                      const int64_t* e_start, int64_t N, int64_t E, float cutoff_radius, uint64_t seed,
                      const float* frame1, const float* frame2, float* frame3, int64_t* sel_edge,
                      void* workspace, int64_t workspace_bytes, void* stream);

/* cfb200_sigma_frames / cfb200_sigma_edges with the per-pair sorted translation lists of cfb200_pair_cache
 * (pair_list (E,5,128), valid for lattice ranges (cache_range)^3; NULL: every pair is swept): the translations that
 * carry weight are a prefix of a pair's list, shared by all heads; pairs whose box the list does not cover are
 * swept as before.  Needs a head count that divides 32 to use the lists. */
int cfb200_sigma_frames_cached(const float* q_scaled, const float* k, const float* a_ik, const float* pos_ij,
                               const float* tvecs, const float* rvlen, const int64_t* batch,
                               const int64_t* edges, const int64_t* e_start, int64_t N, int64_t E,
                               float cutoff_radius, uint64_t seed_noise, uint64_t seed_sign,
                               float* frame1, float* frame2, float* frame3, void* workspace,
                               int64_t workspace_bytes, const float* pair_list, int cache_range,
                               void* stream);
int cfb200_sigma_edges_cached(const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen,
                              const int64_t* batch, const int64_t* edges, int64_t N, int64_t E,
                              float cutoff_radius, uint64_t seed_noise, float* records,
                              const float* pair_list, int cache_range, void* stream);

/* Replaces RealEncodingWithFramedProjFuncCUDA.forward
 * (models/cuda_funcs/real_space_framed_proj.py:21-120; kernels
 * real_enc_frame_proj_fwd_length.cu, real_enc_frame_proj_fwd_angle.cu).
 * W_dist (H,head_dim,dist_dim); W_ang1..3 (H,head_dim,angle_dim) and frame1..3 (N,H,3) may all be
 * NULL (no angle encoding).  Outputs z (E,H) and values (E,H,head_dim) (values may be NULL). */
int cfb200_framed_proj_fwd(const float* a_ik, const float* pos_ij, const float* tvecs,
                           const float* rvlen, const int64_t* batch, const int64_t* edges,
                           int64_t N, int64_t E, float dist_max, float cutoff_radius,
                           const float* W_dist, const float* W_ang1, const float* W_ang2,
                           const float* W_ang3, const float* frame1, const float* frame2,
                           const float* frame3, float* z, float* values, void* stream);

/* Replaces RealEncodingWithFramedProjFuncCUDA.backward
 * (models/cuda_funcs/real_space_framed_proj.py:123-221; kernels
 * real_enc_frame_proj_bwd_length.cu, real_enc_frame_proj_bwd_angle.cu).
 * Outputs ga (N,H) and the weight gradients already summed over atoms, gW_dist
 * (H,head_dim,dist_dim), gW_ang1..3 (H,head_dim,angle_dim).  workspace: at least
 * cfb200_framed_proj_bwd_workspace_bytes(N,E) bytes, 256-byte aligned; need not be cleared. */
int cfb200_framed_proj_bwd(const float* a_ik, const float* pos_ij, const float* tvecs,
                           const float* rvlen, const int64_t* batch, const int64_t* edges,
                           const int64_t* e_start, int64_t N, int64_t E, float dist_max,
                           float cutoff_radius, const float* W_dist, const float* W_ang1,
                           const float* W_ang2, const float* W_ang3, const float* frame1,
                           const float* frame2, const float* frame3, const float* z,
                           const float* gz, const float* gvalues, float* ga, float* gW_dist,
                           float* gW_ang1, float* gW_ang2, float* gW_ang3, void* workspace,
                           int64_t workspace_bytes, void* stream);

/* cfb200_proj_fwd / cfb200_proj_bwd for `heads` heads instead of the configured number: a_ik (N,heads),
 * W_dist (heads,head_dim,dist_dim), z (E,heads), values (E,heads,head_dim) and the gradients likewise.  The
 * "multihead" domain of the plain Crystalformer gives half of the heads to the real-space encoding and half
 * to the reciprocal one (models/indexed_lattice_multi_head_attention_cuda.py:953-963). */
int64_t cfb200_proj_heads_bwd_workspace_bytes(int64_t N, int64_t E, int64_t heads);
int cfb200_proj_heads_fwd(const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen,
                          const int64_t* batch, const int64_t* edges, int64_t N, int64_t E, int64_t heads,
                          float dist_max, float cutoff_radius, const float* W_dist, float* z,
                          float* values, void* stream);
int cfb200_proj_heads_bwd(const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen,
                          const int64_t* batch, const int64_t* edges, const int64_t* e_start, int64_t N,
                          int64_t E, int64_t heads, float dist_max, float cutoff_radius,
                          const float* W_dist, const float* z, const float* gz, const float* gvalues,
                          float* ga, float* gW_dist, void* workspace, int64_t workspace_bytes,
                          void* stream);

/* Host code (no device work, no stream): deals n items with the given costs to `parts` groups of nearly equal
 * total cost -- the most expensive first, each to the group with the smallest total so far (lowest group on
 * ties, earlier item first among equal costs).  The reference spreads a batch over devices by this rule with the
 * squared crystal size as cost (models/latticeformer.py:224-233).  part_of (n) receives the group of every item. */
int cfb200_deal_by_cost(const double* cost, int64_t n, int32_t parts, int32_t* part_of);

/* Replaces ReciPeriodicEncodingFuncCUDA (models/cuda_funcs/reci_space_enc.py:17-97; kernels
 * reci_enc_fwd.cu, reci_enc_bwd.cu): the reciprocal-space lattice sum of the plain Crystalformer's
 * "reci" / "multihead" domains over n1 in [0, lattice_range], n2, n3 in [-lattice_range, lattice_range]
 * (lattice_range <= 3, CFB200_E_UNSUPPORTED above).  a_ik (N,H) must be negative; kr_base (E,3) =
 * rvecs[crystal] @ (pos_j - pos_i); rvecs (B,3,3) reciprocal vectors in rows; vcell (B) cell volumes;
 * e_start (N+1) CSR offsets of the pairs of each atom (pairs sorted by their first atom).  H is the number of
 * heads of a_ik (any H >= 1; the "multihead" domain passes half of the configured heads).
 * Forward: z (E,H) = log(max(sum, 1e-6)) + 1.5 log(-4 pi a) - log(vcell), sumexp (E,H) = sum.
 * Backward: ga (N,H) from gz (E,H) and the forward's sumexp. */
int cfb200_reci_enc_fwd(const float* a_ik, const float* kr_base, const float* rvecs, const float* vcell,
                        const int64_t* batch, const int64_t* e_start, int64_t N, int64_t H, int64_t E,
                        float* z, float* sumexp, void* stream);
int cfb200_reci_enc_bwd(const float* a_ik, const float* kr_base, const float* rvecs, const int64_t* batch,
                        const int64_t* e_start, const float* gz, const float* sumexp, int64_t N,
                        int64_t H, int64_t E, float* ga, void* stream);

/* Replaces RealPeriodicEncodingWithProjFuncCUDA with frame_method "no"
 * (models/cuda_funcs/real_space_enc_proj.py:21-213; kernels real_enc_proj_fwd.cu,
 * real_enc_proj_bwd.cu): the plain Crystalformer encoding -- lattice-sum bias z (E,H) and the
 * distance value encoding over ALL dist_dim Gaussians (no window, no coefficient, no frames).
 * The backward needs the same workspace as cfb200_framed_proj_bwd. */
int cfb200_proj_fwd(const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen,
                    const int64_t* batch, const int64_t* edges, int64_t N, int64_t E, float dist_max,
                    float cutoff_radius, const float* W_dist, float* z, float* values, void* stream);
int cfb200_proj_bwd(const float* a_ik, const float* pos_ij, const float* tvecs, const float* rvlen,
                    const int64_t* batch, const int64_t* edges, const int64_t* e_start, int64_t N,
                    int64_t E, float dist_max, float cutoff_radius, const float* W_dist,
                    const float* z, const float* gz, const float* gvalues, float* ga, float* gW_dist,
                    void* workspace, int64_t workspace_bytes, void* stream);

/* No counterpart in the reference (whose Functions allocate their temporaries with torch).
 * Same computation, arguments and outputs as cfb200_framed_proj_bwd, for hosts that cannot
 * provide a workspace: a plugin under a runtime that owns the device heap and passes only input
 * and output buffers, or a service that forbids device allocation after start-up.  The scratch is
 * a fixed device array of CFB200_NOALLOC_MAX_BYTES inside the library (held on every GPU the
 * process uses it on, until exit); the call allocates nothing.
 *  - Returns CFB200_E_TOO_LARGE when cfb200_framed_proj_bwd_workspace_bytes(N,E) exceeds
 *    CFB200_NOALLOC_MAX_BYTES (about 340 000 pairs with 8 heads).
 *  - The first call on each device looks up the array's device address (the device must be
 *    current); make that first call before any stream capture.
 *  - All calls share the one array: calls that may overlap on the GPU (different streams,
 *    different host threads) race and must be serialised by the caller.  Nothing has to be
 *    cleared between calls; the kernels overwrite what they later read. */
#define CFB200_NOALLOC_MAX_BYTES (16 * 1024 * 1024)
int cfb200_framed_proj_bwd_noalloc(const float* a_ik, const float* pos_ij, const float* tvecs,
                                   const float* rvlen, const int64_t* batch, const int64_t* edges,
                                   const int64_t* e_start, int64_t N, int64_t E, float dist_max,
                                   float cutoff_radius, const float* W_dist, const float* W_ang1,
                                   const float* W_ang2, const float* W_ang3, const float* frame1,
                                   const float* frame2, const float* frame3, const float* z,
                                   const float* gz, const float* gvalues, float* ga, float* gW_dist,
                                   float* gW_ang1, float* gW_ang2, float* gW_ang3, void* stream);

/* Per-pair geometry shared by all heads and layers.  No counterpart in the reference, whose kernels
 * redo this work in every layer and for every head: which lattice translations of a pair are near,
 * and how near, depends only on the pair's separation and the cell.  For the lattice ranges
 * (range, range, range) cfb200_pair_cache fills either or both of
 *   pair_cache (E,4) float, 16-byte aligned:
 *     [0], [1]  smallest and second smallest d^2 > 1e-5 over the translations,
 *     [2]       linear index of the first translation attaining [0] (int32 bits, -1 if none),
 *     [3]       smallest d^2 over all translations;
 *   pair_list (E,5,128) float, only for (2 range + 1)^3 <= 128 (CFB200_E_UNSUPPORTED otherwise):
 *     all translations sorted by squared distance -- planes d^2, x, y, z of the separation vector and
 *     the packed translation (n1+range) | (n2+range) << 8 | (n3+range) << 16 | index << 24 (int32
 *     bits); unused entries have d^2 = 1e30.
 * The *_cached entry points compute what their plain namesakes compute and use the cache for every
 * (atom, head) whose three lattice ranges equal cache_range -- the frame searches also for larger ranges,
 * wherever every translation outside the cached box is provably farther than what decides the search;
 * other tasks are searched as usual.
 * Frames are bit-identical to the plain entry point with either cache; with pair_list the lattice
 * sums are accumulated nearest-first instead of in index order (differences of a few ulp).
 * Either pointer may be NULL. */
int cfb200_pair_cache(const float* pos_ij, const float* tvecs, const int64_t* batch,
                      const int64_t* edges, int64_t N, int64_t E, int range, float* pair_cache,
                      float* pair_list, void* stream);
int cfb200_max_frames_cached(const float* q_scaled, const float* k, const float* a_ik,
                             const float* pos_ij, const float* tvecs, const float* rvlen,
                             const int64_t* batch, const int64_t* edges, const int64_t* e_start,
                             int64_t N, int64_t E, float cutoff_radius, uint64_t seed1,
                             uint64_t seed2, float* frame1, float* frame2, float* frame3,
                             const float* pair_cache, const float* pair_list, int cache_range,
                             void* stream);
int cfb200_max_frame_cached(int axis, const float* q_scaled, const float* k, const float* a_ik,
                            const float* pos_ij, const float* tvecs, const float* rvlen,
                            const int64_t* batch, const int64_t* edges, const int64_t* e_start,
                            int64_t N, int64_t E, float cutoff_radius, uint64_t seed,
                            const float* frame1, float* frame, int64_t* sel_edge, int32_t* sel_image,
                            const float* pair_cache, const float* pair_list, int cache_range,
                            void* stream);
int cfb200_framed_proj_fwd_cached(const float* a_ik, const float* pos_ij, const float* tvecs,
                                  const float* rvlen, const int64_t* batch, const int64_t* edges,
                                  int64_t N, int64_t E, float dist_max, float cutoff_radius,
                                  const float* W_dist, const float* W_ang1, const float* W_ang2,
                                  const float* W_ang3, const float* frame1, const float* frame2,
                                  const float* frame3, float* z, float* values,
                                  const float* pair_cache, const float* pair_list, int cache_range,
                                  void* stream);
int cfb200_framed_proj_bwd_cached(const float* a_ik, const float* pos_ij, const float* tvecs,
                                  const float* rvlen, const int64_t* batch, const int64_t* edges,
                                  const int64_t* e_start, int64_t N, int64_t E, float dist_max,
                                  float cutoff_radius, const float* W_dist, const float* W_ang1,
                                  const float* W_ang2, const float* W_ang3, const float* frame1,
                                  const float* frame2, const float* frame3, const float* z,
                                  const float* gz, const float* gvalues, float* ga, float* gW_dist,
                                  float* gW_ang1, float* gW_ang2, float* gW_ang3, void* workspace,
                                  int64_t workspace_bytes, const float* pair_list, int cache_range,
                                  void* stream);

/* Lattice-sum bias, frame-projected value encoding and ragged attention of one layer in one pass:
 * what RealEncodingWithFramedProjFuncCUDA.forward followed by FusedDotProductAttentionCUDA.forward
 * compute (models/indexed_lattice_multi_head_attention_cuda.py:944-985), without ever forming the
 * (E,H,head_dim) value encoding: it is linear in the 256 basis sums of a pair, so the sums are pooled
 * with the attention weights first and projected once per (atom, head).  For head_dim 16 and 64 distance
 * Gaussians.  order (N) int32 or NULL: the sequence in which atoms are handed to the warps (most
 * expensive first balances best); counters: num_heads int32 of scratch (work-queue heads; the call
 * clears them).  pair_list / cache_range as in cfb200_pair_cache (NULL: every pair is
 * swept).  unwindowed != 0 selects the plain Crystalformer encoding of cfb200_proj_fwd (every distance
 * Gaussian, no coefficient, no angle weights).  Outputs: out (N,H,16); z (E,H); lse (N,H) log-sum-exp of the logits; spool (N,H,256) the
 * attention-pooled basis sums [distance 64 | axis 1..3 64 each], distance part unscaled, angle parts times
 * the angle coefficient -- the weight gradients are  gW[h] (16 x 256) = sum_i gout[i,h,:]^T spool[i,h,:],
 * a GEMM left to the caller.
 * The backward takes the forward's out, z, lse and the upstream gout (N,H,16) and returns gq_scaled, gk,
 * gv (N,H,16), ga (N,H) and gz (E,H) (scratch the column pass reads; also the gradient of the logit bias).
 * val (E,H,16), px (E,H) and upool (N,H,16), all three or none: with them the forward also stores, per (pair,
 * head), the value encoding W s and sum p d^2 (68 bytes), and per (atom, head) the projection of the
 * attention-pooled basis sums weighted with d^2; the backward, given the same three, is a plain ragged-attention
 * backward.  Without them the forward is lighter and the backward recomputes the lattice sums. */
int cfb200_attn_fused_fwd(const float* q_scaled, const float* k, const float* v, const float* a_ik,
                          const float* pos_ij, const float* tvecs, const float* rvlen,
                          const int64_t* batch, const int64_t* edges, const int64_t* e_start,
                          const int32_t* order, int32_t* counters, int64_t N, int64_t E, float dist_max,
                          float cutoff_radius, const float* W_dist, const float* W_ang1,
                          const float* W_ang2, const float* W_ang3, const float* frame1,
                          const float* frame2, const float* frame3, const float* pair_list,
                          int cache_range, float* out, float* z, float* lse, float* spool,
                          float* val, float* px, float* upool, int unwindowed, void* stream);
int cfb200_attn_fused_bwd(const float* q_scaled, const float* k, const float* v, const float* a_ik,
                          const float* pos_ij, const float* tvecs, const float* rvlen,
                          const int64_t* batch, const int64_t* edges, const int64_t* e_start,
                          const int32_t* order, int32_t* counters, int64_t N, int64_t E, float dist_max,
                          float cutoff_radius, const float* W_dist, const float* W_ang1,
                          const float* W_ang2, const float* W_ang3, const float* frame1,
                          const float* frame2, const float* frame3, const float* pair_list,
                          int cache_range, const float* out, const float* z, const float* lse,
                          const float* gout, float* gq_scaled, float* gk, float* gv, float* ga,
                          float* gz, const float* val, const float* px, const float* upool, int unwindowed,
                          void* stream);

/* Replaces FusedDotProductAttentionCUDA.forward (models/cuda_funcs/fused_dpa.py:17-64;
 * kernel fused_dpa_fwd.cu).  q_scaled, k, v (N,H,head_dim); z (E,H) or NULL; values
 * (E,H,head_dim) or NULL.  Outputs out (N,H,head_dim), lse (N,H) = log-sum-exp of the logits
 * (kept for the backward pass), prob (E,H) or NULL. */
int cfb200_dpa_fwd(const float* q_scaled, const float* k, const float* v, const float* z,
                   const float* values, const int64_t* edges, const int64_t* e_start, int64_t N,
                   int64_t E, float* out, float* lse, float* prob, void* stream);

/* Replaces FusedDotProductAttentionCUDA.backward (models/cuda_funcs/fused_dpa.py:66-168;
 * kernels irregular_transpose.cu, fused_dpa_bwd.cu, fused_dpa_bwd_q.cu).  Outputs gq, gk, gv
 * (N,H,head_dim), gz (E,H), gvalues (E,H,head_dim) (NULL when values is NULL). */
int cfb200_dpa_bwd(const float* q_scaled, const float* k, const float* v, const float* z,
                   const float* values, const int64_t* edges, const int64_t* e_start, int64_t N,
                   int64_t E, const float* out, const float* lse, const float* gout, float* gq,
                   float* gk, float* gv, float* gz, float* gvalues, void* stream);

/* Replaces IrregularMeanCUDA (models/cuda_funcs/irregular_mean.py:19-69; kernel
 * irregular_mean_fwd.cu).  x (N,D); start (B+1) atom offsets; out (B,D). */
int cfb200_segment_mean_fwd(const float* x, const int64_t* start, int64_t B, int64_t D, float* out,
                            void* stream);
int cfb200_segment_mean_bwd(const float* gout, const int64_t* start, int64_t B, int64_t D,
                            float* gx, void* stream);

/* Gradient clipping by global norm and the AdamW update on flat fp32 buffers, in two launches (what
 * torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW.step do tensor by tensor for the reference's
 * trainer).  params, grads, exp_avg, exp_avg_sq: n floats each; weight decay applies to the first
 * decay_end elements only; max_norm <= 0 disables clipping; bias_correction{1,2} = 1 - beta{1,2}^step;
 * scratch: 256 floats; grad_norm (1 float, optional): the norm before clipping. */
int cfb200_adamw_clip_step(float* params, const float* grads, float* exp_avg, float* exp_avg_sq,
                           int64_t n, int64_t decay_end, float lr, float beta1, float beta2, float eps,
                           float weight_decay, float max_norm, double bias_correction1,
                           double bias_correction2, float* scratch, float* grad_norm, void* stream);
/* The same step followed, in the same launch, by the running average of the weights that the reference keeps over
 * its last epochs (torch.optim.swa_utils.AveragedModel.update_parameters after opt.step(),
 * models/regression.py:150-152): averaged (n floats) += (params - averaged) * average_weight, with
 * average_weight = 1 / (number of models averaged so far + 1), so the first update copies the weights.
 * averaged == NULL: no average (cfb200_adamw_clip_step). */
int cfb200_adamw_clip_step_avg(float* params, const float* grads, float* exp_avg, float* exp_avg_sq,
                               int64_t n, int64_t decay_end, float lr, float beta1, float beta2, float eps,
                               float weight_decay, float max_norm, double bias_correction1,
                               double bias_correction2, float* scratch, float* grad_norm, float* averaged,
                               float average_weight, void* stream);

/* ---- one host call per batch and per encoder layer -------------------------------------------
 *
 * Replaces get_edge_index and compute_lattice_distances_for_cuda
 * (models/indexed_latticeformer_encoder.py:15-32, :175-245) and the reciprocal-vector lengths of
 * models/indexed_lattice_multi_head_attention_cuda.py:539 with one call: from raw positions pos (N,3),
 * lattice vectors tvecs (B,3,3) and sizes (B) it produces the pair list (edges (2,E), e_start (N+1),
 * batch (N), crystal_start (B+1)), pos_ij (E,3), rvecs (B,3,3) (optional), rvlen (B,3), vcell (B)
 * (optional), the per-pair geometry of cfb200_pair_cache for lattice ranges (range)^3 (pair_cache (E,4),
 * pair_list (E,5,128); either may be NULL, range 0 skips both) and `order`, int32, the work queue of the fused
 * attention kernels: atoms of the crystals with the most attention work first.
 * split == NULL: `order` holds the N atoms.  Otherwise `order` has room for cfb200_queue_entries(N) entries and
 * `split` for cfb200_split_ints(N) int32, and the queue can cut the longest tasks into chunks: one warp walks the
 * pairs of an (atom, head) one after the other, so an atom of a dense cell with many atoms can take several times
 * a warp's average load and the launch would end with that warp alone; such an atom gets an entry per chunk of
 * its pairs, every layer decides from its coefficients which (atom, head) tasks it really cuts, the chunks leave
 * partial results and a small kernel merges them in chunk order (results do not depend on the scheduling).  Hand
 * `split` to the layer calls through cfb200_geometry and give each layer's state a task table.  workspace: at least cfb200_batch_geometry_workspace_bytes(B) bytes. */
int64_t cfb200_batch_geometry_workspace_bytes(int64_t B);
int64_t cfb200_queue_entries(int64_t N);
int64_t cfb200_split_ints(int64_t N);
int64_t cfb200_attn_tasks_bytes(int64_t N);
int cfb200_batch_geometry(const float* pos, const float* tvecs, const int64_t* sizes, int64_t B, int64_t N,
                          int64_t E, int range, int64_t* edges, int64_t* e_start, int64_t* batch,
                          int64_t* crystal_start, float* pos_ij, float* rvecs, float* rvlen, float* vcell,
                          float* pair_cache, float* pair_list, int32_t* order, int32_t* split, void* workspace,
                          int64_t workspace_bytes, void* stream);

/* A dense layer, y (M,N) = x (M,K) op(W) (+ bias (N)) (+ residual (M,N)), then ReLU if relu != 0 -- what the
 * reference computes with torch.nn.functional.linear (models/indexed_lattice_multi_head_attention_cuda.py:869,
 * :987-988; models/indexed_latticeformer_encoder.py:888-890).  weight_is_kn = 0: W is (N,K) as torch stores a
 * Linear weight (y = x W^T); 1: W is (K,N) (y = x W, the data gradient of the same layer).  K and N must be
 * multiples of 4 and all pointers 16-byte aligned.  Runs on the tensor cores (tcgen05, three-product TF32
 * split with FP32 accumulation) when N is a multiple of 128 and K of 32, else on the FP32 pipe. */
int cfb200_linear(const float* x, const float* weight, const float* bias, const float* residual, int64_t M,
                  int64_t N, int64_t K, int relu, int weight_is_kn, float* y, void* stream);

/* Parameters of one encoder layer, laid out as the reference module stores them
 * (models/indexed_lattice_multi_head_attention_cuda.py:1078-1160, models/indexed_latticeformer_encoder.py:783-790):
 * q/k/v_proj (D,D), in_bias (3D), lattice_pos (D), gauss_scale (2) or NULL, out_proj (D,D), out_bias (D),
 * pe_dist and pe_ang1..3 (H,16,64) (pe_ang*: NULL without frames), ff1 (F,D), ff1_bias (F), ff2 (D,F),
 * ff2_bias (D).  Every pointer must be 16-byte aligned. */
typedef struct cfb200_layer_weights {
    const float *q_proj, *k_proj, *v_proj, *in_bias, *lattice_pos, *gauss_scale, *out_proj, *out_bias;
    const float *pe_dist, *pe_ang1, *pe_ang2, *pe_ang3, *ff1, *ff1_bias, *ff2, *ff2_bias;
} cfb200_layer_weights;

/* Destinations of the gradients, same shapes (no gauss_scale: it is not trained). */
typedef struct cfb200_layer_grads {
    float *q_proj, *k_proj, *v_proj, *in_bias, *lattice_pos, *out_proj, *out_bias;
    float *pe_dist, *pe_ang1, *pe_ang2, *pe_ang3, *ff1, *ff1_bias, *ff2, *ff2_bias;
} cfb200_layer_grads;

/* Batch tensors shared by all layers (outputs of cfb200_batch_geometry); counters: 64 int32 of scratch. */
typedef struct cfb200_geometry {
    const float *pos_ij, *tvecs, *rvlen;
    const int64_t *batch, *edges, *e_start;
    const int32_t* order;
    int32_t* counters;
    const float *pair_cache, *pair_list;
    int64_t N, E;
    int32_t cache_range;
    int32_t* split;   /* chunked work queue of cfb200_batch_geometry, or NULL: `order` then holds N atoms */
} cfb200_geometry;

/* Activations a layer's forward leaves for its backward (caller-allocated): q, q_scaled, k, v, attn, x1
 * (N,D); a, lse (N,H); frames (3,N,H,3) (NULL for frame_method 0); z (E,H); spool (N,H,256); h (N,F); tasks:
 * cfb200_attn_tasks_bytes(N) bytes, 16-byte aligned, the layer's task table when the geometry carries a chunked
 * queue (NULL otherwise, or to run the layer on the plain queue); val (E,H,16), px (E,H) and upool (N,H,16):
 * results of the forward lattice sum with which the backward pass needs no second lattice sum (all three or none:
 * with NULL the forward is lighter and the backward recomputes -- the choice for inference and when memory is
 * short). */
typedef struct cfb200_layer_state {
    float *q, *q_scaled, *k, *v, *a, *frames, *z, *spool, *attn, *lse, *x1, *h;
    void* tasks;
    float *val, *px, *upool;
} cfb200_layer_state;

/* frame_method: 0 = none (plain Crystalformer encoding), 1 = max frames, 2 = weighted-PCA frames, 3 = static max
 * frames, 4 = lattice frames, 5 = pca frames.  seed1, seed2: noise seeds of the two max-frame axes (lattice frames:
 * of the first two searches, the third uses seed1 ^ seed2), noise seed and sign seed of the weighted-PCA frames, or
 * (seed1) the sign seed of the pca frames. */
typedef struct cfb200_layer_desc {
    int32_t d_model, ff_dim, frame_method;
    float gauss_lb, beta, scale_real, dist_max, cutoff_radius;
    uint64_t seed1, seed2;
} cfb200_layer_desc;

/* One encoder layer (no layer norm, no dropout, ReLU; the structure of the reference's default
 * configuration), forward and backward, every kernel enqueued by one call.  Replaces
 * CrystalformerEncoderLayerCUDA.forward (models/indexed_latticeformer_encoder.py:848-890) with
 * crystalformer_multi_head_attention_forward_cuda inside it
 * (models/indexed_lattice_multi_head_attention_cuda.py:737-996) and the autograd graph behind them:
 *   q,k,v = x W^T + b;  a, q_scaled = coefficients(q);  frames;  attn = fused lattice-sum attention;
 *   x1 = x + attn Wo^T + bo;  h = relu(x1 Wf1^T + bf1);  x_out = x1 + h Wf2^T + bf2.
 * x, x_out, g_out, g_x: (N,D).  The backward writes every gradient of `grads` (adds to it when
 * accumulate != 0; sums run in a fixed order).  workspace: cfb200_encoder_layer_workspace_bytes bytes. */
int64_t cfb200_encoder_layer_workspace_bytes(int64_t N, int64_t E, int d_model, int ff_dim, int frame_method);
int cfb200_encoder_layer_fwd(const cfb200_layer_desc* desc /* host */, const cfb200_layer_weights* weights /* host */,
                             const cfb200_geometry* geometry /* host */, const float* x,
                             cfb200_layer_state* state /* host */, float* x_out, void* workspace,
                             int64_t workspace_bytes, void* stream);
int cfb200_encoder_layer_bwd(const cfb200_layer_desc* desc /* host */, const cfb200_layer_weights* weights /* host */,
                             const cfb200_geometry* geometry /* host */, const float* x,
                             const cfb200_layer_state* state /* host */, const float* g_out, float* g_x,
                             const cfb200_layer_grads* grads /* host */, int accumulate, void* workspace,
                             int64_t workspace_bytes, void* stream);

/* Measurement aid with no counterpart in the reference: between cfb200_timing_begin() and
 * cfb200_timing_end() every stage of cfb200_batch_geometry and cfb200_encoder_layer_fwd / _bwd is bracketed by
 * CUDA events on the stream it runs on.  cfb200_timing_end waits for them and returns, per stage
 * CFB200_TM_*, the summed milliseconds and the number of brackets (arrays of CFB200_TM_STAGES entries, host).
 * For one host thread; off by default, and then no events are created. */
#define CFB200_TM_GEOMETRY 0       /* cfb200_batch_geometry                                          */
#define CFB200_TM_LINEAR_FWD 1     /* input projections; output projection + feed-forward block      */
#define CFB200_TM_COEF 2           /* Gaussian coefficients, forward and backward                    */
#define CFB200_TM_FRAMES 3         /* max or weighted-PCA frames                                     */
#define CFB200_TM_ATTN_FWD 4       /* fused lattice-sum attention, forward kernel                    */
#define CFB200_TM_LINEAR_BWD 5     /* data gradients of the dense layers                             */
#define CFB200_TM_ATTN_BWD 6       /* fused lattice-sum attention, backward kernel                   */
#define CFB200_TM_ATTN_BWD_COLS 7  /* column pass of the attention backward (gk, gv)                 */
#define CFB200_TM_WGRAD 8          /* weight and bias gradients of the layer                         */
#define CFB200_TM_STAGES 9
int cfb200_timing_begin(void);
int cfb200_timing_end(float* ms_by_stage /* host */, int32_t* calls_by_stage /* host */);

/* Measurement aid with no counterpart in the reference: every thread of `blocks` x 256 threads
 * runs `iters` rounds of 8 independent chains of fused multiply-adds (kind 0) or ex2.approx
 * (kind 1) and writes one float to sink (blocks*256 floats).  Timed by the caller, it gives the
 * FP32 and special-function pipe throughput of the device the roofline fractions refer to. */
int cfb200_probe_throughput(int kind, int blocks, int iters, float* sink, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CFB200_H */
