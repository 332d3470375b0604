/*
 * fsgs.h -- C ABI of libfsgs.so: the B200 (sm_100a) surfel-rendering hot path of Fast-SP-GS.
 *
 * Every entry point takes raw DEVICE pointers (unless a parameter says "host"), plain sizes and a
 * CUDA stream handle, launches asynchronously on that stream and returns FSGS_OK or a negative
 * fsgs_status.  Nothing here allocates or frees device memory, throws, or synchronises the device;
 * scratch memory is passed in by the caller after a *_workspace_bytes() query.  All floating point
 * data is contiguous fp32; quaternions are (x, y, z, w); matrices are row major.
 *
 * Each declaration names the reference interface it stands in for (paths inside the Fast-SP-GS
 * project, fast_2d_gs/_C/...).  The PyTorch-facing operators with the reference's own names live in
 * the python package (fsgs/ops.py) and call only what is declared here.
 */
#ifndef FSGS_H_
#define FSGS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *fsgs_stream_t; /* a cudaStream_t */

typedef enum fsgs_status {
  FSGS_OK = 0,
  FSGS_ERR_INVALID_ARGUMENT = -1, /* null pointer, negative size, unsupported option */
  FSGS_ERR_UNSUPPORTED = -2,      /* e.g. SH degree above the built maximum */
  FSGS_ERR_WORKSPACE = -3,        /* workspace too small */
  FSGS_ERR_LAUNCH = -4,           /* cudaGetLastError() reported a launch failure */
  FSGS_ERR_LIMIT = -5             /* size beyond a documented maximum */
} fsgs_status;

#define FSGS_TILE 16           /* tiles are 16 x 16 pixels (include/gaussian_render.h:27-31) */
#define FSGS_RECORD_FLOATS 32  /* one packed per-Gaussian render record = 128 bytes */
#define FSGS_MAX_SH_DEGREE 7
#define FSGS_KNN_MAX_K 16

/* counters[] written by fsgs_preprocess_forward / fsgs_bin_tiles (int64 each) */
#define FSGS_CNT_SLOTS 0     /* R  = sum of tile-rectangle areas = numel of the reference's point_list */
#define FSGS_CNT_PAIRS 1     /* R* = (Gaussian, tile) pairs that pass the 4-corner test */
#define FSGS_CNT_OVERFLOW 2  /* pairs dropped because point_list capacity < R* (0 when healthy) */
#define FSGS_CNT_STATUS 3    /* device-side error bits (bounded wait ran out, ...), 0 when healthy */
#define FSGS_NUM_COUNTERS 4

const char *fsgs_status_string(int status);
int fsgs_version(void);

/* ------------------------------------------------------------------------------------------------
 * Nearest / farthest control point.
 * Replaces cdist_top / cdist_top_backward   (src/other/cdist_top.cu:34-84, 107-154).
 * x1 [B,N,D], x2 [B,M,D] -> dist [B,N] (sqrt of the squared distance), index [B,N] int64.
 * Exact ties: nearest keeps the LAST index, farthest the FIRST (cdist_top.cu:24).
 * Backward: g1 [B,N,D] is written, g2 [B,M,D] is zeroed then accumulated.
 * ---------------------------------------------------------------------------------------------- */
int fsgs_cdist_top(int B, int N, int M, int D, const float *x1, const float *x2, int largest, float *dist,
    int64_t *index, fsgs_stream_t stream);
int fsgs_cdist_top_backward(int B, int N, int M, int D, const float *x1, const float *x2, const float *dist,
    const int64_t *index, const float *grad_dist, float *g1, float *g2, fsgs_stream_t stream);
/* The same two in double precision (the reference dispatches on the dtype, cdist_top.cu:48,116). */
int fsgs_cdist_top_f64(int B, int N, int M, int D, const double *x1, const double *x2, int largest, double *dist,
    int64_t *index, fsgs_stream_t stream);
int fsgs_cdist_top_backward_f64(int B, int N, int M, int D, const double *x1, const double *x2, const double *dist,
    const int64_t *index, const double *grad_dist, double *g1, double *g2, fsgs_stream_t stream);

/* Exact K nearest control points (3-D), squared L2 by direct differences, ascending by (distance, index):
 * ties go to the lower index.  x [N,3], c [M,3] -> d2 [N,K], index [N,K] int64.  K <= FSGS_KNN_MAX_K.
 * Stands in for the pytorch3d.ops.knn_points call of fast_2d_gs/network.py:504 (third party; additive). */
int fsgs_knn(int N, int M, int K, const float *x, const float *c, float *d2, int64_t *index, fsgs_stream_t stream);
/* The same search, same results bit for bit, through a uniform grid over the control points (built by the call in
 * the workspace: one small launch): a query evaluates only the control points of the cells around it, shell by
 * shell, until no unvisited cell can hold anything closer than its K-th candidate.  Hundreds instead of thousands
 * of distance evaluations per query at M = 4096. */
size_t fsgs_knn_grid_workspace_bytes(int M);
int fsgs_knn_grid(int N, int M, int K, const float *x, const float *c, float *d2, int64_t *index, void *workspace,
    size_t workspace_bytes, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Visibility-masked Adam.
 * Replaces AdamMasksedUpdated   (src/other/adam_masked_update.cu:9-36): one [N,M] tensor per call.
 * fsgs_adam_masked_multi updates up to 8 tensors that share N and the mask in ONE launch
 * (the six per-step launches of fast_2d_gs/sparse_gaussian_adam.py:20-46 folded together).
 * ---------------------------------------------------------------------------------------------- */
int fsgs_adam_masked(float *param, const float *grad, float *exp_avg, float *exp_avg_sq, const uint8_t *visible,
    float lr, float b1, float b2, float eps, int64_t N, int64_t M, fsgs_stream_t stream);

typedef struct fsgs_adam_tensor {
  float *param;
  const float *grad;
  float *exp_avg;
  float *exp_avg_sq;
  int32_t M;    /* elements per Gaussian */
  float lr;     /* bias-corrected learning rate for this tensor */
  float eps;
} fsgs_adam_tensor;

#define FSGS_ADAM_MAX_TENSORS 8
int fsgs_adam_masked_multi(int n_tensors, const fsgs_adam_tensor *tensors /* host */, const uint8_t *visible,
    int64_t N, float b1, float b2, fsgs_stream_t stream);
/* The same with the mask as floats (visible where > 0): the form in which the mask travels with the gradients
 * through one all-reduce (the sum over ranks of 0/1 masks is > 0 exactly where any rank saw the Gaussian). */
int fsgs_adam_masked_multi_fmask(int n_tensors, const fsgs_adam_tensor *tensors /* host */, const float *visible,
    int64_t N, float b1, float b2, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Splat -> screen matrix, standalone.
 * Replaces gs_2d_fast_compute_transmat_forward / gs_2d_fast_compute_trans_mat_backward
 * (src/gaussian_splatting/gs_2d_fast_preprocess.cu:871-909, 923-958).
 * ---------------------------------------------------------------------------------------------- */
int fsgs_transmat_forward(int P, const float *means, const float *scales, const float *rots, const float *Tw2v,
    const float *Tv2s, float *trans_mat, float *normals, fsgs_stream_t stream);
int fsgs_transmat_backward(int P, const float *scales, const float *rots, const float *Tw2v, const float *Tv2s,
    const float *grad_trans_mat, const float *grad_normals, float *grad_means, float *grad_scales, float *grad_rots,
    fsgs_stream_t stream);
/* The same in double precision (the reference dispatches both over the floating types, :889,936). */
int fsgs_transmat_forward_f64(int P, const double *means, const double *scales, const double *rots, const double *Tw2v,
    const double *Tv2s, double *trans_mat, double *normals, fsgs_stream_t stream);
int fsgs_transmat_backward_f64(int P, const double *scales, const double *rots, const double *Tw2v, const double *Tv2s,
    const double *grad_trans_mat, const double *grad_normals, double *grad_means, double *grad_scales,
    double *grad_rots, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Superpoint LBS warp (rigid blend), optionally fused into the preprocess.
 * Restates fast_2d_gs/network.py:545-573, 630-645 (PyTorch + lietorch in the reference; additive).
 *   means  = sum_k w_k (R(q_k) xyz + t_k)          scales = exp(scaling_raw) + sum_k w_k ds_k
 *   rots   = normalize(rotation_raw + sum_k w_k dr_k)
 * ---------------------------------------------------------------------------------------------- */
typedef struct fsgs_lbs {
  int32_t K, M;
  const float *xyz;          /* [P,3] canonical positions */
  const float *scaling_raw;  /* [P,2] log scales */
  const float *rotation_raw; /* [P,4] */
  const int64_t *knn_idx;    /* [P,K] */
  const float *knn_w;        /* [P,K] */
  const float *sp_q;         /* [M,4] unit quaternions */
  const float *sp_t;         /* [M,3] translations */
  const float *sp_dr;        /* [M,4] additive rotation deltas */
  const float *sp_ds;        /* [M,2] additive scale deltas */
  /* Optional (both or neither): the P*K (Gaussian, neighbour) pairs grouped by superpoint, built once per
   * k-NN refresh: sp_pairs holds the pair ids i*K + k ordered by knn_idx, sp_pair_offsets [M+1] where each
   * superpoint's run starts.  With them the backward sums every superpoint's gradient in one block, without
   * atomics and bit-reproducibly; without them it accumulates with floating-point atomics. */
  const int32_t *sp_pair_offsets;
  const int32_t *sp_pairs;
} fsgs_lbs;

int fsgs_lbs_warp_forward(int P, const fsgs_lbs *lbs /* host */, float *means, float *scales, float *rots,
    fsgs_stream_t stream);

typedef struct fsgs_lbs_grads {
  float *g_xyz, *g_scaling_raw, *g_rotation_raw; /* [P,3] [P,2] [P,4]  written */
  float *g_knn_w;                                /* [P,K]              written */
  float *g_sp_q, *g_sp_t, *g_sp_dr, *g_sp_ds;    /* [M,*]              zeroed then accumulated */
  /* accumulate != 0: the per-Gaussian outputs (g_xyz, g_scaling_raw, g_rotation_raw, g_knn_w) are ADDED to instead
   * of written (the gradients of several views summed in place, views in call order); the superpoint rows g_sp_* are
   * written as always, because every view has its own motion.  Needs the grouped pairs of fsgs_lbs and scratch_rot
   * [P,4], which receives this view's rotation gradient. */
  int32_t accumulate;
  float *scratch_rot;
} fsgs_lbs_grads;

int fsgs_lbs_warp_backward(int P, const fsgs_lbs *lbs /* host */, const float *g_means, const float *g_scales,
    const float *g_rots, const fsgs_lbs_grads *grads /* host */, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Per-Gaussian preprocess.
 * Replaces the kernel stage of gs_2d_fast_preprocess_forward
 * (gs_2d_fast_preprocess.cu:160-262 launched at :688) and counts, in the same pass, the tiles
 * each splat really covers (the 4-corner conic test of duplicateWithKeys, :264-327).
 * Every output row is written (zeros for culled Gaussians): no pre-zeroing needed.
 * With sh_degree < 0, shs holds [P,3] colours, colors may alias shs and is left untouched.
 * ---------------------------------------------------------------------------------------------- */
typedef struct fsgs_preprocess_args {
  int32_t P, W, H, sh_degree;
  int32_t n_dc;   /* coefficients per Gaussian in shs (1 when sh_rest is given) */
  int32_t n_rest; /* coefficients per Gaussian in sh_rest, 0 when absent */
  const float *means, *scales, *rots; /* [P,3] [P,2] [P,4]; ignored when lbs != NULL */
  const float *opac;                  /* [P,1] */
  const float *shs, *sh_rest;         /* [P,n_dc,3], [P,n_rest,3] or NULL */
  const float *Tw2v, *Tv2s, *campos;  /* [4,4] [3,3] [3] */
  const float *trans_precomp;         /* [P,3,3] or NULL */
  const uint8_t *culling;             /* [P] or NULL */
  const fsgs_lbs *lbs;                /* host pointer or NULL; when set, warped_* receive the warped set */
  float *warped_means, *warped_scales, *warped_rots;
  /* outputs */
  float *means2D, *colors, *trans_mat, *inverse_m, *normal_opacity, *depths; /* [P,2|3|9|9|4|1] */
  int32_t *radii;         /* [P] */
  int32_t *tiles_touched; /* [P] tile-rectangle area (the reference's slot count) */
  float *records;         /* [P,32] packed render records, or NULL */
  int32_t *tile_counts;   /* [T] pairs per tile; zeroed by the call */
  int64_t *counters;      /* [FSGS_NUM_COUNTERS]; zeroed by the call */
  /* != 0: opac holds logits; the kernel applies the sigmoid the model applies before its render call
   * (fast_2d_gs/network.py:611), in the same float operations (1 / (1 + exp(-x))) */
  int32_t opacity_is_logit;
} fsgs_preprocess_args;

int fsgs_preprocess_forward(const fsgs_preprocess_args *args /* host */, fsgs_stream_t stream);

/* Builds the packed render records from the reference-layout tensors (used when the compositing
 * operators are called on their own, as GS_2D_fast_render_forward is). */
int fsgs_pack_records(int P, const float *means2D, const float *colors, const float *normal_opacity,
    const float *trans_mat, const float *inverse_m, float *records, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Tile binning.
 * Replaces InclusiveSum + duplicateWithKeys + DeviceRadixSort::SortPairs + identifyTileRanges
 * (gs_2d_fast_preprocess.cu:716-778).  Output order is identical to the reference's: per tile by
 * (depth bits, Gaussian index); point_list[R*..min(R,capacity)) = -1; ranges of empty tiles = (0,0).
 * tile_order [T] lists tile ids by decreasing list length (launch order for the compositing kernels).
 * ---------------------------------------------------------------------------------------------- */
typedef struct fsgs_bin_args {
  int32_t P, W, H;
  const float *means2D, *inverse_m, *depths, *opac;
  const int32_t *radii;
  const int32_t *tile_counts; /* from fsgs_preprocess_forward */
  int64_t *counters;
  int64_t capacity;     /* entries available in point_list */
  int32_t *point_list;  /* [capacity] */
  int64_t *ranges;      /* [T,2] */
  int32_t *tile_order;  /* [T] */
  void *workspace;
  size_t workspace_bytes;
  int32_t opac_stride;  /* floats between consecutive opacities; 0 means 1 (4 reads them out of normal_opacity) */
} fsgs_bin_args;

size_t fsgs_bin_workspace_bytes(int W, int H, int64_t capacity);
int fsgs_bin_tiles(const fsgs_bin_args *args /* host */, fsgs_stream_t stream);

/* Tile binning for callers that must not allocate.  No counterpart in the reference.
 *
 * Same inputs, outputs and results as fsgs_bin_tiles, but the scratch memory (pair keys, per-tile cursors and
 * offsets) lives in a fixed array inside the library instead of a caller-provided workspace, and the call makes
 * no cudaMalloc / cudaFree / allocating library call.  It is meant for hosts that get their device memory once at
 * start-up and may not go back to the CUDA allocator while frames are being produced -- a viewer or engine
 * plug-in with a fixed memory budget, or a plain C caller that has no caching allocator and would otherwise pay a
 * device-synchronising cudaMalloc/cudaFree per frame.  args->workspace and args->workspace_bytes are ignored.
 *
 * Limits: capacity <= FSGS_NOALLOC_MAX_PAIRS and tiles <= FSGS_NOALLOC_MAX_TILES, else FSGS_ERR_LIMIT and
 * nothing is launched.  The array (about 10.7 MB) is held by every GPU that loads the library until the process
 * exits.  The first call on each device looks up the array's device address (with that device current); make
 * that first call before any stream capture.  All calls on a device share the array: calls that overlap on the
 * GPU (different streams) race; calls on one stream are safe.  Nothing has to be cleared between calls. */
#define FSGS_NOALLOC_MAX_PAIRS (1 << 20)
#define FSGS_NOALLOC_MAX_TILES 16384
int fsgs_bin_tiles_noalloc(const fsgs_bin_args *args /* host */, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Per-tile alpha compositing.
 * Replaces GS_2D_fast_render_forward / GS_2D_fast_render_backward
 * (src/gaussian_splatting/gs_2d_fast_redner.cu:839-953, 955-1074; kernels :22-271, :273-561).
 * The backward follows the semantics of the per-pixel variant that training uses, with the
 * per-Gaussian sums reduced across each warp and across the tile in shared memory before one global
 * reduction per (Gaussian, tile, component).
 * ---------------------------------------------------------------------------------------------- */
typedef struct fsgs_render_args {
  int32_t P, W, H;
  float near_n, far_n;
  int32_t only_image;         /* 1: colour + opacity only */
  const float *records;       /* [P,32] */
  const int32_t *point_list;
  const int64_t *ranges;      /* [T,2] */
  const int32_t *tile_order;  /* [T] or NULL */
  const float *trans_mat_t2;  /* [P,3,3] or NULL (flow) */
  /* outputs: every pixel is written */
  float *out_color;    /* [3,H,W] */
  float *out_opacity;  /* [H,W] */
  float *out_extras;   /* [8,H,W] or NULL when only_image */
  float *out_flow;     /* [H,W,2] or NULL */
  int32_t *n_contrib;  /* [2,H,W] */
  int32_t *accum_max_count;     /* [P] or NULL */
  float *accum_weights_p;       /* [P] or NULL */
  int32_t *accum_weights_count; /* [P] or NULL */
  /* counters of the binning that made the lists, or NULL.  When given and counters[FSGS_CNT_OVERFLOW] != 0 (the
   * lists were truncated) every output pixel is set to NaN instead of being composited from incomplete lists. */
  int64_t *counters;
} fsgs_render_args;

/* Not provided: the five extra outputs of the reference's bucketed forward (max_contrib, bucket_to_tile, sampled_T,
 * sampled_acc, sampled_aux; gs_2d_fast_redner.cu:872-888), which exist to feed its bucketed backward.  The backward
 * here needs no samples; the Python operator accepts per_tile_bucket_offset, ignores it and returns placeholders in
 * those five positions (max_contrib all zero, the others empty). */
int fsgs_render_forward(const fsgs_render_args *args /* host */, fsgs_stream_t stream);

/* Work counter (diagnostic; no counterpart in the reference): replays every pixel's walk over its tile's list with
 * the forward pass's tests (gs_2d_fast_redner.cu:152-191) and writes counts[3] (device, int64):
 *   [0] traversed (pixel, list entry) pairs: entries visited before the pixel's exit,
 *   [1] contributing pairs: those that are blended,
 *   [2] pairs the backward pass walks: entries up to each pixel's last contributor.
 * Reads records, point_list and ranges of args; the output pointers are ignored. */
int fsgs_render_pair_counts(const fsgs_render_args *args /* host */, int64_t *counts, fsgs_stream_t stream);

typedef struct fsgs_render_bwd_args {
  int32_t P, W, H;
  float near_n, far_n;
  const float *records;
  const int32_t *point_list;
  const int64_t *ranges;
  const int32_t *tile_order;
  const float *trans_mat_t2;
  const float *out_opacity, *out_extras; /* forward outputs; out_extras NULL selects the colour-only adjoint */
  const int32_t *n_contrib;
  /* Upstream gradients, contiguous.  dL_dextras (or out_extras) NULL selects the adjoint without auxiliary
   * channels: 15 instead of 21 gradient components per splat, dL_dtrans_mat and the normal part of
   * dL_dnormal_opacity stay zero.  In that variant dL_dopacity may be NULL, which reproduces the reference kernel
   * instantiated without auxiliary channels (it ignores the opacity gradient, gs_2d_fast_redner.cu:338-341);
   * non-NULL it is honoured.  dL_dflow may be NULL. */
  const float *dL_dcolor, *dL_dopacity, *dL_dextras, *dL_dflow;
  /* outputs, zeroed by the call */
  float *dL_dcolors;         /* [P,3] */
  float *dL_dmeans2D;        /* [P,2] */
  float *dL_dtrans_mat;      /* [P,3,3] (row 2 only) */
  float *dL_dinverse_m;      /* [P,3,3] */
  float *dL_dnormal_opacity; /* [P,4] */
  int64_t *counters;
} fsgs_render_bwd_args;

int fsgs_render_backward(const fsgs_render_bwd_args *args /* host */, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Row compaction of up to FSGS_COMPACT_MAX_TENSORS tensors by one keep mask (rows in order).
 * Replaces the per-tensor boolean indexing of change_optimizer(op='prune') / prune_points
 * (fast_2d_gs/gaussian_splatting.py:495-548, 557-568): parameters and both Adam moments in one launch.
 * fsgs_compact_plan: keep [N] bytes -> workspace (fsgs_compact_workspace_bytes(N)), *count (device,
 * optional) = number of kept rows.  fsgs_compact_rows: dst[k] = src[i_k] for every tensor; rows are
 * row_words 4-byte words wide (any 4-byte type, or 8-byte types counted as two words); dst must hold
 * count rows.  N < 2^31.
 * ---------------------------------------------------------------------------------------------- */
#define FSGS_COMPACT_MAX_TENSORS 24
typedef struct fsgs_row_tensor {
  const void *src;
  void *dst;
  int32_t row_words;
} fsgs_row_tensor;

size_t fsgs_compact_workspace_bytes(int64_t N);
int fsgs_compact_plan(int64_t N, const uint8_t *keep, void *workspace, size_t workspace_bytes, int64_t *count,
                      fsgs_stream_t stream);
int fsgs_compact_rows(int n_tensors, const fsgs_row_tensor *tensors, int64_t N, const uint8_t *keep,
                      const void *workspace, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Densification: clone / split of Gaussians and the surgery on the optimiser state, on the device.
 * Replaces the tensor-by-tensor torch.cat / boolean indexing of densify_and_clone, densify_and_split,
 * densification_postfix and change_optimizer(op='concat' | 'prune')
 * (fast_2d_gs/gaussian_splatting.py:498-548, 570-622; the 2-D split of fast_2d_gs/network.py:1156-1185) and the
 * statistics of add_densification_stats (network.py:1143-1154).
 *  fsgs_densify_stats   one view: for radii > 0, accum += |viewspace_grad[i]| (the densification proxy the
 *                       preprocess backward leaves), denom += 1, max_radii = max(max_radii, radii).
 *  fsgs_densify_select  flags[i] = 1 (clone) when accum/denom (NaN -> 0) >= grad_threshold and
 *                       max(exp(scaling_raw[i])) <= scale_threshold, 2 (split) when >= and larger, else 0.
 *  fsgs_split_children  n children (N per parent, copy-major like torch's repeat(N, 1)): position = parent position
 *                       + R(normalised raw quaternion) (s_x z[k,0], s_y z[k,1], 0), log-scale = log(s / (0.8 N));
 *                       z [n,2] are standard-normal draws supplied by the caller.
 *  fsgs_gather_rows     dst[k] = src[index[k]] for up to FSGS_COMPACT_MAX_TENSORS tensors in one launch; index[k] < 0
 *                       gives a zero row (the fresh Adam moments of new Gaussians).  Rows as in fsgs_compact_rows.
 * The order of the result -- kept originals, clones, split children copy 0, copy 1 -- is the reference's.
 * ---------------------------------------------------------------------------------------------- */
int fsgs_densify_stats(int P, const float *viewspace_grad, const int32_t *radii, float *accum, float *denom,
                       float *max_radii, fsgs_stream_t stream);
int fsgs_densify_select(int P, const float *accum, const float *denom, const float *scaling_raw, float grad_threshold,
                        float scale_threshold, uint8_t *flags, fsgs_stream_t stream);
int fsgs_split_children(int n, int N, const int32_t *parent, const float *z, const float *xyz,
                        const float *scaling_raw, const float *rotation_raw, float *xyz_out, float *scaling_out,
                        fsgs_stream_t stream);
int fsgs_gather_rows(int n_tensors, const fsgs_row_tensor *tensors, int64_t n_out, const int32_t *index,
                     fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Structural similarity, 11x11 Gaussian window (sigma 1.5, zero padding), forward and adjoint.
 * Replaces fusedssim / fusedssim_backward   (src/other/structural_similarity.cu:340-381; callers
 * fast_2d_gs/losses/ssim.py:24-45; the map is that of _ssim, ssim.py:48-67).
 * Images are [B,C,H,W] contiguous.  Forward: ssim_map and, when the three dm_* pointers are given, the
 * partial derivatives of the map with respect to mu1, w*x^2 and w*xy.  `sums` (optional, [2], zeroed by
 * the caller) receives the sum of the map and the sum of |img1 - img2| (for mean reductions without
 * another pass).  Backward: dL_dimg1 from dL_dmap, or from the constant dL_dmap_uniform when dL_dmap is
 * NULL; l1_weight * sign(img1 - img2) is added (0 to leave it out).  B*C <= 65535.
 * ---------------------------------------------------------------------------------------------- */
int fsgs_ssim_forward(int B, int C, int H, int W, float C1, float C2, const float *img1, const float *img2,
                      float *ssim_map, float *dm_dmu1, float *dm_dsigma1_sq, float *dm_dsigma12, float *sums,
                      fsgs_stream_t stream);
int fsgs_ssim_backward(int B, int C, int H, int W, float C1, float C2, const float *img1, const float *img2,
                       const float *dL_dmap, float dL_dmap_uniform, float l1_weight, const float *dm_dmu1,
                       const float *dm_dsigma1_sq, const float *dm_dsigma12, float *dL_dimg1, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Preprocess backward.
 * Replaces gs_2d_fast_preprocess_backward   (gs_2d_fast_preprocess.cu:536-609, 784-859).
 * grad_means2D is consumed and then overwritten with the densification proxy, as in the reference.
 * Every row of every grad_* output is written: zeros for Gaussians the forward pass culled (radii <= 0),
 * so the outputs need no initialisation (the reference's Python zero-fills them before its kernel, which
 * writes visible rows only: same result).  grad_means2D rows of culled Gaussians are left as they are.
 * ---------------------------------------------------------------------------------------------- */
#define FSGS_SH_SOURCE_FLOATS 7 /* row of sh_source: colour gradient 3 | view direction 3 | visibility 1 */
typedef struct fsgs_preprocess_bwd_args {
  int32_t P, W, H, sh_degree, n_dc, n_rest;
  const float *means, *scales, *rots, *shs, *sh_rest;
  const float *Tw2v, *Tv2s, *campos;
  const float *trans_mat, *colors;
  const int32_t *radii;
  float *grad_means2D;
  const float *grad_trans_mat, *grad_inverse_m, *grad_colors, *grad_normal_opacity;
  float *grad_means, *grad_scales, *grad_rots, *grad_opac, *grad_shs, *grad_sh_rest; /* last two may be NULL */
  /* Optional extensions for a training loop that keeps everything on the device (all may stay 0 / NULL):
   *  normal_opacity [P,4] (the forward output): grad_opac then receives the gradient of the opacity LOGIT,
   *    g * o * (1 - o), the adjoint of the sigmoid the model applies (network.py:611);
   *  visible [P] float: 1 for Gaussians with radii > 0, else 0 (the mask of the sparse Adam, in a form that can ride
   *    in the same all-reduce as the gradients);
   *  accumulate != 0: grad_opac, grad_shs, grad_sh_rest are ADDED to (rows of culled Gaussians untouched) and
   *    visible is raised to 1 where visible, never lowered -- the gradients of several views summed in place, in
   *    call order.  grad_means / grad_scales / grad_rots are always written (they feed the LBS adjoint, which has its
   *    own accumulate flag).  Supported for sh_degree < 0 and for degrees 1..3 with SH rows of at most 48 floats;
   *    otherwise FSGS_ERR_UNSUPPORTED;
   *  counters (the binning's, of the view these gradients come from): when counters[FSGS_CNT_OVERFLOW] != 0 the
   *    tile lists were truncated and the gradients are wrong; visible is then written as -infinity on EVERY row, and
   *    a row that is -infinity is never raised again.  -infinity survives the summation over views and over ranks,
   *    is "not visible" to the masked Adam, and so drops the whole step, on every rank, on the device. */
  const float *normal_opacity;
  float *visible;
  int32_t accumulate;
  const int64_t *counters;
  /* sh_source [P,FSGS_SH_SOURCE_FLOATS] (optional, sh_degree >= 0): the two factors of this view's SH gradient, which
   * is their outer product -- the colour gradient after the clamp (3) and the unit direction camera -> Gaussian (3);
   * zeros for culled Gaussians -- and this view's visibility (1: 1 visible, 0 culled, -infinity when counters report
   * an overflow).  grad_shs / grad_sh_rest may then be NULL: seven floats per Gaussian and view travel between ranks
   * instead of 48 + 1, and fsgs_sh_grad_from_views rebuilds the summed gradient and the summed mask on every rank. */
  float *sh_source;
} fsgs_preprocess_bwd_args;

int fsgs_preprocess_backward(const fsgs_preprocess_bwd_args *args /* host */, fsgs_stream_t stream);

/* Summed SH gradient of n_slots views from their factors (the rank-1 structure of preprocess_backward's SH part,
 * gs_2d_fast_preprocess.cu:536-609 with the SH adjoint of utils/ops_3d/spherical_harmonics.py:242-302):
 *   g_sh[i][k][c] = sum over slots s, in the order given, of basis_k(dir[s][i]) * g_colour[s][i][c]
 * sh_source: slot s at sh_source + s * slot_stride floats, [P,FSGS_SH_SOURCE_FLOATS] as written by
 * fsgs_preprocess_backward; a slot of zeros adds nothing.  order[n_slots] (host, values < n_slots): the slots in
 * summation order (view order, so that every rank forms the same bits).  g_sh_dc [P,3] and g_sh_rest [P,n_rest,3] are
 * WRITTEN (zeros beyond the active degree); visible [P] (optional) receives the sum of the slots' visibility
 * entries: > 0 where some view saw the Gaussian, -infinity when any view overflowed -- the float mask of
 * fsgs_adam_masked_multi_fmask.  sh_degree 0..3, n_slots <= FSGS_MAX_VIEW_SLOTS. */
/* The same rows (and, optionally, the same separate mask with the same accumulate / counters semantics) without the
 * preprocess adjoint:
 * from the forward pass's warped means [P,3] and colours [P,3] (pre-clamp sign: colour > 0), the compositing adjoint's
 * colour gradient [P,3] and radii.  Lets the exchange between ranks start before the preprocess adjoint runs. */
int fsgs_sh_factors(int P, const float *means, const float *colors, const float *grad_colors, const int32_t *radii,
                    const float *campos, const int64_t *counters, int accumulate, float *sh_source, float *visible,
                    fsgs_stream_t stream);

#define FSGS_MAX_VIEW_SLOTS 64
int fsgs_sh_grad_from_views(int P, int sh_degree, int n_rest, int n_slots, const int32_t *order /* host */,
                            const float *sh_source, int64_t slot_stride, float *g_sh_dc, float *g_sh_rest,
                            float *visible, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Per-pixel epilogue of GS_2D_fast_render, one kernel each way.
 * Replaces the PyTorch operator chain of renderer/gs_2d_fast_render.py:731-740 with depths_to_points /
 * depth_to_normal (:558-589): normals_world [3,H,W] = view normals (out_extras[1:4]) rotated by Tw2v[:3,:3];
 * surf_depth [1,H,W] = expected depth * (1 - depth_ratio) + depth_ratio * median depth, non-finite values
 * zeroed; surf_normal [3,H,W] = normalised cross product of the central differences of the back-projected
 * depth map, times the pixel's opacity (opacity is treated as a constant, as the reference detaches it),
 * zero on the image border.  The backward writes g_extras [8,H,W] (channels 5..7 zero); any of the three
 * upstream gradients may be NULL.
 * ---------------------------------------------------------------------------------------------- */
int fsgs_epilogue_forward(int W, int H, float depth_ratio, const float *Tw2v, const float *Tv2c,
    const float *out_extras, const float *out_opacity, float *normals_world, float *surf_depth, float *surf_normal,
    fsgs_stream_t stream);
int fsgs_epilogue_backward(int W, int H, float depth_ratio, const float *Tw2v, const float *Tv2c,
    const float *out_extras, const float *out_opacity, const float *g_normals_world, const float *g_surf_depth,
    const float *g_surf_normal, float *g_extras, fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Per-step superpoint motion: the deformation network evaluated on the superpoint centres at one time, and the
 * kernel-weighted LBS weights.
 * Replaces the PyTorch module chain of SC_GS_DeformNetwork.forward (fast_2d_gs/network.py:1748-1776: frequency
 * encodings -- fast_2d_gs/_C/src/nerf/freqencoder.cu:8-32 --, time network, `depth` linear layers of `width` units
 * with ReLU and one skip connection after layer `skip`, heads for translation, scale, rotation and -- local_frame --
 * the superpoint's own rotation) followed by the head of warp() (network.py:545-549: q = normalize(g_rot + (0,0,0,1)),
 * t' = t + c - R(q) c) and the adjoint of all of it; and calc_LBS_weight's kernel form (network.py:506-513).
 * fp32 throughout.  Parameters live in ONE flat buffer (fsgs_motion_param_count floats), every weight matrix stored
 * [inputs, outputs] row major (the transpose of torch.nn.Linear.weight), sections starting on 16-byte boundaries at
 * the offsets fsgs_motion_param_offsets reports; g_params has the same layout.  With time_out == 0 there is no time
 * network and the time encoding itself is appended to the position encoding.  Outputs: sp_q [M,4] unit quaternions
 * ((0,0,0,1) without local_frame), sp_t [M,3], sp_dr [M,4], sp_ds [M,2] -- the motion fsgs_lbs takes.  The
 * backward reads the workspace the forward left (same args), takes the gradients of the four outputs and writes
 * (accumulate != 0: adds to) g_params; positions and time get no gradient (the reference detaches them).
 * Limits: 32 <= width <= 256 (multiple of 32), depth <= 16, position encoding + time features + width <= 384.
 * ---------------------------------------------------------------------------------------------- */
typedef struct fsgs_motion_cfg {
  int32_t M;            /* superpoints */
  int32_t depth, width; /* linear layers, units per layer */
  int32_t skip;         /* the input encodings are concatenated in front of the output of this layer */
  int32_t deg_p, deg_t; /* frequency-encoding degrees of position and time */
  int32_t time_hidden, time_out; /* time network 2*deg_t+1 -> time_hidden -> time_out; time_out == 0: none */
  int32_t local_frame;  /* != 0: fourth head (rotation of the superpoint about its own centre) */
  float scale_p, scale_t; /* encoder input scales (<= 0: 1) */
} fsgs_motion_cfg;

typedef struct fsgs_motion_args {
  fsgs_motion_cfg cfg;
  const float *sp_points; /* [M,3] */
  const float *t;         /* [1] device */
  const float *params;    /* flat parameter buffer */
  float *sp_q, *sp_t, *sp_dr, *sp_ds;
  const float *g_sp_q, *g_sp_t, *g_sp_dr, *g_sp_ds; /* backward only */
  float *g_params;                                  /* backward only */
  int32_t accumulate;
  void *workspace;
  size_t workspace_bytes;
} fsgs_motion_args;

int64_t fsgs_motion_param_count(const fsgs_motion_cfg *cfg);
/* offsets [6 + 2*depth] (floats): time0 W, b, time2 W, b, then W, b of every linear layer, then heads W, b (heads
 * packed column-wise: translation 3 | scale 3 | rotation 4 | local rotation 4); inputs [depth]: inputs per layer */
int fsgs_motion_param_offsets(const fsgs_motion_cfg *cfg, int64_t *offsets, int32_t *inputs);
size_t fsgs_motion_workspace_bytes(const fsgs_motion_cfg *cfg);
int fsgs_motion_forward(const fsgs_motion_args *args /* host */, fsgs_stream_t stream);
int fsgs_motion_backward(const fsgs_motion_args *args /* host */, fsgs_stream_t stream);

/* weights [P,K] = normalise(exp(-d2 / (2 r^2)) * sigma + 1e-7), r = exp(raw_radius[idx]), sigma =
 * sigmoid(raw_weight[idx]) (raw_weight NULL: 1).  Backward: g_weights [P,K] -> g_raw_radius [M], g_raw_weight [M]
 * (written, or added to when accumulate != 0): every pair's term once per Gaussian, then one block per superpoint
 * sums its grouped pairs (the same sp_pair_offsets / sp_pairs as in fsgs_lbs) in a fixed order, no atomics; the
 * distances are treated as constants. */
int fsgs_lbs_weights_forward(int P, int K, const float *d2, const int64_t *idx, const float *raw_radius,
    const float *raw_weight, float *weights, fsgs_stream_t stream);
size_t fsgs_lbs_weights_backward_workspace_bytes(int P, int K); /* 8 P K: one (radius, weight) term per pair */
int fsgs_lbs_weights_backward(int P, int K, int M, const float *d2, const int64_t *idx, const float *raw_radius,
    const float *raw_weight, const float *g_weights, const int32_t *sp_pair_offsets, const int32_t *sp_pairs,
    float *g_raw_radius, float *g_raw_weight, int accumulate, void *workspace, size_t workspace_bytes,
    fsgs_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * One view of a training iteration in two calls (forward, backward), all intermediates in one workspace.
 * Covers the body of the reference's per-view loop, fast_2d_gs/network.py:683-745 -- sigmoid of the opacity
 * logits (:611), superpoint LBS warp (:523-573, 630-645), GS_2D_fast_render -- and the backward autograd derives
 * from it, down to the gradients of the model's leaves (positions, log-scales, raw rotations, opacity logits,
 * SH coefficients) and of the superpoint motion.  Launches only; nothing is allocated or synchronised.
 *
 * fsgs_view_forward writes out_color [3,H,W], out_opacity [H,W], out_extras [8,H,W], n_contrib [2,H,W], radii
 * (optional, [P]) and counters.  fsgs_view_backward needs the same struct again (same workspace, untouched since
 * the forward) plus the upstream gradients: dL_dcolor [3,H,W] is required; dL_dopacity [H,W] may be NULL (zero);
 * dL_dextras [8,H,W] NULL selects the adjoint without auxiliary channels.  Gradients go to the g_* pointers:
 * accumulate == 0 writes every row (zeros for culled Gaussians), accumulate != 0 adds to the per-Gaussian gradients
 * (views summed in call order; g_knn_w must then be given); the superpoint-motion gradients g_sp_* belong to this
 * view's motion and are always written.  visible [P] floats: 1 where radii > 0 (raised, never lowered,
 * when accumulating).  viewspace_grad [P,2] (optional) receives the densification proxy of visible Gaussians
 * (gs_2d_fast_preprocess.cu:605-608).  list_capacity: entries reserved for the tile lists; when
 * counters[FSGS_CNT_OVERFLOW] comes back non-zero the view was composited from truncated lists.
 * ---------------------------------------------------------------------------------------------- */
typedef struct fsgs_view_args {
  int32_t P, W, H, sh_degree, n_dc, n_rest;
  float near_n, far_n;
  const float *opacity_raw;      /* [P,1] logits */
  const float *sh_dc, *sh_rest;  /* [P,n_dc,3], [P,n_rest,3] or NULL */
  const fsgs_lbs *lbs;           /* host pointer: canonical geometry, neighbours, this view's superpoint motion */
  const float *Tw2v, *Tv2s, *campos;
  float *out_color, *out_opacity, *out_extras;
  int32_t *n_contrib;
  int32_t *radii;     /* [P] or NULL */
  int64_t *counters;  /* [FSGS_NUM_COUNTERS] */
  const float *dL_dcolor, *dL_dopacity, *dL_dextras;
  float *g_xyz, *g_scaling_raw, *g_rotation_raw, *g_opacity_raw, *g_sh_dc, *g_sh_rest;
  float *g_knn_w, *g_sp_q, *g_sp_t, *g_sp_dr, *g_sp_ds; /* [P,K], [M,4], [M,3], [M,4], [M,2]; NULL: discarded */
  float *visible;        /* [P] or NULL */
  float *viewspace_grad; /* [P,2] or NULL */
  int32_t accumulate;
  /* backward only: 0 = everything; 1 = up to and including the preprocess adjoint (g_sh_*, g_opacity_raw and visible
   * are then final in stream order: their exchange may start); 2 = the remaining LBS adjoint;
   * 3 = the compositing adjoint, then g_sh_source and visible by fsgs_sh_factors (final in stream order before the
   * preprocess adjoint has run: needs g_sh_source); 4 = the rest after 3: preprocess adjoint (which leaves
   * g_sh_source and visible alone) and LBS adjoint */
  int32_t phase;
  int64_t list_capacity;
  void *workspace;
  size_t workspace_bytes;
  /* backward only, optional: [P,FSGS_SH_SOURCE_FLOATS] factors of this view's SH gradient and its visibility
   * (fsgs_preprocess_bwd_args.sh_source);
   * g_sh_dc / g_sh_rest may then be NULL */
  float *g_sh_source;
} fsgs_view_args;

size_t fsgs_view_workspace_bytes(int P, int W, int H, int64_t list_capacity, int K, int M);
/* fsgs_render_pair_counts on the lists of the view last passed to fsgs_view_forward (same struct, same workspace). */
int fsgs_view_pair_counts(const fsgs_view_args *args /* host */, int64_t *counts, fsgs_stream_t stream);
/* Optional stage timing of the two calls below (a diagnostic): after fsgs_stage_timing(1), every stage they launch
 * is bracketed by CUDA events recorded on the call's stream; fsgs_stage_times() waits for the recorded events and
 * returns, per stage, the summed milliseconds and the number of launches since timing was switched on, then
 * clears them.  Stages: 0 preprocess forward (LBS warp fused), 1 tile binning, 2 compositing forward,
 * 3 compositing backward, 4 preprocess backward, 5 LBS backward.  Process-wide state, one thread at a time. */
#define FSGS_NUM_STAGES 6
int fsgs_stage_timing(int enable);
int fsgs_stage_times(float *ms /* host [FSGS_NUM_STAGES] */, int32_t *launches /* host [FSGS_NUM_STAGES] */);
int fsgs_view_forward(const fsgs_view_args *args /* host */, fsgs_stream_t stream);
int fsgs_view_backward(const fsgs_view_args *args /* host */, fsgs_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FSGS_H_ */
