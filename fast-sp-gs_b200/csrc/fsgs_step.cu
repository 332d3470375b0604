// One view of a training step as two calls: every launch of the forward (LBS warp + preprocess, binning,
// compositing) and of the backward (compositing adjoint, preprocess adjoint, LBS adjoint) issued from C on one
// stream, with all intermediates in one caller-provided workspace.  A host loop then crosses the language boundary
// twice per view instead of once per kernel, allocates nothing per step, and the per-Gaussian gradients of several
// views are summed in place (accumulate), so a rank that renders several views still has ONE buffer to exchange.
// The step these two calls cover is the body of the reference's per-view loop, fast_2d_gs/network.py:683-745
// (render) and the backward that autograd derives from it.
#include "fsgs_common.cuh"

#include <vector>

namespace fsgs {

// ---- optional stage timing -------------------------------------------------------------------------------------
struct StageSpan {
  int stage;
  cudaEvent_t t0, t1;
};
static bool g_timing = false;
static std::vector<StageSpan> g_spans;
static std::vector<cudaEvent_t> g_event_pool;

static cudaEvent_t take_event() {
  if (!g_event_pool.empty()) {
    cudaEvent_t e = g_event_pool.back();
    g_event_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

struct StageTimer {  // brackets one stage when timing is on
  StageSpan span;
  cudaStream_t st;
  bool on;
  StageTimer(int stage, cudaStream_t s) : st(s), on(g_timing) {
    if (!on) return;
    span.stage = stage, span.t0 = take_event(), span.t1 = take_event();
    cudaEventRecord(span.t0, st);
  }
  ~StageTimer() {
    if (!on) return;
    cudaEventRecord(span.t1, st);
    g_spans.push_back(span);
  }
};

struct ViewWorkspace {
  float *warped_means, *warped_scales, *warped_rots;
  float *means2D, *colors, *trans_mat, *inverse_m, *normal_opacity, *depths;
  int32_t *radii, *tiles_touched;
  float *records;
  int32_t *tile_counts, *point_list, *tile_order;
  int64_t *ranges;
  void *bin_ws;
  size_t bin_ws_bytes;
  float *g_colors, *g_means2D, *g_trans_mat, *g_inverse_m, *g_normal_opacity;
  float *g_means, *g_scales, *g_rots, *scratch_rot, *g_knn_w, *g_sp;
  size_t total;
};

static inline size_t up256(size_t n) { return (n + 255) & ~(size_t) 255; }

// Carves (base may be NULL: sizes only).  Every array starts on a 256-byte boundary.
static ViewWorkspace carve_view(void *base, int P, int W, int H, int64_t capacity, int K, int M) {
  const size_t T = (size_t) ((W + kTile - 1) / kTile) * ((H + kTile - 1) / kTile);
  const size_t n = (size_t) (P > 0 ? P : 1);
  size_t off = 0;
  char *b = (char *) base;
  auto take = [&](size_t bytes) {
    void *p = b ? (void *) (b + off) : nullptr;
    off += up256(bytes);
    return p;
  };
  ViewWorkspace w;
  w.warped_means = (float *) take(12 * n), w.warped_scales = (float *) take(8 * n), w.warped_rots = (float *) take(16 * n);
  w.means2D = (float *) take(8 * n), w.colors = (float *) take(12 * n), w.trans_mat = (float *) take(36 * n);
  w.inverse_m = (float *) take(36 * n), w.normal_opacity = (float *) take(16 * n), w.depths = (float *) take(4 * n);
  w.radii = (int32_t *) take(4 * n), w.tiles_touched = (int32_t *) take(4 * n);
  w.records = (float *) take(sizeof(float) * kRecFloats * n);
  w.tile_counts = (int32_t *) take(4 * T);
  w.point_list = (int32_t *) take(4 * (size_t) (capacity > 0 ? capacity : 1));
  w.tile_order = (int32_t *) take(4 * T);
  w.ranges = (int64_t *) take(16 * T);
  w.bin_ws_bytes = fsgs_bin_workspace_bytes(W, H, capacity);
  w.bin_ws = take(w.bin_ws_bytes);
  w.g_colors = (float *) take(12 * n), w.g_means2D = (float *) take(8 * n), w.g_trans_mat = (float *) take(36 * n);
  w.g_inverse_m = (float *) take(36 * n), w.g_normal_opacity = (float *) take(16 * n);
  w.g_means = (float *) take(12 * n), w.g_scales = (float *) take(8 * n), w.g_rots = (float *) take(16 * n);
  w.scratch_rot = (float *) take(16 * n);
  w.g_knn_w = (float *) take(4 * n * (size_t) (K > 0 ? K : 1));
  w.g_sp = (float *) take(4 * 13 * (size_t) (M > 0 ? M : 1) + 4 * 256);
  w.total = off;
  return w;
}

static bool view_args_ok(const fsgs_view_args *a) {
  return a && a->P >= 0 && a->W > 0 && a->H > 0 && a->list_capacity >= 0 && a->workspace && a->lbs && a->opacity_raw &&
         a->sh_dc && a->Tw2v && a->Tv2s && a->campos && a->counters && a->out_color && a->out_opacity &&
         a->out_extras && a->n_contrib;
}

}  // namespace fsgs

using namespace fsgs;

extern "C" size_t fsgs_view_workspace_bytes(int P, int W, int H, int64_t list_capacity, int K, int M) {
  return carve_view(nullptr, P, W, H, list_capacity, K, M).total;
}

extern "C" int fsgs_view_forward(const fsgs_view_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(view_args_ok(a));
  const ViewWorkspace w = carve_view(a->workspace, a->P, a->W, a->H, a->list_capacity, a->lbs->K, a->lbs->M);
  if (a->workspace_bytes < w.total) return FSGS_ERR_WORKSPACE;
  fsgs_preprocess_args p = {};
  p.P = a->P, p.W = a->W, p.H = a->H, p.sh_degree = a->sh_degree, p.n_dc = a->n_dc, p.n_rest = a->n_rest;
  p.opac = a->opacity_raw, p.opacity_is_logit = 1;
  p.shs = a->sh_dc, p.sh_rest = a->sh_rest;
  p.Tw2v = a->Tw2v, p.Tv2s = a->Tv2s, p.campos = a->campos;
  p.lbs = a->lbs, p.warped_means = w.warped_means, p.warped_scales = w.warped_scales, p.warped_rots = w.warped_rots;
  p.means2D = w.means2D, p.colors = w.colors, p.trans_mat = w.trans_mat, p.inverse_m = w.inverse_m;
  p.normal_opacity = w.normal_opacity, p.depths = w.depths;
  p.radii = a->radii ? a->radii : w.radii, p.tiles_touched = w.tiles_touched, p.records = w.records;
  p.tile_counts = w.tile_counts, p.counters = a->counters;
  int rc;
  {
    StageTimer t(0, (cudaStream_t) stream);
    rc = fsgs_preprocess_forward(&p, stream);
  }
  if (rc != FSGS_OK) return rc;

  fsgs_bin_args b = {};
  b.P = a->P, b.W = a->W, b.H = a->H;
  // the activated opacity sits in normal_opacity[:, 3]; the binning reads it with a stride of four floats
  b.means2D = w.means2D, b.inverse_m = w.inverse_m, b.depths = w.depths, b.opac = w.normal_opacity + 3;
  b.opac_stride = 4;
  b.radii = p.radii, b.tile_counts = w.tile_counts, b.counters = a->counters, b.capacity = a->list_capacity;
  b.point_list = w.point_list, b.ranges = w.ranges, b.tile_order = w.tile_order;
  b.workspace = w.bin_ws, b.workspace_bytes = w.bin_ws_bytes;
  {
    StageTimer t(1, (cudaStream_t) stream);
    rc = fsgs_bin_tiles(&b, stream);
  }
  if (rc != FSGS_OK) return rc;

  fsgs_render_args r = {};
  r.P = a->P, r.W = a->W, r.H = a->H, r.near_n = a->near_n, r.far_n = a->far_n, r.only_image = 0;
  r.records = w.records, r.point_list = w.point_list, r.ranges = w.ranges, r.tile_order = w.tile_order;
  r.out_color = a->out_color, r.out_opacity = a->out_opacity, r.out_extras = a->out_extras, r.n_contrib = a->n_contrib;
  r.counters = a->counters;
  StageTimer t(2, (cudaStream_t) stream);
  return fsgs_render_forward(&r, stream);
}

extern "C" int fsgs_view_pair_counts(const fsgs_view_args *a, int64_t *counts, fsgs_stream_t stream) {
  FSGS_REQUIRE(view_args_ok(a) && counts);
  const ViewWorkspace w = carve_view(a->workspace, a->P, a->W, a->H, a->list_capacity, a->lbs->K, a->lbs->M);
  if (a->workspace_bytes < w.total) return FSGS_ERR_WORKSPACE;
  fsgs_render_args r = {};
  r.P = a->P, r.W = a->W, r.H = a->H, r.near_n = a->near_n, r.far_n = a->far_n;
  r.records = w.records, r.point_list = w.point_list, r.ranges = w.ranges;
  return fsgs_render_pair_counts(&r, counts, stream);
}

extern "C" int fsgs_stage_timing(int enable) {
  g_timing = enable != 0;
  if (!g_timing) {
    for (const StageSpan &s : g_spans) g_event_pool.push_back(s.t0), g_event_pool.push_back(s.t1);
    g_spans.clear();
  }
  return FSGS_OK;
}

extern "C" int fsgs_stage_times(float *ms, int32_t *launches) {
  FSGS_REQUIRE(ms && launches);
  for (int k = 0; k < FSGS_NUM_STAGES; ++k) ms[k] = 0.0f, launches[k] = 0;
  for (const StageSpan &s : g_spans) {
    float t = 0.0f;
    if (cudaEventSynchronize(s.t1) != cudaSuccess || cudaEventElapsedTime(&t, s.t0, s.t1) != cudaSuccess)
      return FSGS_ERR_LAUNCH;
    ms[s.stage] += t, launches[s.stage] += 1;
    g_event_pool.push_back(s.t0), g_event_pool.push_back(s.t1);
  }
  g_spans.clear();
  return FSGS_OK;
}

extern "C" int fsgs_view_backward(const fsgs_view_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(view_args_ok(a) && a->dL_dcolor);
  FSGS_REQUIRE(a->g_xyz && a->g_scaling_raw && a->g_rotation_raw && a->g_opacity_raw);
  // the SH gradient leaves either as rows (g_sh_dc, g_sh_rest) or as its two factors (g_sh_source), or both
  FSGS_REQUIRE(a->g_sh_source || (a->g_sh_dc && (a->sh_rest == nullptr || a->n_rest == 0 || a->g_sh_rest)));
  const int K = a->lbs->K, M = a->lbs->M;
  const ViewWorkspace w = carve_view(a->workspace, a->P, a->W, a->H, a->list_capacity, K, M);
  if (a->workspace_bytes < w.total) return FSGS_ERR_WORKSPACE;
  float *g_means2D = a->viewspace_grad ? a->viewspace_grad : w.g_means2D;
  FSGS_REQUIRE(a->phase >= 0 && a->phase <= 4 && (a->phase != 3 || a->g_sh_source));
  int rc = FSGS_OK;
  const bool do_blend = a->phase == 0 || a->phase == 1 || a->phase == 3;
  const bool do_pre = a->phase == 0 || a->phase == 1 || a->phase == 4;
  const bool do_lbs = a->phase == 0 || a->phase == 2 || a->phase == 4;
  if (do_blend) {
  fsgs_render_bwd_args r = {};
  r.P = a->P, r.W = a->W, r.H = a->H, r.near_n = a->near_n, r.far_n = a->far_n;
  r.records = w.records, r.point_list = w.point_list, r.ranges = w.ranges, r.tile_order = w.tile_order;
  r.out_opacity = a->out_opacity, r.out_extras = a->dL_dextras ? a->out_extras : nullptr, r.n_contrib = a->n_contrib;
  r.dL_dcolor = a->dL_dcolor, r.dL_dopacity = a->dL_dopacity, r.dL_dextras = a->dL_dextras;
  r.dL_dcolors = w.g_colors, r.dL_dmeans2D = g_means2D, r.dL_dtrans_mat = w.g_trans_mat;
  r.dL_dinverse_m = w.g_inverse_m, r.dL_dnormal_opacity = w.g_normal_opacity;
  r.counters = a->counters;
  {
    StageTimer t(3, (cudaStream_t) stream);
    rc = fsgs_render_backward(&r, stream);
  }
  if (rc != FSGS_OK) return rc;
  }
  if (a->phase == 3) {
    StageTimer t(4, (cudaStream_t) stream);
    return fsgs_sh_factors(a->P, w.warped_means, w.colors, w.g_colors, a->radii ? a->radii : w.radii, a->campos,
        a->counters, a->accumulate, a->g_sh_source, a->visible, stream);
  }
  if (do_pre) {
  fsgs_preprocess_bwd_args p = {};
  p.P = a->P, p.W = a->W, p.H = a->H, p.sh_degree = a->sh_degree, p.n_dc = a->n_dc, p.n_rest = a->n_rest;
  p.means = w.warped_means, p.scales = w.warped_scales, p.rots = w.warped_rots;
  p.shs = a->sh_dc, p.sh_rest = a->sh_rest;
  p.Tw2v = a->Tw2v, p.Tv2s = a->Tv2s, p.campos = a->campos;
  p.trans_mat = w.trans_mat, p.colors = w.colors, p.radii = a->radii ? a->radii : w.radii;
  p.grad_means2D = g_means2D, p.grad_trans_mat = w.g_trans_mat, p.grad_inverse_m = w.g_inverse_m;
  p.grad_colors = w.g_colors, p.grad_normal_opacity = w.g_normal_opacity;
  p.grad_means = w.g_means, p.grad_scales = w.g_scales, p.grad_rots = w.g_rots;
  p.grad_opac = a->g_opacity_raw, p.grad_shs = a->g_sh_dc, p.grad_sh_rest = a->g_sh_rest;
  p.normal_opacity = w.normal_opacity, p.accumulate = a->accumulate;
  p.counters = a->counters;  // an overflowed view poisons the mask: the optimiser then drops the step
  // after phase 3 the factors and the mask are already out (and may be travelling)
  p.visible = a->phase == 4 ? nullptr : a->visible;
  p.sh_source = a->phase == 4 ? nullptr : a->g_sh_source;
  {
    StageTimer t(4, (cudaStream_t) stream);
    rc = fsgs_preprocess_backward(&p, stream);
  }
  if (rc != FSGS_OK) return rc;
  }
  if (!do_lbs) return FSGS_OK;

  fsgs_lbs_grads g = {};
  g.g_xyz = a->g_xyz, g.g_scaling_raw = a->g_scaling_raw, g.g_rotation_raw = a->g_rotation_raw;
  g.g_knn_w = a->g_knn_w ? a->g_knn_w : w.g_knn_w;
  float *sp = w.g_sp;  // q [M,4] | dr [M,4] | t [M,3] | ds [M,2], the 16-byte rows first
  g.g_sp_q = a->g_sp_q ? a->g_sp_q : sp;
  g.g_sp_dr = a->g_sp_dr ? a->g_sp_dr : sp + 4 * (size_t) M;
  g.g_sp_t = a->g_sp_t ? a->g_sp_t : sp + 8 * (size_t) M;
  g.g_sp_ds = a->g_sp_ds ? a->g_sp_ds : sp + 11 * (size_t) M + (M & 1);
  // an accumulating call adds to a buffer that persists between views: it must be the caller's, not the workspace's
  if (a->accumulate && !a->g_knn_w) return FSGS_ERR_INVALID_ARGUMENT;
  g.accumulate = a->accumulate;
  g.scratch_rot = w.scratch_rot;
  StageTimer t(5, (cudaStream_t) stream);
  return fsgs_lbs_warp_backward(a->P, a->lbs, w.g_means, w.g_scales, w.g_rots, &g, stream);
}
