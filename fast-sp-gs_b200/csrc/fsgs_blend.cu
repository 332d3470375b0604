// Per-tile alpha compositing, forward and backward.
//
// One block of 256 threads per 16x16 tile; each warp owns an 8x4 pixel sub-tile.  A tile's list is staged
// through shared memory in batches of packed 112-byte render records.  Every warp skips the splats of a
// batch whose alpha >= 1/255 box misses its sub-tile (the box is conservative, so results are unchanged),
// pixels stop once their transmittance is spent, warps and blocks stop once all their pixels have.
//
// The backward walks each list back to front like the reference's per-pixel kernel
// (gs_2d_fast_redner.cu:273-561) but sums the 21 gradient components of a splat across the warp with a
// transposing shuffle reduction, then across the tile's warps in shared memory, and issues one global
// reduction per (Gaussian, tile, component) instead of one per (Gaussian, pixel, component).
//
// Per-pixel arithmetic (ray-splat intersection, alpha, thresholds) keeps the reference's expression forms:
// a splat flipping across the alpha >= 1/255 cut would move a pixel by more than the 1e-4 image tolerance.
#include "fsgs_common.cuh"

namespace fsgs {

constexpr int kStage = 128;          // splats per shared-memory batch
constexpr int kQ = kRecQuadsUsed;    // float4 per staged record
// Gradient components per splat.  With upstream gradients on the auxiliary channels: colour 0-2, normal 3-5,
// opacity 6, mean2D 7-8, depth row of trans_mat 9-11, inverse_m 12-20.  Without (colour and opacity upstream only)
// the normal and depth-row components are identically zero and are left out: colour 0-2, opacity 3, mean2D 4-5,
// inverse_m 6-14.
template <bool AUX>
struct GradMap {
  static constexpr int N = AUX ? 21 : 15;
  static constexpr int kNrm = 3, kTw = 9;  // AUX only
  static constexpr int kOpac = AUX ? 6 : 3, kM2d = AUX ? 7 : 4, kIm = AUX ? 12 : 6;
};
constexpr unsigned kFull = 0xffffffffu;

struct FwdDev {
  const long long *counters;  // optional: a non-zero overflow counter poisons the frame (NaN) instead of hiding it
  int P, W, H, gx;
  float near_n, far_n;
  const float4 *records;
  const int32_t *point_list;
  const long long *ranges;
  const int32_t *tile_order;
  const float *m2;  // trans_mat_t2
  float *out_color, *out_opacity, *out_extras;
  float2 *out_flow;
  int32_t *n_contrib;
  int32_t *accum_max_count;
  float *accum_weights_p;
  int32_t *accum_weights_count;
};

// Staging.  A tile's list is consumed in batches of kStage entries.  The Gaussian ids of a batch are fetched two
// batches ahead (plain loads into a register, parked in a small ring in shared memory), its records one batch ahead
// with 16-byte asynchronous copies (global -> shared without passing through registers), so that the gather latency
// of batch k+1 is hidden behind the arithmetic of batch k and the block meets at one barrier per batch.
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned) __cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Starts the copies of one batch: records (kQ float4 each) of the Gaussians in s_gid[0..cnt) and, for flow, their
// 3x3 matrices at t2 (plain loads: 36-byte rows are not 16-byte aligned).
template <bool FLOW>
__device__ __forceinline__ void issue_stage(const float4 *__restrict__ records, const int *s_gid, int cnt,
    const float *__restrict__ m2, float4 *s_rec, float *s_m2) {
  for (int e = threadIdx.x; e < cnt * kQ; e += blockDim.x) {
    const int r = e / kQ, qd = e - r * kQ;
    cp_async16(s_rec + e, records + (size_t) s_gid[r] * (kRecFloats / 4) + qd);
  }
  cp_async_commit();
  if (FLOW) {
    for (int e = threadIdx.x; e < cnt * 9; e += blockDim.x) {
      const int r = e / 9, k = e - r * 9;
      s_m2[e] = __ldg(m2 + (size_t) s_gid[r] * 9 + k);
    }
  }
}

// Can the splat of this record reach alpha >= 1/255 on any pixel of the rectangle [bx0,bx1] x [by0,by1]?
// Conservative (never false when some pixel passes), much tighter than the box for elongated, slanted footprints.
//   alpha >= 1/255  <=>  min(rho3d, rho2d) <= tau  (tau' padded), with
//   rho2d = 2 |x - centre|^2  -> distance from the centre to the rectangle;
//   rho3d = (p0^2 + p1^2) / p2^2, p = IM (x, y, 1)  ->  Q(x, y) = p0^2 + p1^2 - tau' p2^2 <= 0, a quadratic whose
//   minimum over the rectangle is at its unconstrained minimiser if that lies inside, else on one of the four edges.
// If Q is not convex (the splat's disc crosses the camera plane) the answer is "maybe".  A tolerance proportional to
// the cancelling terms covers rounding.
__device__ __forceinline__ bool subtile_may_hit(const float4 q0, const float4 q1, const float4 q2, const float4 q3,
    float bx0, float bx1, float by0, float by1) {
  const float tau = q0.w;
  if (!(tau > 0.0f)) return false;
  // low-pass disc
  const float ddx = fmaxf(fmaxf(bx0 - q0.x, q0.x - bx1), 0.0f), ddy = fmaxf(fmaxf(by0 - q0.y, q0.y - by1), 0.0f);
  if (2.0f * (ddx * ddx + ddy * ddy) <= tau) return true;
  const float xc = 0.5f * (bx0 + bx1), yc = 0.5f * (by0 + by1);
  const float hx = 0.5f * (bx1 - bx0) + 0.01f, hy = 0.5f * (by1 - by0) + 0.01f;
  const float a0 = q1.x, b0 = q1.y, a1 = q1.w, b1 = q2.x, a2 = q2.z, b2 = q2.w;
  const float P0 = a0 * xc + b0 * yc + q1.z, P1 = a1 * xc + b1 * yc + q2.y, P2 = a2 * xc + b2 * yc + q3.x;
  const float tP2 = tau * P2, ta2 = tau * a2, tb2 = tau * b2;
  const float Q0 = P0 * P0 + P1 * P1 - tP2 * P2;
  const float gx = 2.0f * (P0 * a0 + P1 * a1 - tP2 * a2), gy = 2.0f * (P0 * b0 + P1 * b1 - tP2 * b2);
  const float Axx = a0 * a0 + a1 * a1 - ta2 * a2, Ayy = b0 * b0 + b1 * b1 - tb2 * b2;
  const float Axy = 2.0f * (a0 * b0 + a1 * b1 - ta2 * b2);
  const float det = 4.0f * Axx * Ayy - Axy * Axy;
  if (!(Axx > 0.0f && Ayy > 0.0f && det > 1e-6f * (4.0f * Axx * Ayy))) return true;
  const float tol = 1e-4f * (P0 * P0 + P1 * P1 + tP2 * P2);
  const float inv_det = __fdividef(1.0f, det);
  const float ux = (Axy * gy - 2.0f * Ayy * gx) * inv_det, uy = (Axy * gx - 2.0f * Axx * gy) * inv_det;
  float qmin;
  if (fabsf(ux) <= hx && fabsf(uy) <= hy) {
    qmin = Q0 + 0.5f * (gx * ux + gy * uy);
  } else {
    const float inv_2ayy = __fdividef(0.5f, Ayy), inv_2axx = __fdividef(0.5f, Axx);
    qmin = 3.0e38f;
#pragma unroll
    for (int sgn = -1; sgn <= 1; sgn += 2) {
      const float ex = sgn * hx;  // edge x = ex: quadratic in y
      const float ly = gy + Axy * ex, cy = Q0 + ex * (gx + Axx * ex);
      const float ty = fminf(fmaxf(-ly * inv_2ayy, -hy), hy);
      qmin = fminf(qmin, cy + ty * (ly + Ayy * ty));
      const float ey = sgn * hy;  // edge y = ey: quadratic in x
      const float lx = gx + Axy * ey, cx = Q0 + ey * (gy + Ayy * ey);
      const float tx = fminf(fmaxf(-lx * inv_2axx, -hx), hx);
      qmin = fminf(qmin, cx + tx * (lx + Axx * tx));
    }
  }
  return !(qmin > tol);  // also true when anything went NaN
}

struct Hit {
  float sx, sy, pz, rho3d, rho2d, depth, G, alpha, dx, dy;
};

// (pixel, splat) evaluation shared by both passes; false when the pair is skipped.
// Same operations, in the same order, as the reference kernels (gs_2d_fast_redner.cu:152-186).
// FAST replaces the two IEEE divisions and expf by their approximate forms: used by the backward pass only, whose
// tolerance is relative (1e-3 per tensor); the forward pass decides the alpha and transmittance cuts and stays exact,
// and the backward pass falls back to the exact forms wherever an approximate value comes close to a cut.
template <bool FAST>
__device__ __forceinline__ bool eval_pair(const float4 *rec, float px, float py, float near_n, Hit &h, float &opa,
    float3 &Tw) {
  const float4 q0 = rec[0], q1 = rec[1], q2 = rec[2], q3 = rec[3];
  const float p0 = q1.x * px + q1.y * py + q1.z;
  const float p1 = q1.w * px + q2.x * py + q2.y;
  const float p2 = q2.z * px + q2.w * py + q3.x;
  if (p2 == 0.0f) return false;
  h.pz = p2;
  if (FAST) {
    const float inv = __fdividef(1.0f, p2);
    h.sx = p0 * inv, h.sy = p1 * inv;
  } else {
    h.sx = p0 / p2, h.sy = p1 / p2;
  }
  h.rho3d = (h.sx * h.sx + h.sy * h.sy);
  h.dx = q0.x - px, h.dy = q0.y - py;
  h.rho2d = 2.0f * (h.dx * h.dx + h.dy * h.dy);
  const float rho = fminf(h.rho3d, h.rho2d);
  Tw = make_float3(q3.y, q3.z, q3.w);
  h.depth = (h.sx * Tw.x + h.sy * Tw.y) + Tw.z;
  if (h.depth < near_n * (FAST ? 1.0f - 2e-5f : 1.0f)) return false;
  opa = q0.z;
  const float power = -0.5f * rho;
  if (power > 0.0f) return false;
  h.G = FAST ? __expf(power) : expf(power);
  h.alpha = fminf(0.99f, opa * h.G);
  if (FAST) {
    // The forward pass decides the depth and alpha cuts with exact division and expf.  Within a guard band around
    // either cut the approximate forms could land on the other side -- the pair would then be blended by one pass
    // and skipped by the other -- so there the pair is evaluated again exactly (rare: a relative band of 2e-5).
    const float cut = 1.0f / 255.0f, raw = opa * h.G;
    if (raw < cut * (1.0f - 2e-5f)) return false;
    if (raw < cut * (1.0f + 2e-5f) || h.depth < near_n * (1.0f + 2e-5f))
      return eval_pair<false>(rec, px, py, near_n, h, opa, Tw);
    return true;
  }
  if (h.alpha < 1.0f / 255.0f) return false;
  return true;
}

template <bool AUX, bool FLOW>
__global__ void __launch_bounds__(256) blend_forward_kernel(FwdDev a) {
  __shared__ float4 s_recs[2][kStage * kQ];
  __shared__ int s_gids[3][kStage];
  __shared__ float s_m2s[2][FLOW ? kStage * 9 : 1];

  const int tile = a.tile_order ? a.tile_order[blockIdx.x] : blockIdx.x;
  const int tx = tile % a.gx, ty = tile / a.gx;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sx0 = tx * kTile + (warp & 1) * 8, sy0 = ty * kTile + (warp >> 1) * 4;
  const int ix = sx0 + (lane & 7), iy = sy0 + (lane >> 3);
  const bool inside = ix < a.W && iy < a.H;
  const float px = (float) ix, py = (float) iy;
  const float bx0 = (float) sx0, bx1 = (float) (sx0 + 7), by0 = (float) sy0, by1 = (float) (sy0 + 3);
  const size_t HW = (size_t) a.H * a.W;
  const size_t pix = (size_t) iy * a.W + ix;

  const long long r0 = a.ranges[2 * tile], r1 = a.ranges[2 * tile + 1];
  const int n = (int) (r1 - r0);
  if (a.counters && a.counters[FSGS_CNT_OVERFLOW] != 0) {
    // the tile lists were truncated: a frame composited from them would look plausible and be wrong
    if (inside) {
      const float nan = __int_as_float(0x7fc00000);
      a.out_opacity[pix] = nan;
      a.n_contrib[pix] = 0, a.n_contrib[HW + pix] = AUX ? -1 : 0;
      a.out_color[pix] = nan, a.out_color[HW + pix] = nan, a.out_color[2 * HW + pix] = nan;
      if (AUX)
        for (int c = 0; c < 8; ++c) a.out_extras[c * HW + pix] = nan;
      if (FLOW) a.out_flow[pix] = make_float2(nan, nan);
    }
    return;
  }

  const float far_scale = a.far_n / (a.far_n - a.near_n);
  bool done = !inside;
  float T = 1.0f, C0 = 0, C1 = 0, C2 = 0;
  float N0 = 0, N1 = 0, N2 = 0, D = 0, M1 = 0, M2 = 0, dist = 0, med_depth = 0, F0 = 0, F1 = 0;
  int last = 0, med_contrib = -1;
  float wmax = 0;
  int wmax_id = -1;
  bool flag = false;

  // prologue: ids of batches 0 and 1, records of batch 0
  const int32_t *list = a.point_list + r0;
  const int n_st = (n + kStage - 1) / kStage;
  if ((int) threadIdx.x < min(kStage, n)) s_gids[0][threadIdx.x] = list[threadIdx.x];
  if ((int) threadIdx.x < min(kStage, n - kStage)) s_gids[1][threadIdx.x] = list[kStage + threadIdx.x];
  __syncthreads();
  if (n_st > 0) issue_stage<FLOW>(a.records, s_gids[0], min(kStage, n), a.m2, s_recs[0], s_m2s[0]);

  for (int st = 0; st < n_st; ++st) {
    const int base = st * kStage;
    const int cnt = min(kStage, n - base);
    const float4 *s_rec = s_recs[st & 1];
    const int *s_gid = s_gids[st % 3];
    const float *s_m2 = s_m2s[st & 1];
    // the ids of batch st+2 travel while this batch is composited
    int id2 = 0;
    const bool has2 = (int) threadIdx.x < min(kStage, n - base - 2 * kStage);
    if (has2) id2 = list[base + 2 * kStage + threadIdx.x];
    cp_async_wait_all();  // this thread's copies of batch st have landed
    if (__syncthreads_and(done)) break;  // everybody's have, and the other buffer is free again
    if (st + 1 < n_st)
      issue_stage<FLOW>(a.records, s_gids[(st + 1) % 3], min(kStage, n - base - kStage), a.m2, s_recs[(st + 1) & 1],
          s_m2s[(st + 1) & 1]);
    for (int c = 0; c < cnt && !__all_sync(kFull, done); c += 32) {
      const int rr = c + lane;
      bool hit = false;
      if (rr < cnt) {
        const float4 box = s_rec[rr * kQ + 4];
        hit = box.x <= bx1 && box.y >= bx0 && box.z <= by1 && box.w >= by0;
        if (hit)
          hit = subtile_may_hit(s_rec[rr * kQ], s_rec[rr * kQ + 1], s_rec[rr * kQ + 2], s_rec[rr * kQ + 3], bx0, bx1,
              by0, by1);
      }
      unsigned mask = __ballot_sync(kFull, hit);
      while (mask) {
        const int j = __ffs(mask) - 1;
        mask &= mask - 1;
        if (done) continue;
        const int r = c + j;
        const float4 *rec = s_rec + r * kQ;
        Hit h;
        float opa;
        float3 Tw;
        if (!eval_pair<false>(rec, px, py, a.near_n, h, opa, Tw)) continue;
        const float test_T = T * (1 - h.alpha);
        if (test_T < 0.0001f) {
          done = true;
          continue;
        }
        const float w = h.alpha * T;
        const int contributor = base + r + 1;
        const float4 q5 = rec[5];
        if (AUX) {
          const float4 q6 = rec[6];
          const float A = 1 - T;
          // normalised depth for the distortion terms: feeds no cut, so the reciprocal may be approximate
          const float m = far_scale * (1 - a.near_n * __fdividef(1.0f, h.depth));
          dist += (m * m * A + M2 - 2 * m * M1) * w;
          D += h.depth * w;
          M1 += m * w;
          M2 += m * m * w;
          if (T > 0.5f) {
            med_depth = h.depth;
            med_contrib = contributor;
          }
          N0 += q5.w * w, N1 += q6.x * w, N2 += q6.y * w;
          if (a.accum_max_count || a.accum_weights_p || a.accum_weights_count) {
            const int g = s_gid[r];
            if (wmax < w) wmax = w, wmax_id = g, flag = true;
            if (a.accum_weights_p) atomicAdd(a.accum_weights_p + g, w);
            if (a.accum_weights_count) atomicAdd(a.accum_weights_count + g, 1);
            // the flag is never cleared: every later contribution counts (gs_2d_fast_redner.cu:82,211-215,227)
            if (flag && a.accum_max_count) atomicAdd(a.accum_max_count + wmax_id, 1);
          }
          if (FLOW) {
            const float *m2 = s_m2 + r * 9;
            const float u = m2[0] * h.sx + m2[1] * h.sy + m2[2];
            const float v = m2[3] * h.sx + m2[4] * h.sy + m2[5];
            float ww = m2[6] * h.sx + m2[7] * h.sy + m2[8];
            ww = fabsf(ww) < 1e-5f ? 1e-5f : ww;
            F0 += (u / ww - px) * w;
            F1 += (v / ww - py) * w;
          }
        }
        C0 += q5.x * w, C1 += q5.y * w, C2 += q5.z * w;
        T = test_T;
        last = contributor;
      }
    }
    if (has2) s_gids[(st + 2) % 3][threadIdx.x] = id2;  // read after the next barrier
  }

  if (inside) {
    const float A = 1.0f - T;
    a.out_opacity[pix] = A;
    a.n_contrib[pix] = last;
    a.out_color[pix] = C0, a.out_color[HW + pix] = C1, a.out_color[2 * HW + pix] = C2;
    if (AUX) {
      a.n_contrib[HW + pix] = med_contrib;
      a.out_extras[pix] = D;
      a.out_extras[HW + pix] = N0, a.out_extras[2 * HW + pix] = N1, a.out_extras[3 * HW + pix] = N2;
      a.out_extras[4 * HW + pix] = med_depth;
      a.out_extras[5 * HW + pix] = dist;
      a.out_extras[6 * HW + pix] = M1;
      a.out_extras[7 * HW + pix] = M2;
      if (FLOW) a.out_flow[pix] = make_float2(A > 0 ? F0 / A : 0.0f, A > 0 ? F1 / A : 0.0f);
    } else {
      a.n_contrib[HW + pix] = 0;
    }
  }
}

// Work counter for roofline arithmetic (a diagnostic, not part of a frame): replays every pixel's walk over its
// tile's list with the forward pass's own tests and counts
//   [0] traversed pairs: (pixel, list entry) visited before the pixel's exit (transmittance exhausted or list end),
//   [1] contributing pairs: those that pass the depth, power and alpha cuts and are blended,
//   [2] pairs the backward pass walks: entries up to each pixel's last contributor.
// One thread per pixel, records read straight from global memory.
__global__ void __launch_bounds__(256) pair_count_kernel(FwdDev a, unsigned long long *__restrict__ counts) {
  __shared__ unsigned long long s_sum[3][8];
  const int tile = blockIdx.x;
  const int tx = tile % a.gx, ty = tile / a.gx;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ix = tx * kTile + (warp & 1) * 8 + (lane & 7), iy = ty * kTile + (warp >> 1) * 4 + (lane >> 3);
  const bool inside = ix < a.W && iy < a.H;
  const float px = (float) ix, py = (float) iy;
  const long long r0 = a.ranges[2 * tile], r1 = a.ranges[2 * tile + 1];
  unsigned long long traversed = 0, blended = 0, last = 0;
  if (inside) {
    float T = 1.0f;
    for (long long e = r0; e < r1; ++e) {
      ++traversed;
      const float4 *rec = a.records + (size_t) a.point_list[e] * (kRecFloats / 4);
      Hit h;
      float opa;
      float3 Tw;
      if (!eval_pair<false>(rec, px, py, a.near_n, h, opa, Tw)) continue;
      const float test_T = T * (1 - h.alpha);
      if (test_T < 0.0001f) break;
      T = test_T;
      ++blended;
      last = (unsigned long long) (e - r0 + 1);
    }
  }
  unsigned long long v[3] = {traversed, blended, last};
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    for (int o = 16; o > 0; o >>= 1) v[k] += __shfl_xor_sync(kFull, v[k], o);
    if (lane == 0) s_sum[k][warp] = v[k];
  }
  __syncthreads();
  if (threadIdx.x < 3) {
    unsigned long long t = 0;
    for (int w = 0; w < 8; ++w) t += s_sum[threadIdx.x][w];
    atomicAdd(counts + threadIdx.x, t);
  }
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------

struct BwdDev {
  int P, W, H, gx;
  float near_n, far_n;
  const float4 *records;
  const int32_t *point_list;
  const long long *ranges;
  const int32_t *tile_order;
  const float *m2;
  const float *out_opacity, *out_extras;
  const int32_t *n_contrib;
  const float *g_color, *g_opacity, *g_extras;
  const float2 *g_flow;
  float *g_colors, *g_means2D, *g_trans_mat, *g_inverse_m, *g_normal_opacity;
};

// Sums N per-lane components across the warp.  Five exchange rounds; in each, the lanes whose bit `width` is clear
// keep the lower half of the values they carry and the others the upper half, so the count a lane carries goes
// 21 -> 11 -> 6 -> 3 -> 2 -> 1 and the whole reduction takes 11+6+3+2+1 = 23 shuffles.  Afterwards the lane holds the
// warp total of component `comp` (lanes whose path ran into the padding of an odd split hold 0 and a comp that may
// be >= N).
template <int N>
__device__ __forceinline__ float warp_transpose_reduce(float (&v)[32], int lane, int &comp) {
  int n = N;
  comp = 0;
#pragma unroll
  for (int width = 16; width >= 1; width >>= 1) {
    const int h = (n + 1) / 2;
    const bool up = lane & width;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (k < h) {
        const float lo = v[k], hi = (k + h < n) ? v[k + h] : 0.0f;
        const float send = up ? lo : hi;
        const float keep = up ? hi : lo;
        v[k] = keep + __shfl_xor_sync(kFull, send, width);
      }
    }
    comp += up ? h : 0;
    n = h;
  }
  return v[0];
}

template <bool AUX, bool FLOW>
__global__ void __launch_bounds__(256, AUX ? 3 : 4) blend_backward_kernel(BwdDev a) {
  // dynamic shared memory: two record buffers, two gradient buffers, a ring of four id batches (+ flow matrices)
  extern __shared__ float4 s_dyn[];
  float4 *const s_recs = s_dyn;                                               // [2][kStage * kQ]
  using GM = GradMap<AUX>;
  constexpr int kGrad = GM::N;
  float *const s_grads = reinterpret_cast<float *>(s_recs + 2 * kStage * kQ);  // [2][kStage * kGrad]
  int *const s_gids = reinterpret_cast<int *>(s_grads + 2 * kStage * kGrad);   // [4][kStage]
  float *const s_m2s = reinterpret_cast<float *>(s_gids + 4 * kStage);         // [2][kStage * 9] when FLOW
  __shared__ int s_max[8];

  const int tile = a.tile_order ? a.tile_order[blockIdx.x] : blockIdx.x;
  const int tx = tile % a.gx, ty = tile / a.gx;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sx0 = tx * kTile + (warp & 1) * 8, sy0 = ty * kTile + (warp >> 1) * 4;
  const int ix = sx0 + (lane & 7), iy = sy0 + (lane >> 3);
  const bool inside = ix < a.W && iy < a.H;
  const float px = (float) ix, py = (float) iy;
  const float bx0 = (float) sx0, bx1 = (float) (sx0 + 7), by0 = (float) sy0, by1 = (float) (sy0 + 3);
  const size_t HW = (size_t) a.H * a.W;
  const size_t pix = (size_t) iy * a.W + ix;

  const long long r0 = a.ranges[2 * tile], r1 = a.ranges[2 * tile + 1];
  const int n = (int) (r1 - r0);

  const float T_final = inside ? 1 - a.out_opacity[pix] : 0;
  float T = T_final;
  const int last_contributor = inside ? a.n_contrib[pix] : 0;
  const int median_contributor = (AUX && inside) ? a.n_contrib[HW + pix] : 0;

  float gpix0 = 0, gpix1 = 0, gpix2 = 0;
  float g_reg = 0, g_depth = 0, g_acc = 0, g_n0 = 0, g_n1 = 0, g_n2 = 0, g_med = 0;
  float final_D = 0, final_D2 = 0;
  float2 gflow = make_float2(0, 0);
  if (inside) {
    gpix0 = a.g_color[pix], gpix1 = a.g_color[HW + pix], gpix2 = a.g_color[2 * HW + pix];
    if (a.g_opacity) g_acc = a.g_opacity[pix];
    if (AUX) {
      g_depth = a.g_extras[pix];
      g_n0 = a.g_extras[HW + pix], g_n1 = a.g_extras[2 * HW + pix], g_n2 = a.g_extras[3 * HW + pix];
      g_med = a.g_extras[4 * HW + pix];
      g_reg = a.g_extras[5 * HW + pix];
      final_D = a.out_extras[6 * HW + pix];
      final_D2 = a.out_extras[7 * HW + pix];
    }
    if (FLOW) gflow = a.g_flow[pix];
  }
  const float final_A = 1 - T_final;
  const float far_scale = a.far_n / (a.far_n - a.near_n);

  // The reference keeps, per output channel, the colour accumulated behind the current splat
  // (acc = last_alpha * last_value + (1 - last_alpha) * acc) and sums (value - acc) * upstream over channels.
  // The recurrence is linear in the values, so one scalar recurrence on q = sum_ch value_ch * upstream_ch gives
  // the same dL/dalpha with a fifth of the state.
  float acc_q = 0, last_q = 0;
  float last_dL_dT = 0, last_alpha = 0;

  // the deepest list position any pixel of the warp / the tile blended
  int wmax = last_contributor;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wmax = max(wmax, __shfl_xor_sync(kFull, wmax, o));
  if (lane == 0) s_max[warp] = wmax;
  __syncthreads();
  int tmax = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) tmax = max(tmax, s_max[k]);
  if (tmax == 0) return;

  // Batches are taken back to front: step k works on list positions [base_k, base_k + cnt_k), entry r of the batch
  // being position base_k + cnt_k - 1 - r.  Ids are fetched two steps ahead, records one step ahead; the gradients of
  // step k-1 are flushed to global memory (and their buffer cleared) while step k accumulates into the other buffer.
  const int n_stages = (min(n, tmax) + kStage - 1) / kStage;
  const int32_t *list = a.point_list + r0;
  const int tid = threadIdx.x;
  auto step_base = [&](int k) { return (n_stages - 1 - k) * kStage; };
  auto step_cnt = [&](int k) { return min(kStage, n - step_base(k)); };
  auto flush = [&](int k) {
    float *s_grad = s_grads + (k & 1) * (kStage * kGrad);
    const int *s_gid = s_gids + (k & 3) * kStage;
    const int cnt = step_cnt(k);
    // one global reduction per (Gaussian, component) of the batch
    for (int e = tid; e < cnt * kGrad; e += blockDim.x) {
      const float v = s_grad[e];
      if (v == 0.0f) continue;
      s_grad[e] = 0.0f;
      const int r = e / kGrad, c = e - r * kGrad;
      const size_t g = (size_t) s_gid[r];
      float *dst;
      if (c < 3) dst = a.g_colors + g * 3 + c;
      else if (AUX && c < GM::kOpac) dst = a.g_normal_opacity + g * 4 + (c - GM::kNrm);
      else if (c == GM::kOpac) dst = a.g_normal_opacity + g * 4 + 3;
      else if (c < GM::kM2d + 2) dst = a.g_means2D + g * 2 + (c - GM::kM2d);
      else if (AUX && c < GM::kIm) dst = a.g_trans_mat + g * 9 + 6 + (c - GM::kTw);
      else dst = a.g_inverse_m + g * 9 + (c - GM::kIm);
      atomicAdd(dst, v);
    }
  };
  for (int e = tid; e < 2 * kStage * kGrad; e += blockDim.x) s_grads[e] = 0.0f;
  for (int k = 0; k < 2 && k < n_stages; ++k)
    if (tid < step_cnt(k)) s_gids[k * kStage + tid] = list[step_base(k) + step_cnt(k) - 1 - tid];
  __syncthreads();
  issue_stage<FLOW>(a.records, s_gids, step_cnt(0), a.m2, s_recs, s_m2s);

  for (int k = 0; k < n_stages; ++k) {
    const int base = step_base(k), cnt = step_cnt(k);
    const float4 *s_rec = s_recs + (k & 1) * (kStage * kQ);
    float *s_grad = s_grads + (k & 1) * (kStage * kGrad);
    const float *s_m2 = s_m2s + (k & 1) * (kStage * 9);
    int id2 = 0;
    const bool has2 = k + 2 < n_stages && tid < step_cnt(k + 2);
    if (has2) id2 = list[step_base(k + 2) + step_cnt(k + 2) - 1 - tid];
    cp_async_wait_all();
    __syncthreads();  // records of step k are in; step k-1 is complete in its gradient buffer
    if (k + 1 < n_stages)
      issue_stage<FLOW>(a.records, s_gids + ((k + 1) & 3) * kStage, step_cnt(k + 1), a.m2,
          s_recs + ((k + 1) & 1) * (kStage * kQ), s_m2s + ((k + 1) & 1) * (kStage * 9));
    if (k > 0) flush(k - 1);

    if (base < wmax) {
      for (int c = 0; c < cnt; c += 32) {
        const int rr = c + lane;
        bool hit = false;
        if (rr < cnt) {
          const float4 box = s_rec[rr * kQ + 4];
          hit = box.x <= bx1 && box.y >= bx0 && box.z <= by1 && box.w >= by0;
          if (hit)
            hit = subtile_may_hit(s_rec[rr * kQ], s_rec[rr * kQ + 1], s_rec[rr * kQ + 2], s_rec[rr * kQ + 3], bx0,
                bx1, by0, by1);
        }
        unsigned mask = __ballot_sync(kFull, hit);
        while (mask) {
          const int j = __ffs(mask) - 1;
          mask &= mask - 1;
          const int r = c + j;
          const int contributor = base + cnt - 1 - r;  // 0-based list position
          if (contributor >= wmax) continue;            // warp-uniform
          const float4 *rec = s_rec + r * kQ;
          float g[32];
#pragma unroll
          for (int k = 0; k < kGrad; ++k) g[k] = 0.0f;
          bool active = contributor < last_contributor;
          Hit h;
          float opa = 0;
          float3 Tw = make_float3(0, 0, 0);
          if (active) active = eval_pair<true>(rec, px, py, a.near_n, h, opa, Tw);
          if (active) {
            const float alpha = h.alpha, G = h.G;
            T = __fdividef(T, 1.0f - alpha);
            const float w = alpha * T;
            const float4 q5 = rec[5];
            float q = q5.x * gpix0 + q5.y * gpix1 + q5.z * gpix2 + g_acc;
            float dL_dalpha = 0.0f;
            g[0] = w * gpix0, g[1] = w * gpix1, g[2] = w * gpix2;

            float dL_dz = 0.0f, dL_dweight = 0.0f, dL_dsx = 0.0f, dL_dsy = 0.0f;
            if (AUX) {
              const float4 q6 = rec[6];
              const float inv_depth = __fdividef(1.0f, h.depth);
              const float m_d = far_scale * (1 - a.near_n * inv_depth);
              const float dmd_dd = far_scale * a.near_n * inv_depth * inv_depth;
              if (contributor == median_contributor - 1) dL_dz += g_med;
              dL_dweight += (final_D2 + m_d * m_d * final_A - 2 * m_d * final_D) * g_reg;
              dL_dalpha += dL_dweight - last_dL_dT;
              last_dL_dT = dL_dweight * alpha + (1 - alpha) * last_dL_dT;
              const float dL_dmd = 2.0f * (T * alpha) * (m_d * final_A - final_D) * g_reg;
              dL_dz += dL_dmd * dmd_dd;
              q += h.depth * g_depth + q5.w * g_n0 + q6.x * g_n1 + q6.y * g_n2;
              g[GM::kNrm] = w * g_n0, g[GM::kNrm + 1] = w * g_n1, g[GM::kNrm + 2] = w * g_n2;
              dL_dz += w * g_depth;
            }
            if (FLOW) {
              const float *m2 = s_m2 + r * 9;
              const float u = m2[0] * h.sx + m2[1] * h.sy + m2[2];
              const float v = m2[3] * h.sx + m2[4] * h.sy + m2[5];
              float ww = m2[6] * h.sx + m2[7] * h.sy + m2[8];
              ww = fabsf(ww) < 1e-5f ? 1e-5f : ww;
              q += (u / ww - px) * gflow.x + (v / ww - py) * gflow.y;
              const float gu = w / ww * gflow.x, gv = w / ww * gflow.y;
              const float gw = -w / (ww * ww) * (u * gflow.x + v * gflow.y);
              dL_dsx += m2[0] * gu + m2[3] * gv + m2[6] * gw;
              dL_dsy += m2[1] * gu + m2[4] * gv + m2[7] * gw;
            }
            acc_q = last_alpha * last_q + (1.0f - last_alpha) * acc_q;
            last_q = q;
            dL_dalpha += q - acc_q;
            dL_dalpha *= T;
            last_alpha = alpha;
            const float dL_dG = opa * dL_dalpha;
            if (h.rho3d <= h.rho2d) {
              dL_dsx += dL_dG * -G * h.sx + dL_dz * Tw.x;
              dL_dsy += dL_dG * -G * h.sy + dL_dz * Tw.y;
              const float inv_pz = __fdividef(1.0f, h.pz);
              const float ga = dL_dsx * inv_pz, gb = dL_dsy * inv_pz;
              const float gc = -(ga * h.sx + gb * h.sy);
              g[GM::kIm] = ga * px, g[GM::kIm + 1] = ga * py, g[GM::kIm + 2] = ga;
              g[GM::kIm + 3] = gb * px, g[GM::kIm + 4] = gb * py, g[GM::kIm + 5] = gb;
              g[GM::kIm + 6] = gc * px, g[GM::kIm + 7] = gc * py, g[GM::kIm + 8] = gc;
            } else {
              g[GM::kM2d] = dL_dG * (-G * 2.0f * h.dx);
              g[GM::kM2d + 1] = dL_dG * (-G * 2.0f * h.dy);
            }
            if (AUX) g[GM::kTw] = dL_dz * h.sx, g[GM::kTw + 1] = dL_dz * h.sy, g[GM::kTw + 2] = dL_dz;
            g[GM::kOpac] = G * dL_dalpha;
          }
          if (__ballot_sync(kFull, active) == 0) continue;
          int comp;
          const float total = warp_transpose_reduce<kGrad>(g, lane, comp);
          if (comp < kGrad && total != 0.0f) atomicAdd(s_grad + r * kGrad + comp, total);
        }
      }
    }
    if (has2) s_gids[((k + 2) & 3) * kStage + tid] = id2;  // read after the next barrier
  }
  __syncthreads();
  flush(n_stages - 1);
}

static size_t bwd_smem_bytes(bool aux, bool flow) {
  const int n = aux ? GradMap<true>::N : GradMap<false>::N;
  return sizeof(float4) * 2 * kStage * kQ + sizeof(float) * 2 * kStage * n + sizeof(int) * 4 * kStage +
         (flow ? sizeof(float) * 2 * kStage * 9 : 0);
}

}  // namespace fsgs

using namespace fsgs;

extern "C" int fsgs_render_forward(const fsgs_render_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(a && a->P >= 0 && a->W > 0 && a->H > 0);
  FSGS_REQUIRE(a->ranges && a->out_color && a->out_opacity && a->n_contrib);
  FSGS_REQUIRE(a->P == 0 || (a->records && a->point_list));
  FSGS_REQUIRE(a->only_image || a->out_extras);
  FSGS_REQUIRE(!a->trans_mat_t2 || a->only_image || a->out_flow);
  FwdDev d;
  d.P = a->P, d.W = a->W, d.H = a->H, d.gx = (a->W + kTile - 1) / kTile;
  d.near_n = a->near_n, d.far_n = a->far_n;
  d.records = (const float4 *) a->records, d.point_list = a->point_list, d.ranges = (const long long *) a->ranges;
  d.tile_order = a->tile_order, d.m2 = a->trans_mat_t2;
  d.out_color = a->out_color, d.out_opacity = a->out_opacity, d.out_extras = a->out_extras;
  d.out_flow = (float2 *) a->out_flow, d.n_contrib = a->n_contrib;
  d.accum_max_count = a->accum_max_count, d.accum_weights_p = a->accum_weights_p;
  d.accum_weights_count = a->accum_weights_count;
  d.counters = (const long long *) a->counters;
  const int T = d.gx * ((a->H + kTile - 1) / kTile);
  cudaStream_t st = (cudaStream_t) stream;
  if (a->only_image) blend_forward_kernel<false, false><<<T, 256, 0, st>>>(d);
  else if (a->trans_mat_t2) blend_forward_kernel<true, true><<<T, 256, 0, st>>>(d);
  else blend_forward_kernel<true, false><<<T, 256, 0, st>>>(d);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_render_pair_counts(const fsgs_render_args *a, int64_t *counts, fsgs_stream_t stream) {
  FSGS_REQUIRE(a && counts && a->P >= 0 && a->W > 0 && a->H > 0 && a->ranges);
  FSGS_REQUIRE(a->P == 0 || (a->records && a->point_list));
  cudaStream_t st = (cudaStream_t) stream;
  cudaMemsetAsync(counts, 0, sizeof(int64_t) * 3, st);
  FwdDev d = {};
  d.P = a->P, d.W = a->W, d.H = a->H, d.gx = (a->W + kTile - 1) / kTile;
  d.near_n = a->near_n, d.far_n = a->far_n;
  d.records = (const float4 *) a->records, d.point_list = a->point_list, d.ranges = (const long long *) a->ranges;
  const int T = d.gx * ((a->H + kTile - 1) / kTile);
  pair_count_kernel<<<T, 256, 0, st>>>(d, (unsigned long long *) counts);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_render_backward(const fsgs_render_bwd_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(a && a->P >= 0 && a->W > 0 && a->H > 0);
  FSGS_REQUIRE(a->ranges && a->out_opacity && a->n_contrib && a->dL_dcolor);
  FSGS_REQUIRE(a->dL_dcolors && a->dL_dmeans2D && a->dL_dtrans_mat && a->dL_dinverse_m && a->dL_dnormal_opacity);
  const bool aux = a->out_extras && a->dL_dextras;
  FSGS_REQUIRE(!aux || a->dL_dopacity);
  const bool flow = aux && a->dL_dflow && a->trans_mat_t2;
  cudaStream_t st = (cudaStream_t) stream;
  const size_t P = (size_t) a->P;
  cudaMemsetAsync(a->dL_dcolors, 0, sizeof(float) * 3 * P, st);
  cudaMemsetAsync(a->dL_dmeans2D, 0, sizeof(float) * 2 * P, st);
  cudaMemsetAsync(a->dL_dtrans_mat, 0, sizeof(float) * 9 * P, st);
  cudaMemsetAsync(a->dL_dinverse_m, 0, sizeof(float) * 9 * P, st);
  cudaMemsetAsync(a->dL_dnormal_opacity, 0, sizeof(float) * 4 * P, st);
  if (a->P == 0) return FSGS_OK;
  FSGS_REQUIRE(a->records && a->point_list);
  BwdDev d;
  d.P = a->P, d.W = a->W, d.H = a->H, d.gx = (a->W + kTile - 1) / kTile;
  d.near_n = a->near_n, d.far_n = a->far_n;
  d.records = (const float4 *) a->records, d.point_list = a->point_list, d.ranges = (const long long *) a->ranges;
  d.tile_order = a->tile_order, d.m2 = a->trans_mat_t2;
  d.out_opacity = a->out_opacity, d.out_extras = a->out_extras, d.n_contrib = a->n_contrib;
  d.g_color = a->dL_dcolor, d.g_opacity = a->dL_dopacity, d.g_extras = a->dL_dextras;
  d.g_flow = (const float2 *) a->dL_dflow;
  d.g_colors = a->dL_dcolors, d.g_means2D = a->dL_dmeans2D, d.g_trans_mat = a->dL_dtrans_mat;
  d.g_inverse_m = a->dL_dinverse_m, d.g_normal_opacity = a->dL_dnormal_opacity;
  const int T = d.gx * ((a->H + kTile - 1) / kTile);
  const size_t smem_color = bwd_smem_bytes(false, false), smem = bwd_smem_bytes(true, false);
  const size_t smem_flow = bwd_smem_bytes(true, true);
  static bool configured_dev[64] = {};  // the opt-in above 48 KB is a per-function, per-device attribute: set once
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FSGS_ERR_LAUNCH;
  bool &configured = configured_dev[dev];
  if (!configured) {
    if (cudaFuncSetAttribute(blend_backward_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_color) != cudaSuccess ||
        cudaFuncSetAttribute(blend_backward_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess ||
        cudaFuncSetAttribute(blend_backward_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_flow) != cudaSuccess)
      return FSGS_ERR_LAUNCH;
    configured = true;
  }
  if (!aux) blend_backward_kernel<false, false><<<T, 256, smem_color, st>>>(d);
  else if (flow) blend_backward_kernel<true, true><<<T, 256, smem_flow, st>>>(d);
  else blend_backward_kernel<true, false><<<T, 256, smem, st>>>(d);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}
