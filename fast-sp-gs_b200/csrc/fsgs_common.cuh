// Shared device helpers of libfsgs: launch checks, the splat->screen matrix, the render-record layout.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fsgs.h"

#define FSGS_LAUNCH_CHECK()                                  \
  do {                                                       \
    if (cudaGetLastError() != cudaSuccess) return FSGS_ERR_LAUNCH; \
  } while (0)

#define FSGS_REQUIRE(cond) \
  do {                     \
    if (!(cond)) return FSGS_ERR_INVALID_ARGUMENT; \
  } while (0)

namespace fsgs {

constexpr int kTile = FSGS_TILE;
constexpr int kTilePix = kTile * kTile;
constexpr int kRecFloats = FSGS_RECORD_FLOATS;

static inline int ceil_div(int64_t a, int64_t b) { return (int) ((a + b - 1) / b); }

// Render record, 8 float4 per Gaussian (128 B, one cache line):
//  q0: mean2D.x, mean2D.y, opacity, tau' (the padded bound on rho inside which alpha can reach 1/255; 0: never)
//  q1: A.x A.y A.z B.x        rows A, B, C of inverse_m (the adjugate of the splat->screen matrix)
//  q2: B.y B.z C.x C.y
//  q3: C.z Tw.x Tw.y Tw.z     Tw = row 2 of the splat->screen matrix (depth row)
//  q4: xmin xmax ymin ymax    pixel box outside which alpha < 1/255 for certain
//  q5: r g b normal.x
//  q6: normal.y normal.z - -
//  q7: unused
constexpr int kRecQuadsUsed = 7;

struct Mat3 {
  float m[9];
};

// Tile rectangle [x0,x1) x [y0,y1) of a splat: centre +- integer radius, truncated toward zero, clamped.
// (reference include/gaussian_render.h:33-40)
__device__ __forceinline__ void tile_rect(float px, float py, int radius, int gx, int gy, int &x0, int &y0, int &x1,
    int &y1) {
  x0 = min(gx, max(0, (int) ((px - radius) / kTile)));
  y0 = min(gy, max(0, (int) ((py - radius) / kTile)));
  x1 = min(gx, max(0, (int) ((px + radius + kTile - 1) / kTile)));
  y1 = min(gy, max(0, (int) ((py + radius + kTile - 1) / kTile)));
}

// ---- pinned fp32 arithmetic -------------------------------------------------------------------------------
// The binning's corner test flips on the last bit of its inputs, and tile lists have to equal the reference's
// bit for bit.  nvcc decides per kernel which multiply feeds which fused multiply-add, so equal source does not
// give equal bits.  Every operation below that reaches the corner test is therefore written with explicit
// round-to-nearest intrinsics, in the association that reproduces the reference build (-O3, default -fmad,
// sm_100) bit for bit; the sequence was established by comparing against the reference kernels' outputs.
#define FMUL(a, b) __fmul_rn((a), (b))
#define FADD(a, b) __fadd_rn((a), (b))
#define FSUB(a, b) __fsub_rn((a), (b))
#define FFMA(a, b, c) __fmaf_rn((a), (b), (c))

// a0*b0 + a1*b1 + a2*b2 accumulated from zero in index order: fma(a2,b2, fma(a1,b1, a0*b0))
__device__ __forceinline__ float dot3_chain(float a0, float b0, float a1, float b1, float a2, float b2) {
  return FFMA(a2, b2, FFMA(a1, b1, FMUL(a0, b0)));
}
// the same sum written as one expression: fma(a2,b2, fma(a0,b0, a1*b1))
__device__ __forceinline__ float dot3_expr(float a0, float b0, float a1, float b1, float a2, float b2) {
  return FFMA(a2, b2, FFMA(a0, b0, FMUL(a1, b1)));
}

// View-space position; the products are shared with the third column of the splat matrix, so nothing is fused.
__device__ __forceinline__ float3 view_point(const float3 p, const float *__restrict__ Tw2v) {
  float3 v;
  v.x = FADD(FADD(FADD(FMUL(Tw2v[0], p.x), FMUL(Tw2v[1], p.y)), FMUL(Tw2v[2], p.z)), Tw2v[3]);
  v.y = FADD(FADD(FADD(FMUL(Tw2v[4], p.x), FMUL(Tw2v[5], p.y)), FMUL(Tw2v[6], p.z)), Tw2v[7]);
  v.z = FADD(FADD(FADD(FMUL(Tw2v[8], p.x), FMUL(Tw2v[9], p.y)), FMUL(Tw2v[10], p.z)), Tw2v[11]);
  return v;
}

// Splat -> screen matrix M = Tv2s * (Tw2v[:3,:3] * [R(q)*diag(s) | p] + e_z * Tw2v[2,3]) and the view-space
// normal.  Only the z translation of the camera enters M (reference gs_2d_fast_preprocess.cu:60-98).
__device__ __forceinline__ void splat_matrix(const float3 p, const float2 s, const float4 q, const float *__restrict__ Tw2v,
    const float *__restrict__ Tv2s, float *M, float3 &normal) {
  float L[9];
  float3 n;
  const float xx = FMUL(q.x, q.x), yy = FMUL(q.y, q.y), zz = FMUL(q.z, q.z);
  const float xz = FMUL(q.x, q.z), zw = FMUL(q.z, q.w), xw = FMUL(q.x, q.w);
  L[0] = FMUL(FSUB(1.0f, FMUL(2.0f, FADD(yy, zz))), s.x);
  L[1] = FMUL(FMUL(2.0f, FFMA(q.x, q.y, -zw)), s.y);
  L[2] = p.x;
  n.x = FMUL(2.0f, FFMA(q.y, q.w, xz));

  L[3] = FMUL(FMUL(2.0f, FFMA(q.x, q.y, zw)), s.x);
  L[4] = FMUL(FSUB(1.0f, FMUL(2.0f, FFMA(q.x, q.x, zz))), s.y);
  L[5] = p.y;
  n.y = FMUL(2.0f, FFMA(q.y, q.z, -xw));

  L[6] = FMUL(FMUL(2.0f, FFMA(-q.y, q.w, xz)), s.x);
  L[7] = FMUL(FMUL(2.0f, FFMA(q.y, q.z, xw)), s.y);
  L[8] = p.z;
  n.z = FSUB(1.0f, FMUL(2.0f, FFMA(q.x, q.x, yy)));

  float t[9];
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    t[i * 3 + 0] = dot3_chain(Tw2v[i * 4], L[0], Tw2v[i * 4 + 1], L[3], Tw2v[i * 4 + 2], L[6]);
    t[i * 3 + 1] = dot3_chain(Tw2v[i * 4], L[1], Tw2v[i * 4 + 1], L[4], Tw2v[i * 4 + 2], L[7]);
    t[i * 3 + 2] = FADD(FADD(FMUL(Tw2v[i * 4], L[2]), FMUL(Tw2v[i * 4 + 1], L[5])), FMUL(Tw2v[i * 4 + 2], L[8]));
  }
  t[8] = FADD(t[8], Tw2v[11]);
#pragma unroll
  for (int i = 0; i < 3; ++i) {
#pragma unroll
    for (int j = 0; j < 3; ++j)
      M[i * 3 + j] = dot3_chain(Tv2s[i * 3], t[j], Tv2s[i * 3 + 1], t[3 + j], Tv2s[i * 3 + 2], t[6 + j]);
  }
  normal.x = dot3_expr(Tw2v[0], n.x, Tw2v[1], n.y, Tw2v[2], n.z);
  normal.y = dot3_expr(Tw2v[4], n.x, Tw2v[5], n.y, Tw2v[6], n.z);
  normal.z = dot3_expr(Tw2v[8], n.x, Tw2v[9], n.y, Tw2v[10], n.z);
}

// Adjugate of M, rows = cross products of M's columns (reference gs_2d_fast_preprocess.cu:247-255).
__device__ __forceinline__ void adjugate(const float *m, float *im) {
  im[0] = FFMA(m[4], m[8], -FMUL(m[7], m[5]));
  im[1] = FFMA(m[7], m[2], -FMUL(m[1], m[8]));
  im[2] = FFMA(m[1], m[5], -FMUL(m[4], m[2]));
  im[3] = FFMA(m[6], m[5], -FMUL(m[3], m[8]));
  im[4] = FFMA(m[0], m[8], -FMUL(m[6], m[2]));
  im[5] = FFMA(m[3], m[2], -FMUL(m[0], m[5]));
  im[6] = FFMA(m[3], m[7], -FMUL(m[6], m[4]));
  im[7] = FFMA(m[6], m[1], -FMUL(m[0], m[7]));
  im[8] = FFMA(m[0], m[4], -FMUL(m[3], m[1]));
}

// 3-sigma bounding box of the projected splat: centre and ceil'd radius.  false when degenerate.
// (reference gs_2d_fast_preprocess.cu:143-158, 227)
__device__ __forceinline__ bool splat_bounds(const float *M, float2 &ctr, float &radius) {
  const float d = FFMA(-M[8], M[8], FFMA(9.0f, FMUL(M[6], M[6]), FMUL(9.0f, FMUL(M[7], M[7]))));
  if (d == 0.0f) return false;
  const float inv_d = __fdiv_rn(1.0f, d);
  const float f0 = FMUL(inv_d, 9.0f), f2 = -inv_d;
  ctr.x = dot3_expr(f0, FMUL(M[0], M[6]), f0, FMUL(M[1], M[7]), f2, FMUL(M[2], M[8]));
  ctr.y = dot3_expr(f0, FMUL(M[3], M[6]), f0, FMUL(M[4], M[7]), f2, FMUL(M[5], M[8]));
  const float hx = FFMA(ctr.x, ctr.x, -dot3_expr(f0, FMUL(M[0], M[0]), f0, FMUL(M[1], M[1]), f2, FMUL(M[2], M[2])));
  const float hy = FFMA(ctr.y, ctr.y, -dot3_expr(f0, FMUL(M[3], M[3]), f0, FMUL(M[4], M[4]), f2, FMUL(M[5], M[5])));
  const float ex = __fsqrt_rn(fmaxf(1e-4f, hx)), ey = __fsqrt_rn(fmaxf(1e-4f, hy));
  radius = ceilf(fmaxf(fmaxf(ex, ey), 3.0f * float(0.707106)));
  return true;
}

__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm volatile("lg2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The six coefficients (tile units) of the conic  alpha >= 1/255  of a splat
// (reference gs_2d_fast_preprocess.cu:282-300) and the corner test (:301).
//
// The test cancels terms of about 1e10 down to a few rounding steps for a splat that grazes a tile corner, so which
// products are fused into the following addition decides membership.  The reference build evaluates
//   ((((xx*u*u + yy*v*v) + xy*u*v) + x_*u) + y_*v) + __ <= 0
// with only the cross term fused -- except in the first row of a tile rectangle with an odd number of rows (the
// iteration its compiler peels off the two-row loop over y), where the y_*v term is fused as well.  Both forms were
// established against the reference kernels' lists: with them every list is identical on all scenes compared.
struct Conic {
  float xx, yy, xy, x_, y_, __;
  __device__ __forceinline__ bool inside(float u, float v, bool fuse_y) const {
    float s = FADD(FMUL(FMUL(xx, u), u), FMUL(FMUL(yy, v), v));
    s = FFMA(FMUL(xy, u), v, s);
    s = FADD(s, FMUL(x_, u));
    s = fuse_y ? FFMA(y_, v, s) : FADD(s, FMUL(y_, v));
    return FADD(s, __) <= 0;
  }
  // tile (tx, ty) of a rectangle whose first row is y0 and which has `rows` rows: any of its four corners inside
  __device__ __forceinline__ bool covers(int tx, int ty, int y0, int rows) const {
    const bool fuse_y = (rows & 1) && ty == y0;
    const float u0 = (float) tx, u1 = (float) (tx + 1), v0 = (float) ty, v1 = (float) (ty + 1);
    return inside(u0, v0, fuse_y) || inside(u1, v0, fuse_y) || inside(u0, v1, fuse_y) || inside(u1, v1, fuse_y);
  }
};

__device__ __forceinline__ Conic make_conic(const float *IM, float opacity) {
  const float ln2 = 0.69314718055f;
  const float d = FMUL(-2.0f * ln2, FADD(float(7.9886846867721655), lg2_approx(opacity)));
  const float d6 = FMUL(d, IM[6]), d7 = FMUL(d, IM[7]), d8 = FMUL(d, IM[8]);
  Conic c;
  const float Wxx = dot3_expr(IM[0], IM[0], IM[3], IM[3], d6, IM[6]);
  const float Wyy = dot3_expr(IM[1], IM[1], IM[4], IM[4], d7, IM[7]);
  const float W__ = dot3_expr(IM[2], IM[2], IM[5], IM[5], d8, IM[8]);
  const float Wxy = FMUL(2.0f, dot3_expr(IM[0], IM[1], IM[3], IM[4], d6, IM[7]));
  const float Wx_ = FMUL(2.0f, dot3_expr(IM[0], IM[2], IM[3], IM[5], d6, IM[8]));
  const float Wy_ = FMUL(2.0f, dot3_expr(IM[1], IM[2], IM[4], IM[5], d7, IM[8]));
  c.xx = Wxx * (kTile * kTile);
  c.yy = Wyy * (kTile * kTile);
  c.xy = Wxy * (kTile * kTile);
  c.x_ = Wx_ * kTile;
  c.y_ = Wy_ * kTile;
  c.__ = W__;
  return c;
}

// Calls f for every tile of a splat's rectangle with at least one corner inside its conic (reference
// gs_2d_fast_preprocess.cu:301-318), for the 32 splats held by the lanes of a warp, with the work spread evenly: the
// tiles of all 32 rectangles are numbered consecutively (prefix sum of the areas) and handed out 32 per round, so that every lane
// tests one tile per round whatever the shapes of the individual rectangles (one thread walking its own rectangle
// leaves three quarters of the warp idle: rectangle areas range from 1 to over 100).  Lane L passes its conic and
// rectangle (`has` false: none) and two payload words; f(tile_x, tile_y, payload0, payload1) runs on the lane that
// tested the tile, with the payload of the splat the tile belongs to.  Must be called by all 32 lanes.
template <typename F>
__device__ __forceinline__ void warp_for_each_covered_tile(const Conic &c, int x0, int y0, int x1, int y1, bool has,
    unsigned p0, unsigned p1, F f) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const int w = has ? x1 - x0 : 0, h = has ? y1 - y0 : 0;
  const int area = w * h;
  int incl = area;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(full, incl, o);
    if (lane >= o) incl += n;
  }
  const int excl = incl - area;
  const int total = __shfl_sync(full, incl, 31);
  for (int base = 0; base < total; base += 32) {
    const bool valid = base + lane < total;
    const int item = valid ? base + lane : total - 1;
    int s = 0;  // first lane whose inclusive prefix exceeds item
#pragma unroll
    for (int step = 16; step > 0; step >>= 1) {
      const int v = __shfl_sync(full, incl, s + step - 1);
      if (v <= item) s += step;
    }
    const int local = item - __shfl_sync(full, excl, s);
    const int swh = __shfl_sync(full, w | (h << 16), s);
    const int sw = swh & 0xffff, sh = swh >> 16;
    const int sx0 = __shfl_sync(full, x0, s), sy0 = __shfl_sync(full, y0, s);
    Conic cs;
    cs.xx = __shfl_sync(full, c.xx, s), cs.yy = __shfl_sync(full, c.yy, s), cs.xy = __shfl_sync(full, c.xy, s);
    cs.x_ = __shfl_sync(full, c.x_, s), cs.y_ = __shfl_sync(full, c.y_, s), cs.__ = __shfl_sync(full, c.__, s);
    const unsigned q0 = __shfl_sync(full, p0, s), q1 = __shfl_sync(full, p1, s);
    const int ly = local / sw, lx = local - ly * sw;
    const int tx = sx0 + lx, ty = sy0 + ly;
    const bool covered = valid && cs.covers(tx, ty, sy0, sh);
    if (covered) f(tx, ty, q0, q1);
  }
}

// Conservative pixel box of {alpha >= 1/255} for one splat: the projected disc u^2+v^2 <= tau plus the
// low-pass disc around the 3-sigma box centre, padded against rounding.  An empty box (xmin > xmax)
// means the splat can never pass the alpha cut; an infinite box means "cannot bound" (the disc crosses
// the camera plane).  M is the splat->screen matrix, ctr the low-pass centre (means2D).
__device__ __forceinline__ float4 alpha_box(const float *M, float2 ctr, float opacity, float &tau_padded) {
  const float inf = __int_as_float(0x7f800000);
  tau_padded = 0.0f;
  float tau = 2.0f * __logf(255.0f * opacity);  // alpha >= 1/255  <=>  rho <= tau
  if (!(opacity > 0.0f) || !(tau == tau)) return make_float4(1.0f, -1.0f, 1.0f, -1.0f);
  tau = tau * 1.002f + 0.02f;
  if (tau <= 0.0f) return make_float4(1.0f, -1.0f, 1.0f, -1.0f);
  tau_padded = tau;
  const float r2d = sqrtf(0.5f * tau) + 0.5f;
  float4 box = make_float4(ctr.x - r2d, ctr.x + r2d, ctr.y - r2d, ctr.y + r2d);
  const float d = tau * (M[6] * M[6] + M[7] * M[7]) - M[8] * M[8];
  if (!(d < -1e-6f * M[8] * M[8])) return make_float4(-inf, inf, -inf, inf);
  const float fx = tau / d, fz = -1.0f / d;
  const float cx = fx * (M[0] * M[6] + M[1] * M[7]) + fz * (M[2] * M[8]);
  const float cy = fx * (M[3] * M[6] + M[4] * M[7]) + fz * (M[5] * M[8]);
  const float hx2 = cx * cx - (fx * (M[0] * M[0] + M[1] * M[1]) + fz * (M[2] * M[2]));
  const float hy2 = cy * cy - (fx * (M[3] * M[3] + M[4] * M[4]) + fz * (M[5] * M[5]));
  const float hx = sqrtf(fmaxf(hx2, 0.0f)) * 1.01f + 0.5f + 1e-4f * fabsf(cx);
  const float hy = sqrtf(fmaxf(hy2, 0.0f)) * 1.01f + 0.5f + 1e-4f * fabsf(cy);
  if (!(hx == hx) || !(hy == hy)) return make_float4(-inf, inf, -inf, inf);
  box.x = fminf(box.x, cx - hx);
  box.y = fmaxf(box.y, cx + hx);
  box.z = fminf(box.z, cy - hy);
  box.w = fmaxf(box.w, cy + hy);
  return box;
}

__device__ __forceinline__ void write_record(float4 *rec, float2 xy, float opacity, const float *im, const float *M,
    float4 box, float tau_padded, float3 rgb, float3 nrm) {
  rec[0] = make_float4(xy.x, xy.y, opacity, tau_padded);
  rec[1] = make_float4(im[0], im[1], im[2], im[3]);
  rec[2] = make_float4(im[4], im[5], im[6], im[7]);
  rec[3] = make_float4(im[8], M[6], M[7], M[8]);
  rec[4] = box;
  rec[5] = make_float4(rgb.x, rgb.y, rgb.z, nrm.x);
  rec[6] = make_float4(nrm.y, nrm.z, 0.0f, 0.0f);
}

}  // namespace fsgs
