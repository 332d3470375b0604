/*
 * fsgs_oracle.c -- CPU restatement of the Fast-SP-GS surfel-rendering hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: it is
 * linked by the test-suite, by the smoke test and by the CPU-baseline leg of the
 * benchmark, never by the product path.
 *
 * Every function restates, in plain scalar C (fp32, no FMA contraction:
 * build with -ffp-contract=off), the algorithm of the reference file/lines named
 * in its header comment.  Paths are relative to the reference project root.
 *
 * Pinning: checked against golden vectors produced by the reference's own
 * PyTorch twins (tests/golden/make_golden.py) and, on a GPU box, against the
 * reference CUDA kernels built by oracle/build_ref.py.
 *
 * Known, deliberate deviations from the reference CUDA arithmetic:
 *   - lg2.approx.f32 is replaced by log2f (CPU has no such instruction);
 *   - nvcc contracts a*b+c into FMA; this file does not, except where a result is an index or a list membership
 *     that a rounding step can flip (the conic corner test of the binning, cdist_top): there the fused operations of
 *     the reference's CUDA build are written out with fmaf.
 * The first only matters for conic corner tests that land within a few ulp of zero.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define TILE 16
/* accumulation shared between threads that work on different tiles */
#define ATOMIC_ADD(dst, val)        \
  do {                              \
    const float v_ = (val);         \
    _Pragma("omp atomic")(dst) += v_; \
  } while (0)
#define TILE_PIX 256

/* ------------------------------------------------------------------------- */
/* small helpers                                                             */
/* ------------------------------------------------------------------------- */

static inline int imin(int a, int b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Threads the parallel loops below use from now on (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void) n;
#endif
}

/* Tile rectangle of a splat.  fast_2d_gs/_C/include/gaussian_render.h:33-40
 * (C truncation toward zero, then clamp to the grid). */
static void tile_rect(float px, float py, int radius, int gx, int gy, int *x0, int *y0, int *x1, int *y1) {
  *x0 = imin(gx, imax(0, (int) ((px - radius) / TILE)));
  *y0 = imin(gy, imax(0, (int) ((py - radius) / TILE)));
  *x1 = imin(gx, imax(0, (int) ((px + radius + TILE - 1) / TILE)));
  *y1 = imin(gy, imax(0, (int) ((py + radius + TILE - 1) / TILE)));
}

/* Unit quaternion (x,y,z,w) -> rotation matrix, row major.
 * fast_2d_gs/_C/src/gaussian_splatting/gs_2d_fast_preprocess.cu:67-80 */
static void quat_to_rot(const float *q, float *R) {
  const float x = q[0], y = q[1], z = q[2], w = q[3];
  R[0] = 1 - 2 * (y * y + z * z);
  R[1] = 2 * (x * y - z * w);
  R[2] = 2 * (y * w + x * z);
  R[3] = 2 * (x * y + z * w);
  R[4] = 1 - 2 * (x * x + z * z);
  R[5] = 2 * (y * z - x * w);
  R[6] = 2 * (x * z - y * w);
  R[7] = 2 * (x * w + y * z);
  R[8] = 1 - 2 * (x * x + y * y);
}

/* Splat -> screen matrix M (3x3) and view-space normal.
 * gs_2d_fast_preprocess.cu:60-98.  Only the z translation of Tw2v enters M. */
static void splat_matrix(const float *p, const float *s, const float *q, const float *Tw2v, const float *Tv2s,
    float *M, float *normal) {
  float R[9], L[9], t[9];
  quat_to_rot(q, R);
  for (int r = 0; r < 3; ++r) {
    L[r * 3 + 0] = R[r * 3 + 0] * s[0];
    L[r * 3 + 1] = R[r * 3 + 1] * s[1];
    L[r * 3 + 2] = p[r];
  }
  for (int i = 0; i < 3; ++i)
    for (int j = 0; j < 3; ++j) {
      float acc = 0;
      for (int k = 0; k < 3; ++k) acc += Tw2v[i * 4 + k] * L[k * 3 + j];
      t[i * 3 + j] = acc;
    }
  t[8] += Tw2v[11];
  for (int i = 0; i < 3; ++i)
    for (int j = 0; j < 3; ++j) {
      float acc = 0;
      for (int k = 0; k < 3; ++k) acc += Tv2s[i * 3 + k] * t[k * 3 + j];
      M[i * 3 + j] = acc;
    }
  const float n[3] = {R[2], R[5], R[8]};
  for (int i = 0; i < 3; ++i) normal[i] = Tw2v[i * 4 + 0] * n[0] + Tw2v[i * 4 + 1] * n[1] + Tw2v[i * 4 + 2] * n[2];
}

void orc_transmat(int P, const float *means, const float *scales, const float *quats, const float *Tw2v,
    const float *Tv2s, float *M, float *normals) {
  for (int i = 0; i < P; ++i) splat_matrix(means + 3 * i, scales + 2 * i, quats + 4 * i, Tw2v, Tv2s, M + 9 * i, normals + 3 * i);
}

/* ------------------------------------------------------------------------- */
/* spherical harmonics, degree <= 3                                          */
/* fast_2d_gs/_C/include/spherical_harmonic.h:18-202 (forward), 204-677 (bwd) */
/* ------------------------------------------------------------------------- */

#define SH_C0 0.28209479177387814f
#define SH_C1 0.48860251190291987f
#define SH_C2A 1.0925484305920792f
#define SH_C2B 0.94617469575755997f
#define SH_C2C 0.31539156525251999f
#define SH_C2D 0.54627421529603959f
#define SH_C3A 0.59004358992664352f
#define SH_C3B 2.8906114426405538f
#define SH_C3C 0.45704579946446572f
#define SH_C3D 0.3731763325901154f
#define SH_C3E 1.4453057213202769f

/* Degrees 4..7 by the general definition the reference states (utils/ops_3d/spherical_harmonics.py:16-67; its CUDA
 * header tabulates the same functions as polynomials, include/spherical_harmonic.h:81-202): associated Legendre
 * functions by the upward recurrence, Condon-Shortley phase included, in double precision. */
#define SH_MAX 64

static double sh_legendre(int l, int m, double x) {
  double pmm = 1.0;
  if (m > 0) {
    const double somx2 = sqrt((1.0 - x) * (1.0 + x));
    double fact = 1.0;
    for (int i = 1; i <= m; ++i) {
      pmm *= -fact * somx2;
      fact += 2.0;
    }
  }
  if (l == m) return pmm;
  double pmmp1 = x * (2.0 * m + 1.0) * pmm;
  if (l == m + 1) return pmmp1;
  double pll = 0.0;
  for (int ll = m + 2; ll <= l; ++ll) {
    pll = ((2.0 * ll - 1.0) * x * pmmp1 - (ll + m - 1.0) * pmm) / (ll - m);
    pmm = pmmp1;
    pmmp1 = pll;
  }
  return pll;
}

static double sh_norm(int l, int m) {
  double f = 1.0; /* (l-m)! / (l+m)! */
  for (int i = l - m + 1; i <= l + m; ++i) f /= (double) i;
  return sqrt((2.0 * l + 1.0) * f / (4.0 * 3.14159265358979323846));
}

/* Y_l^m at the unit vector (x, y, z) */
static double sh_general(int l, int m, double x, double y, double z) {
  const double phi = atan2(y, x);
  const double ct = z > 1.0 ? 1.0 : (z < -1.0 ? -1.0 : z);
  if (m == 0) return sh_norm(l, 0) * sh_legendre(l, 0, ct);
  if (m > 0) return 1.4142135623730951 * sh_norm(l, m) * sh_legendre(l, m, ct) * cos(m * phi);
  return 1.4142135623730951 * sh_norm(l, -m) * sh_legendre(l, -m, ct) * sin(-m * phi);
}

/* sum over the coefficients of degrees 4..deg of t[k] * Y_k(normalize(p)), for the adjoint by differences */
static double sh_high_sum(int deg, const float *t, double px, double py, double pz) {
  const double n = 1.0 / sqrt(px * px + py * py + pz * pz + 1e-12);
  double acc = 0.0;
  for (int l = 4; l <= deg; ++l)
    for (int m = -l; m <= l; ++m) acc += (double) t[l * l + l + m] * sh_general(l, m, px * n, py * n, pz * n);
  return acc;
}

static void sh_basis(int deg, float x, float y, float z, float *b) {
  const float x2 = x * x, y2 = y * y, z2 = z * z;
  b[0] = SH_C0;
  if (deg > 0) {
    b[1] = -SH_C1 * y;
    b[2] = SH_C1 * z;
    b[3] = -SH_C1 * x;
  }
  if (deg > 1) {
    b[4] = SH_C2A * (x * y);
    b[5] = -SH_C2A * (y * z);
    b[6] = SH_C2B * z2 - SH_C2C;
    b[7] = -SH_C2A * (x * z);
    b[8] = SH_C2D * x2 - SH_C2D * y2;
  }
  if (deg > 2) {
    b[9] = SH_C3A * y * (-3.0f * x2 + y2);
    b[10] = SH_C3B * (x * y) * z;
    b[11] = SH_C3C * y * (1.0f - 5.0f * z2);
    b[12] = SH_C3D * z * (5.0f * z2 - 3.0f);
    b[13] = SH_C3C * x * (1.0f - 5.0f * z2);
    b[14] = SH_C3E * z * (x2 - y2);
    b[15] = SH_C3A * x * (-x2 + 3.0f * y2);
  }
  for (int l = 4; l <= deg; ++l)
    for (int m = -l; m <= l; ++m) b[l * l + l + m] = (float) sh_general(l, m, x, y, z);
}

void orc_sh_basis(int n, int deg, const float *dirs, float *out /* [n, (deg+1)^2] */) {
  const int nb = (deg + 1) * (deg + 1);
  for (int i = 0; i < n; ++i) {
    float b[SH_MAX];
    sh_basis(deg, dirs[3 * i], dirs[3 * i + 1], dirs[3 * i + 2], b);
    for (int k = 0; k < nb; ++k) out[(size_t) i * nb + k] = b[k];
  }
}

/* d basis / d (x,y,z) treating the polynomials above as functions of three free variables */
static void sh_basis_grad(int deg, float x, float y, float z, float *dx, float *dy, float *dz) {
  const float x2 = x * x, y2 = y * y, z2 = z * z;
  for (int k = 0; k < 16; ++k) dx[k] = dy[k] = dz[k] = 0;
  if (deg > 0) {
    dy[1] = -SH_C1;
    dz[2] = SH_C1;
    dx[3] = -SH_C1;
  }
  if (deg > 1) {
    dx[4] = SH_C2A * y, dy[4] = SH_C2A * x;
    dy[5] = -SH_C2A * z, dz[5] = -SH_C2A * y;
    dz[6] = 2.0f * SH_C2B * z;
    dx[7] = -SH_C2A * z, dz[7] = -SH_C2A * x;
    dx[8] = 2.0f * SH_C2D * x, dy[8] = -2.0f * SH_C2D * y;
  }
  if (deg > 2) {
    dx[9] = SH_C3A * (-6.0f * x * y), dy[9] = SH_C3A * (-3.0f * x2 + 3.0f * y2);
    dx[10] = SH_C3B * y * z, dy[10] = SH_C3B * x * z, dz[10] = SH_C3B * x * y;
    dy[11] = SH_C3C * (1.0f - 5.0f * z2), dz[11] = SH_C3C * (-10.0f * y * z);
    dz[12] = SH_C3D * (15.0f * z2 - 3.0f);
    dx[13] = SH_C3C * (1.0f - 5.0f * z2), dz[13] = SH_C3C * (-10.0f * x * z);
    dx[14] = SH_C3E * 2.0f * x * z, dy[14] = -SH_C3E * 2.0f * y * z, dz[14] = SH_C3E * (x2 - y2);
    dx[15] = SH_C3A * (-3.0f * x2 + 3.0f * y2), dy[15] = SH_C3A * 6.0f * x * y;
  }
}

/* coefficient k of Gaussian i: k==0 from sh_dc, k>=1 from sh_rest (or from sh_dc when it holds all) */
static inline const float *sh_coef(const float *sh_dc, const float *sh_rest, int n_dc, int n_rest, int i, int k) {
  if (sh_rest == NULL) return sh_dc + ((size_t) i * n_dc + k) * 3;
  return k == 0 ? sh_dc + (size_t) i * n_dc * 3 : sh_rest + ((size_t) i * n_rest + (k - 1)) * 3;
}

static void sh_to_rgb(int deg, const float *pos, const float *campos, const float *sh_dc, const float *sh_rest,
    int n_dc, int n_rest, int i, float *rgb) {
  float x = pos[0] - campos[0], y = pos[1] - campos[1], z = pos[2] - campos[2];
  const float n = 1.0f / sqrtf(x * x + y * y + z * z + 1e-12f);
  x *= n, y *= n, z *= n;
  float b[SH_MAX];
  sh_basis(deg, x, y, z, b);
  const int nb = (deg + 1) * (deg + 1);
  float r[3] = {0, 0, 0};
  for (int k = 0; k < nb; ++k) {
    const float *c = sh_coef(sh_dc, sh_rest, n_dc, n_rest, i, k);
    for (int ch = 0; ch < 3; ++ch) r[ch] += c[ch] * b[k];
  }
  for (int ch = 0; ch < 3; ++ch) {
    r[ch] += 0.5f;
    rgb[ch] = r[ch] > 0 ? r[ch] : 0;
  }
}

void orc_sh_to_rgb(int P, int deg, const float *pos, const float *campos, const float *sh_dc, const float *sh_rest,
    int n_dc, int n_rest, float *rgb) {
  for (int i = 0; i < P; ++i) sh_to_rgb(deg, pos + 3 * i, campos, sh_dc, sh_rest, n_dc, n_rest, i, rgb + 3 * i);
}

/* ------------------------------------------------------------------------- */
/* preprocess forward: gs_2d_fast_preprocess.cu:143-158 (AABB), 160-262       */
/* ------------------------------------------------------------------------- */

/* All outputs must be zero-initialised by the caller (the reference host does the same,
 * gs_2d_fast_preprocess.cu:664-671).  With sh_degree < 0, sh_dc holds [P,3] colours and
 * `colors` is left untouched (the reference aliases its input). */
void orc_preprocess_fwd(int P, int W, int H, int sh_degree, int n_dc, int n_rest, const float *means,
    const float *scales, const float *quats, const float *opac, const float *sh_dc, const float *sh_rest,
    const float *Tw2v, const float *Tv2s, const float *campos, const uint8_t *culling, float *means2D, float *colors,
    float *trans_mat, float *inverse_m, float *normal_opacity, float *depths, int32_t *radii, int32_t *tiles_touched) {
  const int gx = (W + TILE - 1) / TILE, gy = (H + TILE - 1) / TILE;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < P; ++i) {
    if (culling && culling[i]) continue;
    radii[i] = 0;
    tiles_touched[i] = 0;
    const float *p = means + 3 * i;
    const float vx = Tw2v[0] * p[0] + Tw2v[1] * p[1] + Tw2v[2] * p[2] + Tw2v[3];
    const float vy = Tw2v[4] * p[0] + Tw2v[5] * p[1] + Tw2v[6] * p[2] + Tw2v[7];
    const float vz = Tw2v[8] * p[0] + Tw2v[9] * p[1] + Tw2v[10] * p[2] + Tw2v[11];
    if (vz <= 0.2f) continue;
    float m[9], nrm[3];
    splat_matrix(p, scales + 2 * i, quats + 4 * i, Tw2v, Tv2s, m, nrm);
    const float c = -(vx * nrm[0] + vy * nrm[1] + vz * nrm[2]);
    if (c == 0) continue;
    const float sgn = c > 0 ? 1.0f : -1.0f;
    for (int k = 0; k < 3; ++k) nrm[k] = sgn * nrm[k];

    /* bounding box at cutoff 3 (gs_2d_fast_preprocess.cu:143-158) */
    const float tv[3] = {9.0f, 9.0f, -1.0f};
    const float d = tv[0] * (m[6] * m[6]) + tv[1] * (m[7] * m[7]) + tv[2] * (m[8] * m[8]);
    if (d == 0.0f) continue;
    const float inv_d = 1 / d;
    const float f[3] = {inv_d * tv[0], inv_d * tv[1], inv_d * tv[2]};
    const float cx = f[0] * (m[0] * m[6]) + f[1] * (m[1] * m[7]) + f[2] * (m[2] * m[8]);
    const float cy = f[0] * (m[3] * m[6]) + f[1] * (m[4] * m[7]) + f[2] * (m[5] * m[8]);
    const float hx = cx * cx - (f[0] * (m[0] * m[0]) + f[1] * (m[1] * m[1]) + f[2] * (m[2] * m[2]));
    const float hy = cy * cy - (f[0] * (m[3] * m[3]) + f[1] * (m[4] * m[4]) + f[2] * (m[5] * m[5]));
    const float ex = sqrtf(fmaxf(1e-4f, hx)), ey = sqrtf(fmaxf(1e-4f, hy));
    const float radius = ceilf(fmaxf(fmaxf(ex, ey), 3.0f * (float) 0.707106));

    int x0, y0, x1, y1;
    tile_rect(cx, cy, (int) radius, gx, gy, &x0, &y0, &x1, &y1);
    if ((x1 - x0) * (y1 - y0) == 0) continue;

    if (sh_degree >= 0) sh_to_rgb(sh_degree, p, campos, sh_dc, sh_rest, n_dc, n_rest, i, colors + 3 * i);
    for (int k = 0; k < 9; ++k) trans_mat[9 * i + k] = m[k];
    float *im = inverse_m + 9 * i;
    /* adjugate of M: rows are cross products of M's columns (gs_2d_fast_preprocess.cu:247-255) */
    im[0] = m[4] * m[8] - m[7] * m[5];
    im[1] = m[7] * m[2] - m[1] * m[8];
    im[2] = m[1] * m[5] - m[4] * m[2];
    im[3] = m[6] * m[5] - m[3] * m[8];
    im[4] = m[0] * m[8] - m[6] * m[2];
    im[5] = m[3] * m[2] - m[0] * m[5];
    im[6] = m[3] * m[7] - m[6] * m[4];
    im[7] = m[6] * m[1] - m[0] * m[7];
    im[8] = m[0] * m[4] - m[3] * m[1];
    depths[i] = vz;
    radii[i] = (int) radius;
    means2D[2 * i] = cx, means2D[2 * i + 1] = cy;
    normal_opacity[4 * i + 0] = nrm[0];
    normal_opacity[4 * i + 1] = nrm[1];
    normal_opacity[4 * i + 2] = nrm[2];
    normal_opacity[4 * i + 3] = opac[i];
    tiles_touched[i] = (y1 - y0) * (x1 - x0);
  }
}

/* ------------------------------------------------------------------------- */
/* tile binning: gs_2d_fast_preprocess.cu:264-327 (keys), 757-765 (sort),     */
/* 484-514 (ranges); gaussian_prepare.cu:32-44 (bit count, irrelevant here    */
/* because a full 64-bit comparison sort gives the same order).               */
/* ------------------------------------------------------------------------- */

/* Six conic coefficients of the alpha >= 1/255 footprint, in tile units.
 * gs_2d_fast_preprocess.cu:282-300.  The corner test below cancels terms of about 1e10 down to a few rounding
 * steps for a splat that grazes a tile corner, so the fused multiply-adds of the reference's CUDA build (nvcc,
 * default -fmad) are restated with fmaf: each coefficient is fma(d*c, c', fma(a, a', b*b')). */
static inline float dot3_cuda(float a0, float b0, float a1, float b1, float a2, float b2) {
  return fmaf(a2, b2, fmaf(a0, b0, a1 * b1));
}

static void conic_coeffs(const float *im, float opacity, float *w6) {
  const float ln2 = 0.69314718055f;
  const float d = -2.0f * ln2 * (7.9886846867721655f + log2f(opacity));
  const float d6 = d * im[6], d7 = d * im[7], d8 = d * im[8];
  float Wxx = dot3_cuda(im[0], im[0], im[3], im[3], d6, im[6]);
  float Wyy = dot3_cuda(im[1], im[1], im[4], im[4], d7, im[7]);
  float W__ = dot3_cuda(im[2], im[2], im[5], im[5], d8, im[8]);
  float Wxy = 2 * dot3_cuda(im[0], im[1], im[3], im[4], d6, im[7]);
  float Wx_ = 2 * dot3_cuda(im[0], im[2], im[3], im[5], d6, im[8]);
  float Wy_ = 2 * dot3_cuda(im[1], im[2], im[4], im[5], d7, im[8]);
  w6[0] = Wxx * TILE * TILE;
  w6[1] = Wyy * TILE * TILE;
  w6[2] = Wxy * TILE * TILE;
  w6[3] = Wx_ * TILE;
  w6[4] = Wy_ * TILE;
  w6[5] = W__;
}

/* The corner test of :301 as the reference's CUDA build evaluates it: only the cross term is fused, except in the
 * first row of a rectangle with an odd number of rows (the iteration peeled off its two-row loop over y), where the
 * w[4]*v term is fused too. */
static inline float conic_eval(const float *w, float u, float v, int fuse_y) {
  float s = (w[0] * u) * u + (w[1] * v) * v;
  s = fmaf(w[2] * u, v, s);
  s = s + w[3] * u;
  s = fuse_y ? fmaf(w[4], v, s) : s + w[4] * v;
  return s + w[5];
}

void orc_conic(int P, const float *inverse_m, const float *opac, const int32_t *radii, float *w6) {
  for (int i = 0; i < P; ++i) {
    if (radii[i] > 0) conic_coeffs(inverse_m + 9 * i, opac[i], w6 + 6 * i);
    else memset(w6 + 6 * i, 0, 6 * sizeof(float));
  }
}

typedef struct {
  uint64_t key;
  int32_t val;
  int64_t seq;
} pair_t;

static int pair_cmp(const void *a, const void *b) {
  const pair_t *x = (const pair_t *) a, *y = (const pair_t *) b;
  if (x->key != y->key) return x->key < y->key ? -1 : 1;
  return x->seq < y->seq ? -1 : (x->seq > y->seq);
}

/* Returns R = sum of tile-rectangle areas (size of point_list). */
int64_t orc_bin_size(int P, const int32_t *tiles_touched) {
  int64_t r = 0;
  for (int i = 0; i < P; ++i) r += tiles_touched[i];
  return r;
}

/* point_list[R]: Gaussian ids sorted by (tile, depth bits), ties by emission order, then the -1 padding.
 * ranges[T,2]: must be zero-initialised.  Returns the number of real (non-padding) pairs. */
int64_t orc_bin(int P, int W, int H, const float *means2D, const float *inverse_m, const float *depths,
    const float *opac, const int32_t *radii, const int32_t *tiles_touched, int32_t *point_list, int64_t *ranges,
    uint64_t *keys_out) {
  const int gx = (W + TILE - 1) / TILE, gy = (H + TILE - 1) / TILE;
  const int64_t R = orc_bin_size(P, tiles_touched);
  pair_t *pairs = (pair_t *) malloc(sizeof(pair_t) * (size_t) (R > 0 ? R : 1));
  int64_t off = 0;
  int64_t real = 0;
  for (int i = 0; i < P; ++i) {
    if (radii[i] <= 0) continue;
    const int64_t end = off + tiles_touched[i];
    int x0, y0, x1, y1;
    tile_rect(means2D[2 * i], means2D[2 * i + 1], radii[i], gx, gy, &x0, &y0, &x1, &y1);
    float w[6];
    conic_coeffs(inverse_m + 9 * i, opac[i], w);
    uint32_t dbits;
    memcpy(&dbits, depths + i, 4);
    for (int x = x0; x < x1; ++x)
      for (int y = y0; y < y1; ++y) {
        const int fy = ((y1 - y0) & 1) && y == y0;
        if (conic_eval(w, x, y, fy) <= 0 || conic_eval(w, x + 1, y, fy) <= 0 || conic_eval(w, x, y + 1, fy) <= 0 ||
            conic_eval(w, x + 1, y + 1, fy) <= 0) {
          pairs[off].key = ((uint64_t) (y * gx + x) << 32) | dbits;
          pairs[off].val = i;
          pairs[off].seq = off;
          ++off, ++real;
        }
      }
    for (; off < end; ++off) {
      pairs[off].key = (uint64_t) (gx * gy) << 32;
      pairs[off].val = -1;
      pairs[off].seq = off;
    }
  }
  qsort(pairs, (size_t) R, sizeof(pair_t), pair_cmp);
  const uint32_t T = (uint32_t) (gx * gy);
  for (int64_t k = 0; k < R; ++k) {
    point_list[k] = pairs[k].val;
    if (keys_out) keys_out[k] = pairs[k].key;
    const uint32_t cur = (uint32_t) (pairs[k].key >> 32);
    if (k == 0) {
      if (cur < T) ranges[2 * cur] = 0;
    } else {
      const uint32_t prev = (uint32_t) (pairs[k - 1].key >> 32);
      if (cur != prev) {
        ranges[2 * prev + 1] = k;
        if (cur < T) ranges[2 * cur] = k;
      }
    }
    if (k == R - 1 && cur < T) ranges[2 * cur + 1] = R;
  }
  free(pairs);
  return real;
}

/* ------------------------------------------------------------------------- */
/* compositing forward: gs_2d_fast_redner.cu:22-271                           */
/* ------------------------------------------------------------------------- */

typedef struct {
  float sx, sy, rho3d, rho2d, depth, G, alpha, pz, dx, dy;
} hit_t;

/* Per (pixel, splat) evaluation shared by forward and backward; returns 0 when the pair is skipped.
 * gs_2d_fast_redner.cu:152-186 */
static int eval_pair(float px, float py, const float *xy, const float *im, const float *Tw, float opa, float near_n,
    hit_t *h) {
  const float p0 = im[0] * px + im[1] * py + im[2];
  const float p1 = im[3] * px + im[4] * py + im[5];
  const float p2 = im[6] * px + im[7] * py + im[8];
  if (p2 == 0.0f) return 0;
  h->pz = p2;
  h->sx = p0 / p2, h->sy = p1 / p2;
  h->rho3d = h->sx * h->sx + h->sy * h->sy;
  h->dx = xy[0] - px, h->dy = xy[1] - py;
  h->rho2d = 2.0f * (h->dx * h->dx + h->dy * h->dy);
  const float rho = fminf(h->rho3d, h->rho2d);
  h->depth = (h->sx * Tw[0] + h->sy * Tw[1]) + Tw[2];
  if (h->depth < near_n) return 0;
  const float power = -0.5f * rho;
  if (power > 0.0f) return 0;
  h->G = expf(power);
  h->alpha = fminf(0.99f, opa * h->G);
  if (h->alpha < 1.0f / 255.0f) return 0;
  return 1;
}

/* aux != 0 renders the 8 extra channels (depth, normal x3, median depth, distortion, M1, M2) and, when
 * trans_mat_t2 != NULL, the flow map.  All outputs zero-initialised by the caller.
 * accum_* may be NULL; they are only touched in aux mode (as in the reference). */
void orc_blend_fwd(int W, int H, float near_n, float far_n, int aux, const float *means2D, const float *colors,
    const float *normal_opacity, const float *trans_mat, const float *inverse_m, const int32_t *point_list,
    const int64_t *ranges, const float *trans_mat_t2, float *out_color, float *out_opacity, float *out_extras,
    float *out_flow, int32_t *n_contrib, int32_t *accum_max_count, float *accum_weights_p,
    int32_t *accum_weights_count) {
  const int gx = (W + TILE - 1) / TILE, gy = (H + TILE - 1) / TILE;
  const size_t HW = (size_t) H * W;
  const int serial = accum_max_count || accum_weights_p || accum_weights_count;
#pragma omp parallel for schedule(dynamic, 1) if (!serial)
  for (int tile = 0; tile < gx * gy; ++tile) {
    const int tx = tile % gx, ty = tile / gx;
    const int64_t r0 = ranges[2 * tile], r1 = ranges[2 * tile + 1];
    for (int ly = 0; ly < TILE; ++ly)
      for (int lx = 0; lx < TILE; ++lx) {
        const int ix = tx * TILE + lx, iy = ty * TILE + ly;
        if (ix >= W || iy >= H) continue;
        const size_t pix = (size_t) iy * W + ix;
        const float px = (float) ix, py = (float) iy;
        float T = 1.0f, C[3] = {0, 0, 0}, N[3] = {0, 0, 0};
        float D = 0, M1 = 0, M2 = 0, dist = 0, med_depth = 0, flow[2] = {0, 0};
        int32_t contributor = 0, last = 0, med_contrib = -1;
        float wmax = 0;
        int32_t wmax_id = -1;
        int flag = 0;
        for (int64_t k = r0; k < r1; ++k) {
          ++contributor;
          const int g = point_list[k];
          hit_t h;
          if (!eval_pair(px, py, means2D + 2 * g, inverse_m + 9 * g, trans_mat + 9 * g + 6, normal_opacity[4 * g + 3],
                  near_n, &h))
            continue;
          const float test_T = T * (1 - h.alpha);
          if (test_T < 0.0001f) break;
          const float w = h.alpha * T;
          if (aux) {
            const float A = 1 - T;
            const float m = far_n / (far_n - near_n) * (1 - near_n / h.depth);
            dist += (m * m * A + M2 - 2 * m * M1) * w;
            D += h.depth * w;
            M1 += m * w;
            M2 += m * m * w;
            if (T > 0.5f) {
              med_depth = h.depth;
              med_contrib = contributor;
            }
            for (int ch = 0; ch < 3; ++ch) N[ch] += normal_opacity[4 * g + ch] * w;
            if (wmax < w) {
              wmax = w;
              wmax_id = g;
              flag = 1;
            }
            if (accum_weights_p) accum_weights_p[g] += w;
            if (accum_weights_count) accum_weights_count[g] += 1;
            if (trans_mat_t2) {
              const float *m2 = trans_mat_t2 + 9 * g;
              const float u = m2[0] * h.sx + m2[1] * h.sy + m2[2];
              const float v = m2[3] * h.sx + m2[4] * h.sy + m2[5];
              float ww = m2[6] * h.sx + m2[7] * h.sy + m2[8];
              ww = fabsf(ww) < 1e-5f ? 1e-5f : ww;
              flow[0] += (u / ww - px) * w;
              flow[1] += (v / ww - py) * w;
            }
          }
          /* the flag is never cleared: every later contribution counts (gs_2d_fast_redner.cu:82,211-215,227) */
          if (flag && accum_max_count) accum_max_count[wmax_id] += 1;
          for (int ch = 0; ch < 3; ++ch) C[ch] += colors[3 * g + ch] * w;
          T = test_T;
          last = contributor;
        }
        const float A = 1.0f - T;
        out_opacity[pix] = A;
        n_contrib[pix] = last;
        for (int ch = 0; ch < 3; ++ch) out_color[ch * HW + pix] = C[ch];
        if (aux) {
          n_contrib[HW + pix] = med_contrib;
          out_extras[0 * HW + pix] = D;
          for (int ch = 0; ch < 3; ++ch) out_extras[(1 + ch) * HW + pix] = N[ch];
          out_extras[4 * HW + pix] = med_depth;
          out_extras[5 * HW + pix] = dist;
          out_extras[6 * HW + pix] = M1;
          out_extras[7 * HW + pix] = M2;
          if (trans_mat_t2 && out_flow) {
            out_flow[2 * pix + 0] = A > 0 ? flow[0] / A : 0.0f;
            out_flow[2 * pix + 1] = A > 0 ? flow[1] / A : 0.0f;
          }
        }
      }
  }
}

/* ------------------------------------------------------------------------- */
/* compositing backward (the per-pixel back-to-front variant that training    */
/* uses): gs_2d_fast_redner.cu:273-561                                        */
/* ------------------------------------------------------------------------- */

/* Gradient outputs must be zero-initialised.  dL_dextras / dL_dflow may be NULL (then aux terms are off,
 * matching the kernel instantiated without auxiliary channels).  dL_dtrans_mat only receives row 2. */
void orc_blend_bwd(int W, int H, float near_n, float far_n, const float *means2D, const float *colors,
    const float *normal_opacity, const float *trans_mat, const float *inverse_m, const int32_t *point_list,
    const int64_t *ranges, const float *trans_mat_t2, const float *out_opacity, const float *out_extras,
    const int32_t *n_contrib, const float *dL_dcolor, const float *dL_dopacity, const float *dL_dextras,
    const float *dL_dflow, float *g_means2D, float *g_colors, float *g_normal_opacity, float *g_trans_mat,
    float *g_inverse_m) {
  const int gx = (W + TILE - 1) / TILE, gy = (H + TILE - 1) / TILE;
  const size_t HW = (size_t) H * W;
  const int aux = dL_dextras != NULL && out_extras != NULL;
#pragma omp parallel for schedule(dynamic, 1)
  for (int tile = 0; tile < gx * gy; ++tile) {
    const int tx = tile % gx, ty = tile / gx;
    const int64_t r0 = ranges[2 * tile], r1 = ranges[2 * tile + 1];
    for (int ly = 0; ly < TILE; ++ly)
      for (int lx = 0; lx < TILE; ++lx) {
        const int ix = tx * TILE + lx, iy = ty * TILE + ly;
        if (ix >= W || iy >= H) continue;
        const size_t pix = (size_t) iy * W + ix;
        const float px = (float) ix, py = (float) iy;
        const float T_final = 1 - out_opacity[pix];
        float T = T_final;
        const int last_contributor = n_contrib[pix];
        const int median_contributor = aux ? n_contrib[HW + pix] : 0;
        float gpix[3], accum_rec[3] = {0, 0, 0}, last_color[3] = {0, 0, 0};
        for (int ch = 0; ch < 3; ++ch) gpix[ch] = dL_dcolor[ch * HW + pix];
        float g_reg = 0, g_depth = 0, g_acc = 0, g_n2d[3] = {0, 0, 0}, g_med = 0;
        if (aux) {
          g_acc = dL_dopacity[pix];
          g_depth = dL_dextras[0 * HW + pix];
          g_reg = dL_dextras[5 * HW + pix];
          for (int ch = 0; ch < 3; ++ch) g_n2d[ch] = dL_dextras[(1 + ch) * HW + pix];
          g_med = dL_dextras[4 * HW + pix];
        }
        float last_depth = 0, last_normal[3] = {0, 0, 0}, acc_depth = 0, acc_alpha = 0, acc_normal[3] = {0, 0, 0};
        const float final_D = aux ? out_extras[6 * HW + pix] : 0;
        const float final_D2 = aux ? out_extras[7 * HW + pix] : 0;
        const float final_A = 1 - T_final;
        float last_dL_dT = 0, last_alpha = 0;
        float acc_flow[2] = {0, 0}, last_flow[2] = {0, 0}, gflow[2] = {0, 0};
        if (dL_dflow) gflow[0] = dL_dflow[2 * pix], gflow[1] = dL_dflow[2 * pix + 1];

        for (int64_t k = r1 - 1; k >= r0; --k) {
          const int contributor = (int) (k - r0); /* 0-based list position */
          if (contributor >= last_contributor) continue;
          const int g = point_list[k];
          const float *Tw = trans_mat + 9 * g + 6;
          const float opa = normal_opacity[4 * g + 3];
          hit_t h;
          if (!eval_pair(px, py, means2D + 2 * g, inverse_m + 9 * g, Tw, opa, near_n, &h)) continue;
          const float alpha = h.alpha, G = h.G;
          T = T / (1.0f - alpha);
          const float w = alpha * T;
          float dL_dalpha = 0;
          for (int ch = 0; ch < 3; ++ch) {
            const float c = colors[3 * g + ch];
            accum_rec[ch] = last_alpha * last_color[ch] + (1.0f - last_alpha) * accum_rec[ch];
            last_color[ch] = c;
            dL_dalpha += (c - accum_rec[ch]) * gpix[ch];
            ATOMIC_ADD(g_colors[3 * g + ch], w * gpix[ch]);
          }
          float dL_dz = 0, dL_dweight = 0, dL_dsx = 0, dL_dsy = 0;
          if (aux) {
            const float m_d = far_n / (far_n - near_n) * (1 - near_n / h.depth);
            const float dmd_dd = (far_n * near_n) / ((far_n - near_n) * h.depth * h.depth);
            if (contributor == median_contributor - 1) dL_dz += g_med;
            dL_dweight += (final_D2 + m_d * m_d * final_A - 2 * m_d * final_D) * g_reg;
            dL_dalpha += dL_dweight - last_dL_dT;
            last_dL_dT = dL_dweight * alpha + (1 - alpha) * last_dL_dT;
            const float dL_dmd = 2.0f * (T * alpha) * (m_d * final_A - final_D) * g_reg;
            dL_dz += dL_dmd * dmd_dd;
            acc_depth = last_alpha * last_depth + (1.0f - last_alpha) * acc_depth;
            last_depth = h.depth;
            dL_dalpha += (h.depth - acc_depth) * g_depth;
            acc_alpha = last_alpha * 1.0f + (1.0f - last_alpha) * acc_alpha;
            dL_dalpha += (1 - acc_alpha) * g_acc;
            for (int ch = 0; ch < 3; ++ch) {
              const float nc = normal_opacity[4 * g + ch];
              acc_normal[ch] = last_alpha * last_normal[ch] + (1.0f - last_alpha) * acc_normal[ch];
              last_normal[ch] = nc;
              dL_dalpha += (nc - acc_normal[ch]) * g_n2d[ch];
              ATOMIC_ADD(g_normal_opacity[4 * g + ch], w * g_n2d[ch]);
            }
            dL_dz += w * g_depth;
          }
          if (dL_dflow) {
            const float *m2 = trans_mat_t2 + 9 * g;
            const float u = m2[0] * h.sx + m2[1] * h.sy + m2[2];
            const float v = m2[3] * h.sx + m2[4] * h.sy + m2[5];
            float ww = m2[6] * h.sx + m2[7] * h.sy + m2[8];
            ww = fabsf(ww) < 1e-5f ? 1e-5f : ww;
            acc_flow[0] = last_alpha * last_flow[0] + (1.0f - last_alpha) * acc_flow[0];
            acc_flow[1] = last_alpha * last_flow[1] + (1.0f - last_alpha) * acc_flow[1];
            last_flow[0] = u / ww - px, last_flow[1] = v / ww - py;
            dL_dalpha += (last_flow[0] - acc_flow[0]) * gflow[0] + (last_flow[1] - acc_flow[1]) * gflow[1];
            const float gu = w / ww * gflow[0], gv = w / ww * gflow[1];
            const float gw = -w / (ww * ww) * (u * gflow[0] + v * gflow[1]);
            dL_dsx += m2[0] * gu + m2[3] * gv + m2[6] * gw;
            dL_dsy += m2[1] * gu + m2[4] * gv + m2[7] * gw;
          }
          dL_dalpha *= T;
          last_alpha = alpha;
          const float dL_dG = opa * dL_dalpha;
          if (h.rho3d <= h.rho2d) {
            dL_dsx += dL_dG * -G * h.sx + dL_dz * Tw[0];
            dL_dsy += dL_dG * -G * h.sy + dL_dz * Tw[1];
            const float a = dL_dsx / h.pz, b = dL_dsy / h.pz;
            const float c = -(a * h.sx + b * h.sy);
            float *gi = g_inverse_m + 9 * g;
            ATOMIC_ADD(gi[0], a * px); ATOMIC_ADD(gi[1], a * py); ATOMIC_ADD(gi[2], a);
            ATOMIC_ADD(gi[3], b * px); ATOMIC_ADD(gi[4], b * py); ATOMIC_ADD(gi[5], b);
            ATOMIC_ADD(gi[6], c * px); ATOMIC_ADD(gi[7], c * py); ATOMIC_ADD(gi[8], c);
          } else {
            ATOMIC_ADD(g_means2D[2 * g + 0], dL_dG * (-G * 2.0f * h.dx));
            ATOMIC_ADD(g_means2D[2 * g + 1], dL_dG * (-G * 2.0f * h.dy));
          }
          ATOMIC_ADD(g_trans_mat[9 * g + 6], dL_dz * h.sx);
          ATOMIC_ADD(g_trans_mat[9 * g + 7], dL_dz * h.sy);
          ATOMIC_ADD(g_trans_mat[9 * g + 8], dL_dz);
          ATOMIC_ADD(g_normal_opacity[4 * g + 3], G * dL_dalpha);
        }
      }
  }
}

/* ------------------------------------------------------------------------- */
/* preprocess backward: gs_2d_fast_preprocess.cu:100-139, 516-609;            */
/* include/ops_3d.h:126-134 (quaternion adjoint)                              */
/* ------------------------------------------------------------------------- */

static inline void cross3(const float *a, const float *b, float *o) {
  o[0] = a[1] * b[2] - a[2] * b[1];
  o[1] = a[2] * b[0] - a[0] * b[2];
  o[2] = a[0] * b[1] - a[1] * b[0];
}

/* Adjoint of inverse_m = adj(M) = [c1 x c2 ; c2 x c0 ; c0 x c1], c_j the columns of M: adds dL/dM into gT.
 * gs_2d_fast_preprocess.cu:561-569 */
static void adjugate_adjoint(const float *m, const float *G, float *gT) {
  float c[3][3], dc[3][3] = {{0}};
  for (int j = 0; j < 3; ++j)
    for (int r = 0; r < 3; ++r) c[j][r] = m[r * 3 + j];
  float t[3];
  for (int r = 0; r < 3; ++r) { /* row r = c[(r+1)%3] x c[(r+2)%3] */
    const int a = (r + 1) % 3, b = (r + 2) % 3;
    cross3(c[b], G + 3 * r, t);
    for (int k = 0; k < 3; ++k) dc[a][k] += t[k];
    cross3(G + 3 * r, c[a], t);
    for (int k = 0; k < 3; ++k) dc[b][k] += t[k];
  }
  for (int j = 0; j < 3; ++j)
    for (int r = 0; r < 3; ++r) gT[r * 3 + j] += dc[j][r];
}

/* g_trans_mat += adjoint of the adjugate applied to g_inverse_m (test helper) */
void orc_fold_inverse_grad(int P, const float *trans_mat, const float *g_inverse_m, float *g_trans_mat) {
  for (int i = 0; i < P; ++i) adjugate_adjoint(trans_mat + 9 * i, g_inverse_m + 9 * i, g_trans_mat + 9 * i);
}

/* g_means2D is read (gradient of the low-pass branch) and then overwritten with the densification proxy,
 * as the reference does.  g_sh_dc / g_sh_rest may be NULL. */
void orc_preprocess_bwd(int P, int W, int H, int sh_degree, int n_dc, int n_rest, const float *means,
    const float *scales, const float *quats, const float *sh_dc, const float *sh_rest, const float *Tw2v,
    const float *Tv2s, const float *campos, const float *trans_mat, const int32_t *radii, const float *colors,
    float *g_means2D, const float *g_trans_mat, const float *g_inverse_m, const float *g_colors,
    const float *g_normal_opacity, float *g_means, float *g_scales, float *g_quats, float *g_opac, float *g_sh_dc,
    float *g_sh_rest) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < P; ++i) {
    if (radii[i] <= 0) continue;
    g_opac[i] = g_normal_opacity[4 * i + 3];
    const float *m = trans_mat + 9 * i;
    float gT[9];
    for (int k = 0; k < 9; ++k) gT[k] = g_trans_mat[9 * i + k];
    adjugate_adjoint(m, g_inverse_m + 9 * i, gT);
    /* adjoint of the bounding-box centre (gs_2d_fast_preprocess.cu:516-534) */
    {
      const float gx = g_means2D[2 * i], gy = g_means2D[2 * i + 1];
      const float tv[3] = {9.0f, 9.0f, -1.0f};
      const float d = tv[0] * (m[6] * m[6]) + tv[1] * (m[7] * m[7]) + tv[2] * (m[8] * m[8]);
      const float inv_d = 1.0f / d;
      float f[3], df[3];
      for (int k = 0; k < 3; ++k) f[k] = tv[k] * inv_d;
      for (int k = 0; k < 3; ++k) {
        gT[0 + k] += gx * f[k] * m[6 + k];
        gT[3 + k] += gy * f[k] * m[6 + k];
        df[k] = gx * m[0 + k] * m[6 + k] + gy * m[3 + k] * m[6 + k];
      }
      const float dd = (df[0] * f[0] + df[1] * f[1] + df[2] * f[2]) * -(1.0f / d);
      for (int k = 0; k < 3; ++k)
        gT[6 + k] += (gx * f[k] * m[0 + k] + gy * f[k] * m[3 + k]) + dd * (tv[k] * m[6 + k] * 2.0f);
    }
    /* normal flip */
    const float *q = quats + 4 * i, *p = means + 3 * i, *s = scales + 2 * i;
    float R[9];
    quat_to_rot(q, R);
    float gn[3] = {g_normal_opacity[4 * i], g_normal_opacity[4 * i + 1], g_normal_opacity[4 * i + 2]};
    {
      const float n[3] = {R[2], R[5], R[8]};
      float nv[3], pv[3];
      for (int r = 0; r < 3; ++r) {
        nv[r] = Tw2v[r * 4] * n[0] + Tw2v[r * 4 + 1] * n[1] + Tw2v[r * 4 + 2] * n[2];
        pv[r] = Tw2v[r * 4] * p[0] + Tw2v[r * 4 + 1] * p[1] + Tw2v[r * 4 + 2] * p[2] + Tw2v[r * 4 + 3];
      }
      const float c = -(pv[0] * nv[0] + pv[1] * nv[1] + pv[2] * nv[2]);
      const float sgn = c > 0 ? 1.0f : -1.0f;
      for (int k = 0; k < 3; ++k) gn[k] *= sgn;
    }
    /* adjoint of splat_matrix (gs_2d_fast_preprocess.cu:100-139) */
    float gL[9], dR[9];
    for (int a = 0; a < 3; ++a)
      for (int b = 0; b < 3; ++b) {
        float acc = 0;
        for (int k = 0; k < 3; ++k) acc += Tv2s[k * 3 + a] * gT[k * 3 + b];
        gL[a * 3 + b] = acc;
      }
    for (int a = 0; a < 3; ++a)
      for (int b = 0; b < 3; ++b) {
        float acc = 0;
        for (int k = 0; k < 3; ++k) acc += Tw2v[k * 4 + a] * gL[k * 3 + b];
        dR[a * 3 + b] = acc;
      }
    float gp[3] = {dR[2], dR[5], dR[8]};
    for (int a = 0; a < 3; ++a) dR[a * 3 + 2] = gn[0] * Tw2v[0 + a] + gn[1] * Tw2v[4 + a] + gn[2] * Tw2v[8 + a];
    g_scales[2 * i + 0] = dR[0] * R[0] + dR[3] * R[3] + dR[6] * R[6];
    g_scales[2 * i + 1] = dR[1] * R[1] + dR[4] * R[4] + dR[7] * R[7];
    for (int a = 0; a < 3; ++a) dR[a * 3] *= s[0], dR[a * 3 + 1] *= s[1];
    {
      const float x = q[0], y = q[1], z = q[2], w = q[3];
      g_quats[4 * i + 0] =
          2 * (-2 * x * (dR[4] + dR[8]) + y * (dR[1] + dR[3]) + z * (dR[2] + dR[6]) + w * (dR[7] - dR[5]));
      g_quats[4 * i + 1] =
          2 * (x * (dR[1] + dR[3]) - 2 * y * (dR[0] + dR[8]) + z * (dR[5] + dR[7]) + w * (dR[2] - dR[6]));
      g_quats[4 * i + 2] =
          2 * (x * (dR[2] + dR[6]) + y * (dR[5] + dR[7]) - 2 * z * (dR[0] + dR[4]) + w * (dR[3] - dR[1]));
      g_quats[4 * i + 3] = 2 * (x * (dR[7] - dR[5]) + y * (dR[2] - dR[6]) + z * (dR[3] - dR[1]));
    }
    /* SH adjoint (spherical_harmonic.h:204-677) */
    if (sh_degree >= 0) {
      float x = p[0] - campos[0], y = p[1] - campos[1], z = p[2] - campos[2];
      const float ux = x, uy = y, uz = z;
      const float n = 1.0f / sqrtf(x * x + y * y + z * z + 1e-12f);
      x *= n, y *= n, z *= n;
      float grgb[3];
      for (int ch = 0; ch < 3; ++ch) grgb[ch] = colors[3 * i + ch] > 0 ? g_colors[3 * i + ch] : 0.0f;
      float b[SH_MAX], bx[16], by[16], bz[16], tk[SH_MAX];
      sh_basis(sh_degree, x, y, z, b);
      sh_basis_grad(sh_degree, x, y, z, bx, by, bz);
      const int nb = (sh_degree + 1) * (sh_degree + 1);
      float dx = 0, dy = 0, dz = 0;
      for (int k = 0; k < nb; ++k) {
        const float *c = sh_coef(sh_dc, sh_rest, n_dc, n_rest, i, k);
        float *gc = NULL;
        if (g_sh_dc) gc = (float *) sh_coef(g_sh_dc, g_sh_rest, n_dc, n_rest, i, k);
        if (gc && !(sh_rest && k > 0 && !g_sh_rest))
          for (int ch = 0; ch < 3; ++ch) gc[ch] = grgb[ch] * b[k];
        const float tdot = grgb[0] * c[0] + grgb[1] * c[1] + grgb[2] * c[2];
        tk[k] = tdot;
        if (k < 16) dx += tdot * bx[k], dy += tdot * by[k], dz += tdot * bz[k];
      }
      const float t = -(ux * dx + uy * dy + uz * dz) * n * n * n;
      gp[0] += dx * n + t * ux;
      gp[1] += dy * n + t * uy;
      gp[2] += dz * n + t * uz;
      if (sh_degree > 3) {
        /* degrees 4..: central differences of the general definition with respect to the position, in double */
        const double h = 1e-5 / (double) n;
        const double u[3] = {ux, uy, uz};
        for (int a = 0; a < 3; ++a) {
          double up[3] = {u[0], u[1], u[2]}, um[3] = {u[0], u[1], u[2]};
          up[a] += h, um[a] -= h;
          gp[a] += (float) ((sh_high_sum(sh_degree, tk, up[0], up[1], up[2]) -
                             sh_high_sum(sh_degree, tk, um[0], um[1], um[2])) / (2.0 * h));
        }
      }
    }
    for (int k = 0; k < 3; ++k) g_means[3 * i + k] = gp[k];
    g_means2D[2 * i + 0] = gT[2] * m[8] * 0.5f * (float) W;
    g_means2D[2 * i + 1] = gT[5] * m[8] * 0.5f * (float) H;
  }
}

/* ------------------------------------------------------------------------- */
/* nearest / farthest control point: src/other/cdist_top.cu:3-32, 57-81       */
/* ------------------------------------------------------------------------- */

/* The reference has two builds of this loop.  Its CPU branch (:57-81, gcc) rounds the product and the sum
 * separately; its CUDA kernel (:19-23, nvcc with the default -fmad) contracts them into sum = fma(t, t, sum).  The two
 * can pick different control points on near-ties, so both forms are restated: `fused` selects the CUDA build's. */
#define ORC_CDIST_TOP(NAME, T, FMA, SQRT)                                                                      \
  void NAME(int B, int N, int M, int D, const T *x1, const T *x2, int largest, int fused, T *dist,             \
      int64_t *index) {                                                                                         \
    for (int b = 0; b < B; ++b) {                                                                               \
      _Pragma("omp parallel for schedule(static)") for (int n = 0; n < N; ++n) {                                \
        const T *p = x1 + ((size_t) b * N + n) * D;                                                             \
        T best = 0;                                                                                             \
        int besti = 0;                                                                                          \
        for (int m = 0; m < M; ++m) {                                                                           \
          const T *c = x2 + ((size_t) b * M + m) * D;                                                           \
          T sum = 0;                                                                                            \
          for (int k = 0; k < D; ++k) {                                                                         \
            const T t = p[k] - c[k];                                                                            \
            if (fused) sum = FMA(t, t, sum);                                                                    \
            else sum += t * t;                                                                                  \
          }                                                                                                     \
          /* replace when (sum > best) == largest: exact ties go to the LAST index for largest == 0 */          \
          if (m == 0 || ((sum > best) ? 1 : 0) == (largest ? 1 : 0)) {                                          \
            best = sum;                                                                                         \
            besti = m;                                                                                          \
          }                                                                                                     \
        }                                                                                                       \
        dist[(size_t) b * N + n] = SQRT(best);                                                                  \
        index[(size_t) b * N + n] = besti;                                                                      \
      }                                                                                                         \
    }                                                                                                           \
  }
ORC_CDIST_TOP(orc_cdist_top, float, fmaf, sqrtf)

/* src/other/cdist_top.cu:86-105, 130-150 */
void orc_cdist_top_bwd(int B, int N, int M, int D, const float *x1, const float *x2, const float *dist,
    const int64_t *index, const float *grad_dist, float *g1, float *g2) {
  for (int b = 0; b < B; ++b)
    for (int n = 0; n < N; ++n) {
      const size_t i = (size_t) b * N + n;
      const int64_t j = index[i];
      const float g = grad_dist[i] / dist[i];
      for (int k = 0; k < D; ++k) {
        const float t = g * (x1[i * D + k] - x2[((size_t) b * M + j) * D + k]);
        g1[i * D + k] = t;
        g2[((size_t) b * M + j) * D + k] -= t;
      }
    }
}

/* the same two functions in double precision (the reference dispatches on the dtype, cdist_top.cu:48,116) */
ORC_CDIST_TOP(orc_cdist_top_f64, double, fma, sqrt)

/* src/other/cdist_top.cu:86-105, 130-150 */
void orc_cdist_top_bwd_f64(int B, int N, int M, int D, const double *x1, const double *x2, const double *dist,
    const int64_t *index, const double *grad_dist, double *g1, double *g2) {
  for (int b = 0; b < B; ++b)
    for (int n = 0; n < N; ++n) {
      const size_t i = (size_t) b * N + n;
      const int64_t j = index[i];
      const double g = grad_dist[i] / dist[i];
      for (int k = 0; k < D; ++k) {
        const double t = g * (x1[i * D + k] - x2[((size_t) b * M + j) * D + k]);
        g1[i * D + k] = t;
        g2[((size_t) b * M + j) * D + k] -= t;
      }
    }
}

/* Exact K nearest control points by squared L2 (direct differences, accumulation order of
 * cdist_top.cu:19-23), ascending by (distance, index): ties go to the LOWER index.
 * This is the contract of the K-NN used for LBS weights (fast_2d_gs/network.py:504), whose
 * third-party implementation (pytorch3d.ops.knn_points, unpinned) is not part of the reference tree. */
void orc_knn(int N, int M, int D, int K, const float *x, const float *c, float *d2, int64_t *index) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float bd[64];
    int bi[64];
    int cnt = 0;
    for (int m = 0; m < M; ++m) {
      float sum = 0;
      for (int k = 0; k < D; ++k) {
        const float t = x[(size_t) n * D + k] - c[(size_t) m * D + k];
        sum += t * t;
      }
      if (cnt < K || sum < bd[cnt - 1]) {
        int pos = cnt < K ? cnt : K - 1;
        while (pos > 0 && bd[pos - 1] > sum) {
          bd[pos] = bd[pos - 1];
          bi[pos] = bi[pos - 1];
          --pos;
        }
        bd[pos] = sum;
        bi[pos] = m;
        if (cnt < K) ++cnt;
      }
    }
    for (int k = 0; k < K; ++k) {
      d2[(size_t) n * K + k] = k < cnt ? bd[k] : INFINITY;
      index[(size_t) n * K + k] = k < cnt ? bi[k] : -1;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* masked Adam: src/other/adam_masked_update.cu:9-28                          */
/* ------------------------------------------------------------------------- */

void orc_adam(float *param, const float *grad, float *exp_avg, float *exp_avg_sq, const uint8_t *visible, float lr,
    float b1, float b2, float eps, int64_t N, int64_t M) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n) {
    if (!visible[n]) continue;
    for (int64_t k = 0; k < M; ++k) {
      const int64_t i = n * M + k;
      const float g = grad[i];
      const float m = b1 * exp_avg[i] + (1.0f - b1) * g;
      const float v = b2 * exp_avg_sq[i] + (1.0f - b2) * g * g;
      const float step = -lr * m / (sqrtf(v) + eps);
      param[i] += step;
      exp_avg[i] = m;
      exp_avg_sq[i] = v;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* SSIM map and its adjoint: fast_2d_gs/losses/ssim.py:12-22 (window), 48-67   */
/* (_ssim: five zero-padded 11x11 convolutions); derivative maps and adjoint   */
/* as bound by FusedSSIM (ssim.py:24-45; src/other/structural_similarity.cu)   */
/* ------------------------------------------------------------------------- */

static void ssim_window(float *w2 /* [11*11] */) {
  float g[11], sum = 0.0f;
  for (int i = 0; i < 11; ++i) {
    g[i] = (float) exp(-(double) ((i - 5) * (i - 5)) / (2.0 * 1.5 * 1.5));
    sum += g[i];
  }
  for (int i = 0; i < 11; ++i) g[i] /= sum;
  for (int i = 0; i < 11; ++i)
    for (int j = 0; j < 11; ++j) w2[i * 11 + j] = g[i] * g[j];
}

/* images [planes, H, W]; outputs the map and d map / d(mu1, w*x^2, w*xy) */
void orc_ssim_forward(int planes, int H, int W, float C1, float C2, const float *x, const float *y, float *map,
    float *d_mu1, float *d_s11, float *d_s12) {
  float w2[121];
  ssim_window(w2);
#pragma omp parallel for schedule(static)
  for (int p = 0; p < planes * H; ++p) {
    const int pl = p / H, r = p % H;
    const float *xp = x + (size_t) pl * H * W, *yp = y + (size_t) pl * H * W;
    for (int c = 0; c < W; ++c) {
      float mu1 = 0, mu2 = 0, q11 = 0, q22 = 0, q12 = 0;
      for (int i = 0; i < 11; ++i) {
        const int rr = r + i - 5;
        if (rr < 0 || rr >= H) continue;
        for (int j = 0; j < 11; ++j) {
          const int cc = c + j - 5;
          if (cc < 0 || cc >= W) continue;
          const float w = w2[i * 11 + j], u = xp[(size_t) rr * W + cc], v = yp[(size_t) rr * W + cc];
          mu1 += w * u, mu2 += w * v, q11 += w * (u * u), q22 += w * (v * v), q12 += w * (u * v);
        }
      }
      const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2, mu12 = mu1 * mu2;
      const float s11 = q11 - mu1_sq, s22 = q22 - mu2_sq, s12 = q12 - mu12;
      const float A = mu1_sq + mu2_sq + C1, B = s11 + s22 + C2, Cn = 2 * mu12 + C1, D = 2 * s12 + C2;
      const size_t o = (size_t) pl * H * W + (size_t) r * W + c;
      map[o] = (Cn * D) / (A * B);
      if (d_mu1) {
        d_mu1[o] = 2 * mu2 * (D - Cn) / (A * B) - 2 * mu1 * Cn * D / (A * A * B) + 2 * mu1 * Cn * D / (A * B * B);
        d_s11[o] = -Cn * D / (A * B * B);
        d_s12[o] = 2 * Cn / (A * B);
      }
    }
  }
}

/* dL/dx = w * (g d_mu1) + 2 x (w * (g d_s11)) + y (w * (g d_s12)) */
void orc_ssim_backward(int planes, int H, int W, const float *x, const float *y, const float *g_map,
    const float *d_mu1, const float *d_s11, const float *d_s12, float *g_x) {
  float w2[121];
  ssim_window(w2);
#pragma omp parallel for schedule(static)
  for (int p = 0; p < planes * H; ++p) {
    const int pl = p / H, r = p % H;
    const size_t base = (size_t) pl * H * W;
    for (int c = 0; c < W; ++c) {
      float t0 = 0, t1 = 0, t2 = 0;
      for (int i = 0; i < 11; ++i) {
        const int rr = r + i - 5;
        if (rr < 0 || rr >= H) continue;
        for (int j = 0; j < 11; ++j) {
          const int cc = c + j - 5;
          if (cc < 0 || cc >= W) continue;
          const size_t q = base + (size_t) rr * W + cc;
          const float w = w2[i * 11 + j] * g_map[q];
          t0 += w * d_mu1[q], t1 += w * d_s11[q], t2 += w * d_s12[q];
        }
      }
      const size_t o = base + (size_t) r * W + c;
      g_x[o] = t0 + 2 * x[o] * t1 + y[o] * t2;
    }
  }
}
