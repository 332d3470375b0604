// Real spherical-harmonic colour, forward and adjoint: degrees 0..3 here, 4..7 in the generated fsgs_sh_high.h.
// Basis and sign convention of the reference (fast_2d_gs/_C/include/spherical_harmonic.h:18-202, 204-677):
// colour = max(0, 0.5 + sum_k c_k * Y_k(dir)),  dir = normalize(position - camera position).
#pragma once
#include "fsgs_common.cuh"
#include "fsgs_sh_high.h"

namespace fsgs {

constexpr float kSH0 = 0.28209479177387814f;
constexpr float kSH1 = 0.48860251190291987f;
constexpr float kSH2a = 1.0925484305920792f;
constexpr float kSH2b = 0.94617469575755997f;
constexpr float kSH2c = 0.31539156525251999f;
constexpr float kSH2d = 0.54627421529603959f;
constexpr float kSH3a = 0.59004358992664352f;
constexpr float kSH3b = 2.8906114426405538f;
constexpr float kSH3c = 0.45704579946446572f;
constexpr float kSH3d = 0.3731763325901154f;
constexpr float kSH3e = 1.4453057213202769f;

// Y_k for k < (deg+1)^2
__device__ __forceinline__ void sh_basis(int deg, float x, float y, float z, float *b) {
  const float x2 = x * x, y2 = y * y, z2 = z * z;
  b[0] = kSH0;
  if (deg > 0) {
    b[1] = -kSH1 * y;
    b[2] = kSH1 * z;
    b[3] = -kSH1 * x;
  }
  if (deg > 1) {
    b[4] = kSH2a * (x * y);
    b[5] = -kSH2a * (y * z);
    b[6] = kSH2b * z2 - kSH2c;
    b[7] = -kSH2a * (x * z);
    b[8] = kSH2d * x2 - kSH2d * y2;
  }
  if (deg > 2) {
    b[9] = kSH3a * y * (-3.0f * x2 + y2);
    b[10] = kSH3b * (x * y) * z;
    b[11] = kSH3c * y * (1.0f - 5.0f * z2);
    b[12] = kSH3d * z * (5.0f * z2 - 3.0f);
    b[13] = kSH3c * x * (1.0f - 5.0f * z2);
    b[14] = kSH3e * z * (x2 - y2);
    b[15] = kSH3a * x * (-x2 + 3.0f * y2);
  }
}

// gradient of Y_k with respect to (x, y, z) as free variables
__device__ __forceinline__ float3 sh_basis_grad(int k, float x, float y, float z) {
  const float x2 = x * x, y2 = y * y, z2 = z * z;
  switch (k) {
    case 1: return make_float3(0, -kSH1, 0);
    case 2: return make_float3(0, 0, kSH1);
    case 3: return make_float3(-kSH1, 0, 0);
    case 4: return make_float3(kSH2a * y, kSH2a * x, 0);
    case 5: return make_float3(0, -kSH2a * z, -kSH2a * y);
    case 6: return make_float3(0, 0, 2.0f * kSH2b * z);
    case 7: return make_float3(-kSH2a * z, 0, -kSH2a * x);
    case 8: return make_float3(2.0f * kSH2d * x, -2.0f * kSH2d * y, 0);
    case 9: return make_float3(kSH3a * (-6.0f * x * y), kSH3a * (-3.0f * x2 + 3.0f * y2), 0);
    case 10: return make_float3(kSH3b * y * z, kSH3b * x * z, kSH3b * x * y);
    case 11: return make_float3(0, kSH3c * (1.0f - 5.0f * z2), kSH3c * (-10.0f * y * z));
    case 12: return make_float3(0, 0, kSH3d * (15.0f * z2 - 3.0f));
    case 13: return make_float3(kSH3c * (1.0f - 5.0f * z2), 0, kSH3c * (-10.0f * x * z));
    case 14: return make_float3(kSH3e * 2.0f * x * z, -kSH3e * 2.0f * y * z, kSH3e * (x2 - y2));
    case 15: return make_float3(kSH3a * (-3.0f * x2 + 3.0f * y2), kSH3a * 6.0f * x * y, 0);
    default: return make_float3(0, 0, 0);
  }
}

// Degrees 4..deg of the colour: rgb += sum_k c_k * Y_k, coefficient k at coef + 3 * k.
__device__ __forceinline__ void sh_high_colour(int deg, float x, float y, float z, const float *coef, float3 &rgb) {
  float bb[15];
#define FSGS_SH_BAND(L)                                                                  \
  if (deg >= L) {                                                                        \
    fsgs_sh_band##L(x, y, z, bb);                                                        \
    _Pragma("unroll") for (int m = 0; m < 2 * L + 1; ++m) {                              \
      const float *c = coef + 3 * (L * L + m);                                           \
      rgb.x += c[0] * bb[m], rgb.y += c[1] * bb[m], rgb.z += c[2] * bb[m];               \
    }                                                                                    \
  }
  FSGS_SH_BAND(4)
  FSGS_SH_BAND(5)
  FSGS_SH_BAND(6)
  FSGS_SH_BAND(7)
#undef FSGS_SH_BAND
}

// Adjoint of the above for degrees 4..deg: writes g_coef[k] = grgb * Y_k (when g_coef is not null) and accumulates
// (dx, dy, dz) += sum_k (grgb . c_k) dY_k / d(x, y, z).
__device__ __forceinline__ void sh_high_adjoint(int deg, float x, float y, float z, const float *coef, float *g_coef,
    float3 grgb, float &dx, float &dy, float &dz) {
  float bb[15], t[15];
#define FSGS_SH_BAND(L)                                                                  \
  if (deg >= L) {                                                                        \
    fsgs_sh_band##L(x, y, z, bb);                                                        \
    _Pragma("unroll") for (int m = 0; m < 2 * L + 1; ++m) {                              \
      const float *c = coef + 3 * (L * L + m);                                           \
      t[m] = grgb.x * c[0] + grgb.y * c[1] + grgb.z * c[2];                              \
      if (g_coef) {                                                                      \
        float *g = g_coef + 3 * (L * L + m);                                             \
        g[0] = grgb.x * bb[m], g[1] = grgb.y * bb[m], g[2] = grgb.z * bb[m];             \
      }                                                                                  \
    }                                                                                    \
    fsgs_sh_band##L##_adjoint(x, y, z, t, &dx, &dy, &dz);                                \
  }
  FSGS_SH_BAND(4)
  FSGS_SH_BAND(5)
  FSGS_SH_BAND(6)
  FSGS_SH_BAND(7)
#undef FSGS_SH_BAND
}

}  // namespace fsgs
