// Image loss epilogue: structural similarity with an 11x11 Gaussian window (sigma 1.5, zero padding) forward and
// adjoint, with the L1 term and both mean reductions folded in.
//
// The map and its three partial-derivative maps follow the operators the reference binds as `fusedssim` /
// `fusedssim_backward` (fast_2d_gs/losses/ssim.py:24-45, src/other/structural_similarity.cu:187-381; the map itself
// is the one of `_ssim`, ssim.py:48-67):
//   mu1 = w * x, mu2 = w * y, s11 = w * x^2 - mu1^2, s22 = w * y^2 - mu2^2, s12 = w * xy - mu1 mu2
//   map = (2 mu1 mu2 + C1)(2 s12 + C2) / ((mu1^2 + mu2^2 + C1)(s11 + s22 + C2))
// and, holding the raw moments w*x^2 and w*xy fixed,
//   dm_dmu1, dm_dsigma1_sq, dm_dsigma12  = d map / d mu1, d (w*x^2), d (w*xy),
// so that  dL/dx = w * (g dm_dmu1) + 2 x (w * (g dm_dsigma1_sq)) + y (w * (g dm_dsigma12)),  g = dL/dmap.
//
// One block of 32x8 threads per 32x32 tile of one channel: the tile and its 5-pixel apron are staged in shared
// memory, the separable window is applied along x into a second buffer and along y from there.  Bandwidth bound:
// every input pixel is fetched (32+10)^2 / 32^2 = 1.7 times.
#include "fsgs_common.cuh"

namespace fsgs {

constexpr int kWin = 11, kHalf = 5;
constexpr int kLT = 32;                 // tile edge
constexpr int kLA = kLT + 2 * kHalf;    // tile + apron
constexpr int kLThreads = 256;

__constant__ float c_window[kWin];

struct SsimFwd {
  int B, C, H, W;
  float C1, C2;
  const float *x, *y;
  float *map, *d_mu1, *d_s11, *d_s12;  // derivative maps may be null
  float *sums;                         // [2]: sum of the map, sum of |x - y|; may be null
};

__device__ __forceinline__ float block_sum(float v, float *scratch) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0;
  if (threadIdx.x < kLThreads / 32) t = scratch[threadIdx.x];
  if (warp == 0)
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;  // valid in thread 0
}

__global__ void __launch_bounds__(kLThreads) ssim_forward_kernel(SsimFwd a) {
  __shared__ float s_x[kLA][kLA + 1], s_y[kLA][kLA + 1];
  __shared__ float s_h[5][kLA][kLT + 1];
  __shared__ float s_red[kLThreads / 32];
  const int plane = blockIdx.z;  // b * C + c
  const size_t off = (size_t) plane * a.H * a.W;
  const int tx0 = blockIdx.x * kLT, ty0 = blockIdx.y * kLT;
  const float *x = a.x + off, *y = a.y + off;
  for (int e = threadIdx.x; e < kLA * kLA; e += kLThreads) {
    const int r = e / kLA, c = e - r * kLA;
    const int gy = ty0 + r - kHalf, gx = tx0 + c - kHalf;
    const bool in = gy >= 0 && gy < a.H && gx >= 0 && gx < a.W;
    s_x[r][c] = in ? __ldg(x + (size_t) gy * a.W + gx) : 0.0f;
    s_y[r][c] = in ? __ldg(y + (size_t) gy * a.W + gx) : 0.0f;
  }
  __syncthreads();
  // along x
  for (int e = threadIdx.x; e < kLA * kLT; e += kLThreads) {
    const int r = e / kLT, c = e - r * kLT;
    float m1 = 0, m2 = 0, q11 = 0, q22 = 0, q12 = 0;
#pragma unroll
    for (int k = 0; k < kWin; ++k) {
      const float w = c_window[k], u = s_x[r][c + k], v = s_y[r][c + k];
      m1 += w * u, m2 += w * v, q11 += w * (u * u), q22 += w * (v * v), q12 += w * (u * v);
    }
    s_h[0][r][c] = m1, s_h[1][r][c] = m2, s_h[2][r][c] = q11, s_h[3][r][c] = q22, s_h[4][r][c] = q12;
  }
  __syncthreads();
  // along y, then the map
  float sum_map = 0, sum_l1 = 0;
  for (int e = threadIdx.x; e < kLT * kLT; e += kLThreads) {
    const int r = e / kLT, c = e - r * kLT;
    const int gy = ty0 + r, gx = tx0 + c;
    if (gy >= a.H || gx >= a.W) continue;
    float mu1 = 0, mu2 = 0, q11 = 0, q22 = 0, q12 = 0;
#pragma unroll
    for (int k = 0; k < kWin; ++k) {
      const float w = c_window[k];
      mu1 += w * s_h[0][r + k][c], mu2 += w * s_h[1][r + k][c], q11 += w * s_h[2][r + k][c];
      q22 += w * s_h[3][r + k][c], q12 += w * s_h[4][r + k][c];
    }
    const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2, mu12 = mu1 * mu2;
    const float s11 = q11 - mu1_sq, s22 = q22 - mu2_sq, s12 = q12 - mu12;
    const float A = mu1_sq + mu2_sq + a.C1, Bv = s11 + s22 + a.C2;
    const float Cv = 2.0f * mu12 + a.C1, D = 2.0f * s12 + a.C2;
    const float m = (Cv * D) / (A * Bv);
    const size_t p = off + (size_t) gy * a.W + gx;
    a.map[p] = m;
    if (a.d_mu1) {
      a.d_mu1[p] = (mu2 * 2.0f * D) / (A * Bv) - (mu2 * 2.0f * Cv) / (A * Bv) - (mu1 * 2.0f * Cv * D) / (A * A * Bv) +
                   (mu1 * 2.0f * Cv * D) / (A * Bv * Bv);
      a.d_s11[p] = (-Cv * D) / (A * Bv * Bv);
      a.d_s12[p] = (2.0f * Cv) / (A * Bv);
    }
    sum_map += m;
    sum_l1 += fabsf(s_x[r + kHalf][c + kHalf] - s_y[r + kHalf][c + kHalf]);
  }
  if (a.sums) {
    const float t0 = block_sum(sum_map, s_red);
    const float t1 = block_sum(sum_l1, s_red);
    if (threadIdx.x == 0) atomicAdd(a.sums, t0), atomicAdd(a.sums + 1, t1);
  }
}

struct SsimBwd {
  int B, C, H, W;
  const float *x, *y, *g_map;  // g_map may be null: then g_uniform everywhere
  float g_uniform, l1_weight;  // l1_weight * sign(x - y) is added to the result
  const float *d_mu1, *d_s11, *d_s12;
  float *g_x;
};

__global__ void __launch_bounds__(kLThreads) ssim_backward_kernel(SsimBwd a) {
  __shared__ float s_d[3][kLA][kLA + 1];
  __shared__ float s_h[3][kLA][kLT + 1];
  const int plane = blockIdx.z;
  const size_t off = (size_t) plane * a.H * a.W;
  const int tx0 = blockIdx.x * kLT, ty0 = blockIdx.y * kLT;
  for (int e = threadIdx.x; e < kLA * kLA; e += kLThreads) {
    const int r = e / kLA, c = e - r * kLA;
    const int gy = ty0 + r - kHalf, gx = tx0 + c - kHalf;
    float d0 = 0, d1 = 0, d2 = 0;
    if (gy >= 0 && gy < a.H && gx >= 0 && gx < a.W) {
      const size_t p = off + (size_t) gy * a.W + gx;
      const float g = a.g_map ? __ldg(a.g_map + p) : a.g_uniform;
      d0 = g * __ldg(a.d_mu1 + p), d1 = g * __ldg(a.d_s11 + p), d2 = g * __ldg(a.d_s12 + p);
    }
    s_d[0][r][c] = d0, s_d[1][r][c] = d1, s_d[2][r][c] = d2;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < kLA * kLT; e += kLThreads) {
    const int r = e / kLT, c = e - r * kLT;
    float t0 = 0, t1 = 0, t2 = 0;
#pragma unroll
    for (int k = 0; k < kWin; ++k) {
      const float w = c_window[k];
      t0 += w * s_d[0][r][c + k], t1 += w * s_d[1][r][c + k], t2 += w * s_d[2][r][c + k];
    }
    s_h[0][r][c] = t0, s_h[1][r][c] = t1, s_h[2][r][c] = t2;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < kLT * kLT; e += kLThreads) {
    const int r = e / kLT, c = e - r * kLT;
    const int gy = ty0 + r, gx = tx0 + c;
    if (gy >= a.H || gx >= a.W) continue;
    float t0 = 0, t1 = 0, t2 = 0;
#pragma unroll
    for (int k = 0; k < kWin; ++k) {
      const float w = c_window[k];
      t0 += w * s_h[0][r + k][c], t1 += w * s_h[1][r + k][c], t2 += w * s_h[2][r + k][c];
    }
    const size_t p = off + (size_t) gy * a.W + gx;
    const float xv = a.x[p], yv = a.y[p];
    float g = t0 + 2.0f * xv * t1 + yv * t2;
    if (a.l1_weight != 0.0f) g += a.l1_weight * (xv > yv ? 1.0f : (xv < yv ? -1.0f : 0.0f));
    a.g_x[p] = g;
  }
}

// The window of the reference (losses/ssim.py:12-14): exp(-(i-5)^2 / (2 * 1.5^2)) normalised, in float.
static int upload_window() {
  static bool done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FSGS_ERR_LAUNCH;
  if (done[dev]) return FSGS_OK;
  float w[kWin], sum = 0.0f;
  for (int i = 0; i < kWin; ++i) {
    w[i] = (float) exp(-(double) ((i - kHalf) * (i - kHalf)) / (2.0 * 1.5 * 1.5));
    sum += w[i];
  }
  for (int i = 0; i < kWin; ++i) w[i] /= sum;
  if (cudaMemcpyToSymbol(c_window, w, sizeof(w)) != cudaSuccess) return FSGS_ERR_LAUNCH;
  done[dev] = true;
  return FSGS_OK;
}

}  // namespace fsgs

using namespace fsgs;

extern "C" int fsgs_ssim_forward(int B, int C, int H, int W, float C1, float C2, const float *img1, const float *img2,
    float *ssim_map, float *dm_dmu1, float *dm_dsigma1_sq, float *dm_dsigma12, float *sums, fsgs_stream_t stream) {
  FSGS_REQUIRE(B >= 0 && C >= 0 && H >= 0 && W >= 0 && (size_t) B * C <= 65535);
  if ((size_t) B * C * H * W == 0) return FSGS_OK;
  FSGS_REQUIRE(img1 && img2 && ssim_map);
  FSGS_REQUIRE((dm_dmu1 && dm_dsigma1_sq && dm_dsigma12) || (!dm_dmu1 && !dm_dsigma1_sq && !dm_dsigma12));
  const int rc = upload_window();
  if (rc != FSGS_OK) return rc;
  SsimFwd a = {B, C, H, W, C1, C2, img1, img2, ssim_map, dm_dmu1, dm_dsigma1_sq, dm_dsigma12, sums};
  const dim3 grid(ceil_div(W, kLT), ceil_div(H, kLT), B * C);
  ssim_forward_kernel<<<grid, kLThreads, 0, (cudaStream_t) stream>>>(a);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_ssim_backward(int B, int C, int H, int W, float C1, float C2, const float *img1, const float *img2,
    const float *dL_dmap, float dL_dmap_uniform, float l1_weight, const float *dm_dmu1, const float *dm_dsigma1_sq,
    const float *dm_dsigma12, float *dL_dimg1, fsgs_stream_t stream) {
  (void) C1, (void) C2;
  FSGS_REQUIRE(B >= 0 && C >= 0 && H >= 0 && W >= 0 && (size_t) B * C <= 65535);
  if ((size_t) B * C * H * W == 0) return FSGS_OK;
  FSGS_REQUIRE(img1 && img2 && dm_dmu1 && dm_dsigma1_sq && dm_dsigma12 && dL_dimg1);
  const int rc = upload_window();
  if (rc != FSGS_OK) return rc;
  SsimBwd a = {B, C, H, W, img1, img2, dL_dmap, dL_dmap_uniform, l1_weight, dm_dmu1, dm_dsigma1_sq, dm_dsigma12, dL_dimg1};
  const dim3 grid(ceil_div(W, kLT), ceil_div(H, kLT), B * C);
  ssim_backward_kernel<<<grid, kLThreads, 0, (cudaStream_t) stream>>>(a);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}
