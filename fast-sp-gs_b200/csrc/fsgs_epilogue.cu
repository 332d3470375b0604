// Per-pixel epilogue of GS_2D_fast_render in one kernel each way: normals to world space, the expected /
// median depth blend with non-finite values zeroed, and the pseudo surface normal of the back-projected depth
// map (reference renderer/gs_2d_fast_render.py:558-589, 731-740, a chain of ~25 PyTorch kernels there).
#include "fsgs_common.cuh"

namespace fsgs {

struct EpiCam {
  float R[9];    // Tw2v[:3,:3]
  float K[9];    // pixel (x, y, 1) -> world ray direction: inv(intrinsics)^T * c2w[:3,:3]^T
  float o[3];    // camera position
};

__device__ __forceinline__ void inv3(const float *m, float *out) {
  const float c0 = m[4] * m[8] - m[5] * m[7], c1 = m[5] * m[6] - m[3] * m[8], c2 = m[3] * m[7] - m[4] * m[6];
  const float inv_det = 1.0f / (m[0] * c0 + m[1] * c1 + m[2] * c2);
  out[0] = c0 * inv_det, out[1] = (m[2] * m[7] - m[1] * m[8]) * inv_det, out[2] = (m[1] * m[5] - m[2] * m[4]) * inv_det;
  out[3] = c1 * inv_det, out[4] = (m[0] * m[8] - m[2] * m[6]) * inv_det, out[5] = (m[2] * m[3] - m[0] * m[5]) * inv_det;
  out[6] = c2 * inv_det, out[7] = (m[1] * m[6] - m[0] * m[7]) * inv_det, out[8] = (m[0] * m[4] - m[1] * m[3]) * inv_det;
}

// Thread 0 of every block derives the three small matrices from the two camera matrices.
__device__ __forceinline__ void make_cam(const float *__restrict__ Tw2v, const float *__restrict__ Tv2c, int W, int H,
    EpiCam &c) {
  float R[9], Ri[9];
  for (int i = 0; i < 3; ++i)
    for (int j = 0; j < 3; ++j) R[i * 3 + j] = Tw2v[i * 4 + j];
  inv3(R, Ri);  // rotation part of the view-to-world matrix
  for (int i = 0; i < 9; ++i) c.R[i] = R[i];
  for (int i = 0; i < 3; ++i) c.o[i] = -(Ri[i * 3] * Tw2v[3] + Ri[i * 3 + 1] * Tw2v[7] + Ri[i * 3 + 2] * Tw2v[11]);
  // intrinsics = ([[W/2,0,0,W/2],[0,H/2,0,H/2],[0,0,0,1]] * Tv2c)[:, :3]
  float In[9], Ii[9];
  for (int b = 0; b < 3; ++b) {
    In[0 * 3 + b] = 0.5f * W * Tv2c[0 * 4 + b] + 0.5f * W * Tv2c[3 * 4 + b];
    In[1 * 3 + b] = 0.5f * H * Tv2c[1 * 4 + b] + 0.5f * H * Tv2c[3 * 4 + b];
    In[2 * 3 + b] = Tv2c[3 * 4 + b];
  }
  inv3(In, Ii);
  for (int a = 0; a < 3; ++a)
    for (int j = 0; j < 3; ++j)
      c.K[a * 3 + j] = Ii[0 * 3 + a] * Ri[j * 3 + 0] + Ii[1 * 3 + a] * Ri[j * 3 + 1] + Ii[2 * 3 + a] * Ri[j * 3 + 2];
}

__device__ __forceinline__ float zero_nonfinite(float v) {
  // torch.nan_to_num(v, 0, 0): nan -> 0, +inf -> 0, -inf -> lowest finite
  if (v != v || v == __int_as_float(0x7f800000)) return 0.0f;
  if (v == __int_as_float(0xff800000)) return -3.4028234663852886e38f;
  return v;
}

__device__ __forceinline__ float surf_depth_at(const float *__restrict__ extras, size_t HW, size_t pix, float ratio) {
  return zero_nonfinite(extras[pix]) * (1.0f - ratio) + ratio * zero_nonfinite(extras[4 * HW + pix]);
}

__device__ __forceinline__ float3 ray_dir(const EpiCam &c, int x, int y) {
  const float fx = (float) x, fy = (float) y;
  return make_float3(fx * c.K[0] + fy * c.K[3] + c.K[6], fx * c.K[1] + fy * c.K[4] + c.K[7],
      fx * c.K[2] + fy * c.K[5] + c.K[8]);
}

__device__ __forceinline__ float3 world_point(const EpiCam &c, int x, int y, float d) {
  const float3 r = ray_dir(c, x, y);
  return make_float3(d * r.x + c.o[0], d * r.y + c.o[1], d * r.z + c.o[2]);
}

__device__ __forceinline__ float3 sub3(float3 a, float3 b) { return make_float3(a.x - b.x, a.y - b.y, a.z - b.z); }
__device__ __forceinline__ float3 crs3(float3 a, float3 b) {
  return make_float3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}

__global__ void __launch_bounds__(256) epilogue_forward_kernel(int W, int H, float ratio, const float *__restrict__ Tw2v,
    const float *__restrict__ Tv2c, const float *__restrict__ extras, const float *__restrict__ opacity,
    float *__restrict__ normals_world, float *__restrict__ surf_depth, float *__restrict__ surf_normal) {
  __shared__ EpiCam cam;
  if (threadIdx.x == 0 && threadIdx.y == 0) make_cam(Tw2v, Tv2c, W, H, cam);
  __syncthreads();
  const int x = blockIdx.x * blockDim.x + threadIdx.x, y = blockIdx.y * blockDim.y + threadIdx.y;
  if (x >= W || y >= H) return;
  const size_t HW = (size_t) H * W, pix = (size_t) y * W + x;
  const float n0 = extras[HW + pix], n1 = extras[2 * HW + pix], n2 = extras[3 * HW + pix];
  normals_world[pix] = n0 * cam.R[0] + n1 * cam.R[3] + n2 * cam.R[6];
  normals_world[HW + pix] = n0 * cam.R[1] + n1 * cam.R[4] + n2 * cam.R[7];
  normals_world[2 * HW + pix] = n0 * cam.R[2] + n1 * cam.R[5] + n2 * cam.R[8];
  surf_depth[pix] = surf_depth_at(extras, HW, pix, ratio);
  float3 n = make_float3(0, 0, 0);
  if (x >= 1 && x <= W - 2 && y >= 1 && y <= H - 2) {
    const float3 pu = world_point(cam, x, y - 1, surf_depth_at(extras, HW, pix - W, ratio));
    const float3 pd = world_point(cam, x, y + 1, surf_depth_at(extras, HW, pix + W, ratio));
    const float3 pl = world_point(cam, x - 1, y, surf_depth_at(extras, HW, pix - 1, ratio));
    const float3 pr = world_point(cam, x + 1, y, surf_depth_at(extras, HW, pix + 1, ratio));
    const float3 c = crs3(sub3(pd, pu), sub3(pr, pl));
    const float inv = 1.0f / fmaxf(sqrtf(c.x * c.x + c.y * c.y + c.z * c.z), 1e-12f);
    const float o = opacity[pix];
    n = make_float3(c.x * inv * o, c.y * inv * o, c.z * inv * o);
  }
  surf_normal[pix] = n.x, surf_normal[HW + pix] = n.y, surf_normal[2 * HW + pix] = n.z;
}

// Gradients of the cross product's two arguments at centre pixel (x, y): dL/d(dx), dL/d(dy) with
// dx = P(y+1) - P(y-1), dy = P(x+1) - P(x-1).  Zero outside the interior.
__device__ __forceinline__ void centre_grads(const EpiCam &cam, int W, int H, float ratio, const float *__restrict__ extras,
    const float *__restrict__ opacity, const float *__restrict__ g_sn, int x, int y, float3 &g_dx, float3 &g_dy) {
  g_dx = g_dy = make_float3(0, 0, 0);
  if (x < 1 || x > W - 2 || y < 1 || y > H - 2) return;
  const size_t HW = (size_t) H * W, pix = (size_t) y * W + x;
  const float3 dx = sub3(world_point(cam, x, y + 1, surf_depth_at(extras, HW, pix + W, ratio)),
      world_point(cam, x, y - 1, surf_depth_at(extras, HW, pix - W, ratio)));
  const float3 dy = sub3(world_point(cam, x + 1, y, surf_depth_at(extras, HW, pix + 1, ratio)),
      world_point(cam, x - 1, y, surf_depth_at(extras, HW, pix - 1, ratio)));
  const float3 c = crs3(dx, dy);
  const float len = sqrtf(c.x * c.x + c.y * c.y + c.z * c.z);
  const float o = opacity[pix];
  const float3 gn = make_float3(g_sn[pix] * o, g_sn[HW + pix] * o, g_sn[2 * HW + pix] * o);
  float3 gc;
  if (len > 1e-12f) {
    const float inv = 1.0f / len;
    const float3 n = make_float3(c.x * inv, c.y * inv, c.z * inv);
    const float d = n.x * gn.x + n.y * gn.y + n.z * gn.z;
    gc = make_float3((gn.x - n.x * d) * inv, (gn.y - n.y * d) * inv, (gn.z - n.z * d) * inv);
  } else {
    gc = make_float3(gn.x * 1e12f, gn.y * 1e12f, gn.z * 1e12f);  // v / eps branch of the clamped normalisation
  }
  g_dx = crs3(dy, gc);
  g_dy = crs3(gc, dx);
}

__global__ void __launch_bounds__(256) epilogue_backward_kernel(int W, int H, float ratio, const float *__restrict__ Tw2v,
    const float *__restrict__ Tv2c, const float *__restrict__ extras, const float *__restrict__ opacity,
    const float *__restrict__ g_nw, const float *__restrict__ g_sd, const float *__restrict__ g_sn,
    float *__restrict__ g_extras) {
  __shared__ EpiCam cam;
  if (threadIdx.x == 0 && threadIdx.y == 0) make_cam(Tw2v, Tv2c, W, H, cam);
  __syncthreads();
  const int x = blockIdx.x * blockDim.x + threadIdx.x, y = blockIdx.y * blockDim.y + threadIdx.y;
  if (x >= W || y >= H) return;
  const size_t HW = (size_t) H * W, pix = (size_t) y * W + x;
  float gN[3] = {0, 0, 0};
  if (g_nw) {
    const float a = g_nw[pix], b = g_nw[HW + pix], c = g_nw[2 * HW + pix];
    gN[0] = a * cam.R[0] + b * cam.R[1] + c * cam.R[2];
    gN[1] = a * cam.R[3] + b * cam.R[4] + c * cam.R[5];
    gN[2] = a * cam.R[6] + b * cam.R[7] + c * cam.R[8];
  }
  float gd = g_sd ? g_sd[pix] : 0.0f;
  if (g_sn) {
    // this pixel is the lower / upper / right / left neighbour of up to four interior centres
    float3 gp = make_float3(0, 0, 0), a, b;
    centre_grads(cam, W, H, ratio, extras, opacity, g_sn, x, y - 1, a, b);
    gp.x += a.x, gp.y += a.y, gp.z += a.z;
    centre_grads(cam, W, H, ratio, extras, opacity, g_sn, x, y + 1, a, b);
    gp.x -= a.x, gp.y -= a.y, gp.z -= a.z;
    centre_grads(cam, W, H, ratio, extras, opacity, g_sn, x - 1, y, a, b);
    gp.x += b.x, gp.y += b.y, gp.z += b.z;
    centre_grads(cam, W, H, ratio, extras, opacity, g_sn, x + 1, y, a, b);
    gp.x -= b.x, gp.y -= b.y, gp.z -= b.z;
    const float3 r = ray_dir(cam, x, y);
    gd += gp.x * r.x + gp.y * r.y + gp.z * r.z;
  }
  const float D = extras[pix], Dm = extras[4 * HW + pix];
  const bool fD = D == D && fabsf(D) != __int_as_float(0x7f800000);
  const bool fM = Dm == Dm && fabsf(Dm) != __int_as_float(0x7f800000);
  g_extras[pix] = fD ? gd * (1.0f - ratio) : 0.0f;
  g_extras[HW + pix] = gN[0], g_extras[2 * HW + pix] = gN[1], g_extras[3 * HW + pix] = gN[2];
  g_extras[4 * HW + pix] = fM ? gd * ratio : 0.0f;
  g_extras[5 * HW + pix] = 0.0f, g_extras[6 * HW + pix] = 0.0f, g_extras[7 * HW + pix] = 0.0f;
}

}  // namespace fsgs

using namespace fsgs;

extern "C" int fsgs_epilogue_forward(int W, int H, float depth_ratio, const float *Tw2v, const float *Tv2c,
    const float *out_extras, const float *out_opacity, float *normals_world, float *surf_depth, float *surf_normal,
    fsgs_stream_t stream) {
  FSGS_REQUIRE(W > 0 && H > 0 && Tw2v && Tv2c && out_extras && out_opacity && normals_world && surf_depth && surf_normal);
  const dim3 block(32, 8), grid(ceil_div(W, 32), ceil_div(H, 8));
  epilogue_forward_kernel<<<grid, block, 0, (cudaStream_t) stream>>>(W, H, depth_ratio, Tw2v, Tv2c, out_extras,
      out_opacity, normals_world, surf_depth, surf_normal);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_epilogue_backward(int W, int H, float depth_ratio, const float *Tw2v, const float *Tv2c,
    const float *out_extras, const float *out_opacity, const float *g_normals_world, const float *g_surf_depth,
    const float *g_surf_normal, float *g_extras, fsgs_stream_t stream) {
  FSGS_REQUIRE(W > 0 && H > 0 && Tw2v && Tv2c && out_extras && out_opacity && g_extras);
  const dim3 block(32, 8), grid(ceil_div(W, 32), ceil_div(H, 8));
  epilogue_backward_kernel<<<grid, block, 0, (cudaStream_t) stream>>>(W, H, depth_ratio, Tw2v, Tv2c, out_extras,
      out_opacity, g_normals_world, g_surf_depth, g_surf_normal, g_extras);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}
