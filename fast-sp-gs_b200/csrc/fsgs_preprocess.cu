// Per-Gaussian stages of the surfel renderer: LBS warp, projection (splat->screen matrix, bounds, SH colour),
// their adjoints, and the packed render record.  One thread per Gaussian; every kernel is HBM bound.
#include "fsgs_common.cuh"
#include "fsgs_sh.cuh"
#include "fsgs_tma.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace fsgs {

// ------------------------------------------------------------------------------------------------
// LBS warp
// ------------------------------------------------------------------------------------------------

struct LbsDev {
  int K, M;
  const float *xyz, *scaling_raw, *rotation_raw;
  const int64_t *knn_idx;
  const float *knn_w;
  const float4 *sp_q;
  const float *sp_t;
  const float4 *sp_dr;
  const float2 *sp_ds;
  const int32_t *pair_offsets, *pairs;  // optional: pairs grouped by superpoint
};

static LbsDev to_dev(const fsgs_lbs *l) {
  LbsDev d;
  d.K = l->K, d.M = l->M;
  d.xyz = l->xyz, d.scaling_raw = l->scaling_raw, d.rotation_raw = l->rotation_raw;
  d.knn_idx = l->knn_idx, d.knn_w = l->knn_w;
  d.sp_q = (const float4 *) l->sp_q, d.sp_t = l->sp_t;
  d.sp_dr = (const float4 *) l->sp_dr, d.sp_ds = (const float2 *) l->sp_ds;
  d.pair_offsets = l->sp_pair_offsets, d.pairs = l->sp_pairs;
  return d;
}

static bool lbs_valid(const fsgs_lbs *l) {
  return l->K > 0 && l->K <= FSGS_KNN_MAX_K && l->M > 0 && l->xyz && l->scaling_raw && l->rotation_raw &&
         l->knn_idx && l->knn_w && l->sp_q && l->sp_t && l->sp_dr && l->sp_ds;
}

__device__ __forceinline__ float3 quat_rotate(const float4 q, const float3 p) {
  const float r00 = 1 - 2 * (q.y * q.y + q.z * q.z), r01 = 2 * (q.x * q.y - q.z * q.w), r02 = 2 * (q.y * q.w + q.x * q.z);
  const float r10 = 2 * (q.x * q.y + q.z * q.w), r11 = 1 - 2 * (q.x * q.x + q.z * q.z), r12 = 2 * (q.y * q.z - q.x * q.w);
  const float r20 = 2 * (q.x * q.z - q.y * q.w), r21 = 2 * (q.x * q.w + q.y * q.z), r22 = 1 - 2 * (q.x * q.x + q.y * q.y);
  return make_float3(r00 * p.x + r01 * p.y + r02 * p.z, r10 * p.x + r11 * p.y + r12 * p.z,
      r20 * p.x + r21 * p.y + r22 * p.z);
}

__device__ __forceinline__ float3 quat_rotate_T(const float4 q, const float3 p) {
  return quat_rotate(make_float4(-q.x, -q.y, -q.z, q.w), p);
}

// Adjoint of q -> R(q) given dL/dR (row major 3x3).  (reference include/ops_3d.h:126-134)
__device__ __forceinline__ float4 quat_adjoint(const float4 q, const float *dR) {
  float4 g;
  g.x = 2 * (-2 * q.x * (dR[4] + dR[8]) + q.y * (dR[1] + dR[3]) + q.z * (dR[2] + dR[6]) + q.w * (dR[7] - dR[5]));
  g.y = 2 * (q.x * (dR[1] + dR[3]) - 2 * q.y * (dR[0] + dR[8]) + q.z * (dR[5] + dR[7]) + q.w * (dR[2] - dR[6]));
  g.z = 2 * (q.x * (dR[2] + dR[6]) + q.y * (dR[5] + dR[7]) - 2 * q.z * (dR[0] + dR[4]) + q.w * (dR[3] - dR[1]));
  g.w = 2 * (q.x * (dR[7] - dR[5]) + q.y * (dR[2] - dR[6]) + q.z * (dR[3] - dR[1]));
  return g;
}

__device__ __forceinline__ void lbs_warp_one(const LbsDev &l, int i, float3 &mean, float2 &scale, float4 &rot) {
  const float3 p = make_float3(l.xyz[3 * i], l.xyz[3 * i + 1], l.xyz[3 * i + 2]);
  // issued before the gathers below so that their latency overlaps
  const float ls0 = __ldg(l.scaling_raw + 2 * i), ls1 = __ldg(l.scaling_raw + 2 * i + 1);
  const float4 r0 = __ldg(reinterpret_cast<const float4 *>(l.rotation_raw) + i);
  float3 acc = make_float3(0, 0, 0);
  float4 dr = make_float4(0, 0, 0, 0);
  float2 ds = make_float2(0, 0);
  for (int k = 0; k < l.K; ++k) {
    const int m = (int) l.knn_idx[(size_t) i * l.K + k];
    const float w = l.knn_w[(size_t) i * l.K + k];
    const float4 q = __ldg(l.sp_q + m);
    const float3 r = quat_rotate(q, p);
    acc.x += (r.x + __ldg(l.sp_t + 3 * m + 0)) * w;
    acc.y += (r.y + __ldg(l.sp_t + 3 * m + 1)) * w;
    acc.z += (r.z + __ldg(l.sp_t + 3 * m + 2)) * w;
    const float4 a = __ldg(l.sp_dr + m);
    dr.x += a.x * w, dr.y += a.y * w, dr.z += a.z * w, dr.w += a.w * w;
    const float2 b = __ldg(l.sp_ds + m);
    ds.x += b.x * w, ds.y += b.y * w;
  }
  mean = make_float3(p.x + (acc.x - p.x), p.y + (acc.y - p.y), p.z + (acc.z - p.z));
  scale = make_float2(expf(ls0) + ds.x, expf(ls1) + ds.y);
  const float4 r = make_float4(r0.x + dr.x, r0.y + dr.y, r0.z + dr.z, r0.w + dr.w);
  const float inv = 1.0f / fmaxf(sqrtf(r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w), 1e-12f);
  rot = make_float4(r.x * inv, r.y * inv, r.z * inv, r.w * inv);
}

__global__ void __launch_bounds__(256) lbs_warp_forward_kernel(int P, LbsDev l, float *__restrict__ means,
    float2 *__restrict__ scales, float4 *__restrict__ rots) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  float3 m;
  float2 s;
  float4 q;
  lbs_warp_one(l, i, m, s, q);
  means[3 * i] = m.x, means[3 * i + 1] = m.y, means[3 * i + 2] = m.z;
  scales[i] = s;
  rots[i] = q;
}

__device__ __forceinline__ void red_add_v4(float *p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void red_add_v2(float *p, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(a), "f"(b) : "memory");
}

// Superpoint gradient table row: q(4) t(3) dr(4) ds(2) = 13 floats.
constexpr int kSpRow = 13;
constexpr int kLbsCluster = 8;  // blocks per cluster in the backward (portable maximum)

template <bool SMEM_TABLE>
__global__ void __launch_bounds__(256) lbs_warp_backward_kernel(int P, LbsDev l, const float *__restrict__ g_means,
    const float2 *__restrict__ g_scales, const float4 *__restrict__ g_rots, float *__restrict__ g_xyz,
    float2 *__restrict__ g_scaling_raw, float4 *__restrict__ g_rotation_raw, float *__restrict__ g_knn_w,
    float *__restrict__ g_sp_q, float *__restrict__ g_sp_t, float *__restrict__ g_sp_dr, float *__restrict__ g_sp_ds) {
  extern __shared__ float table[];  // [M, 13] when SMEM_TABLE
  if (SMEM_TABLE) {
    for (int k = threadIdx.x; k < l.M * kSpRow; k += blockDim.x) table[k] = 0.0f;
    __syncthreads();
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < P; i += gridDim.x * blockDim.x) {
    const float3 p = make_float3(l.xyz[3 * i], l.xyz[3 * i + 1], l.xyz[3 * i + 2]);
    const float3 gm = make_float3(g_means[3 * i], g_means[3 * i + 1], g_means[3 * i + 2]);
    const float2 gs = g_scales[i];
    // adjoint of the quaternion normalisation
    float4 dr = make_float4(0, 0, 0, 0);
    for (int k = 0; k < l.K; ++k) {
      const int m = (int) l.knn_idx[(size_t) i * l.K + k];
      const float w = l.knn_w[(size_t) i * l.K + k];
      const float4 a = __ldg(l.sp_dr + m);
      dr.x += a.x * w, dr.y += a.y * w, dr.z += a.z * w, dr.w += a.w * w;
    }
    const float4 r0 = reinterpret_cast<const float4 *>(l.rotation_raw)[i];
    const float4 r = make_float4(r0.x + dr.x, r0.y + dr.y, r0.z + dr.z, r0.w + dr.w);
    const float nrm = fmaxf(sqrtf(r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w), 1e-12f);
    const float inv = 1.0f / nrm;
    const float4 y = make_float4(r.x * inv, r.y * inv, r.z * inv, r.w * inv);
    const float4 gy = g_rots[i];
    const float yd = y.x * gy.x + y.y * gy.y + y.z * gy.z + y.w * gy.w;
    const float4 gr = make_float4((gy.x - y.x * yd) * inv, (gy.y - y.y * yd) * inv, (gy.z - y.z * yd) * inv,
        (gy.w - y.w * yd) * inv);
    g_rotation_raw[i] = gr;
    g_scaling_raw[i] = make_float2(gs.x * expf(l.scaling_raw[2 * i]), gs.y * expf(l.scaling_raw[2 * i + 1]));

    float3 gx = make_float3(0, 0, 0);
    for (int k = 0; k < l.K; ++k) {
      const int m = (int) l.knn_idx[(size_t) i * l.K + k];
      const float w = l.knn_w[(size_t) i * l.K + k];
      const float4 q = __ldg(l.sp_q + m);
      const float3 rp = quat_rotate(q, p);
      const float3 moved = make_float3(rp.x + __ldg(l.sp_t + 3 * m), rp.y + __ldg(l.sp_t + 3 * m + 1),
          rp.z + __ldg(l.sp_t + 3 * m + 2));
      const float4 a = __ldg(l.sp_dr + m);
      const float2 b = __ldg(l.sp_ds + m);
      g_knn_w[(size_t) i * l.K + k] = gm.x * moved.x + gm.y * moved.y + gm.z * moved.z +
                                      (gr.x * a.x + gr.y * a.y + gr.z * a.z + gr.w * a.w) + (gs.x * b.x + gs.y * b.y);
      const float3 back = quat_rotate_T(q, gm);
      gx.x += w * back.x, gx.y += w * back.y, gx.z += w * back.z;
      // dL/dR = w * gm (outer) p
      float dR[9];
      dR[0] = w * gm.x * p.x, dR[1] = w * gm.x * p.y, dR[2] = w * gm.x * p.z;
      dR[3] = w * gm.y * p.x, dR[4] = w * gm.y * p.y, dR[5] = w * gm.y * p.z;
      dR[6] = w * gm.z * p.x, dR[7] = w * gm.z * p.y, dR[8] = w * gm.z * p.z;
      const float4 gq = quat_adjoint(q, dR);
      const float row[kSpRow] = {gq.x, gq.y, gq.z, gq.w, w * gm.x, w * gm.y, w * gm.z, w * gr.x, w * gr.y, w * gr.z,
          w * gr.w, w * gs.x, w * gs.y};
      if (SMEM_TABLE) {
#pragma unroll
        for (int c = 0; c < kSpRow; ++c) atomicAdd(table + m * kSpRow + c, row[c]);
      } else {
        // vector reductions in L2: the [M,4] and [M,2] rows are 16- and 8-byte aligned
        red_add_v4(g_sp_q + 4 * m, row[0], row[1], row[2], row[3]);
#pragma unroll
        for (int c = 0; c < 3; ++c) atomicAdd(g_sp_t + 3 * m + c, row[4 + c]);
        red_add_v4(g_sp_dr + 4 * m, row[7], row[8], row[9], row[10]);
        red_add_v2(g_sp_ds + 2 * m, row[11], row[12]);
      }
    }
    g_xyz[3 * i] = gx.x, g_xyz[3 * i + 1] = gx.y, g_xyz[3 * i + 2] = gx.z;
  }
  if (SMEM_TABLE) {
    // The blocks of a cluster add their tables up through distributed shared memory, each block taking one slice
    // of the rows, so that global memory sees one reduction per (cluster, entry) instead of one per (block, entry).
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int nr = (int) cluster.num_blocks(), len = l.M * kSpRow;
    const int per = (len + nr - 1) / nr, lo = (int) cluster.block_rank() * per, hi = min(len, lo + per);
    for (int k = lo + threadIdx.x; k < hi; k += blockDim.x) {
      float v = 0.0f;
      for (int r = 0; r < nr; ++r) v += cluster.map_shared_rank(table, r)[k];
      if (v == 0.0f) continue;
      const int m = k / kSpRow, c = k % kSpRow;
      if (c < 4) atomicAdd(g_sp_q + 4 * m + c, v);
      else if (c < 7) atomicAdd(g_sp_t + 3 * m + (c - 4), v);
      else if (c < 11) atomicAdd(g_sp_dr + 4 * m + (c - 7), v);
      else atomicAdd(g_sp_ds + 2 * m + (c - 11), v);
    }
    cluster.sync();  // no block leaves while its table may still be read
  }
}

// The same adjoint without atomics, for callers that supply the (Gaussian, neighbour) pairs grouped by superpoint
// (offsets [M+1] and pair ids i*K + k, built once per k-NN refresh).  Pass 1: one thread per Gaussian writes the
// per-Gaussian gradients.  Pass 2: one block per superpoint walks its pairs, every thread sums its share of
//   S_R = sum w (g_mean (x) p)   S_t = sum w g_mean   S_dr = sum w g_rot_raw   S_ds = sum w g_scale
// (the quaternion adjoint is linear in dL/dR, so it is applied once to S_R), the block adds the partial sums up and
// writes the superpoint's row: every output written exactly once, in a fixed order -- bit-reproducible.
// With `scratch_rot` the rotation gradient of this view goes there (pass 2 reads it) and, like the other per-Gaussian
// outputs, is ADDED to what g_* already hold (several views accumulated into one gradient).
template <bool ACC>
__global__ void __launch_bounds__(256) lbs_backward_points_kernel(int P, LbsDev l, const float *__restrict__ g_means,
    const float2 *__restrict__ g_scales, const float4 *__restrict__ g_rots, float *__restrict__ g_xyz,
    float2 *__restrict__ g_scaling_raw, float4 *__restrict__ g_rotation_raw, float *__restrict__ g_knn_w,
    float4 *__restrict__ scratch_rot) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const float3 p = make_float3(l.xyz[3 * i], l.xyz[3 * i + 1], l.xyz[3 * i + 2]);
  const float3 gm = make_float3(g_means[3 * i], g_means[3 * i + 1], g_means[3 * i + 2]);
  const float2 gs = g_scales[i];
  float4 dr = make_float4(0, 0, 0, 0);
  for (int k = 0; k < l.K; ++k) {
    const int m = (int) l.knn_idx[(size_t) i * l.K + k];
    const float w = l.knn_w[(size_t) i * l.K + k];
    const float4 a = __ldg(l.sp_dr + m);
    dr.x += a.x * w, dr.y += a.y * w, dr.z += a.z * w, dr.w += a.w * w;
  }
  const float4 r0 = reinterpret_cast<const float4 *>(l.rotation_raw)[i];
  const float4 r = make_float4(r0.x + dr.x, r0.y + dr.y, r0.z + dr.z, r0.w + dr.w);
  const float nrm = fmaxf(sqrtf(r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w), 1e-12f);
  const float inv = 1.0f / nrm;
  const float4 y = make_float4(r.x * inv, r.y * inv, r.z * inv, r.w * inv);
  const float4 gy = g_rots[i];
  const float yd = y.x * gy.x + y.y * gy.y + y.z * gy.z + y.w * gy.w;
  const float4 gr = make_float4((gy.x - y.x * yd) * inv, (gy.y - y.y * yd) * inv, (gy.z - y.z * yd) * inv,
      (gy.w - y.w * yd) * inv);
  const float2 gsr = make_float2(gs.x * expf(l.scaling_raw[2 * i]), gs.y * expf(l.scaling_raw[2 * i + 1]));
  if (ACC) {
    scratch_rot[i] = gr;
    const float4 o = g_rotation_raw[i];
    g_rotation_raw[i] = make_float4(o.x + gr.x, o.y + gr.y, o.z + gr.z, o.w + gr.w);
    const float2 os = g_scaling_raw[i];
    g_scaling_raw[i] = make_float2(os.x + gsr.x, os.y + gsr.y);
  } else {
    g_rotation_raw[i] = gr;
    g_scaling_raw[i] = gsr;
  }
  float3 gx = make_float3(0, 0, 0);
  for (int k = 0; k < l.K; ++k) {
    const int m = (int) l.knn_idx[(size_t) i * l.K + k];
    const float w = l.knn_w[(size_t) i * l.K + k];
    const float4 q = __ldg(l.sp_q + m);
    const float3 rp = quat_rotate(q, p);
    const float3 moved = make_float3(rp.x + __ldg(l.sp_t + 3 * m), rp.y + __ldg(l.sp_t + 3 * m + 1),
        rp.z + __ldg(l.sp_t + 3 * m + 2));
    const float4 a = __ldg(l.sp_dr + m);
    const float2 b = __ldg(l.sp_ds + m);
    const float gw = gm.x * moved.x + gm.y * moved.y + gm.z * moved.z +
                     (gr.x * a.x + gr.y * a.y + gr.z * a.z + gr.w * a.w) + (gs.x * b.x + gs.y * b.y);
    if (ACC) g_knn_w[(size_t) i * l.K + k] += gw;
    else g_knn_w[(size_t) i * l.K + k] = gw;
    const float3 back = quat_rotate_T(q, gm);
    gx.x += w * back.x, gx.y += w * back.y, gx.z += w * back.z;
  }
  if (ACC) g_xyz[3 * i] += gx.x, g_xyz[3 * i + 1] += gx.y, g_xyz[3 * i + 2] += gx.z;
  else g_xyz[3 * i] = gx.x, g_xyz[3 * i + 1] = gx.y, g_xyz[3 * i + 2] = gx.z;
}

constexpr int kSpSums = 18;
// kSpThreads threads per superpoint: many when there are few superpoints (few blocks would leave the GPU idle), fewer
// when there are thousands (the block reduction then weighs more than the latency it hides)
template <int kSpThreads, bool ACC>
__global__ void __launch_bounds__(kSpThreads) lbs_backward_superpoints_kernel(LbsDev l,
    const int32_t *__restrict__ offsets, const int32_t *__restrict__ pairs, const float *__restrict__ g_means,
    const float2 *__restrict__ g_scales, const float4 *__restrict__ g_rotation_raw, float *__restrict__ g_sp_q,
    float *__restrict__ g_sp_t, float *__restrict__ g_sp_dr, float *__restrict__ g_sp_ds) {
  __shared__ float s_part[kSpThreads / 32][kSpSums];
  const int m = blockIdx.x;
  const int lo = offsets[m], hi = offsets[m + 1];
  float acc[kSpSums];
#pragma unroll
  for (int c = 0; c < kSpSums; ++c) acc[c] = 0.0f;
  for (int e = lo + threadIdx.x; e < hi; e += kSpThreads) {
    const int pair = pairs[e];
    const int i = pair / l.K;
    const float w = l.knn_w[pair];
    const float3 p = make_float3(l.xyz[3 * i], l.xyz[3 * i + 1], l.xyz[3 * i + 2]);
    const float3 gm = make_float3(w * g_means[3 * i], w * g_means[3 * i + 1], w * g_means[3 * i + 2]);
    const float4 gr = g_rotation_raw[i];
    const float2 gs = g_scales[i];
    acc[0] += gm.x * p.x, acc[1] += gm.x * p.y, acc[2] += gm.x * p.z;
    acc[3] += gm.y * p.x, acc[4] += gm.y * p.y, acc[5] += gm.y * p.z;
    acc[6] += gm.z * p.x, acc[7] += gm.z * p.y, acc[8] += gm.z * p.z;
    acc[9] += gm.x, acc[10] += gm.y, acc[11] += gm.z;
    acc[12] += w * gr.x, acc[13] += w * gr.y, acc[14] += w * gr.z, acc[15] += w * gr.w;
    acc[16] += w * gs.x, acc[17] += w * gs.y;
  }
#pragma unroll
  for (int c = 0; c < kSpSums; ++c)
    for (int o = 16; o > 0; o >>= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int c = 0; c < kSpSums; ++c) s_part[threadIdx.x >> 5][c] = acc[c];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float t[kSpSums];
#pragma unroll
    for (int c = 0; c < kSpSums; ++c) {
      t[c] = 0.0f;
      for (int w = 0; w < kSpThreads / 32; ++w) t[c] += s_part[w][c];
    }
    float4 gq = quat_adjoint(l.sp_q[m], t);
    if (ACC) {  // this block is the only writer of row m: a plain read-modify-write
      const float4 oq = reinterpret_cast<float4 *>(g_sp_q)[m], od = reinterpret_cast<float4 *>(g_sp_dr)[m];
      const float2 os = reinterpret_cast<float2 *>(g_sp_ds)[m];
      gq = make_float4(gq.x + oq.x, gq.y + oq.y, gq.z + oq.z, gq.w + oq.w);
      t[9] += g_sp_t[3 * m], t[10] += g_sp_t[3 * m + 1], t[11] += g_sp_t[3 * m + 2];
      t[12] += od.x, t[13] += od.y, t[14] += od.z, t[15] += od.w;
      t[16] += os.x, t[17] += os.y;
    }
    reinterpret_cast<float4 *>(g_sp_q)[m] = gq;
    g_sp_t[3 * m] = t[9], g_sp_t[3 * m + 1] = t[10], g_sp_t[3 * m + 2] = t[11];
    reinterpret_cast<float4 *>(g_sp_dr)[m] = make_float4(t[12], t[13], t[14], t[15]);
    reinterpret_cast<float2 *>(g_sp_ds)[m] = make_float2(t[16], t[17]);
  }
}

// ------------------------------------------------------------------------------------------------
// preprocess forward
// ------------------------------------------------------------------------------------------------

struct PreDev {
  int P, W, H, sh_degree, n_dc, n_rest, gx, gy;
  const float *means;
  const float2 *scales;
  const float4 *rots;
  const float *opac, *shs, *sh_rest, *Tw2v, *Tv2s, *campos, *trans_precomp;
  const uint8_t *culling;
  float *warped_means;
  float2 *warped_scales;
  float4 *warped_rots;
  float2 *means2D;
  float *colors, *trans_mat, *inverse_m;
  float4 *normal_opacity;
  float *depths;
  int32_t *radii, *tiles_touched;
  float4 *records;
  int32_t *tile_counts;
  unsigned long long *counters;
  int opacity_is_logit;
};

// sigmoid in the operation order of the framework's own CUDA kernel (1 / (1 + exp(-x)) in float)
__device__ __forceinline__ float sigmoid_f32(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }

__device__ __forceinline__ const float *sh_coef(const PreDev &a, int i, int k) {
  if (a.sh_rest == nullptr) return a.shs + ((size_t) i * a.n_dc + k) * 3;
  return k == 0 ? a.shs + (size_t) i * a.n_dc * 3 : a.sh_rest + ((size_t) i * a.n_rest + (k - 1)) * 3;
}

// One Gaussian per thread, 128 per block.  The wide AoS arrays go through shared memory so that global memory sees
// only contiguous traffic: the block's slice of the SH coefficients arrives by one bulk asynchronous copy that is in
// flight while the threads do the geometry, and the 9-float matrices, the colours, the warped means and the 128-byte
// render records leave through a staging buffer (records by one bulk store).
constexpr int kPreBlock = 128;
constexpr int kShSourceFloats = FSGS_SH_SOURCE_FLOATS;  // colour gradient 3 | direction 3 | visibility 1
constexpr int kWideMax = 48;                                    // SH floats per Gaussian that can be staged
constexpr int kStageTm = 0, kStageIm = kPreBlock * 9, kStageCol = kPreBlock * 18, kStageWm = kPreBlock * 21;
constexpr int kStageRec = kPreBlock * 24;                       // float offset of the record staging (16-B aligned)
constexpr int kStageFloats = kStageRec + kPreBlock * kRecFloats;

// rows x N floats, contiguous in global memory, from the staging buffer
template <int N>
__device__ __forceinline__ void store_rows(float *__restrict__ dst, const float *src, int rows) {
  const int n = rows * N;
  for (int e = threadIdx.x; e < n; e += kPreBlock) dst[e] = src[e];
}
template <int N>
__device__ __forceinline__ void add_rows(float *__restrict__ dst, const float *src, int rows) {
  const int n = rows * N;
  for (int e = threadIdx.x; e < n; e += kPreBlock) dst[e] += src[e];
}

template <bool LBS, bool HIGH_SH>
__global__ void __launch_bounds__(kPreBlock) preprocess_forward_kernel(PreDev a, LbsDev lbs) {
  // the SH slice is dead once the colours are known; the output staging reuses its space
  __shared__ __align__(128) float s_mem[kStageFloats > kPreBlock * kWideMax ? kStageFloats : kPreBlock * kWideMax];
  float *s_wide = s_mem, *s_stage = s_mem;
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ float cam[16 + 9 + 3];
  __shared__ int s_area[kPreBlock / 32], s_real[kPreBlock / 32];
  const int t = threadIdx.x, base = blockIdx.x * kPreBlock, rows = min(kPreBlock, a.P - base), i = base + t;
  if (t < 16) cam[t] = a.Tw2v[t];
  else if (t < 25) cam[t] = a.Tv2s[t - 16];
  else if (t < 28) cam[t] = a.campos[t - 25];
  const float *Tw2v = cam, *Tv2s = cam + 16, *campos = cam + 25;

  // the wide SH array: sh_rest when the caller keeps DC and the rest apart, else shs
  const int wide = a.sh_rest ? a.n_rest * 3 : a.n_dc * 3;
  const float *wide_src = (a.sh_rest ? a.sh_rest : a.shs) + (size_t) base * wide;
  const bool staged = a.sh_degree >= 1 && wide <= kWideMax;
  const uint32_t wide_bytes = (uint32_t) rows * wide * 4u;
  const bool bulk = staged && ((uintptr_t) wide_src & 15) == 0 && (wide_bytes & 15u) == 0;
  if (bulk && t == 0) mbar_init(&s_bar, 1);
  __syncthreads();
  if (bulk) {
    if (t == 0) {
      mbar_arrive_expect_tx(&s_bar, wide_bytes);
      bulk_load(s_wide, wide_src, wide_bytes, &s_bar);
    }
  } else if (staged) {
    for (int e = t; e < rows * wide; e += kPreBlock) s_wide[e] = __ldg(wide_src + e);
  }

  int area = 0, real = 0;
  float3 p = make_float3(0, 0, 0);
  float2 s = make_float2(0, 0);
  float4 q = make_float4(0, 0, 0, 0);
  bool vis = false;
  float M[9], IM[9];
  float3 nrm = make_float3(0, 0, 0), rgb = make_float3(0, 0, 0);
  float2 ctr = make_float2(0, 0);
  float vz = 0, opacity = 0, radius = 0;
  int x0 = 0, y0 = 0, x1 = 0, y1 = 0;
  Conic cn = {};
  // loads that the culled path would not need are issued up front all the same: one round trip instead of a chain
  float opac_in = 0.0f, dc0 = 0.0f, dc1 = 0.0f, dc2 = 0.0f;
  if (i < a.P) {
    opac_in = __ldg(a.opac + i);
    if (a.sh_degree >= 0) {
      const float *c0 = a.shs + (size_t) i * (a.sh_degree >= 0 ? a.n_dc : 1) * 3;
      dc0 = __ldg(c0), dc1 = __ldg(c0 + 1), dc2 = __ldg(c0 + 2);
    }
  }
  if (i < a.P) {
    if (LBS) lbs_warp_one(lbs, i, p, s, q);
    else p = make_float3(a.means[3 * i], a.means[3 * i + 1], a.means[3 * i + 2]);
    vis = !(a.culling && a.culling[i]);
    if (vis) {
      const float3 pv = view_point(p, Tw2v);
      vz = pv.z;
      vis = !(vz <= 0.2f);
      if (vis) {
        opacity = a.opacity_is_logit ? sigmoid_f32(opac_in) : opac_in;
        if (a.trans_precomp == nullptr) {
          if (!LBS) s = a.scales[i], q = a.rots[i];
          splat_matrix(p, s, q, Tw2v, Tv2s, M, nrm);
        } else {
#pragma unroll
          for (int k = 0; k < 9; ++k) M[k] = a.trans_precomp[(size_t) 9 * i + k];
          nrm = make_float3(0.0f, 0.0f, 1.0f);
        }
        const float c = -(pv.x * nrm.x + pv.y * nrm.y + pv.z * nrm.z);
        if (c == 0) vis = false;
        const float sgn = c > 0 ? 1.0f : -1.0f;
        nrm = make_float3(sgn * nrm.x, sgn * nrm.y, sgn * nrm.z);
      }
      if (vis) {
        if (!splat_bounds(M, ctr, radius)) {
          vis = false;
        } else {
          tile_rect(ctr.x, ctr.y, (int) radius, a.gx, a.gy, x0, y0, x1, y1);
          if ((x1 - x0) * (y1 - y0) == 0) vis = false;
        }
      }
    }
    if (vis) {
      adjugate(M, IM);
      area = (y1 - y0) * (x1 - x0);
      cn = make_conic(IM, opacity);
    } else {
#pragma unroll
      for (int k = 0; k < 9; ++k) M[k] = 0.0f, IM[k] = 0.0f;
      nrm = make_float3(0, 0, 0);
      ctr = make_float2(0, 0);
      vz = 0, opacity = 0, radius = 0;
    }
  }

  // count (and histogram) the tiles with a corner inside the alpha >= 1/255 conic, the warp's 32 splats together
  {
    const int gx = a.gx;
    int32_t *tc = a.tile_counts;
    warp_for_each_covered_tile(cn, x0, y0, x1, y1, vis, 0u, 0u, [&](int x, int y, unsigned, unsigned) {
      atomicAdd(tc + y * gx + x, 1);
      ++real;
    });
  }

  // the SH slice must have landed before the colours are evaluated
  if (staged) {
    const bool late = bulk && !mbar_wait_bounded(&s_bar, 0);
    if (__syncthreads_or(late)) {
      // the copy never reported completion: note it and read the slice with plain loads instead
      if (t == 0) atomicOr(a.counters + FSGS_CNT_STATUS, 1ull);
      for (int e = t; e < rows * wide; e += kPreBlock) s_wide[e] = __ldg(wide_src + e);
      __syncthreads();
    }
  }
  if (vis) {
    if (a.sh_degree >= 0) {
      float x = p.x - campos[0], y = p.y - campos[1], z = p.z - campos[2];
      const float n = rsqrtf(x * x + y * y + z * z + 1e-12f);
      x *= n, y *= n, z *= n;
      float b[16];
      sh_basis(a.sh_degree, x, y, z, b);
      const int nb = (a.sh_degree + 1) * (a.sh_degree + 1);
      const float *c0 = a.shs + (size_t) i * a.n_dc * 3;          // coefficient 0
      const float *cw = staged ? s_wide + t * wide : (a.sh_rest ? a.sh_rest + (size_t) i * wide : c0);
      if (a.sh_rest) cw -= 3;                                     // the rest array starts at coefficient 1
      rgb.x += dc0 * b[0], rgb.y += dc1 * b[0], rgb.z += dc2 * b[0];
#pragma unroll
      for (int k = 1; k < 16; ++k) {
        if (k < nb) {
          const float *c = cw + 3 * k;
          rgb.x += c[0] * b[k], rgb.y += c[1] * b[k], rgb.z += c[2] * b[k];
        }
      }
      if (HIGH_SH) sh_high_colour(a.sh_degree, x, y, z, cw, rgb);
      rgb = make_float3(fmaxf(rgb.x + 0.5f, 0.0f), fmaxf(rgb.y + 0.5f, 0.0f), fmaxf(rgb.z + 0.5f, 0.0f));
    } else {
      rgb = make_float3(a.shs[3 * i], a.shs[3 * i + 1], a.shs[3 * i + 2]);
    }
  }

  if (staged) __syncthreads();   // all reads of the SH slice are done
  // every row is written: zeros for culled Gaussians
  if (i < a.P) {
#pragma unroll
    for (int k = 0; k < 9; ++k) s_stage[kStageTm + 9 * t + k] = M[k], s_stage[kStageIm + 9 * t + k] = IM[k];
    s_stage[kStageCol + 3 * t] = rgb.x, s_stage[kStageCol + 3 * t + 1] = rgb.y, s_stage[kStageCol + 3 * t + 2] = rgb.z;
    if (LBS) s_stage[kStageWm + 3 * t] = p.x, s_stage[kStageWm + 3 * t + 1] = p.y, s_stage[kStageWm + 3 * t + 2] = p.z;
    if (a.records) {
      float tau = 0.0f;
      const float4 box = vis ? alpha_box(M, ctr, opacity, tau) : make_float4(1.0f, -1.0f, 1.0f, -1.0f);
      float4 *rec = reinterpret_cast<float4 *>(s_stage + kStageRec) + t * (kRecFloats / 4);
      write_record(rec, ctr, opacity, IM, M, box, tau, rgb, nrm);
      rec[7] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    a.means2D[i] = ctr;
    a.normal_opacity[i] = make_float4(nrm.x, nrm.y, nrm.z, opacity);
    a.depths[i] = vz;
    a.radii[i] = (int) radius;
    a.tiles_touched[i] = area;
    if (LBS) a.warped_scales[i] = s, a.warped_rots[i] = q;
  }
  for (int o = 16; o > 0; o >>= 1) {
    area += __shfl_xor_sync(0xffffffffu, area, o);
    real += __shfl_xor_sync(0xffffffffu, real, o);
  }
  if ((t & 31) == 0) s_area[t >> 5] = area, s_real[t >> 5] = real;
  fence_async_smem();
  __syncthreads();

  bool rec_bulk = false;
  if (a.records) {
    float4 *dst = a.records + (size_t) base * (kRecFloats / 4);
    rec_bulk = ((uintptr_t) dst & 15) == 0;
    if (rec_bulk) {
      if (t == 0) bulk_store(dst, s_stage + kStageRec, (uint32_t) rows * kRecFloats * 4u);
    } else {
      store_rows<kRecFloats>(reinterpret_cast<float *>(dst), s_stage + kStageRec, rows);
    }
  }
  if (a.trans_precomp == nullptr) store_rows<9>(a.trans_mat + (size_t) base * 9, s_stage + kStageTm, rows);
  store_rows<9>(a.inverse_m + (size_t) base * 9, s_stage + kStageIm, rows);
  if (a.sh_degree >= 0) store_rows<3>(a.colors + (size_t) base * 3, s_stage + kStageCol, rows);
  if (LBS) store_rows<3>(a.warped_means + (size_t) base * 3, s_stage + kStageWm, rows);
  // block totals -> two global atomics per block
  if (t == 0) {
    long long ta = 0, tr = 0;
    for (int w = 0; w < kPreBlock / 32; ++w) ta += s_area[w], tr += s_real[w];
    if (ta) atomicAdd(a.counters + FSGS_CNT_SLOTS, (unsigned long long) ta);
    if (tr) atomicAdd(a.counters + FSGS_CNT_PAIRS, (unsigned long long) tr);
    if (rec_bulk) bulk_store_wait();   // the staging buffer must outlive the copy
  }
}

__global__ void __launch_bounds__(256) pack_records_kernel(int P, const float2 *__restrict__ means2D,
    const float *__restrict__ colors, const float4 *__restrict__ normal_opacity, const float *__restrict__ trans_mat,
    const float *__restrict__ inverse_m, float4 *__restrict__ records) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  float M[9], IM[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) M[k] = trans_mat[(size_t) 9 * i + k], IM[k] = inverse_m[(size_t) 9 * i + k];
  const float4 no = normal_opacity[i];
  const float2 ctr = means2D[i];
  const float3 rgb = make_float3(colors[3 * i], colors[3 * i + 1], colors[3 * i + 2]);
  float tau = 0.0f;
  const float4 box = alpha_box(M, ctr, no.w, tau);
  write_record(records + (size_t) i * (kRecFloats / 4), ctr, no.w, IM, M, box, tau, rgb,
      make_float3(no.x, no.y, no.z));
}

// ------------------------------------------------------------------------------------------------
// standalone splat matrix, forward / backward
// ------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256) transmat_forward_kernel(int P, const float *__restrict__ means,
    const float2 *__restrict__ scales, const float4 *__restrict__ rots, const float *__restrict__ Tw2v,
    const float *__restrict__ Tv2s, float *__restrict__ trans_mat, float *__restrict__ normals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  float M[9];
  float3 n;
  splat_matrix(make_float3(means[3 * i], means[3 * i + 1], means[3 * i + 2]), scales[i], rots[i], Tw2v, Tv2s, M, n);
#pragma unroll
  for (int k = 0; k < 9; ++k) trans_mat[(size_t) 9 * i + k] = M[k];
  normals[3 * i] = n.x, normals[3 * i + 1] = n.y, normals[3 * i + 2] = n.z;
}

// Adjoint of splat_matrix: gT = dL/dM, gn = dL/dnormal (view space).
// (reference gs_2d_fast_preprocess.cu:100-139)
__device__ __forceinline__ void splat_matrix_adjoint(const float2 s, const float4 q, const float *__restrict__ Tw2v,
    const float *__restrict__ Tv2s, const float *gT, const float3 gn, float3 &g_mean, float2 &g_scale, float4 &g_rot) {
  float gL[9], dR[9];
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      float acc = 0;
#pragma unroll
      for (int k = 0; k < 3; ++k) acc += Tv2s[k * 3 + a] * gT[k * 3 + b];
      gL[a * 3 + b] = acc;
    }
#pragma unroll
  for (int a = 0; a < 3; ++a)
#pragma unroll
    for (int b = 0; b < 3; ++b) {
      float acc = 0;
#pragma unroll
      for (int k = 0; k < 3; ++k) acc += Tw2v[k * 4 + a] * gL[k * 3 + b];
      dR[a * 3 + b] = acc;
    }
  g_mean = make_float3(dR[2], dR[5], dR[8]);
  dR[2] = gn.x * Tw2v[0] + gn.y * Tw2v[4] + gn.z * Tw2v[8];
  dR[5] = gn.x * Tw2v[1] + gn.y * Tw2v[5] + gn.z * Tw2v[9];
  dR[8] = gn.x * Tw2v[2] + gn.y * Tw2v[6] + gn.z * Tw2v[10];
  g_scale.x = dR[0] * (1 - 2 * (q.y * q.y + q.z * q.z)) + dR[3] * (2 * (q.x * q.y + q.z * q.w)) +
              dR[6] * (2 * (q.x * q.z - q.y * q.w));
  g_scale.y = dR[1] * (2 * (q.x * q.y - q.z * q.w)) + dR[4] * (1 - 2 * (q.x * q.x + q.z * q.z)) +
              dR[7] * (2 * (q.x * q.w + q.y * q.z));
  dR[0] *= s.x, dR[3] *= s.x, dR[6] *= s.x;
  dR[1] *= s.y, dR[4] *= s.y, dR[7] *= s.y;
  g_rot = quat_adjoint(q, dR);
}

__global__ void __launch_bounds__(256) transmat_backward_kernel(int P, const float2 *__restrict__ scales,
    const float4 *__restrict__ rots, const float *__restrict__ Tw2v, const float *__restrict__ Tv2s,
    const float *__restrict__ g_trans_mat, const float *__restrict__ g_normals, float *__restrict__ g_means,
    float2 *__restrict__ g_scales, float4 *__restrict__ g_rots) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  float gT[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) gT[k] = g_trans_mat[(size_t) 9 * i + k];
  float3 gm;
  float2 gs;
  float4 gq;
  splat_matrix_adjoint(scales[i], rots[i], Tw2v, Tv2s, gT,
      make_float3(g_normals[3 * i], g_normals[3 * i + 1], g_normals[3 * i + 2]), gm, gs, gq);
  g_means[3 * i] = gm.x, g_means[3 * i + 1] = gm.y, g_means[3 * i + 2] = gm.z;
  g_scales[i] = gs;
  g_rots[i] = gq;
}

// The same two operators in double precision (the reference dispatches them over the floating types,
// gs_2d_fast_preprocess.cu:889,936).  Nothing on the rendering path calls them; plain arithmetic, no contraction pins.
__device__ __forceinline__ void rot_columns_f64(const double *q, double *R) {  // q = (x, y, z, w), R row major
  const double x = q[0], y = q[1], z = q[2], w = q[3];
  R[0] = 1 - 2 * (y * y + z * z), R[1] = 2 * (x * y - z * w), R[2] = 2 * (y * w + x * z);
  R[3] = 2 * (x * y + z * w), R[4] = 1 - 2 * (x * x + z * z), R[5] = 2 * (y * z - x * w);
  R[6] = 2 * (x * z - y * w), R[7] = 2 * (x * w + y * z), R[8] = 1 - 2 * (x * x + y * y);
}

__global__ void __launch_bounds__(256) transmat_forward_f64_kernel(int P, const double *__restrict__ means,
    const double *__restrict__ scales, const double *__restrict__ rots, const double *__restrict__ Tw2v,
    const double *__restrict__ Tv2s, double *__restrict__ trans_mat, double *__restrict__ normals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  double R[9], L[9], t[9];
  rot_columns_f64(rots + 4 * (size_t) i, R);
  const double sx = scales[2 * (size_t) i], sy = scales[2 * (size_t) i + 1];
  for (int r = 0; r < 3; ++r) L[3 * r] = R[3 * r] * sx, L[3 * r + 1] = R[3 * r + 1] * sy, L[3 * r + 2] = means[3 * (size_t) i + r];
  for (int a = 0; a < 3; ++a)
    for (int b = 0; b < 3; ++b)
      t[3 * a + b] = Tw2v[4 * a] * L[b] + Tw2v[4 * a + 1] * L[3 + b] + Tw2v[4 * a + 2] * L[6 + b];
  t[8] += Tw2v[11];
  for (int a = 0; a < 3; ++a)
    for (int b = 0; b < 3; ++b)
      trans_mat[9 * (size_t) i + 3 * a + b] = Tv2s[3 * a] * t[b] + Tv2s[3 * a + 1] * t[3 + b] + Tv2s[3 * a + 2] * t[6 + b];
  for (int a = 0; a < 3; ++a)
    normals[3 * (size_t) i + a] = Tw2v[4 * a] * R[2] + Tw2v[4 * a + 1] * R[5] + Tw2v[4 * a + 2] * R[8];
}

__global__ void __launch_bounds__(256) transmat_backward_f64_kernel(int P, const double *__restrict__ scales,
    const double *__restrict__ rots, const double *__restrict__ Tw2v, const double *__restrict__ Tv2s,
    const double *__restrict__ g_trans_mat, const double *__restrict__ g_normals, double *__restrict__ g_means,
    double *__restrict__ g_scales, double *__restrict__ g_rots) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const double *gT = g_trans_mat + 9 * (size_t) i, *q = rots + 4 * (size_t) i;
  double gt[9], dL[9], R[9];
  for (int a = 0; a < 3; ++a)       // dL/dt = Tv2s^T gT
    for (int b = 0; b < 3; ++b) gt[3 * a + b] = Tv2s[a] * gT[b] + Tv2s[3 + a] * gT[3 + b] + Tv2s[6 + a] * gT[6 + b];
  for (int a = 0; a < 3; ++a)       // dL/dL = Tw2v[:3,:3]^T dL/dt
    for (int b = 0; b < 3; ++b) dL[3 * a + b] = Tw2v[a] * gt[b] + Tw2v[4 + a] * gt[3 + b] + Tw2v[8 + a] * gt[6 + b];
  for (int r = 0; r < 3; ++r) g_means[3 * (size_t) i + r] = dL[3 * r + 2];
  rot_columns_f64(q, R);
  const double sx = scales[2 * (size_t) i], sy = scales[2 * (size_t) i + 1];
  g_scales[2 * (size_t) i] = dL[0] * R[0] + dL[3] * R[3] + dL[6] * R[6];
  g_scales[2 * (size_t) i + 1] = dL[1] * R[1] + dL[4] * R[4] + dL[7] * R[7];
  double dR[9];                     // dL/dR: scaled columns 0, 1; column 2 from the normal
  for (int r = 0; r < 3; ++r) {
    dR[3 * r] = dL[3 * r] * sx, dR[3 * r + 1] = dL[3 * r + 1] * sy;
    dR[3 * r + 2] = g_normals[3 * (size_t) i] * Tw2v[r] + g_normals[3 * (size_t) i + 1] * Tw2v[4 + r] +
                    g_normals[3 * (size_t) i + 2] * Tw2v[8 + r];
  }
  const double x = q[0], y = q[1], z = q[2], w = q[3];
  double *g = g_rots + 4 * (size_t) i;
  g[0] = 2 * (-2 * x * (dR[4] + dR[8]) + y * (dR[1] + dR[3]) + z * (dR[2] + dR[6]) + w * (dR[7] - dR[5]));
  g[1] = 2 * (x * (dR[1] + dR[3]) - 2 * y * (dR[0] + dR[8]) + z * (dR[5] + dR[7]) + w * (dR[2] - dR[6]));
  g[2] = 2 * (x * (dR[2] + dR[6]) + y * (dR[5] + dR[7]) - 2 * z * (dR[0] + dR[4]) + w * (dR[3] - dR[1]));
  g[3] = 2 * (x * (dR[7] - dR[5]) + y * (dR[2] - dR[6]) + z * (dR[3] - dR[1]));
}

// ------------------------------------------------------------------------------------------------
// preprocess backward  (reference gs_2d_fast_preprocess.cu:516-609)
// ------------------------------------------------------------------------------------------------

struct PreBwdDev {
  int P, W, H, sh_degree, n_dc, n_rest;
  const float *means;
  const float2 *scales;
  const float4 *rots;
  const float *shs, *sh_rest, *Tw2v, *Tv2s, *campos, *trans_mat, *colors;
  const int32_t *radii;
  float2 *g_means2D;
  const float *g_trans_mat, *g_inverse_m, *g_colors;
  const float4 *g_normal_opacity;
  float *g_means;
  float2 *g_scales;
  float4 *g_rots;
  float *g_opac, *g_shs, *g_sh_rest;
  const float4 *normal_opacity;  // with it, g_opac is the gradient of the opacity LOGIT: g * o * (1 - o)
  float *visible;                // optional [P] 0/1 mask of the Gaussians with radii > 0
  const long long *overflow;     // optional: != 0 -> the lists were truncated, visible = -inf on every row
  float *sh_source;              // optional [P,6]: clamped colour gradient and view direction
  int accumulate;                // add to g_opac / g_shs / g_sh_rest / visible instead of writing them
};

__device__ __forceinline__ float3 cross3(const float3 a, const float3 b) {
  return make_float3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}

// Adjoint of the preprocess, one Gaussian per thread, 128 per block.  All per-Gaussian rows that are wider than a
// vector load come in by bulk asynchronous copies on one mbarrier (SH coefficients, the three 3x3 matrices, means,
// colours and their gradients); the SH gradient is formed in place over the coefficients it was computed from and
// leaves by one bulk store.  Every output row is written, zeros for Gaussians that were culled in the forward pass,
// except grad_means2D, which is updated in place for visible Gaussians only.
constexpr int kBwdWide = 0, kBwdTm = kPreBlock * kWideMax, kBwdGtm = kBwdTm + kPreBlock * 9;
constexpr int kBwdGim = kBwdGtm + kPreBlock * 9, kBwdMeans = kBwdGim + kPreBlock * 9;
constexpr int kBwdCol = kBwdMeans + kPreBlock * 3, kBwdGcol = kBwdCol + kPreBlock * 3;
constexpr int kBwdFloats = kBwdGcol + kPreBlock * 3;

__device__ __forceinline__ bool bulk_ok(const void *g, uint32_t bytes) {
  return ((uintptr_t) g & 15) == 0 && (bytes & 15u) == 0 && bytes > 0;
}

template <bool HIGH_SH>
__global__ void __launch_bounds__(kPreBlock) preprocess_backward_kernel(PreBwdDev a) {
  __shared__ __align__(128) float s_mem[kBwdFloats];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ float cam[16 + 9 + 3];
  const int t = threadIdx.x, base = blockIdx.x * kPreBlock, rows = min(kPreBlock, a.P - base), i = base + t;
  if (t < 16) cam[t] = a.Tw2v[t];
  else if (t < 25) cam[t] = a.Tv2s[t - 16];
  else if (t < 28) cam[t] = a.campos[t - 25];
  const float *Tw2v = cam, *Tv2s = cam + 16, *campos = cam + 25;

  const bool want_sh = a.sh_degree >= 0;
  const int wide = a.sh_rest ? a.n_rest * 3 : a.n_dc * 3;
  const bool staged = a.sh_degree >= 1 && wide <= kWideMax;
  // slices staged through shared memory: {destination offset, source, floats per row}
  const float *src[7] = {(a.sh_rest ? a.sh_rest : a.shs) + (size_t) base * wide, a.trans_mat + (size_t) base * 9,
      a.g_trans_mat + (size_t) base * 9, a.g_inverse_m + (size_t) base * 9, a.means + (size_t) base * 3,
      want_sh ? a.colors + (size_t) base * 3 : nullptr, want_sh ? a.g_colors + (size_t) base * 3 : nullptr};
  const int dst[7] = {kBwdWide, kBwdTm, kBwdGtm, kBwdGim, kBwdMeans, kBwdCol, kBwdGcol};
  const int per_row[7] = {staged ? wide : 0, 9, 9, 9, 3, want_sh ? 3 : 0, want_sh ? 3 : 0};
  uint32_t bulk_bytes = 0;
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    const uint32_t bytes = (uint32_t) rows * per_row[k] * 4u;
    if (bulk_ok(src[k], bytes)) bulk_bytes += bytes;
  }
  if (bulk_bytes && t == 0) mbar_init(&s_bar, 1);
  __syncthreads();
  if (bulk_bytes && t == 0) {
    mbar_arrive_expect_tx(&s_bar, bulk_bytes);
#pragma unroll
    for (int k = 0; k < 7; ++k) {
      const uint32_t bytes = (uint32_t) rows * per_row[k] * 4u;
      if (bulk_ok(src[k], bytes)) bulk_load(s_mem + dst[k], src[k], bytes, &s_bar);
    }
  }
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    const int n = rows * per_row[k];
    if (n > 0 && !bulk_ok(src[k], (uint32_t) n * 4u))
      for (int e = t; e < n; e += kPreBlock) s_mem[dst[k] + e] = __ldg(src[k] + e);
  }
  // rows that need no staging are fetched while the copies fly
  const bool live = i < a.P && a.radii[i] > 0;
  float4 gno = make_float4(0, 0, 0, 0), q = make_float4(0, 0, 0, 1);
  float2 s = make_float2(0, 0), g2 = make_float2(0, 0);
  if (live) gno = a.g_normal_opacity[i], q = a.rots[i], s = a.scales[i], g2 = a.g_means2D[i];
  {
    const bool late = bulk_bytes && !mbar_wait_bounded(&s_bar, 0);
    if (__syncthreads_or(late)) {
      // a copy never reported completion: read everything with plain loads (no status word on this path; the
      // forward kernel of the same frame reports the condition)
#pragma unroll
      for (int k = 0; k < 7; ++k) {
        const int n = rows * per_row[k];
        for (int e = t; e < n; e += kPreBlock) s_mem[dst[k] + e] = __ldg(src[k] + e);
      }
      __syncthreads();
    }
  }

  float *w_row = s_mem + kBwdWide + t * wide;   // this thread's SH coefficients, then their gradient
  float3 gm = make_float3(0, 0, 0), gdc = make_float3(0, 0, 0);
  float3 src_g = make_float3(0, 0, 0), src_d = make_float3(0, 0, 0);  // the SH gradient's two factors
  float2 gs = make_float2(0, 0);
  float4 gq = make_float4(0, 0, 0, 0);
  if (live) {
    float m[9], gT[9], G[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) {
      m[k] = s_mem[kBwdTm + 9 * t + k];
      gT[k] = s_mem[kBwdGtm + 9 * t + k];
      G[k] = s_mem[kBwdGim + 9 * t + k];
    }
    // adjoint of the adjugate: inverse_m rows are c1 x c2, c2 x c0, c0 x c1 with c_j the columns of M
    {
      const float3 c0 = make_float3(m[0], m[3], m[6]), c1 = make_float3(m[1], m[4], m[7]), c2 = make_float3(m[2], m[5], m[8]);
      const float3 G0 = make_float3(G[0], G[1], G[2]), G1 = make_float3(G[3], G[4], G[5]), G2 = make_float3(G[6], G[7], G[8]);
      const float3 a0 = cross3(G1, c2), b0 = cross3(c1, G2);   // d/dc0
      const float3 a1 = cross3(c2, G0), b1 = cross3(G2, c0);   // d/dc1
      const float3 a2 = cross3(G0, c1), b2 = cross3(c0, G1);   // d/dc2
      gT[0] += a0.x + b0.x, gT[3] += a0.y + b0.y, gT[6] += a0.z + b0.z;
      gT[1] += a1.x + b1.x, gT[4] += a1.y + b1.y, gT[7] += a1.z + b1.z;
      gT[2] += a2.x + b2.x, gT[5] += a2.y + b2.y, gT[8] += a2.z + b2.z;
    }
    // adjoint of the bounding-box centre
    {
      const float2 g = g2;
      const float tv[3] = {9.0f, 9.0f, -1.0f};
      const float d = tv[0] * (m[6] * m[6]) + tv[1] * (m[7] * m[7]) + tv[2] * (m[8] * m[8]);
      const float inv_d = 1.0f / d;
      float f[3], df[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        f[k] = tv[k] * inv_d;
        df[k] = g.x * m[k] * m[6 + k] + g.y * m[3 + k] * m[6 + k];
      }
      const float dd = (df[0] * f[0] + df[1] * f[1] + df[2] * f[2]) * -inv_d;
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        gT[k] += g.x * f[k] * m[6 + k];
        gT[3 + k] += g.y * f[k] * m[6 + k];
        gT[6 + k] += (g.x * f[k] * m[k] + g.y * f[k] * m[3 + k]) + dd * (tv[k] * m[6 + k] * 2.0f);
      }
    }
    const float3 p = make_float3(s_mem[kBwdMeans + 3 * t], s_mem[kBwdMeans + 3 * t + 1], s_mem[kBwdMeans + 3 * t + 2]);
    // the stored normal was flipped to face the camera
    float3 gn = make_float3(gno.x, gno.y, gno.z);
    {
      const float3 n = make_float3(2 * (q.y * q.w + q.x * q.z), 2 * (q.y * q.z - q.x * q.w), 1 - 2 * (q.x * q.x + q.y * q.y));
      const float nx = Tw2v[0] * n.x + Tw2v[1] * n.y + Tw2v[2] * n.z;
      const float ny = Tw2v[4] * n.x + Tw2v[5] * n.y + Tw2v[6] * n.z;
      const float nz = Tw2v[8] * n.x + Tw2v[9] * n.y + Tw2v[10] * n.z;
      const float vx = Tw2v[0] * p.x + Tw2v[1] * p.y + Tw2v[2] * p.z + Tw2v[3];
      const float vy = Tw2v[4] * p.x + Tw2v[5] * p.y + Tw2v[6] * p.z + Tw2v[7];
      const float vz = Tw2v[8] * p.x + Tw2v[9] * p.y + Tw2v[10] * p.z + Tw2v[11];
      const float c = -(vx * nx + vy * ny + vz * nz);
      const float sgn = c > 0 ? 1.0f : -1.0f;
      gn = make_float3(sgn * gn.x, sgn * gn.y, sgn * gn.z);
    }
    splat_matrix_adjoint(s, q, Tw2v, Tv2s, gT, gn, gm, gs, gq);

    if (want_sh) {
      const float ux = p.x - campos[0], uy = p.y - campos[1], uz = p.z - campos[2];
      const float n = rsqrtf(ux * ux + uy * uy + uz * uz + 1e-12f);
      const float x = ux * n, y = uy * n, z = uz * n;
      float3 grgb;
      grgb.x = s_mem[kBwdCol + 3 * t] > 0 ? s_mem[kBwdGcol + 3 * t] : 0.0f;
      grgb.y = s_mem[kBwdCol + 3 * t + 1] > 0 ? s_mem[kBwdGcol + 3 * t + 1] : 0.0f;
      grgb.z = s_mem[kBwdCol + 3 * t + 2] > 0 ? s_mem[kBwdGcol + 3 * t + 2] : 0.0f;
      float b[16];
      sh_basis(a.sh_degree, x, y, z, b);
      const int nb = (a.sh_degree + 1) * (a.sh_degree + 1);
      gdc = make_float3(grgb.x * b[0], grgb.y * b[0], grgb.z * b[0]);
      src_g = grgb, src_d = make_float3(x, y, z);
      float dx = 0, dy = 0, dz = 0;
      // coefficient k >= 1 lives at row offset 3*(k - first)
      const int first = a.sh_rest ? 1 : 0;
      const float *c_g = (a.sh_rest ? a.sh_rest : a.shs) + (size_t) i * wide;           // unstaged source
      float *g_g = a.sh_rest ? a.g_sh_rest : a.g_shs;                                    // unstaged destination
      if (g_g) g_g += (size_t) i * wide;
#pragma unroll
      for (int k = 1; k < 16; ++k) {
        if (k < nb) {
          const int o = 3 * (k - first);
          float c0, c1, c2;
          if (staged) c0 = w_row[o], c1 = w_row[o + 1], c2 = w_row[o + 2];
          else c0 = __ldg(c_g + o), c1 = __ldg(c_g + o + 1), c2 = __ldg(c_g + o + 2);
          const float tt = grgb.x * c0 + grgb.y * c1 + grgb.z * c2;
          const float3 db = sh_basis_grad(k, x, y, z);
          dx += tt * db.x, dy += tt * db.y, dz += tt * db.z;
          if (staged) w_row[o] = grgb.x * b[k], w_row[o + 1] = grgb.y * b[k], w_row[o + 2] = grgb.z * b[k];
          else if (g_g) g_g[o] = grgb.x * b[k], g_g[o + 1] = grgb.y * b[k], g_g[o + 2] = grgb.z * b[k];
        }
      }
      if (HIGH_SH) sh_high_adjoint(a.sh_degree, x, y, z, c_g - 3 * first, g_g ? g_g - 3 * first : nullptr, grgb, dx, dy, dz);
      // coefficients beyond the active degree get no gradient
      if (staged) {
        for (int o = 3 * (nb - first); o < wide; ++o) w_row[o] = 0.0f;
        if (!a.sh_rest) w_row[0] = gdc.x, w_row[1] = gdc.y, w_row[2] = gdc.z;
      } else if (g_g) {
        for (int o = 3 * (nb - first); o < wide; ++o) g_g[o] = 0.0f;
        if (!a.sh_rest) g_g[0] = gdc.x, g_g[1] = gdc.y, g_g[2] = gdc.z;
      }
      const float tt = -(ux * dx + uy * dy + uz * dz) * n * n * n;
      gm.x += dx * n + tt * ux;
      gm.y += dy * n + tt * uy;
      gm.z += dz * n + tt * uz;
    }
    // densification proxy replaces the consumed mean2D gradient (reference gs_2d_fast_preprocess.cu:605-608)
    a.g_means2D[i] = make_float2(gT[2] * m[8] * 0.5f * (float) a.W, gT[5] * m[8] * 0.5f * (float) a.H);
  } else if (i < a.P && want_sh) {
    if (staged) {
      for (int o = 0; o < wide; ++o) w_row[o] = 0.0f;
    } else if (!a.accumulate) {
      float *g_g = a.sh_rest ? a.g_sh_rest : a.g_shs;
      if (g_g)
        for (int o = 0; o < wide; ++o) g_g[(size_t) i * wide + o] = 0.0f;
    }
  }
  if (i < a.P) {
    const bool poisoned = a.overflow && *a.overflow != 0;
    if (a.sh_source) {
      float *o = a.sh_source + (size_t) i * kShSourceFloats;
      o[0] = src_g.x, o[1] = src_g.y, o[2] = src_g.z, o[3] = src_d.x, o[4] = src_d.y, o[5] = src_d.z;
      o[6] = poisoned ? -INFINITY : (live ? 1.0f : 0.0f);
    }
    float g_o = gno.w;
    if (a.normal_opacity) {
      const float o = a.normal_opacity[i].w;
      g_o = g_o * (1.0f - o) * o;
    }
    if (a.accumulate) {
      if (live) a.g_opac[i] += g_o;
      if (a.visible) {
        if (poisoned) a.visible[i] = -INFINITY;
        else if (live && a.visible[i] >= 0.0f) a.visible[i] = 1.0f;  // a poisoned row stays poisoned
      }
    } else {
      a.g_opac[i] = g_o;
      if (a.visible) a.visible[i] = poisoned ? -INFINITY : (live ? 1.0f : 0.0f);
    }
    a.g_scales[i] = gs;
    a.g_rots[i] = gq;
    s_mem[kBwdMeans + 3 * t] = gm.x, s_mem[kBwdMeans + 3 * t + 1] = gm.y, s_mem[kBwdMeans + 3 * t + 2] = gm.z;
    s_mem[kBwdCol + 3 * t] = gdc.x, s_mem[kBwdCol + 3 * t + 1] = gdc.y, s_mem[kBwdCol + 3 * t + 2] = gdc.z;
  }
  fence_async_smem();
  __syncthreads();
  bool out_bulk = false;
  if (want_sh && staged) {
    float *g_wide = a.sh_rest ? a.g_sh_rest : a.g_shs;
    if (g_wide) {
      g_wide += (size_t) base * wide;
      const uint32_t bytes = (uint32_t) rows * wide * 4u;
      out_bulk = bulk_ok(g_wide, bytes);
      if (out_bulk) {
        if (t == 0) {
          if (a.accumulate) bulk_reduce_add_f32(g_wide, s_mem + kBwdWide, bytes);
          else bulk_store(g_wide, s_mem + kBwdWide, bytes);
        }
      } else if (a.accumulate) {
        for (int e = t; e < rows * wide; e += kPreBlock) g_wide[e] += s_mem[kBwdWide + e];
      } else {
        for (int e = t; e < rows * wide; e += kPreBlock) g_wide[e] = s_mem[kBwdWide + e];
      }
    }
  }
  store_rows<3>(a.g_means + (size_t) base * 3, s_mem + kBwdMeans, rows);
  if (want_sh && a.sh_rest && a.g_shs) {
    // the DC gradient; n_dc is 1 in this layout
    if (a.n_dc == 1 && a.accumulate) add_rows<3>(a.g_shs + (size_t) base * 3, s_mem + kBwdCol, rows);
    else if (a.n_dc == 1) store_rows<3>(a.g_shs + (size_t) base * 3, s_mem + kBwdCol, rows);
    else if (i < a.P) {
      float *g = a.g_shs + (size_t) i * a.n_dc * 3;
      g[0] = s_mem[kBwdCol + 3 * t], g[1] = s_mem[kBwdCol + 3 * t + 1], g[2] = s_mem[kBwdCol + 3 * t + 2];
      for (int o = 3; o < a.n_dc * 3; ++o) g[o] = 0.0f;
    }
  }
  if (out_bulk && t == 0) bulk_store_wait();
}

// The two factors of a view's SH gradient and the visibility mask, straight from what the compositing adjoint and the
// forward pass left behind: everything the exchange between ranks needs from this view, available before the
// preprocess adjoint has run.  Same values as preprocess_backward_kernel writes (sh_source, visible).
__global__ void __launch_bounds__(256) sh_factors_kernel(int P, const float *__restrict__ means,
    const float *__restrict__ colors, const float *__restrict__ g_colors, const int32_t *__restrict__ radii,
    const float *__restrict__ campos, const long long *__restrict__ overflow, int accumulate,
    float *__restrict__ sh_source, float *__restrict__ visible) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const bool live = radii[i] > 0;
  float3 g = make_float3(0, 0, 0), d = make_float3(0, 0, 0);
  if (live) {
    const float ux = means[3 * i] - campos[0], uy = means[3 * i + 1] - campos[1], uz = means[3 * i + 2] - campos[2];
    const float n = rsqrtf(ux * ux + uy * uy + uz * uz + 1e-12f);
    d = make_float3(ux * n, uy * n, uz * n);
    g.x = colors[3 * i] > 0 ? g_colors[3 * i] : 0.0f;
    g.y = colors[3 * i + 1] > 0 ? g_colors[3 * i + 1] : 0.0f;
    g.z = colors[3 * i + 2] > 0 ? g_colors[3 * i + 2] : 0.0f;
  }
  const bool poisoned = overflow && *overflow != 0;
  float *o = sh_source + (size_t) i * kShSourceFloats;
  o[0] = g.x, o[1] = g.y, o[2] = g.z, o[3] = d.x, o[4] = d.y, o[5] = d.z;
  o[6] = poisoned ? -INFINITY : (live ? 1.0f : 0.0f);
  if (visible) {
    if (poisoned) visible[i] = -INFINITY;
    else if (!accumulate) visible[i] = live ? 1.0f : 0.0f;
    else if (live && visible[i] >= 0.0f) visible[i] = 1.0f;  // a poisoned row stays poisoned
  }
}

// Summed SH gradient of several views from their factors: one Gaussian per thread, 128 per block; the 48 sums of a
// Gaussian stay in registers over the views, then leave through shared memory as whole 16-byte vectors.
struct ShSlots {
  int n;
  int order[FSGS_MAX_VIEW_SLOTS];
};

__global__ void __launch_bounds__(kPreBlock) sh_grad_from_views_kernel(int P, int sh_degree, int n_rest, ShSlots slots,
    const float *__restrict__ sh_source, long long slot_stride, float *__restrict__ g_dc, float *__restrict__ g_rest,
    float *__restrict__ visible) {
  __shared__ __align__(16) float s_out[kPreBlock * 45];
  const int t = threadIdx.x, base = blockIdx.x * kPreBlock, rows = min(kPreBlock, P - base), i = base + t;
  const int nb = (sh_degree + 1) * (sh_degree + 1);
  float acc[16][3];
#pragma unroll
  for (int k = 0; k < 16; ++k) acc[k][0] = acc[k][1] = acc[k][2] = 0.0f;
  if (i < P) {
    float seen = 0.0f;  // sum of the slots' visibility: > 0 where some view saw the Gaussian, -inf when one overflowed
    for (int s = 0; s < slots.n; ++s) {
      const float *src = sh_source + (size_t) slots.order[s] * slot_stride + (size_t) i * kShSourceFloats;
      const float gr = __ldg(src), gg = __ldg(src + 1), gb = __ldg(src + 2);
      seen += __ldg(src + 6);
      if (gr == 0.0f && gg == 0.0f && gb == 0.0f) continue;
      float b[16];
      sh_basis(sh_degree, __ldg(src + 3), __ldg(src + 4), __ldg(src + 5), b);
#pragma unroll
      for (int k = 0; k < 16; ++k)
        if (k < nb) acc[k][0] += gr * b[k], acc[k][1] += gg * b[k], acc[k][2] += gb * b[k];
    }
    g_dc[(size_t) i * 3] = acc[0][0], g_dc[(size_t) i * 3 + 1] = acc[0][1], g_dc[(size_t) i * 3 + 2] = acc[0][2];
    if (visible) visible[i] = seen;
  }
  if (n_rest <= 0 || !g_rest) return;
  const int wide = n_rest * 3;  // <= 45
#pragma unroll
  for (int k = 1; k < 16; ++k)
    if (k - 1 < n_rest) {
      s_out[t * wide + 3 * (k - 1)] = acc[k][0];
      s_out[t * wide + 3 * (k - 1) + 1] = acc[k][1];
      s_out[t * wide + 3 * (k - 1) + 2] = acc[k][2];
    }
  __syncthreads();
  float *dst = g_rest + (size_t) base * wide;
  const int n = rows * wide;
  if ((((uintptr_t) dst) & 15) == 0 && (n & 3) == 0) {
    for (int e = t; e < n / 4; e += kPreBlock) reinterpret_cast<float4 *>(dst)[e] = reinterpret_cast<const float4 *>(s_out)[e];
  } else {
    for (int e = t; e < n; e += kPreBlock) dst[e] = s_out[e];
  }
}

}  // namespace fsgs

using namespace fsgs;

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------

extern "C" int fsgs_lbs_warp_forward(int P, const fsgs_lbs *lbs, float *means, float *scales, float *rots,
    fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && lbs && means && scales && rots && lbs_valid(lbs));
  if (P == 0) return FSGS_OK;
  lbs_warp_forward_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, to_dev(lbs), means, (float2 *) scales,
      (float4 *) rots);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_lbs_warp_backward(int P, const fsgs_lbs *lbs, const float *g_means, const float *g_scales,
    const float *g_rots, const fsgs_lbs_grads *g, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && lbs && g && lbs_valid(lbs) && g_means && g_scales && g_rots);
  FSGS_REQUIRE(g->g_xyz && g->g_scaling_raw && g->g_rotation_raw && g->g_knn_w && g->g_sp_q && g->g_sp_t &&
               g->g_sp_dr && g->g_sp_ds);
  cudaStream_t st = (cudaStream_t) stream;
  const int M = lbs->M;
  const bool acc = g->accumulate != 0;
  if (acc) FSGS_REQUIRE(lbs->sp_pair_offsets && lbs->sp_pairs && g->scratch_rot);  // grouped pairs only
  if (lbs->sp_pair_offsets && lbs->sp_pairs) {
    const LbsDev d = to_dev(lbs);
    float4 *view_rot = acc ? (float4 *) g->scratch_rot : (float4 *) g->g_rotation_raw;  // this view's, read by pass 2
    if (P > 0) {
      if (acc)
        lbs_backward_points_kernel<true><<<ceil_div(P, 256), 256, 0, st>>>(P, d, g_means, (const float2 *) g_scales,
            (const float4 *) g_rots, g->g_xyz, (float2 *) g->g_scaling_raw, (float4 *) g->g_rotation_raw, g->g_knn_w,
            view_rot);
      else
        lbs_backward_points_kernel<false><<<ceil_div(P, 256), 256, 0, st>>>(P, d, g_means, (const float2 *) g_scales,
            (const float4 *) g_rots, g->g_xyz, (float2 *) g->g_scaling_raw, (float4 *) g->g_rotation_raw, g->g_knn_w,
            nullptr);
    }
#define FSGS_SP_LAUNCH(T, A)                                                                                       \
  lbs_backward_superpoints_kernel<T, A><<<M, T, 0, st>>>(d, lbs->sp_pair_offsets, lbs->sp_pairs, g_means,         \
      (const float2 *) g_scales, view_rot, g->g_sp_q, g->g_sp_t, g->g_sp_dr, g->g_sp_ds)
    // the superpoint rows are written, never accumulated: every view has its own motion, hence its own gradient
    if (M < 1024) FSGS_SP_LAUNCH(512, false);
    else FSGS_SP_LAUNCH(128, false);
#undef FSGS_SP_LAUNCH
    FSGS_LAUNCH_CHECK();
    return FSGS_OK;
  }
  cudaMemsetAsync(g->g_sp_q, 0, sizeof(float) * 4 * M, st);
  cudaMemsetAsync(g->g_sp_t, 0, sizeof(float) * 3 * M, st);
  cudaMemsetAsync(g->g_sp_dr, 0, sizeof(float) * 4 * M, st);
  cudaMemsetAsync(g->g_sp_ds, 0, sizeof(float) * 2 * M, st);
  if (P == 0) return FSGS_OK;
  const size_t table_bytes = sizeof(float) * kSpRow * (size_t) M;
  if (table_bytes <= 40 * 1024) {
    // one table per block in shared memory; few, fat blocks so that the flush stays cheap
    const int blocks = ceil_div(min(ceil_div(P, 256), 148 * 4), kLbsCluster) * kLbsCluster;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks), cfg.blockDim = dim3(256), cfg.dynamicSmemBytes = table_bytes, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kLbsCluster, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, lbs_warp_backward_kernel<true>, P, to_dev(lbs), g_means,
        (const float2 *) g_scales, (const float4 *) g_rots, g->g_xyz, (float2 *) g->g_scaling_raw,
        (float4 *) g->g_rotation_raw, g->g_knn_w, g->g_sp_q, g->g_sp_t, g->g_sp_dr, g->g_sp_ds);
    if (err != cudaSuccess) return FSGS_ERR_LAUNCH;
  } else {
    lbs_warp_backward_kernel<false><<<ceil_div(P, 256), 256, 0, st>>>(P, to_dev(lbs), g_means,
        (const float2 *) g_scales, (const float4 *) g_rots, g->g_xyz, (float2 *) g->g_scaling_raw,
        (float4 *) g->g_rotation_raw, g->g_knn_w, g->g_sp_q, g->g_sp_t, g->g_sp_dr, g->g_sp_ds);
  }
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_preprocess_forward(const fsgs_preprocess_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(a && a->P >= 0 && a->W > 0 && a->H > 0);
  FSGS_REQUIRE(a->tile_counts && a->counters);
  if (a->P == 0) {
    const size_t T = (size_t) ((a->W + kTile - 1) / kTile) * ((a->H + kTile - 1) / kTile);
    cudaMemsetAsync(a->tile_counts, 0, sizeof(int32_t) * T, (cudaStream_t) stream);
    cudaMemsetAsync(a->counters, 0, sizeof(int64_t) * FSGS_NUM_COUNTERS, (cudaStream_t) stream);
    return FSGS_OK;
  }
  FSGS_REQUIRE(a->opac && a->shs && a->Tw2v && a->Tv2s && a->campos);
  FSGS_REQUIRE(a->means2D && a->inverse_m && a->normal_opacity && a->depths && a->radii && a->tiles_touched);
  FSGS_REQUIRE(a->trans_precomp || a->trans_mat);
  if (a->sh_degree > FSGS_MAX_SH_DEGREE) return FSGS_ERR_UNSUPPORTED;
  if (a->sh_degree >= 0) {
    FSGS_REQUIRE(a->colors);
    const int nb = (a->sh_degree + 1) * (a->sh_degree + 1);
    if (a->sh_rest && a->n_rest > 0) FSGS_REQUIRE(a->n_dc >= 1 && a->n_rest >= nb - 1);
    else FSGS_REQUIRE(a->n_dc >= nb);
  }
  if (a->lbs) FSGS_REQUIRE(lbs_valid(a->lbs) && a->warped_means && a->warped_scales && a->warped_rots);
  else FSGS_REQUIRE(a->means && (a->trans_precomp || (a->scales && a->rots)));
  cudaStream_t st = (cudaStream_t) stream;
  PreDev d;
  d.P = a->P, d.W = a->W, d.H = a->H, d.sh_degree = a->sh_degree, d.n_dc = a->n_dc, d.n_rest = a->n_rest;
  d.gx = (a->W + kTile - 1) / kTile, d.gy = (a->H + kTile - 1) / kTile;
  d.means = a->lbs ? a->warped_means : a->means;
  d.scales = (const float2 *) a->scales, d.rots = (const float4 *) a->rots;
  d.opac = a->opac, d.shs = a->shs, d.sh_rest = a->n_rest > 0 ? a->sh_rest : nullptr;
  d.Tw2v = a->Tw2v, d.Tv2s = a->Tv2s, d.campos = a->campos, d.trans_precomp = a->trans_precomp;
  d.culling = a->culling;
  d.warped_means = a->warped_means, d.warped_scales = (float2 *) a->warped_scales, d.warped_rots = (float4 *) a->warped_rots;
  d.means2D = (float2 *) a->means2D, d.colors = a->colors, d.trans_mat = a->trans_mat, d.inverse_m = a->inverse_m;
  d.normal_opacity = (float4 *) a->normal_opacity, d.depths = a->depths, d.radii = a->radii;
  d.tiles_touched = a->tiles_touched, d.records = (float4 *) a->records, d.tile_counts = a->tile_counts;
  d.counters = (unsigned long long *) a->counters;
  d.opacity_is_logit = a->opacity_is_logit;
  cudaMemsetAsync(a->tile_counts, 0, sizeof(int32_t) * (size_t) d.gx * d.gy, st);
  cudaMemsetAsync(a->counters, 0, sizeof(int64_t) * FSGS_NUM_COUNTERS, st);
  if (a->P == 0) return FSGS_OK;
  const int blocks = ceil_div(a->P, kPreBlock);
  const bool high = a->sh_degree > 3;  // degrees 4..7: rare, kept out of the common instantiation
  if (a->lbs && high) preprocess_forward_kernel<true, true><<<blocks, kPreBlock, 0, st>>>(d, to_dev(a->lbs));
  else if (a->lbs) preprocess_forward_kernel<true, false><<<blocks, kPreBlock, 0, st>>>(d, to_dev(a->lbs));
  else if (high) preprocess_forward_kernel<false, true><<<blocks, kPreBlock, 0, st>>>(d, LbsDev());
  else preprocess_forward_kernel<false, false><<<blocks, kPreBlock, 0, st>>>(d, LbsDev());
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_pack_records(int P, const float *means2D, const float *colors, const float *normal_opacity,
    const float *trans_mat, const float *inverse_m, float *records, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && means2D && colors && normal_opacity && trans_mat && inverse_m && records);
  if (P == 0) return FSGS_OK;
  pack_records_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, (const float2 *) means2D, colors,
      (const float4 *) normal_opacity, trans_mat, inverse_m, (float4 *) records);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_transmat_forward(int P, const float *means, const float *scales, const float *rots,
    const float *Tw2v, const float *Tv2s, float *trans_mat, float *normals, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && means && scales && rots && Tw2v && Tv2s && trans_mat && normals);
  if (P == 0) return FSGS_OK;
  transmat_forward_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, means, (const float2 *) scales,
      (const float4 *) rots, Tw2v, Tv2s, trans_mat, normals);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_transmat_backward(int P, const float *scales, const float *rots, const float *Tw2v,
    const float *Tv2s, const float *grad_trans_mat, const float *grad_normals, float *grad_means, float *grad_scales,
    float *grad_rots, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && scales && rots && Tw2v && Tv2s && grad_trans_mat && grad_normals && grad_means &&
               grad_scales && grad_rots);
  if (P == 0) return FSGS_OK;
  transmat_backward_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, (const float2 *) scales,
      (const float4 *) rots, Tw2v, Tv2s, grad_trans_mat, grad_normals, grad_means, (float2 *) grad_scales,
      (float4 *) grad_rots);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_preprocess_backward(const fsgs_preprocess_bwd_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(a && a->P >= 0 && a->W > 0 && a->H > 0);
  FSGS_REQUIRE(a->means && a->scales && a->rots && a->Tw2v && a->Tv2s && a->campos && a->trans_mat && a->radii);
  FSGS_REQUIRE(a->grad_means2D && a->grad_trans_mat && a->grad_inverse_m && a->grad_normal_opacity);
  FSGS_REQUIRE(a->grad_means && a->grad_scales && a->grad_rots && a->grad_opac);
  if (a->sh_degree > FSGS_MAX_SH_DEGREE) return FSGS_ERR_UNSUPPORTED;
  if (a->sh_degree >= 0) FSGS_REQUIRE(a->shs && a->colors && a->grad_colors);
  if (a->P == 0) return FSGS_OK;
  PreBwdDev d;
  d.P = a->P, d.W = a->W, d.H = a->H, d.sh_degree = a->sh_degree, d.n_dc = a->n_dc, d.n_rest = a->n_rest;
  d.means = a->means, d.scales = (const float2 *) a->scales, d.rots = (const float4 *) a->rots;
  d.shs = a->shs, d.sh_rest = a->n_rest > 0 ? a->sh_rest : nullptr;
  d.Tw2v = a->Tw2v, d.Tv2s = a->Tv2s, d.campos = a->campos, d.trans_mat = a->trans_mat, d.colors = a->colors;
  d.radii = a->radii, d.g_means2D = (float2 *) a->grad_means2D, d.g_trans_mat = a->grad_trans_mat;
  d.g_inverse_m = a->grad_inverse_m, d.g_colors = a->grad_colors;
  d.g_normal_opacity = (const float4 *) a->grad_normal_opacity;
  d.g_means = a->grad_means, d.g_scales = (float2 *) a->grad_scales, d.g_rots = (float4 *) a->grad_rots;
  d.g_opac = a->grad_opac, d.g_shs = a->grad_shs, d.g_sh_rest = d.sh_rest ? a->grad_sh_rest : nullptr;
  d.normal_opacity = (const float4 *) a->normal_opacity, d.visible = a->visible, d.accumulate = a->accumulate;
  d.overflow = a->counters ? (const long long *) a->counters + FSGS_CNT_OVERFLOW : nullptr;
  d.sh_source = a->sh_degree >= 0 ? a->sh_source : nullptr;
  if (a->accumulate && a->sh_degree >= 0) {
    // only the layouts whose SH rows are staged through shared memory accumulate: degree 1..3, rows of at most 48
    // floats, the DC coefficient either inside those rows or alone in shs
    const int wide = d.sh_rest ? a->n_rest * 3 : a->n_dc * 3;
    if (a->sh_degree < 1 || a->sh_degree > 3 || wide > kWideMax || (d.sh_rest && a->n_dc != 1)) return FSGS_ERR_UNSUPPORTED;
  }
  if (a->sh_degree > 3) preprocess_backward_kernel<true><<<ceil_div(a->P, kPreBlock), kPreBlock, 0, (cudaStream_t) stream>>>(d);
  else preprocess_backward_kernel<false><<<ceil_div(a->P, kPreBlock), kPreBlock, 0, (cudaStream_t) stream>>>(d);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}


extern "C" int fsgs_sh_grad_from_views(int P, int sh_degree, int n_rest, int n_slots, const int32_t *order,
    const float *sh_source, int64_t slot_stride, float *g_sh_dc, float *g_sh_rest, float *visible,
    fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && sh_degree >= 0 && sh_degree <= 3 && n_rest >= 0 && n_rest <= 15);
  FSGS_REQUIRE(n_slots >= 0 && n_slots <= FSGS_MAX_VIEW_SLOTS && (n_slots == 0 || (order && sh_source)) && g_sh_dc);
  FSGS_REQUIRE(n_rest == 0 || g_sh_rest);
  FSGS_REQUIRE((sh_degree + 1) * (sh_degree + 1) - 1 <= n_rest || n_rest == 0);
  if (P == 0) return FSGS_OK;
  ShSlots slots;
  slots.n = n_slots;
  for (int s = 0; s < n_slots; ++s) {
    FSGS_REQUIRE(order[s] >= 0 && order[s] < n_slots);
    slots.order[s] = order[s];
  }
  sh_grad_from_views_kernel<<<ceil_div(P, kPreBlock), kPreBlock, 0, (cudaStream_t) stream>>>(P, sh_degree, n_rest, slots,
      sh_source, (long long) slot_stride, g_sh_dc, g_sh_rest, visible);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_sh_factors(int P, const float *means, const float *colors, const float *grad_colors,
    const int32_t *radii, const float *campos, const int64_t *counters, int accumulate, float *sh_source,
    float *visible, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && (P == 0 || (means && colors && grad_colors && radii && campos && sh_source)));
  if (P == 0) return FSGS_OK;
  sh_factors_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, means, colors, grad_colors, radii, campos,
      counters ? (const long long *) counters + FSGS_CNT_OVERFLOW : nullptr, accumulate, sh_source, visible);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_transmat_forward_f64(int P, const double *means, const double *scales, const double *rots,
    const double *Tw2v, const double *Tv2s, double *trans_mat, double *normals, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && means && scales && rots && Tw2v && Tv2s && trans_mat && normals);
  if (P == 0) return FSGS_OK;
  transmat_forward_f64_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, means, scales, rots, Tw2v, Tv2s,
      trans_mat, normals);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_transmat_backward_f64(int P, const double *scales, const double *rots, const double *Tw2v,
    const double *Tv2s, const double *grad_trans_mat, const double *grad_normals, double *grad_means,
    double *grad_scales, double *grad_rots, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && scales && rots && Tw2v && Tv2s && grad_trans_mat && grad_normals && grad_means &&
               grad_scales && grad_rots);
  if (P == 0) return FSGS_OK;
  transmat_backward_f64_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, scales, rots, Tw2v, Tv2s,
      grad_trans_mat, grad_normals, grad_means, grad_scales, grad_rots);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}
