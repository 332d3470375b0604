// Row compaction of many tensors at once: keep the rows whose mask byte is non-zero, in order.
//
// The reference prunes Gaussians by boolean-indexing every parameter tensor and both Adam moments one after the other
// (fast_2d_gs/gaussian_splatting.py:495-548 `change_optimizer(op='prune')`, 557-568 `prune_points`): some forty
// index kernels and as many host synchronisations.  Here one plan (three small kernels: per-block counts, their scan,
// the total) serves every tensor, and one gather launch moves all of them.
//
// Rows are handled in blocks of 1024: a block compacts its kept row numbers into shared memory, its destination rows
// are contiguous, so for every tensor the block writes one contiguous span (coalesced) and reads whole source rows.
#include "fsgs_common.cuh"

namespace fsgs {

constexpr int kCompactRows = 1024;  // rows per block

struct CompactWs {
  int32_t *block_offsets;  // [blocks + 1] exclusive prefix of kept rows per block; last = total
};

__global__ void __launch_bounds__(kCompactRows) compact_count_kernel(long long N, const uint8_t *__restrict__ keep,
    int32_t *__restrict__ block_counts) {
  const long long i = (long long) blockIdx.x * kCompactRows + threadIdx.x;
  const int k = i < N && keep[i] != 0;
  const int total = __syncthreads_count(k);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = total;
}

// One block: exclusive scan of the block counts in place (+ the total at [blocks]), total also to *count.
__global__ void __launch_bounds__(1024) compact_scan_kernel(int blocks, int32_t *__restrict__ counts,
    long long *__restrict__ count) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < blocks; base += 1024) {
    const int idx = base + threadIdx.x;
    const int v = idx < blocks ? counts[idx] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += n;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    const int carry = s_carry;
    const int excl = carry + (warp > 0 ? s_warp[warp - 1] : 0) + inc - v;
    if (idx < blocks) counts[idx] = excl;
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = carry + s_warp[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    counts[blocks] = s_carry;
    if (count) *count = s_carry;
  }
}

struct CompactTensors {
  const uint32_t *src[FSGS_COMPACT_MAX_TENSORS];
  uint32_t *dst[FSGS_COMPACT_MAX_TENSORS];
  int words[FSGS_COMPACT_MAX_TENSORS];  // 4-byte words per row
  int n;
};

__global__ void __launch_bounds__(kCompactRows) compact_gather_kernel(CompactTensors t, long long N,
    const uint8_t *__restrict__ keep, const int32_t *__restrict__ block_offsets) {
  __shared__ int s_rows[kCompactRows];
  __shared__ int s_warp[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long i = (long long) blockIdx.x * kCompactRows + threadIdx.x;
  const bool k = i < N && keep[i] != 0;
  const unsigned ballot = __ballot_sync(0xffffffffu, k);
  if (lane == 0) s_warp[warp] = __popc(ballot);
  __syncthreads();
  if (warp == 0) {
    int w = s_warp[lane], inc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    s_warp[lane] = inc - w;  // exclusive
  }
  __syncthreads();
  if (k) s_rows[s_warp[warp] + __popc(ballot & ((1u << lane) - 1u))] = threadIdx.x;
  __syncthreads();
  const long long row0 = (long long) blockIdx.x * kCompactRows;
  const long long off = block_offsets[blockIdx.x];
  const int kept = block_offsets[blockIdx.x + 1] - block_offsets[blockIdx.x];
  for (int a = 0; a < t.n; ++a) {
    const int W = t.words[a];
    const uint32_t *src = t.src[a] + row0 * W;
    uint32_t *dst = t.dst[a] + off * W;
    for (int e = threadIdx.x; e < kept * W; e += kCompactRows) {
      const int r = e / W, c = e - r * W;
      dst[e] = src[(long long) s_rows[r] * W + c];
    }
  }
}

// dst[k] = src[index[k]] for every tensor (rows of `words` 4-byte words); index[k] < 0 gives a row of zeros.
// One block per kCompactRows output rows, every tensor walked with consecutive threads on consecutive words.
__global__ void __launch_bounds__(kCompactRows) gather_rows_kernel(CompactTensors t, long long n_out,
    const int32_t *__restrict__ index) {
  __shared__ int s_src[kCompactRows];
  const long long row0 = (long long) blockIdx.x * kCompactRows;
  const int rows = (int) (n_out - row0 < kCompactRows ? n_out - row0 : kCompactRows);
  if ((int) threadIdx.x < rows) s_src[threadIdx.x] = index[row0 + threadIdx.x];
  __syncthreads();
  for (int a = 0; a < t.n; ++a) {
    const int W = t.words[a];
    uint32_t *dst = t.dst[a] + row0 * W;
    for (int e = threadIdx.x; e < rows * W; e += kCompactRows) {
      const int r = e / W, c = e - r * W;
      const int s = s_src[r];
      dst[e] = s >= 0 ? t.src[a][(long long) s * W + c] : 0u;
    }
  }
}

// Clone / split selection of the densification (fast_2d_gs/gaussian_splatting.py:581-622): flags[i] = 1 clone,
// 2 split, 0 neither.  grad = accum / denom with NaN -> 0; clone when grad >= threshold and the larger activated
// scale <= scale_threshold, split when grad >= threshold and it is larger.
__global__ void __launch_bounds__(256) densify_select_kernel(int P, const float *__restrict__ accum,
    const float *__restrict__ denom, const float2 *__restrict__ scaling_raw, float grad_threshold,
    float scale_threshold, uint8_t *__restrict__ flags) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  float g = accum[i] / denom[i];
  if (g != g) g = 0.0f;
  const float2 s = scaling_raw[i];
  const float big = fmaxf(expf(s.x), expf(s.y));
  uint8_t f = 0;
  if (g >= grad_threshold) f = big <= scale_threshold ? 1 : 2;
  flags[i] = f;
}

// Children of the split Gaussians (network.py:1156-1185, 2-D scales): child k of `n` (N copies of every parent,
// copy-major as torch's repeat(N, 1) lays them out) gets position = parent + R(q) (s_x z_0, s_y z_1, 0) with z the
// given standard-normal draws, and log-scale = log(scale / (0.8 N)).
__global__ void __launch_bounds__(256) split_children_kernel(int n, int N, const int32_t *__restrict__ parent,
    const float *__restrict__ z, const float *__restrict__ xyz, const float2 *__restrict__ scaling_raw,
    const float4 *__restrict__ rotation_raw, float *__restrict__ xyz_out, float2 *__restrict__ scaling_out) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  const int p = parent[k];
  const float2 ls = scaling_raw[p];
  const float sx = expf(ls.x), sy = expf(ls.y);
  const float4 r = rotation_raw[p];
  // the reference rotates by the matrix of the RAW quaternion normalised (quaternion_to_R normalises)
  const float inv = rsqrtf(fmaxf(r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w, 1e-24f));
  const float4 q = make_float4(r.x * inv, r.y * inv, r.z * inv, r.w * inv);
  const float a = sx * z[2 * k], b = sy * z[2 * k + 1];
  const float r00 = 1 - 2 * (q.y * q.y + q.z * q.z), r01 = 2 * (q.x * q.y - q.z * q.w);
  const float r10 = 2 * (q.x * q.y + q.z * q.w), r11 = 1 - 2 * (q.x * q.x + q.z * q.z);
  const float r20 = 2 * (q.x * q.z - q.y * q.w), r21 = 2 * (q.x * q.w + q.y * q.z);
  xyz_out[3 * k] = xyz[3 * p] + r00 * a + r01 * b;
  xyz_out[3 * k + 1] = xyz[3 * p + 1] + r10 * a + r11 * b;
  xyz_out[3 * k + 2] = xyz[3 * p + 2] + r20 * a + r21 * b;
  const float f = 0.8f * (float) N;
  scaling_out[k] = make_float2(logf(sx / f), logf(sy / f));
}

// Densification statistics of one view (network.py:1143-1154): for Gaussians with radii > 0,
// accum += |viewspace gradient|, denom += 1, max_radii = max(max_radii, radii).
__global__ void __launch_bounds__(256) densify_stats_kernel(int P, const float2 *__restrict__ viewspace_grad,
    const int32_t *__restrict__ radii, float *__restrict__ accum, float *__restrict__ denom,
    float *__restrict__ max_radii) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const int r = radii[i];
  if (r <= 0) return;
  const float2 g = viewspace_grad[i];
  accum[i] += sqrtf(g.x * g.x + g.y * g.y);
  denom[i] += 1.0f;
  max_radii[i] = fmaxf(max_radii[i], (float) r);
}

}  // namespace fsgs

using namespace fsgs;

extern "C" int fsgs_gather_rows(int n_tensors, const fsgs_row_tensor *tensors, int64_t n_out, const int32_t *index,
    fsgs_stream_t stream) {
  FSGS_REQUIRE(n_tensors >= 0 && (tensors || n_tensors == 0) && n_out >= 0 && n_out < (1ll << 31));
  if (n_tensors > FSGS_COMPACT_MAX_TENSORS) return FSGS_ERR_LIMIT;
  if (n_out == 0 || n_tensors == 0) return FSGS_OK;
  FSGS_REQUIRE(index);
  CompactTensors t;
  t.n = n_tensors;
  for (int k = 0; k < n_tensors; ++k) {
    FSGS_REQUIRE(tensors[k].src && tensors[k].dst && tensors[k].row_words > 0);
    t.src[k] = (const uint32_t *) tensors[k].src, t.dst[k] = (uint32_t *) tensors[k].dst;
    t.words[k] = tensors[k].row_words;
  }
  const int blocks = (int) ((n_out + kCompactRows - 1) / kCompactRows);
  gather_rows_kernel<<<blocks, kCompactRows, 0, (cudaStream_t) stream>>>(t, (long long) n_out, index);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_densify_select(int P, const float *accum, const float *denom, const float *scaling_raw,
    float grad_threshold, float scale_threshold, uint8_t *flags, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && accum && denom && scaling_raw && flags);
  if (P == 0) return FSGS_OK;
  densify_select_kernel<<<(P + 255) / 256, 256, 0, (cudaStream_t) stream>>>(P, accum, denom,
      (const float2 *) scaling_raw, grad_threshold, scale_threshold, flags);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_split_children(int n, int N, const int32_t *parent, const float *z, const float *xyz,
    const float *scaling_raw, const float *rotation_raw, float *xyz_out, float *scaling_out, fsgs_stream_t stream) {
  FSGS_REQUIRE(n >= 0 && N > 0);
  if (n == 0) return FSGS_OK;
  FSGS_REQUIRE(parent && z && xyz && scaling_raw && rotation_raw && xyz_out && scaling_out);
  split_children_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t) stream>>>(n, N, parent, z, xyz,
      (const float2 *) scaling_raw, (const float4 *) rotation_raw, xyz_out, (float2 *) scaling_out);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_densify_stats(int P, const float *viewspace_grad, const int32_t *radii, float *accum,
    float *denom, float *max_radii, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && viewspace_grad && radii && accum && denom && max_radii);
  if (P == 0) return FSGS_OK;
  densify_stats_kernel<<<(P + 255) / 256, 256, 0, (cudaStream_t) stream>>>(P, (const float2 *) viewspace_grad, radii,
      accum, denom, max_radii);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" size_t fsgs_compact_workspace_bytes(int64_t N) {
  const int64_t blocks = (N + kCompactRows - 1) / kCompactRows;
  return sizeof(int32_t) * (size_t) (blocks + 1);
}

extern "C" int fsgs_compact_plan(int64_t N, const uint8_t *keep, void *workspace, size_t workspace_bytes,
    int64_t *count, fsgs_stream_t stream) {
  FSGS_REQUIRE(N >= 0 && N < (1ll << 31) && workspace && (keep || N == 0));
  if (workspace_bytes < fsgs_compact_workspace_bytes(N)) return FSGS_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t) stream;
  const int blocks = (int) ((N + kCompactRows - 1) / kCompactRows);
  int32_t *counts = (int32_t *) workspace;
  if (blocks > 0) compact_count_kernel<<<blocks, kCompactRows, 0, st>>>((long long) N, keep, counts);
  compact_scan_kernel<<<1, 1024, 0, st>>>(blocks, counts, (long long *) count);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_compact_rows(int n_tensors, const fsgs_row_tensor *tensors, int64_t N, const uint8_t *keep,
    const void *workspace, fsgs_stream_t stream) {
  FSGS_REQUIRE(n_tensors >= 0 && (tensors || n_tensors == 0) && N >= 0 && N < (1ll << 31) && workspace);
  if (n_tensors > FSGS_COMPACT_MAX_TENSORS) return FSGS_ERR_LIMIT;
  if (N == 0 || n_tensors == 0) return FSGS_OK;
  FSGS_REQUIRE(keep);
  CompactTensors t;
  t.n = n_tensors;
  for (int k = 0; k < n_tensors; ++k) {
    FSGS_REQUIRE(tensors[k].src && tensors[k].dst && tensors[k].row_words > 0);
    t.src[k] = (const uint32_t *) tensors[k].src, t.dst[k] = (uint32_t *) tensors[k].dst;
    t.words[k] = tensors[k].row_words;
  }
  const int blocks = (int) ((N + kCompactRows - 1) / kCompactRows);
  compact_gather_kernel<<<blocks, kCompactRows, 0, (cudaStream_t) stream>>>(t, (long long) N, keep,
      (const int32_t *) workspace);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}
