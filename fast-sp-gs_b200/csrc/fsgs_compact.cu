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

}  // namespace fsgs

using namespace fsgs;

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
