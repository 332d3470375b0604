// Tile binning: per-tile list offsets, pair emission, per-tile depth sort (bucket / radix pass on the depth bits
// plus in-bucket ranking; bitonic network for lists beyond 2048 entries).
//
// The reference builds one global list of 64-bit keys (tile << 32 | depth bits), pads every Gaussian's
// slot range up to its rectangle area, and radix-sorts all slots.  Here the tile histogram is already known
// from the preprocess pass, so pairs are scattered straight into their tile's segment and each segment is
// sorted on its own in shared memory by the 64-bit key (depth bits << 32 | Gaussian index).  A Gaussian
// enters a tile at most once, so these keys are unique and the result equals the reference's stable sort:
// within a tile ascending depth bits, ties by ascending Gaussian index.
#include "fsgs_common.cuh"

namespace fsgs {

constexpr int kOrderBins = 4096;     // tile_order buckets: list length >> 4, saturating
constexpr int kSortSmall = 4096;     // keys sorted in static shared memory
constexpr int kSortLarge = 16384;    // keys sorted in opt-in dynamic shared memory
constexpr int kCursorStride = 32;    // ints between the slot cursors of consecutive tiles: one 128-byte line each

struct BinWorkspace {
  unsigned long long *keys;  // [capacity]
  int32_t *cursors;          // [T * kCursorStride]
  long long *starts;         // [T]
  int32_t *eff_counts;       // [T]
};

static size_t align_up(size_t x) { return (x + 255) & ~(size_t) 255; }

static BinWorkspace carve(void *ws, int T, int64_t capacity) {
  BinWorkspace w;
  char *p = (char *) ws;
  w.keys = (unsigned long long *) p;
  p += align_up(sizeof(unsigned long long) * (size_t) (capacity > 0 ? capacity : 1));
  w.cursors = (int32_t *) p;
  p += align_up(sizeof(int32_t) * (size_t) T * kCursorStride);
  w.starts = (long long *) p;
  p += align_up(sizeof(long long) * (size_t) T);
  w.eff_counts = (int32_t *) p;
  return w;
}

// Exclusive prefix sum across the 1024 threads of a block (one value per thread).
__device__ __forceinline__ long long block_exclusive_scan_1024(long long v, long long *s_warp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const long long n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();  // s_warp may still be read from a previous call
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    long long w = s_warp[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const long long n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    s_warp[lane] = w;
  }
  __syncthreads();
  return (warp > 0 ? s_warp[warp - 1] : 0) + inc - v;
}

// One block: exclusive scan of the tile histogram -> list offsets, ranges, zeroed cursors, and the launch
// order of tiles by decreasing list length (bucketed).
__global__ void __launch_bounds__(1024) tile_scan_kernel(int T, const int32_t *__restrict__ tile_counts,
    long long capacity, long long *__restrict__ ranges, long long *__restrict__ starts,
    int32_t *__restrict__ eff_counts, int32_t *__restrict__ cursors, int32_t *__restrict__ tile_order,
    unsigned long long *__restrict__ counters) {
  __shared__ long long s_warp[32];
  __shared__ int s_hist[kOrderBins];
  const int tid = threadIdx.x;
  const int per = (T + 1023) / 1024;
  const int lo = min(T, tid * per), hi = min(T, lo + per);
  long long sum = 0;
  for (int t = lo; t < hi; ++t) sum += tile_counts[t];
  for (int k = tid; k < kOrderBins; k += 1024) s_hist[k] = 0;
  long long off = block_exclusive_scan_1024(sum, s_warp);
  long long dropped = 0;
  for (int t = lo; t < hi; ++t) {
    const int c = tile_counts[t];
    const long long e = off + c;
    const long long e_clip = e < capacity ? e : capacity;
    const long long s_clip = off < capacity ? off : capacity;
    const int eff = (int) (e_clip - s_clip);
    dropped += c - eff;
    starts[t] = s_clip;
    eff_counts[t] = eff;
    cursors[(size_t) t * kCursorStride] = 0;
    ranges[2 * t] = eff > 0 ? s_clip : 0;
    ranges[2 * t + 1] = eff > 0 ? e_clip : 0;
    atomicAdd(&s_hist[min(eff >> 4, kOrderBins - 1)], 1);
    off = e;
  }
  if (dropped) atomicAdd(counters + FSGS_CNT_OVERFLOW, (unsigned long long) dropped);
  __syncthreads();
  // bucket offsets in DEcreasing bucket order: thread t owns buckets 4095-4t .. 4092-4t
  {
    constexpr int kPer = kOrderBins / 1024;
    int h[kPer];
    long long tot = 0;
#pragma unroll
    for (int k = 0; k < kPer; ++k) h[k] = s_hist[kOrderBins - 1 - (tid * kPer + k)], tot += h[k];
    long long acc = block_exclusive_scan_1024(tot, s_warp);
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      s_hist[kOrderBins - 1 - (tid * kPer + k)] = (int) acc;
      acc += h[k];
    }
  }
  __syncthreads();
  for (int t = lo; t < hi; ++t) {
    const int pos = atomicAdd(&s_hist[min(eff_counts[t] >> 4, kOrderBins - 1)], 1);
    tile_order[pos] = t;
  }
}

// One thread per Gaussian: scatter (depth bits, index) into the tile segments; then pad the tail of point_list.
__global__ void __launch_bounds__(256) emit_pairs_kernel(int P, int gx, int gy, const float2 *__restrict__ means2D,
    const float *__restrict__ inverse_m, const float *__restrict__ depths, const float *__restrict__ opac,
    const int32_t *__restrict__ radii, const long long *__restrict__ starts, const int32_t *__restrict__ eff_counts,
    int32_t *__restrict__ cursors, unsigned long long *__restrict__ keys, int32_t *__restrict__ point_list,
    long long capacity, const unsigned long long *__restrict__ counters, int opac_stride) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool has = false;
  int x0 = 0, y0 = 0, x1 = 0, y1 = 0;
  Conic cn = {};
  unsigned long long key = 0;
  if (i < P) {
    const int r = radii[i];
    if (r > 0) {
      const float2 c = means2D[i];
      tile_rect(c.x, c.y, r, gx, gy, x0, y0, x1, y1);
      float IM[9];
#pragma unroll
      for (int k = 0; k < 9; ++k) IM[k] = inverse_m[(size_t) 9 * i + k];
      cn = make_conic(IM, opac[(size_t) i * opac_stride]);
      key = ((unsigned long long) __float_as_uint(depths[i]) << 32) | (unsigned int) i;
      has = true;
    }
  }
  // the warp walks the tiles of its 32 splats together; a slot claimed in one round is filled in the next, so the
  // atomic's round trip overlaps the next round's corner tests
  long long pend_at = -1;
  unsigned long long pend_key = 0;
  warp_for_each_covered_tile(cn, x0, y0, x1, y1, has, (unsigned) (key >> 32), (unsigned) key,
      [&](int x, int y, unsigned k_hi, unsigned k_lo) {
        if (pend_at >= 0) keys[pend_at] = pend_key;
        const int t = y * gx + x;
        const int slot = atomicAdd(cursors + (size_t) t * kCursorStride, 1);
        pend_at = slot < eff_counts[t] ? starts[t] + slot : -1;
        pend_key = ((unsigned long long) k_hi << 32) | k_lo;
      });
  if (pend_at >= 0) keys[pend_at] = pend_key;
  // padding entries of the reference's list: point_list[R* .. min(R, capacity)) = -1
  const long long n_pairs = (long long) counters[FSGS_CNT_PAIRS];
  const long long n_slots = (long long) counters[FSGS_CNT_SLOTS];
  const long long hi = n_slots < capacity ? n_slots : capacity;
  for (long long k = n_pairs + (long long) blockIdx.x * blockDim.x + threadIdx.x; k < hi;
       k += (long long) gridDim.x * blockDim.x)
    point_list[k] = -1;
}

// Bitonic sort of n <= CAP 64-bit keys held in shared memory (padded with all-ones to a power of two).
template <int CAP>
__device__ __forceinline__ void smem_bitonic(unsigned long long *s, int n, const unsigned long long *__restrict__ src,
    int32_t *__restrict__ dst) {
  int np2 = 32;
  while (np2 < n) np2 <<= 1;
  for (int k = threadIdx.x; k < np2; k += blockDim.x) s[k] = k < n ? src[k] : ~0ull;
  __syncthreads();
  // Comparator t of a step with stride j works on elements i and i + j of the 2j-block that holds i; for j <= 32 the
  // 32 comparators of a warp stay inside 64 consecutive elements that no other warp touches, whatever j is, so runs
  // of such steps need only a warp barrier.  A block barrier is paid only around steps with j >= 64 (and at the end).
  for (int k = 2; k <= np2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < (np2 >> 1); t += blockDim.x) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
        const int l = i | j;
        const unsigned long long a = s[i], b = s[l];
        const bool asc = (i & k) == 0;
        if ((a > b) == asc) s[i] = b, s[l] = a;
      }
      const int next_j = j > 1 ? (j >> 1) : k;  // first stride of the next stage is k
      if (j > 32 || next_j > 32 || (j == 1 && k == np2)) __syncthreads();
      else __syncwarp();
    }
  }
  for (int k = threadIdx.x; k < n; k += blockDim.x) dst[k] = (int32_t) (unsigned int) (s[k] & 0xffffffffull);
}

// Bucket sort of n <= kBucketKeys unique 64-bit keys (depth bits << 32 | index) in shared memory, 256 threads:
// a radix pass on the depth bits scaled to the tile's own depth range (kBuckets buckets, monotone in the key), then
// every key finds its rank among the few keys of its bucket by direct comparison of the full key.  About a tenth of
// the instructions of a bitonic network at the list lengths that matter (a few hundred keys).
constexpr int kBuckets = 1024;
constexpr int kBucketKeys = kSortSmall / 2;  // the scattered copy lives in the second half of the key buffer

__device__ __forceinline__ int depth_bucket(unsigned long long key, unsigned lo, float scale) {
  const float d = (float) ((unsigned) (key >> 32) - lo);  // conversions and the product round monotonically
  return min(kBuckets - 1, (int) (d * scale));
}

__device__ __forceinline__ void smem_bucket_sort(unsigned long long *s, int *s_start, int *s_cursor, unsigned *s_red,
    int n, const unsigned long long *__restrict__ src, int32_t *__restrict__ dst) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned lo = 0xffffffffu, hi = 0u;
  for (int k = tid; k < n; k += 256) {
    const unsigned long long key = src[k];
    s[k] = key;
    const unsigned d = (unsigned) (key >> 32);
    lo = min(lo, d), hi = max(hi, d);
  }
  for (int k = tid; k < kBuckets; k += 256) s_cursor[k] = 0;
  for (int o = 16; o > 0; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if (lane == 0) s_red[warp] = lo, s_red[8 + warp] = hi;
  __syncthreads();
  lo = s_red[0], hi = s_red[8];
#pragma unroll
  for (int w = 1; w < 8; ++w) lo = min(lo, s_red[w]), hi = max(hi, s_red[8 + w]);
  const float scale = (float) kBuckets / ((float) (hi - lo) + 1.0f);
  // histogram
  for (int k = tid; k < n; k += 256) atomicAdd(&s_cursor[depth_bucket(s[k], lo, scale)], 1);
  __syncthreads();
  // exclusive scan of the kBuckets counts: four per thread, warp scan, then the eight warp totals
  {
    int c[kBuckets / 256], sum = 0;
#pragma unroll
    for (int k = 0; k < kBuckets / 256; ++k) c[k] = s_cursor[tid * (kBuckets / 256) + k], sum += c[k];
    int inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += v;
    }
    __syncthreads();  // s_red was read above
    if (lane == 31) s_red[warp] = (unsigned) inc;
    __syncthreads();
    int base = inc - sum;
    for (int w = 0; w < warp; ++w) base += (int) s_red[w];
#pragma unroll
    for (int k = 0; k < kBuckets / 256; ++k) {
      s_start[tid * (kBuckets / 256) + k] = base;
      s_cursor[tid * (kBuckets / 256) + k] = base;
      base += c[k];
    }
    if (tid == 255) s_start[kBuckets] = base;
  }
  __syncthreads();
  // scatter into bucket order (any order inside a bucket)
  unsigned long long *t = s + kBucketKeys;
  for (int k = tid; k < n; k += 256) {
    const unsigned long long key = s[k];
    t[atomicAdd(&s_cursor[depth_bucket(key, lo, scale)], 1)] = key;
  }
  __syncthreads();
  // rank inside the bucket by the full key (keys are unique)
  for (int k = tid; k < n; k += 256) {
    const unsigned long long key = t[k];
    const int b = depth_bucket(key, lo, scale);
    const int b0 = s_start[b], b1 = s_start[b + 1];
    int rank = 0;
    for (int e = b0; e < b1; ++e) rank += t[e] < key;
    dst[b0 + rank] = (int32_t) (unsigned int) (key & 0xffffffffull);
  }
}

__global__ void __launch_bounds__(256) tile_sort_small_kernel(int T, const int32_t *__restrict__ tile_order,
    const long long *__restrict__ starts, const int32_t *__restrict__ eff_counts,
    const unsigned long long *__restrict__ keys, int32_t *__restrict__ point_list) {
  __shared__ unsigned long long s[kSortSmall];
  __shared__ int s_start[kBuckets + 1], s_cursor[kBuckets];
  __shared__ unsigned s_red[16];
  const int tile = tile_order[blockIdx.x];
  const int n = eff_counts[tile];
  if (n == 0 || n > kSortSmall) return;
  const long long st = starts[tile];
  if (n <= kBucketKeys) smem_bucket_sort(s, s_start, s_cursor, s_red, n, keys + st, point_list + st);
  else smem_bitonic<kSortSmall>(s, n, keys + st, point_list + st);
}

// Lists longer than kSortSmall sit at the front of tile_order.  Up to kSortLarge keys: shared-memory sort;
// beyond: rank by counting smaller keys (keys are unique), slow but exact and needs no extra memory.
__global__ void __launch_bounds__(1024) tile_sort_large_kernel(int T, const int32_t *__restrict__ tile_order,
    const long long *__restrict__ starts, const int32_t *__restrict__ eff_counts,
    const unsigned long long *__restrict__ keys, int32_t *__restrict__ point_list) {
  extern __shared__ unsigned long long s_dyn[];
  for (int b = blockIdx.x; b < T; b += gridDim.x) {
    const int tile = tile_order[b];
    const int n = eff_counts[tile];
    if (n < kSortSmall) break;  // tile_order is bucketed by n >> 4 in decreasing order
    if (n == kSortSmall) continue;
    const long long st = starts[tile];
    if (n <= kSortLarge) {
      __syncthreads();
      smem_bitonic<kSortLarge>(s_dyn, n, keys + st, point_list + st);
    } else {
      const unsigned long long *src = keys + st;
      for (int e = threadIdx.x; e < n; e += blockDim.x) {
        const unsigned long long mine = src[e];
        int rank = 0;
        for (int k = 0; k < n; ++k) rank += src[k] < mine;
        point_list[st + rank] = (int32_t) (unsigned int) (mine & 0xffffffffull);
      }
    }
  }
}

}  // namespace fsgs

using namespace fsgs;

extern "C" size_t fsgs_bin_workspace_bytes(int W, int H, int64_t capacity) {
  const int T = ((W + kTile - 1) / kTile) * ((H + kTile - 1) / kTile);
  return align_up(sizeof(unsigned long long) * (size_t) (capacity > 0 ? capacity : 1)) +
         align_up(sizeof(int32_t) * (size_t) T * kCursorStride) + align_up(sizeof(long long) * (size_t) T) +
         align_up(sizeof(int32_t) * (size_t) T);
}

// The four launches of the binning on a carved workspace: scan, pair emission, the two per-tile sorts.
static int launch_binning(const fsgs_bin_args *a, const BinWorkspace &w, cudaStream_t st) {
  const int gx = (a->W + kTile - 1) / kTile, gy = (a->H + kTile - 1) / kTile, T = gx * gy;
  tile_scan_kernel<<<1, 1024, 0, st>>>(T, a->tile_counts, (long long) a->capacity, (long long *) a->ranges, w.starts,
      w.eff_counts, w.cursors, a->tile_order, (unsigned long long *) a->counters);
  FSGS_LAUNCH_CHECK();
  const int blocks = max(1, ceil_div(a->P, 256));
  emit_pairs_kernel<<<blocks, 256, 0, st>>>(a->P, gx, gy, (const float2 *) a->means2D, a->inverse_m, a->depths, a->opac,
      a->radii, w.starts, w.eff_counts, w.cursors, w.keys, a->point_list, (long long) a->capacity,
      (const unsigned long long *) a->counters, a->opac_stride > 0 ? a->opac_stride : 1);
  FSGS_LAUNCH_CHECK();
  tile_sort_small_kernel<<<T, 256, 0, st>>>(T, a->tile_order, w.starts, w.eff_counts, w.keys, a->point_list);
  FSGS_LAUNCH_CHECK();
  // the opt-in to 128 KB of dynamic shared memory is a per-device attribute of the kernel
  constexpr int kMaxDev = 64;
  static bool attr_set[kMaxDev] = {false};
  const size_t dyn = sizeof(unsigned long long) * kSortLarge;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return FSGS_ERR_LAUNCH;
  if (dev < 0 || dev >= kMaxDev || !attr_set[dev]) {
    if (cudaFuncSetAttribute(tile_sort_large_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) dyn) !=
        cudaSuccess)
      return FSGS_ERR_LAUNCH;
    if (dev >= 0 && dev < kMaxDev) attr_set[dev] = true;
  }
  tile_sort_large_kernel<<<min(T, 148), 1024, dyn, st>>>(T, a->tile_order, w.starts, w.eff_counts, w.keys,
      a->point_list);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_bin_tiles(const fsgs_bin_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(a && a->P >= 0 && a->W > 0 && a->H > 0 && a->capacity >= 0);
  FSGS_REQUIRE(a->tile_counts && a->counters);
  FSGS_REQUIRE(a->P == 0 || (a->means2D && a->inverse_m && a->depths && a->opac && a->radii));
  FSGS_REQUIRE(a->ranges && a->tile_order && a->workspace && (a->point_list || a->capacity == 0));
  if (a->workspace_bytes < fsgs_bin_workspace_bytes(a->W, a->H, a->capacity)) return FSGS_ERR_WORKSPACE;
  const int T = ((a->W + kTile - 1) / kTile) * ((a->H + kTile - 1) / kTile);
  return launch_binning(a, carve(a->workspace, T, a->capacity), (cudaStream_t) stream);
}

// ------------------------------------------------------------------------------------------------
// Binning without a caller workspace: the scratch is a fixed device array of this library.
// ------------------------------------------------------------------------------------------------

namespace fsgs {
constexpr size_t kNoallocKeysBytes = sizeof(unsigned long long) * (size_t) FSGS_NOALLOC_MAX_PAIRS;
constexpr size_t kNoallocTileBytes =
    (sizeof(int32_t) * kCursorStride + sizeof(long long) + sizeof(int32_t)) * (size_t) FSGS_NOALLOC_MAX_TILES;
constexpr size_t kNoallocBytes = kNoallocKeysBytes + kNoallocTileBytes + 3 * 256;
// Held by every device that loads the library.  In host code this name is only a handle: the device address
// comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_bin_scratch[kNoallocBytes];
constexpr int kMaxDevices = 64;
static void *g_bin_scratch_ptr[kMaxDevices] = {nullptr};
}  // namespace fsgs

extern "C" int fsgs_bin_tiles_noalloc(const fsgs_bin_args *a, fsgs_stream_t stream) {
  FSGS_REQUIRE(a && a->P >= 0 && a->W > 0 && a->H > 0 && a->capacity >= 0);
  FSGS_REQUIRE(a->tile_counts && a->counters);
  FSGS_REQUIRE(a->P == 0 || (a->means2D && a->inverse_m && a->depths && a->opac && a->radii));
  FSGS_REQUIRE(a->ranges && a->tile_order && (a->point_list || a->capacity == 0));
  const int T = ((a->W + kTile - 1) / kTile) * ((a->H + kTile - 1) / kTile);
  if (a->capacity > FSGS_NOALLOC_MAX_PAIRS || T > FSGS_NOALLOC_MAX_TILES) return FSGS_ERR_LIMIT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FSGS_ERR_LAUNCH;
  if (g_bin_scratch_ptr[dev] == nullptr) {  // set-up: first call on this device
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_bin_scratch) != cudaSuccess || ptr == nullptr) return FSGS_ERR_LAUNCH;
    g_bin_scratch_ptr[dev] = ptr;
  }
  cudaStream_t st = (cudaStream_t) stream;
  // same layout as a caller workspace sized for the maximum: keys | cursors | starts | effective counts
  BinWorkspace w;
  char *p = (char *) g_bin_scratch_ptr[dev];
  w.keys = (unsigned long long *) p;
  p += align_up(kNoallocKeysBytes);
  w.cursors = (int32_t *) p;
  p += align_up(sizeof(int32_t) * (size_t) FSGS_NOALLOC_MAX_TILES * kCursorStride);
  w.starts = (long long *) p;
  p += align_up(sizeof(long long) * (size_t) FSGS_NOALLOC_MAX_TILES);
  w.eff_counts = (int32_t *) p;
  // every scratch word that is read is written first: the scan kernel fills cursors / starts / counts for all
  // tiles, the emit kernel fills exactly the key slots the sort kernels read
  return launch_binning(a, w, st);
}
