// Exact nearest control-point search in fp32 SIMT: top-1 (any dimension) and top-K (3-D).
// Control points are staged through shared memory in chunks; every thread owns one query and scans the chunk
// with broadcast reads.  Squared distances are accumulated by direct differences in dimension order
// (reference src/other/cdist_top.cu:19-23).  cdist_top fuses each square into the running sum, sum = fma(t, t, sum),
// as the reference's CUDA build does: indices and distances equal that kernel's bit for bit.  The K-nearest search
// (no counterpart in the reference's own code) keeps multiply and add separate and so equals a plain CPU loop.
#include "fsgs_common.cuh"

namespace fsgs {

constexpr int kChunk = 1024;  // control points per shared-memory chunk (3-D path)

// sum + t * t as one fused multiply-add, float and double
__device__ __forceinline__ float add_sq(float sum, float t) { return __fmaf_rn(t, t, sum); }
__device__ __forceinline__ double add_sq(double sum, double t) { return __fma_rn(t, t, sum); }
__device__ __forceinline__ float root(float v) { return sqrtf(v); }
__device__ __forceinline__ double root(double v) { return sqrt(v); }

template <typename T, int D>
__global__ void __launch_bounds__(128) cdist_top_kernel(int N, int M, const T *__restrict__ x1,
    const T *__restrict__ x2, int largest, T *__restrict__ dist, int64_t *__restrict__ index) {
  __shared__ T s_c[kChunk * D];
  const int b = blockIdx.y;
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const T *c = x2 + (size_t) b * M * D;
  T p[D];
  if (n < N) {
#pragma unroll
    for (int k = 0; k < D; ++k) p[k] = x1[((size_t) b * N + n) * D + k];
  }
  T best = 0;
  int besti = 0;
  for (int m0 = 0; m0 < M; m0 += kChunk) {
    const int cnt = min(kChunk, M - m0);
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * D; e += blockDim.x) s_c[e] = c[(size_t) m0 * D + e];
    __syncthreads();
    if (n < N) {
      for (int m = 0; m < cnt; ++m) {
        T sum = 0;
#pragma unroll
        for (int k = 0; k < D; ++k) sum = add_sq(sum, p[k] - s_c[m * D + k]);
        // replace when (sum > best) == largest: exact ties go to the last index when searching the nearest
        if ((m0 + m) == 0 || (int) (sum > best) == largest) best = sum, besti = m0 + m;
      }
    }
  }
  if (n < N) {
    dist[(size_t) b * N + n] = root(best);
    index[(size_t) b * N + n] = besti;
  }
}

// any dimension: control points read through the cache
template <typename T>
__global__ void __launch_bounds__(128) cdist_top_generic_kernel(int N, int M, int D, const T *__restrict__ x1,
    const T *__restrict__ x2, int largest, T *__restrict__ dist, int64_t *__restrict__ index) {
  const int b = blockIdx.y;
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const T *p = x1 + ((size_t) b * N + n) * D;
  const T *c = x2 + (size_t) b * M * D;
  T best = 0;
  int besti = 0;
  for (int m = 0; m < M; ++m) {
    T sum = 0;
    for (int k = 0; k < D; ++k) sum = add_sq(sum, p[k] - __ldg(c + (size_t) m * D + k));
    if (m == 0 || (int) (sum > best) == largest) best = sum, besti = m;
  }
  dist[(size_t) b * N + n] = root(best);
  index[(size_t) b * N + n] = besti;
}

// (reference src/other/cdist_top.cu:86-105)
template <typename T>
__global__ void __launch_bounds__(256) cdist_top_backward_kernel(int B, int N, int M, int D, const T *__restrict__ x1,
    const T *__restrict__ x2, const T *__restrict__ dist, const int64_t *__restrict__ index,
    const T *__restrict__ grad_dist, T *__restrict__ g1, T *__restrict__ g2) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * N) return;
  const int b = i / N;
  const size_t j = (size_t) b * M + (size_t) index[i];
  const T g = grad_dist[i] / dist[i];
  for (int k = 0; k < D; ++k) {
    const T t = g * (x1[(size_t) i * D + k] - x2[j * D + k]);
    g1[(size_t) i * D + k] = t;
    atomicAdd(g2 + j * D + k, -t);
  }
}

// K nearest, ascending by (distance, index).  A candidate replaces the current worst only when strictly
// closer, and is inserted after entries of equal distance, so ties keep the lower index first.
template <int K>
__global__ void __launch_bounds__(128) knn3_kernel(int N, int M, const float *__restrict__ x, const float *__restrict__ c,
    float *__restrict__ d2, int64_t *__restrict__ index) {
  __shared__ float s_c[kChunk * 3];
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  float px = 0, py = 0, pz = 0;
  if (n < N) px = x[3 * (size_t) n], py = x[3 * (size_t) n + 1], pz = x[3 * (size_t) n + 2];
  float bd[K];
  int bi[K];
#pragma unroll
  for (int k = 0; k < K; ++k) bd[k] = __int_as_float(0x7f800000), bi[k] = -1;
  for (int m0 = 0; m0 < M; m0 += kChunk) {
    const int cnt = min(kChunk, M - m0);
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * 3; e += blockDim.x) s_c[e] = c[(size_t) m0 * 3 + e];
    __syncthreads();
    if (n < N) {
      for (int m = 0; m < cnt; ++m) {
        const float tx = px - s_c[3 * m], ty = py - s_c[3 * m + 1], tz = pz - s_c[3 * m + 2];
        const float sum = __fadd_rn(__fadd_rn(__fmul_rn(tx, tx), __fmul_rn(ty, ty)), __fmul_rn(tz, tz));
        if (sum < bd[K - 1]) {
          bd[K - 1] = sum, bi[K - 1] = m0 + m;
#pragma unroll
          for (int k = K - 1; k > 0; --k) {
            if (bd[k - 1] > bd[k]) {
              const float td = bd[k];
              bd[k] = bd[k - 1], bd[k - 1] = td;
              const int ti = bi[k];
              bi[k] = bi[k - 1], bi[k - 1] = ti;
            }
          }
        }
      }
    }
  }
  if (n < N) {
#pragma unroll
    for (int k = 0; k < K; ++k) d2[(size_t) n * K + k] = bd[k], index[(size_t) n * K + k] = bi[k];
  }
}

template <int K>
static void launch_knn(int N, int M, const float *x, const float *c, float *d2, int64_t *index, cudaStream_t st) {
  knn3_kernel<K><<<ceil_div(N, 128), 128, 0, st>>>(N, M, x, c, d2, index);
}

// ------------------------------------------------------------------------------------------------
// The same K-nearest search through a uniform grid over the control points: exact, same distances (identical
// arithmetic per pair), same order -- ascending by (distance, index) -- but a query only evaluates the control
// points of the grid cells around it, shell by shell, until no unvisited cell can hold anything closer than its
// current K-th candidate.  At 4096 control points that is a few hundred evaluations per query instead of 4096.
// ------------------------------------------------------------------------------------------------

constexpr int kGridMax = 16;  // cells per axis at most (16^3 cell counters fit one block's shared memory)

struct GridHeader {
  float lo[3], h[3], inv_h[3];
  int G, M;
};

// workspace: GridHeader | cell_start [G^3 + 1] | points [M] float4 (x, y, z, index bits), grouped by cell
__global__ void __launch_bounds__(1024) knn_grid_build_kernel(int M, int G, const float *__restrict__ c, GridHeader *hdr,
    int *__restrict__ cell_start, float4 *__restrict__ sorted) {
  __shared__ float s_red[6][32];
  __shared__ int s_count[kGridMax * kGridMax * kGridMax];
  __shared__ int s_warp[32];
  __shared__ GridHeader s_h;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float inf = __int_as_float(0x7f800000);
  float lo[3] = {inf, inf, inf}, hi[3] = {-inf, -inf, -inf};
  for (int m = tid; m < M; m += 1024)
    for (int a = 0; a < 3; ++a) lo[a] = fminf(lo[a], c[3 * m + a]), hi[a] = fmaxf(hi[a], c[3 * m + a]);
  for (int a = 0; a < 3; ++a) {
    for (int o = 16; o > 0; o >>= 1) {
      lo[a] = fminf(lo[a], __shfl_xor_sync(0xffffffffu, lo[a], o));
      hi[a] = fmaxf(hi[a], __shfl_xor_sync(0xffffffffu, hi[a], o));
    }
    if (lane == 0) s_red[a][warp] = lo[a], s_red[3 + a][warp] = hi[a];
  }
  __syncthreads();
  if (tid == 0) {
    for (int a = 0; a < 3; ++a) {
      float l = inf, u = -inf;
      for (int w = 0; w < 32; ++w) l = fminf(l, s_red[a][w]), u = fmaxf(u, s_red[3 + a][w]);
      s_h.lo[a] = l;
      s_h.h[a] = fmaxf((u - l) / (float) G, 1e-20f);
      s_h.inv_h[a] = 1.0f / s_h.h[a];
    }
    s_h.G = G, s_h.M = M;
    *hdr = s_h;
  }
  const int cells = G * G * G;
  for (int k = tid; k < cells; k += 1024) s_count[k] = 0;
  __syncthreads();
  auto cell_of = [&](int m) {
    int id[3];
    for (int a = 0; a < 3; ++a) id[a] = min(G - 1, max(0, (int) ((c[3 * m + a] - s_h.lo[a]) * s_h.inv_h[a])));
    return (id[2] * G + id[1]) * G + id[0];
  };
  for (int m = tid; m < M; m += 1024) atomicAdd(&s_count[cell_of(m)], 1);
  __syncthreads();
  // exclusive scan of up to 4096 counters: four per thread
  int v[4], sum = 0;
  for (int u = 0; u < 4; ++u) {
    const int k = tid * 4 + u;
    v[u] = k < cells ? s_count[k] : 0;
    sum += v[u];
  }
  int inc = sum;
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = s_warp[lane], wi = w;
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    s_warp[lane] = wi - w;
  }
  __syncthreads();
  int run = s_warp[warp] + inc - sum;
  for (int u = 0; u < 4; ++u) {
    const int k = tid * 4 + u;
    if (k < cells) cell_start[k] = run, s_count[k] = run;  // s_count becomes the scatter cursor
    run += v[u];
  }
  if (tid == 0) cell_start[cells] = M;
  __syncthreads();
  for (int m = tid; m < M; m += 1024) {
    const int pos = atomicAdd(&s_count[cell_of(m)], 1);
    sorted[pos] = make_float4(c[3 * m], c[3 * m + 1], c[3 * m + 2], __int_as_float(m));
  }
}

template <int K>
__global__ void __launch_bounds__(128) knn_grid_query_kernel(int N, const float *__restrict__ x,
    const GridHeader *__restrict__ hdr, const int *__restrict__ cell_start, const float4 *__restrict__ sorted,
    float *__restrict__ d2, int64_t *__restrict__ index) {
  __shared__ int s_start[kGridMax * kGridMax * kGridMax + 1];
  const GridHeader H = *hdr;
  const int G = H.G, cells = G * G * G;
  for (int k = threadIdx.x; k <= cells; k += blockDim.x) s_start[k] = cell_start[k];
  __syncthreads();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const float q[3] = {x[3 * (size_t) n], x[3 * (size_t) n + 1], x[3 * (size_t) n + 2]};
  int cq[3];
  for (int a = 0; a < 3; ++a) cq[a] = min(G - 1, max(0, (int) ((q[a] - H.lo[a]) * H.inv_h[a])));
  const float inf = __int_as_float(0x7f800000);
  float bd[K];
  int bi[K];
#pragma unroll
  for (int k = 0; k < K; ++k) bd[k] = inf, bi[k] = 0x7fffffff;
  for (int r = 0; r < G; ++r) {
    const int z0 = max(0, cq[2] - r), z1 = min(G - 1, cq[2] + r);
    const int y0 = max(0, cq[1] - r), y1 = min(G - 1, cq[1] + r);
    const int x0 = max(0, cq[0] - r), x1 = min(G - 1, cq[0] + r);
    for (int cz = z0; cz <= z1; ++cz)
      for (int cy = y0; cy <= y1; ++cy) {
        const bool face = abs(cz - cq[2]) == r || abs(cy - cq[1]) == r;
        // on a face row every cell belongs to the shell; otherwise only the two ends of the row do
        for (int cx = x0; cx <= x1; cx += (face || r == 0) ? 1 : max(1, x1 - x0)) {
          if (!face && abs(cx - cq[0]) != r) continue;
          const int cell = (cz * G + cy) * G + cx;
          for (int e = s_start[cell]; e < s_start[cell + 1]; ++e) {
            const float4 p = __ldg(sorted + e);
            const float tx = q[0] - p.x, ty = q[1] - p.y, tz = q[2] - p.z;
            const float sum = __fadd_rn(__fadd_rn(__fmul_rn(tx, tx), __fmul_rn(ty, ty)), __fmul_rn(tz, tz));
            const int id = __float_as_int(p.w);
            if (sum < bd[K - 1] || (sum == bd[K - 1] && id < bi[K - 1])) {
              bd[K - 1] = sum, bi[K - 1] = id;
#pragma unroll
              for (int k = K - 1; k > 0; --k) {
                if (bd[k - 1] > bd[k] || (bd[k - 1] == bd[k] && bi[k - 1] > bi[k])) {
                  const float td = bd[k];
                  bd[k] = bd[k - 1], bd[k - 1] = td;
                  const int ti = bi[k];
                  bi[k] = bi[k - 1], bi[k - 1] = ti;
                }
              }
            }
          }
        }
      }
    // Everything not yet visited lies outside the cube of cells [cq - r, cq + r]: at least `margin` away along some
    // axis (sides of the cube that coincide with the grid's boundary have nothing beyond them).
    float margin = inf;
    for (int a = 0; a < 3; ++a) {
      // rounding: a control point is assigned to its cell by a rounded product, and the faces below are rounded
      // sums; both errors are a few units in the last place of the coordinates involved
      const float slack = 4e-6f * (fabsf(q[a]) + fabsf(H.lo[a]) + (float) G * H.h[a]);
      if (cq[a] - r > 0) margin = fminf(margin, q[a] - (H.lo[a] + (float) (cq[a] - r) * H.h[a]) - slack);
      if (cq[a] + r < G - 1) margin = fminf(margin, (H.lo[a] + (float) (cq[a] + r + 1) * H.h[a]) - q[a] - slack);
    }
    if (margin == inf) break;                       // the cube covers the grid
    margin *= 1.0f - 1e-5f;                         // and the squared bound stays below the true squared distance
    if (margin > 0.0f && bd[K - 1] < margin * margin) break;
  }
#pragma unroll
  for (int k = 0; k < K; ++k) {
    d2[(size_t) n * K + k] = bd[k];
    index[(size_t) n * K + k] = bi[k] == 0x7fffffff ? -1 : bi[k];
  }
}

template <int K>
static void launch_knn_grid(int N, const float *x, const GridHeader *hdr, const int *cell_start, const float4 *sorted,
    float *d2, int64_t *index, cudaStream_t st) {
  knn_grid_query_kernel<K><<<ceil_div(N, 128), 128, 0, st>>>(N, x, hdr, cell_start, sorted, d2, index);
}

// ------------------------------------------------------------------------------------------------
// masked Adam (reference src/other/adam_masked_update.cu:9-28): same operation order per element
// ------------------------------------------------------------------------------------------------

// m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g g ; p += -lr m / (sqrt(v) + eps).  The two accumulations are fused the
// way the reference build fuses them, so parameters and moments equal the reference's bit for bit.
__device__ __forceinline__ void adam_element(float &p, float g, float &m, float &v, float lr, float b1, float b2,
    float eps) {
  m = __fmaf_rn(__fsub_rn(1.0f, b1), g, __fmul_rn(b1, m));
  v = __fmaf_rn(__fmul_rn(__fsub_rn(1.0f, b2), g), g, __fmul_rn(b2, v));
  const float step = __fdiv_rn(__fmul_rn(-lr, m), __fadd_rn(__fsqrt_rn(v), eps));
  p = __fadd_rn(p, step);
}

__global__ void __launch_bounds__(256) adam_masked_kernel(float *__restrict__ param, const float *__restrict__ grad,
    float *__restrict__ exp_avg, float *__restrict__ exp_avg_sq, const uint8_t *__restrict__ visible, float lr, float b1,
    float b2, float eps, long long N, int M) {
  const long long total = N * M;
  for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long) gridDim.x * blockDim.x) {
    if (!visible[i / M]) continue;
    float p = param[i], m = exp_avg[i], v = exp_avg_sq[i];
    adam_element(p, grad[i], m, v, lr, b1, b2, eps);
    param[i] = p, exp_avg[i] = m, exp_avg_sq[i] = v;
  }
}

struct AdamMulti {
  fsgs_adam_tensor t[FSGS_ADAM_MAX_TENSORS];
  long long chunk_start[FSGS_ADAM_MAX_TENSORS + 1];  // prefix sums of ceil(N * M / 4)
  int vec[FSGS_ADAM_MAX_TENSORS];                     // all four arrays 16-byte aligned
  unsigned magic[FSGS_ADAM_MAX_TENSORS];              // floor(2^32 / M), or 0: divide the slow way
  int n;
};

// the visibility mask as bytes (non-zero: visible) or as floats (> 0: visible)
__device__ __forceinline__ bool is_visible(const uint8_t *m, long long row) { return m[row] != 0; }
__device__ __forceinline__ bool is_visible(const float *m, long long row) { return m[row] > 0.0f; }

// e / M and e % M for e < 2^32 with magic = floor(2^32 / M): the high product is the quotient or one less.
__device__ __forceinline__ void divmod(long long e, int M, unsigned magic, long long &q, int &r) {
  if (magic != 0 && e < (1ll << 32)) {
    unsigned qq = __umulhi((unsigned) e, magic);
    unsigned rr = (unsigned) e - qq * (unsigned) M;
    if (rr >= (unsigned) M) ++qq, rr -= (unsigned) M;
    q = qq, r = (int) rr;
  } else {
    q = e / M, r = (int) (e - q * M);
  }
}

// One launch for all tensors.  Each tensor is walked as a flat array in chunks of four consecutive floats (one
// 16-byte access per array), consecutive threads taking consecutive chunks, so every access is fully coalesced
// whatever the row length.  A chunk may straddle two Gaussians: elements of an invisible one keep their bits.
// Chunks without a visible element touch nothing but the mask.
template <typename MaskT>
__global__ void __launch_bounds__(256) adam_masked_multi_kernel(AdamMulti a, const MaskT *__restrict__ visible,
    long long N, float b1, float b2) {
  const long long total = a.chunk_start[a.n];
  for (long long chunk = (long long) blockIdx.x * blockDim.x + threadIdx.x; chunk < total;
       chunk += (long long) gridDim.x * blockDim.x) {
    int k = 0;
    while (k + 1 < a.n && chunk >= a.chunk_start[k + 1]) ++k;
    const fsgs_adam_tensor &t = a.t[k];
    const long long e0 = (chunk - a.chunk_start[k]) * 4;
    const long long n_el = N * t.M;
    const int cnt = (int) (n_el - e0 < 4 ? n_el - e0 : 4);
    long long row;
    int col;
    divmod(e0, t.M, a.magic[k], row, col);
    bool vis[4];
    bool any = false;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      vis[u] = u < cnt && is_visible(visible, row);
      any |= vis[u];
      if (++col == t.M) col = 0, ++row;
    }
    if (!any) continue;
    if (a.vec[k] && cnt == 4) {
      float4 p = *reinterpret_cast<const float4 *>(t.param + e0);
      const float4 g = *reinterpret_cast<const float4 *>(t.grad + e0);
      float4 m = *reinterpret_cast<const float4 *>(t.exp_avg + e0);
      float4 v = *reinterpret_cast<const float4 *>(t.exp_avg_sq + e0);
      if (vis[0]) adam_element(p.x, g.x, m.x, v.x, t.lr, b1, b2, t.eps);
      if (vis[1]) adam_element(p.y, g.y, m.y, v.y, t.lr, b1, b2, t.eps);
      if (vis[2]) adam_element(p.z, g.z, m.z, v.z, t.lr, b1, b2, t.eps);
      if (vis[3]) adam_element(p.w, g.w, m.w, v.w, t.lr, b1, b2, t.eps);
      *reinterpret_cast<float4 *>(t.param + e0) = p;
      *reinterpret_cast<float4 *>(t.exp_avg + e0) = m;
      *reinterpret_cast<float4 *>(t.exp_avg_sq + e0) = v;
    } else {
      for (int u = 0; u < cnt; ++u) {
        if (!vis[u]) continue;
        const long long i = e0 + u;
        float p = t.param[i], m = t.exp_avg[i], v = t.exp_avg_sq[i];
        adam_element(p, t.grad[i], m, v, t.lr, b1, b2, t.eps);
        t.param[i] = p, t.exp_avg[i] = m, t.exp_avg_sq[i] = v;
      }
    }
  }
}

}  // namespace fsgs

using namespace fsgs;

extern "C" const char *fsgs_status_string(int status) {
  switch (status) {
    case FSGS_OK: return "ok";
    case FSGS_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FSGS_ERR_UNSUPPORTED: return "unsupported option";
    case FSGS_ERR_WORKSPACE: return "workspace too small";
    case FSGS_ERR_LAUNCH: return "kernel launch failed";
    case FSGS_ERR_LIMIT: return "size beyond the documented maximum";
    default: return "unknown status";
  }
}

extern "C" int fsgs_version(void) { return 100; }

template <typename T>
static int cdist_top_impl(int B, int N, int M, int D, const T *x1, const T *x2, int largest, T *dist, int64_t *index,
    fsgs_stream_t stream) {
  FSGS_REQUIRE(B >= 0 && N >= 0 && M > 0 && D > 0);
  if (B == 0 || N == 0) return FSGS_OK;
  FSGS_REQUIRE(x1 && x2 && dist && index);
  cudaStream_t st = (cudaStream_t) stream;
  const dim3 grid(ceil_div(N, 128), B);
  largest = largest ? 1 : 0;
  if (D == 3) cdist_top_kernel<T, 3><<<grid, 128, 0, st>>>(N, M, x1, x2, largest, dist, index);
  else if (D == 2) cdist_top_kernel<T, 2><<<grid, 128, 0, st>>>(N, M, x1, x2, largest, dist, index);
  else cdist_top_generic_kernel<T><<<grid, 128, 0, st>>>(N, M, D, x1, x2, largest, dist, index);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

template <typename T>
static int cdist_top_backward_impl(int B, int N, int M, int D, const T *x1, const T *x2, const T *dist,
    const int64_t *index, const T *grad_dist, T *g1, T *g2, fsgs_stream_t stream) {
  FSGS_REQUIRE(B >= 0 && N >= 0 && M > 0 && D > 0 && x1 && x2 && dist && index && grad_dist && g1 && g2);
  cudaStream_t st = (cudaStream_t) stream;
  cudaMemsetAsync(g2, 0, sizeof(T) * (size_t) B * M * D, st);
  if (B == 0 || N == 0) return FSGS_OK;
  cdist_top_backward_kernel<T><<<ceil_div((int64_t) B * N, 256), 256, 0, st>>>(B, N, M, D, x1, x2, dist, index,
      grad_dist, g1, g2);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_cdist_top(int B, int N, int M, int D, const float *x1, const float *x2, int largest, float *dist,
    int64_t *index, fsgs_stream_t stream) {
  return cdist_top_impl<float>(B, N, M, D, x1, x2, largest, dist, index, stream);
}

extern "C" int fsgs_cdist_top_f64(int B, int N, int M, int D, const double *x1, const double *x2, int largest,
    double *dist, int64_t *index, fsgs_stream_t stream) {
  return cdist_top_impl<double>(B, N, M, D, x1, x2, largest, dist, index, stream);
}

extern "C" int fsgs_cdist_top_backward(int B, int N, int M, int D, const float *x1, const float *x2,
    const float *dist, const int64_t *index, const float *grad_dist, float *g1, float *g2, fsgs_stream_t stream) {
  return cdist_top_backward_impl<float>(B, N, M, D, x1, x2, dist, index, grad_dist, g1, g2, stream);
}

extern "C" int fsgs_cdist_top_backward_f64(int B, int N, int M, int D, const double *x1, const double *x2,
    const double *dist, const int64_t *index, const double *grad_dist, double *g1, double *g2, fsgs_stream_t stream) {
  return cdist_top_backward_impl<double>(B, N, M, D, x1, x2, dist, index, grad_dist, g1, g2, stream);
}

extern "C" int fsgs_knn(int N, int M, int K, const float *x, const float *c, float *d2, int64_t *index,
    fsgs_stream_t stream) {
  FSGS_REQUIRE(N >= 0 && M > 0 && K > 0 && x && c && d2 && index);
  if (K > FSGS_KNN_MAX_K) return FSGS_ERR_LIMIT;
  if (N == 0) return FSGS_OK;
  cudaStream_t st = (cudaStream_t) stream;
  switch (K) {
    case 1: launch_knn<1>(N, M, x, c, d2, index, st); break;
    case 2: launch_knn<2>(N, M, x, c, d2, index, st); break;
    case 3: launch_knn<3>(N, M, x, c, d2, index, st); break;
    case 4: launch_knn<4>(N, M, x, c, d2, index, st); break;
    case 5: launch_knn<5>(N, M, x, c, d2, index, st); break;
    case 6: launch_knn<6>(N, M, x, c, d2, index, st); break;
    case 7: launch_knn<7>(N, M, x, c, d2, index, st); break;
    case 8: launch_knn<8>(N, M, x, c, d2, index, st); break;
    case 9: launch_knn<9>(N, M, x, c, d2, index, st); break;
    case 10: launch_knn<10>(N, M, x, c, d2, index, st); break;
    case 11: launch_knn<11>(N, M, x, c, d2, index, st); break;
    case 12: launch_knn<12>(N, M, x, c, d2, index, st); break;
    case 13: launch_knn<13>(N, M, x, c, d2, index, st); break;
    case 14: launch_knn<14>(N, M, x, c, d2, index, st); break;
    case 15: launch_knn<15>(N, M, x, c, d2, index, st); break;
    default: launch_knn<16>(N, M, x, c, d2, index, st); break;
  }
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

static int knn_grid_cells(int M) {
  int G = (int) (cbrt((double) M / 2.0) + 0.5);
  return G < 1 ? 1 : (G > kGridMax ? kGridMax : G);
}

static size_t up256_knn(size_t n) { return (n + 255) & ~(size_t) 255; }

extern "C" size_t fsgs_knn_grid_workspace_bytes(int M) {
  const int G = knn_grid_cells(M > 0 ? M : 1);
  return up256_knn(sizeof(GridHeader)) + up256_knn(sizeof(int) * ((size_t) G * G * G + 1)) +
         up256_knn(sizeof(float4) * (size_t) (M > 0 ? M : 1));
}

extern "C" int fsgs_knn_grid(int N, int M, int K, const float *x, const float *c, float *d2, int64_t *index,
    void *workspace, size_t workspace_bytes, fsgs_stream_t stream) {
  FSGS_REQUIRE(N >= 0 && M > 0 && K > 0 && x && c && d2 && index && workspace);
  if (K > FSGS_KNN_MAX_K) return FSGS_ERR_LIMIT;
  if (workspace_bytes < fsgs_knn_grid_workspace_bytes(M)) return FSGS_ERR_WORKSPACE;
  if (N == 0) return FSGS_OK;
  cudaStream_t st = (cudaStream_t) stream;
  const int G = knn_grid_cells(M);
  char *w = (char *) workspace;
  GridHeader *hdr = (GridHeader *) w;
  w += up256_knn(sizeof(GridHeader));
  int *cell_start = (int *) w;
  w += up256_knn(sizeof(int) * ((size_t) G * G * G + 1));
  float4 *sorted = (float4 *) w;
  knn_grid_build_kernel<<<1, 1024, 0, st>>>(M, G, c, hdr, cell_start, sorted);
  FSGS_LAUNCH_CHECK();
  switch (K) {
    case 1: launch_knn_grid<1>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 2: launch_knn_grid<2>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 3: launch_knn_grid<3>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 4: launch_knn_grid<4>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 5: launch_knn_grid<5>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 6: launch_knn_grid<6>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 7: launch_knn_grid<7>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 8: launch_knn_grid<8>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 9: launch_knn_grid<9>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 10: launch_knn_grid<10>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 11: launch_knn_grid<11>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 12: launch_knn_grid<12>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 13: launch_knn_grid<13>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 14: launch_knn_grid<14>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    case 15: launch_knn_grid<15>(N, x, hdr, cell_start, sorted, d2, index, st); break;
    default: launch_knn_grid<16>(N, x, hdr, cell_start, sorted, d2, index, st); break;
  }
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_adam_masked(float *param, const float *grad, float *exp_avg, float *exp_avg_sq,
    const uint8_t *visible, float lr, float b1, float b2, float eps, int64_t N, int64_t M, fsgs_stream_t stream) {
  FSGS_REQUIRE(param && grad && exp_avg && exp_avg_sq && visible && N >= 0 && M > 0 && M < (1ll << 31));
  if (N == 0) return FSGS_OK;
  const int64_t total = N * M;
  const int blocks = (int) (total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  adam_masked_kernel<<<blocks, 256, 0, (cudaStream_t) stream>>>(param, grad, exp_avg, exp_avg_sq, visible, lr, b1, b2,
      eps, (long long) N, (int) M);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

template <typename MaskT>
static int adam_multi_impl(int n_tensors, const fsgs_adam_tensor *tensors, const MaskT *visible, int64_t N, float b1,
    float b2, fsgs_stream_t stream) {
  FSGS_REQUIRE(n_tensors > 0 && tensors && visible && N >= 0);
  if (n_tensors > FSGS_ADAM_MAX_TENSORS) return FSGS_ERR_LIMIT;
  AdamMulti a;
  a.n = n_tensors;
  a.chunk_start[0] = 0;
  for (int k = 0; k < n_tensors; ++k) {
    const fsgs_adam_tensor &t = tensors[k];
    FSGS_REQUIRE(t.param && t.grad && t.exp_avg && t.exp_avg_sq && t.M > 0);
    a.t[k] = t;
    a.chunk_start[k + 1] = a.chunk_start[k] + (N * t.M + 3) / 4;
    a.vec[k] = ((((uintptr_t) t.param) | ((uintptr_t) t.grad) | ((uintptr_t) t.exp_avg) | ((uintptr_t) t.exp_avg_sq)) & 15) == 0;
    a.magic[k] = t.M > 1 ? (unsigned) ((1ull << 32) / (unsigned long long) t.M) : 0u;
  }
  if (N == 0) return FSGS_OK;
  const long long total = a.chunk_start[n_tensors];
  const int blocks = (int) ((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
  adam_masked_multi_kernel<MaskT><<<blocks, 256, 0, (cudaStream_t) stream>>>(a, visible, (long long) N, b1, b2);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_adam_masked_multi(int n_tensors, const fsgs_adam_tensor *tensors, const uint8_t *visible,
    int64_t N, float b1, float b2, fsgs_stream_t stream) {
  return adam_multi_impl<uint8_t>(n_tensors, tensors, visible, N, b1, b2, stream);
}

extern "C" int fsgs_adam_masked_multi_fmask(int n_tensors, const fsgs_adam_tensor *tensors, const float *visible,
    int64_t N, float b1, float b2, fsgs_stream_t stream) {
  return adam_multi_impl<float>(n_tensors, tensors, visible, N, b1, b2, stream);
}
