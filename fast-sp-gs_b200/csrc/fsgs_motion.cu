// Per-step superpoint motion: frequency encoding of the superpoint centres and of the time, the time network, the
// deformation MLP (depth x width, one skip connection), its heads, quaternion normalisation and the re-centring of
// the translation about each superpoint's own centre -- one kernel forward; backward: transposed weight copies, the
// row blocks back through the layers, the weight gradients -- and the kernel-weighted LBS weights with their
// two-pass adjoint.  Restates, in fp32 SIMT,
//   fast_2d_gs/network.py:1670-1776  (SC_GS_DeformNetwork: encoders, timenet, linear[], heads)
//   fast_2d_gs/_C/src/nerf/freqencoder.cu:8-32  (output order: x, then sin(2^d s x), cos(2^d s x) per degree)
//   fast_2d_gs/network.py:545-549    (q = normalize(g_rot + (0,0,0,1)); t' = t + c - R(q) c, 'LBS_c')
//   fast_2d_gs/network.py:506-513    (weights = exp(-d^2 / (2 r^2)) * sigma + 1e-7, normalised; r = exp(raw), sigma = sigmoid(raw))
// The network is 0.5 GFLOP per evaluation on M = 512 rows: a latency problem, not a throughput one.  Each block owns
// 8 rows and carries them through every layer with the activations in shared memory, so the eight dependent layers
// cost no launches and no grid synchronisation; the weights ([in, out] row major) stream from L2 through shared
// memory by bulk asynchronous copies issued by a producer warp, and every worker thread keeps an 8 x 4 block of
// partial outputs in registers (column threads x k groups).  Tensor cores are not used: the path is specified in fp32
// and the whole evaluation is tens of microseconds on the FP32 pipe.
#include "fsgs_common.cuh"
#include "fsgs_tma.cuh"

namespace fsgs {

constexpr int kMotionRows = 8;      // rows (superpoints) per block
constexpr int kMotionMaxWidth = 256;
constexpr int kMotionMaxIn = 384;   // widest layer input: width + encodings
constexpr int kHeadsMax = 16;

struct MotionLayout {
  int Ep, Et, in0, NH, depth, width, skip, Ht, To;
  long long time0_W, time0_b, time2_W, time2_b, heads_W, heads_b, total;
  long long lin_W[16], lin_b[16];
  int lin_in[16];
};

static inline long long pad4(long long n) { return (n + 3) & ~3ll; }

static bool motion_layout(const fsgs_motion_cfg *c, MotionLayout &L) {
  if (!c || c->depth < 2 || c->depth > 16 || c->width < 32 || c->width > kMotionMaxWidth || (c->width & 31)) return false;
  if (c->skip < 0 || c->skip >= c->depth - 1 || c->deg_p < 0 || c->deg_t < 0) return false;
  L.Ep = 3 * (2 * c->deg_p + 1), L.Et = 2 * c->deg_t + 1;
  L.Ht = c->time_out > 0 ? c->time_hidden : 0, L.To = c->time_out > 0 ? c->time_out : L.Et;
  L.in0 = L.Ep + L.To;
  L.NH = c->local_frame ? 14 : 10;
  L.depth = c->depth, L.width = c->width, L.skip = c->skip;
  if (L.in0 + L.width > kMotionMaxIn || L.in0 > 128 || L.Et > 32 || L.To > 64) return false;
  if (c->time_out > 0 && (c->time_hidden <= 0 || c->time_hidden > 1024)) return false;
  long long off = 0;
  auto take = [&](long long n) {
    const long long o = off;
    off += pad4(n);
    return o;
  };
  L.time0_W = L.time0_b = L.time2_W = L.time2_b = 0;
  if (c->time_out > 0) {
    L.time0_W = take((long long) L.Et * L.Ht), L.time0_b = take(L.Ht);
    L.time2_W = take((long long) L.Ht * L.To), L.time2_b = take(L.To);
  }
  for (int i = 0; i < L.depth; ++i) {
    L.lin_in[i] = i == 0 ? L.in0 : (i == L.skip + 1 ? L.width + L.in0 : L.width);
    L.lin_W[i] = take((long long) L.lin_in[i] * L.width), L.lin_b[i] = take(L.width);
  }
  L.heads_W = take((long long) L.width * L.NH), L.heads_b = take(L.NH);
  L.total = off;
  return true;
}

struct MotionDev {
  MotionLayout L;
  int M, local_frame;
  float scale_p, scale_t;
  const float *points;  // [M,3] superpoint centres
  const float *t;       // [1]
  const float *params;
  float *x0;            // [M, in0]  layer-0 input (encodings + time features)
  float *h;             // [depth, M, width] post-ReLU activations
  float *heads;         // [M, NH] raw head outputs: d_xyz 3 | d_scale 3 | d_rot 4 | g_rot 4
  float *time_hidden;   // [Ht] post-ReLU hidden layer of the time network
  float4 *sp_q;
  float *sp_t;
  float4 *sp_dr;
  float2 *sp_ds;
};

// rotation by the unit quaternion q = (x, y, z, w)
__device__ __forceinline__ float3 q_rot(const float4 q, const float3 p) {
  const float r00 = 1 - 2 * (q.y * q.y + q.z * q.z), r01 = 2 * (q.x * q.y - q.z * q.w), r02 = 2 * (q.y * q.w + q.x * q.z);
  const float r10 = 2 * (q.x * q.y + q.z * q.w), r11 = 1 - 2 * (q.x * q.x + q.z * q.z), r12 = 2 * (q.y * q.z - q.x * q.w);
  const float r20 = 2 * (q.x * q.z - q.y * q.w), r21 = 2 * (q.x * q.w + q.y * q.z), r22 = 1 - 2 * (q.x * q.x + q.y * q.y);
  return make_float3(r00 * p.x + r01 * p.y + r02 * p.z, r10 * p.x + r11 * p.y + r12 * p.z,
      r20 * p.x + r21 * p.y + r22 * p.z);
}

// dL/dq of R(q) given dL/dR (row major)
__device__ __forceinline__ float4 q_adjoint(const float4 q, const float *dR) {
  float4 g;
  g.x = 2 * (-2 * q.x * (dR[4] + dR[8]) + q.y * (dR[1] + dR[3]) + q.z * (dR[2] + dR[6]) + q.w * (dR[7] - dR[5]));
  g.y = 2 * (q.x * (dR[1] + dR[3]) - 2 * q.y * (dR[0] + dR[8]) + q.z * (dR[5] + dR[7]) + q.w * (dR[2] - dR[6]));
  g.z = 2 * (q.x * (dR[2] + dR[6]) + q.y * (dR[5] + dR[7]) - 2 * q.z * (dR[0] + dR[4]) + q.w * (dR[3] - dR[1]));
  g.w = 2 * (q.x * (dR[7] - dR[5]) + q.y * (dR[2] - dR[6]) + q.z * (dR[3] - dR[1]));
  return g;
}

// out[e] for one scalar x: x, then (sin, cos)(2^d * scale * x), interleaved with stride `dim` like the reference
__device__ __forceinline__ void freq_encode(float x, int deg, float scale, int dim, int c, float *out) {
  out[c] = x;
  const float xs = x * scale;
  for (int d = 0; d < deg; ++d) {
    const float a = scalbnf(xs, d);
    out[(1 + 2 * d) * dim + c] = sinf(a);
    out[(2 + 2 * d) * dim + c] = cosf(a);
  }
}

// ---- the row-block GEMM both passes are built on ---------------------------------------------------------------
// A block carries R = 8 rows through a chain of matrices.  For one matrix Wm [K, N] (row major, N a multiple of 4)
//   out[r][n] = sum_k act[k][r] * Wm[k][n]                 r < 8
// is computed by C = N / 4 column threads x G k-groups (G = 5 .. 8, the split of the block's 512 worker threads):
// thread (g, c) keeps an 8 x 4 block of partial sums over the rows k = g, g + G, ... of every slab in registers -- one
// 16-byte weight load and two broadcast activation loads feed 32 multiply-adds -- the G partial blocks meet in shared
// memory and a second pass adds them up, lanes along n.
// The matrices stream from L2 through a ring of four shared-memory buffers by bulk asynchronous copies.  A seventeenth
// warp is the producer: one thread that waits until all sixteen worker warps have released a buffer and refills it,
// running up to four slabs ahead of the slowest worker, across matrix boundaries.  The workers never meet at a block
// barrier for a slab: a warp waits for the slab's "full" barrier, multiplies, arrives on its "empty" barrier and
// goes on, so that the chain of eight dependent layers is covered by copies already in flight and the warps absorb
// each other's jitter; they meet (a named barrier over the 512 workers) only where a layer's partial sums are added.
// Every wait is bounded: a worker whose slab does not arrive reads it from global memory instead, a producer whose
// buffer is never released stops producing and says so, and the workers then read everything from global memory.
// History: one column per thread was bound by the broadcast loads (0.15 ms forward at 512 rows); 8 x 4 register
// blocks without a split over k left two warps per SM with work (same time); with the split and a block barrier
// per slab 0.080 ms.
constexpr int kWorkers = 512;                  // 16 warps
constexpr int kMotionThreads = kWorkers + 32;  // + the producer warp
constexpr int kSlabBufs = 4;
constexpr int kSlabFloats = 8192;              // 32 KB per buffer: 32 rows of a 256-wide matrix
constexpr int kSplitMax = 8;
constexpr int kPartFloats = kSplitMax * kMotionRows * (kMotionMaxWidth + 4);
constexpr int kMotionDynFloats = kSlabBufs * kSlabFloats + kPartFloats;
static_assert(kMotionRows == 8, "the register blocks and the [k][8] activation layout assume 8 rows per block");
constexpr int kItemSlots = (2 * kMotionMaxIn + kWorkers - 1) / kWorkers;  // reduction items per thread, at most
constexpr int kHeadGroups = kWorkers / 128;                              // k-groups of the heads product

// barrier over the worker warps only (the producer warp never joins)
__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(smem_u32(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}

struct MatSeq {  // the matrices a pass consumes, in order (shared memory)
  const float *ptr[18];
  int rows[18], stride[18], srows[18];
  int n, total;  // matrices, slabs
};

// slab height and slab count of every matrix (one thread, after ptr / rows / stride are filled in)
__device__ __forceinline__ void seq_finish(MatSeq &s) {
  s.total = 0;
  for (int m = 0; m < s.n; ++m) {
    s.srows[m] = max(8, (kSlabFloats / s.stride[m]) & ~7);
    s.total += (s.rows[m] + s.srows[m] - 1) / s.srows[m];
  }
}

__device__ __forceinline__ int gemm_split(int N) {
  return min(kSplitMax, min(kWorkers / (N >> 2), kPartFloats / (kMotionRows * (N + 4))));
}

struct SlabRing {
  float *buf;            // [kSlabBufs][kSlabFloats]
  uint64_t *full;        // [kSlabBufs] one arrival (the producer) + the copy's bytes
  uint64_t *empty;       // [kSlabBufs] sixteen arrivals (one per worker warp)
  const MatSeq *seq;
  volatile int *dead;    // set by the producer when it gives up
  int next;              // worker: index of the next slab to consume

  // Worker: waits for the slab `next` of the sequence; false when it did not arrive (the caller then reads those rows
  // from global memory).  Every lane tests once -- the slab was requested three slabs ago and is normally there --
  // and only then does lane 0 poll, with the producer's give-up flag in view.
  __device__ __forceinline__ bool acquire() {
    uint64_t *bar = &full[next % kSlabBufs];
    const uint32_t parity = (uint32_t) ((next / kSlabBufs) & 1);
    bool ok = mbar_test(bar, parity);
    if (__all_sync(0xffffffffu, ok)) return true;
    if ((threadIdx.x & 31) == 0)
      for (int i = 0; i < (1 << 20) && !ok && !*dead; ++i) ok = mbar_test(bar, parity);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok) ok = mbar_test(bar, parity);
    return __all_sync(0xffffffffu, ok);
  }
  __device__ __forceinline__ int slot() const { return next % kSlabBufs; }
  // Worker: this warp is done with the slab `next`
  __device__ __forceinline__ void release() {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(&empty[next % kSlabBufs]);
    ++next;
  }
};

// Producer (one thread): issues every slab of the sequence in order, each as soon as its buffer has been released.
__device__ __forceinline__ void slab_producer(float *buf, uint64_t *full, uint64_t *empty, const MatSeq *seq,
    volatile int *dead) {
  int m = 0, k = 0, s = 0;
  for (; s < seq->total; ++s) {
    const int b = s % kSlabBufs;
    if (s >= kSlabBufs) {
      // the previous occupant: released by every worker warp, and its own copy complete (a worker that gave up
      // waiting releases early)
      const uint32_t parity = (uint32_t) (((s / kSlabBufs) - 1) & 1);
      if (!mbar_wait_bounded(&empty[b], parity) || !mbar_wait_bounded(&full[b], parity)) break;
    }
    const int stride = seq->stride[m], rows = min(seq->srows[m], seq->rows[m] - k);
    const uint32_t bytes = (uint32_t) rows * stride * 4u;
    mbar_arrive_expect_tx(&full[b], bytes);
    bulk_load(buf + b * kSlabFloats, seq->ptr[m] + (size_t) k * stride, bytes, &full[b]);
    k += rows;
    if (k >= seq->rows[m]) ++m, k = 0;
  }
  if (s < seq->total) {  // gave up: tell the workers, and give the copies still in flight one more bounded wait
    *dead = 1;
    for (int q = max(0, s - kSlabBufs); q < s; ++q) mbar_wait_bounded(&full[q % kSlabBufs], (uint32_t) ((q / kSlabBufs) & 1));
  }
}

// Every thread of the block calls this once, after s_seq is complete (it contains the block's only full barrier).
// The producer warp does its whole job inside and returns true: the caller returns from the kernel.
__device__ __forceinline__ bool ring_start(SlabRing &ring, float *buf, uint64_t *full, uint64_t *empty,
    const MatSeq *seq, int *dead) {
  if (threadIdx.x == 0) {
    for (int b = 0; b < kSlabBufs; ++b) mbar_init(&full[b], 1), mbar_init(&empty[b], kWorkers / 32);
    *dead = 0;
  }
  __syncthreads();
  ring.buf = buf, ring.full = full, ring.empty = empty, ring.seq = seq, ring.dead = dead, ring.next = 0;
  if (threadIdx.x >= kWorkers) {
    if (threadIdx.x == kWorkers) slab_producer(buf, full, empty, seq, dead);
    return true;
  }
  return false;
}

// acc += act^T-block x rows kg, kg + G, ... (n_it of them) of the slab at w (this thread's four columns); act_k0 = the
// activations of the slab's first row.  Inlined once with w in shared memory and once with w in global memory, so
// that each copy uses the loads of its own address space.
__device__ __forceinline__ void slab_fma(const float *w, const float *act_k0, int N, int kg, int G, int n_it,
    float (&acc)[8][4]) {
#pragma unroll 4
  for (int it = 0; it < n_it; ++it) {
    const int kk = kg + it * G;
    const float4 wv = *reinterpret_cast<const float4 *>(w + kk * N);
    const float4 a0 = *reinterpret_cast<const float4 *>(act_k0 + kk * 8);
    const float4 a1 = *reinterpret_cast<const float4 *>(act_k0 + kk * 8 + 4);
    const float ar[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
    for (int r = 0; r < 8; ++r)
      acc[r][0] += ar[r] * wv.x, acc[r][1] += ar[r] * wv.y, acc[r][2] += ar[r] * wv.z, acc[r][3] += ar[r] * wv.w;
  }
}

// Partial sums of act^T-block x matrix m (all its rows) into s_part[g][r][N + 4].  Every worker thread calls it; on
// return the partial sums are complete and s_act is free.  s_slabs = the ring's buffers (the kernel's own shared
// array, so that the compiler sees the address space).
__device__ __forceinline__ void rowblock_gemm(SlabRing &ring, const float *s_slabs, int m, const float *s_act,
    float *s_part) {
  const int K = ring.seq->rows[m], N = ring.seq->stride[m], sr = ring.seq->srows[m], t = threadIdx.x;
  const int C = N >> 2, G = gemm_split(N);
  const int kg = t / C, ct = t - kg * C;
  const bool mine = kg < G;
  const int it_full = mine ? (sr - kg + G - 1) / G : 0;  // this thread's rows of a full slab
  float acc[8][4];
#pragma unroll
  for (int r = 0; r < 8; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += sr) {
    const int rows = K - k0;
    const int n_it = rows >= sr ? it_full : (mine ? (rows - kg + G - 1) / G : 0);
    if (ring.acquire()) slab_fma(s_slabs + ring.slot() * kSlabFloats + 4 * ct, s_act + k0 * 8, N, kg, G, n_it, acc);
    else slab_fma(ring.seq->ptr[m] + (size_t) k0 * N + 4 * ct, s_act + k0 * 8, N, kg, G, n_it, acc);
    ring.release();
  }
  if (mine) {
    const int Np = N + 4;
#pragma unroll
    for (int r = 0; r < 8; ++r)
      *reinterpret_cast<float4 *>(s_part + (kg * 8 + r) * Np + 4 * ct) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
  }
  workers_sync();
}

// Adds the G partial blocks: item (n, half) -- column n, rows 4 half .. 4 half + 3 -- goes to epi(slot, n, half, sums)
// with slot = 0, 1, .. counting the items of this thread (so that the caller can pair them with values it fetched ahead).
template <class F>
__device__ __forceinline__ void rowblock_reduce(const float *s_part, int N, F epi) {
  const int G = gemm_split(N), Np = N + 4;
#pragma unroll
  for (int slot = 0; slot < kItemSlots; ++slot) {
    const int e = threadIdx.x + slot * kWorkers;
    if (e >= 2 * N) break;
    const int half = e >= N ? 1 : 0, n = e - half * N;
    float4 s = make_float4(0, 0, 0, 0);
    const float *p = s_part + (4 * half) * Np + n;
    for (int g = 0; g < G; ++g, p += 8 * Np) s.x += p[0], s.y += p[Np], s.z += p[2 * Np], s.w += p[3 * Np];
    epi(slot, n, half, s);
  }
}

// One block = kMotionRows rows through the whole network, kMotionThreads threads.
__global__ void __launch_bounds__(kMotionThreads) motion_forward_kernel(MotionDev a) {
  constexpr int R = kMotionRows;
  extern __shared__ __align__(128) float s_dyn[];            // slabs [kSlabBufs][kSlabFloats] | partial sums
  float *s_part = s_dyn + kSlabBufs * kSlabFloats;
  __shared__ __align__(8) uint64_t s_full[kSlabBufs], s_empty[kSlabBufs];
  __shared__ int s_dead;
  __shared__ MatSeq s_seq;
  __shared__ __align__(16) float s_in[kMotionMaxIn * R];     // [k][r]: the layer's input, k major
  __shared__ float s_x0[R][128];                             // row major copy of the layer-0 input (for the skip)
  __shared__ float s_te[32];                                 // time encoding
  __shared__ float s_th[1024];                               // time-network hidden layer
  __shared__ float s_tf[64];                                 // time features
  __shared__ float s_heads[R][kHeadsMax];
  const MotionLayout &L = a.L;
  const int j = threadIdx.x, nt = kWorkers, row0 = blockIdx.x * R;
  const int W = L.width;
  const float *P = a.params;
  if (j == 0) {
    s_seq.n = L.depth + 1;
    for (int i = 0; i < L.depth; ++i) s_seq.ptr[i] = P + L.lin_W[i], s_seq.rows[i] = L.lin_in[i], s_seq.stride[i] = W;
    s_seq.ptr[L.depth] = P + L.heads_W, s_seq.rows[L.depth] = W, s_seq.stride[L.depth] = L.NH;
    seq_finish(s_seq);
  }
  SlabRing ring;
  if (ring_start(ring, s_dyn, s_full, s_empty, &s_seq, &s_dead)) return;  // the producer warp: the slabs start to travel

  // encodings
  if (j == 0) freq_encode(a.t[0], (L.Et - 1) / 2, a.scale_t, 1, 0, s_te);
  for (int e = j; e < R * 3; e += nt) {
    const int r = e / 3, c = e - 3 * r;
    const int m = row0 + r;
    freq_encode(m < a.M ? a.points[3 * m + c] : 0.0f, (L.Ep / 3 - 1) / 2, a.scale_p, 3, c, s_x0[r]);
  }
  workers_sync();
  // time network (the same for every row): hidden = relu(W0^T te + b0), features = W2^T hidden + b2
  if (L.Ht > 0) {
    for (int u = j; u < L.Ht; u += nt) {
      float acc = P[L.time0_b + u];
      for (int k = 0; k < L.Et; ++k) acc += s_te[k] * P[L.time0_W + (long long) k * L.Ht + u];
      s_th[u] = fmaxf(acc, 0.0f);
    }
    workers_sync();
    // every warp sums its share of the hidden units for all outputs, then the shares are added
    {
      const int lane = j & 31, warp = j >> 5, nw = nt >> 5;
      float *part = s_part;  // [nw][64] scratch
      for (int u = lane; u < L.To; u += 32) {
        float acc = 0.0f;
        for (int k = warp; k < L.Ht; k += nw) acc += s_th[k] * P[L.time2_W + (long long) k * L.To + u];
        part[warp * 64 + u] = acc;
      }
      workers_sync();
      for (int u = j; u < L.To; u += nt) {
        float acc = P[L.time2_b + u];
        for (int w = 0; w < nw; ++w) acc += part[w * 64 + u];
        s_tf[u] = acc;
      }
    }
    if (blockIdx.x == 0)
      for (int u = j; u < L.Ht; u += nt) a.time_hidden[u] = s_th[u];
  } else {
    for (int u = j; u < L.To; u += nt) s_tf[u] = s_te[u];
  }
  workers_sync();
  for (int e = j; e < R * L.To; e += nt) {
    const int r = e / L.To, u = e - r * L.To;
    s_x0[r][L.Ep + u] = s_tf[u];
  }
  workers_sync();
  for (int e = j; e < R * L.in0; e += nt) {
    const int r = e / L.in0, k = e - r * L.in0;
    s_in[k * R + r] = s_x0[r][k];
    if (row0 + r < a.M) a.x0[(size_t) (row0 + r) * L.in0 + k] = s_x0[r][k];
  }
  workers_sync();

  for (int i = 0; i < L.depth; ++i) {
    rowblock_gemm(ring, s_dyn, i, s_in, s_part);
    // bias, ReLU; the activations become the next layer's input, preceded by the encodings after the skip layer
    const int lead = (i == L.skip) ? L.in0 : 0;
    rowblock_reduce(s_part, W, [&](int, int n, int half, float4 s) {
      const float bias = P[L.lin_b[i] + n];
      const float4 v = make_float4(fmaxf(s.x + bias, 0.0f), fmaxf(s.y + bias, 0.0f), fmaxf(s.z + bias, 0.0f),
          fmaxf(s.w + bias, 0.0f));
      *reinterpret_cast<float4 *>(s_in + (lead + n) * R + 4 * half) = v;
      const int m = row0 + 4 * half;
      float *h = a.h + ((size_t) i * a.M + m) * W + n;
      if (m < a.M) h[0] = v.x;
      if (m + 1 < a.M) h[W] = v.y;
      if (m + 2 < a.M) h[2 * W] = v.z;
      if (m + 3 < a.M) h[3 * W] = v.w;
    });
    if (lead)
      for (int e = j; e < R * lead; e += nt) {
        const int r = e / lead, k = e - r * lead;
        s_in[k * R + r] = s_x0[r][k];
      }
    workers_sync();
  }

  // heads on the last activations (s_in[0 .. W*R), k major): kHeadGroups k-groups x (row, output) pairs, matrix from the ring
  {
    const int NH = L.NH, E = R * NH, kg = j >> 7, e = j & 127;
    const int r = e / NH, o = e - r * NH;
    const bool mine = e < E;
    const int sr = s_seq.srows[L.depth];
    float acc = 0.0f;
    for (int k0 = 0; k0 < W; k0 += sr) {
      const int rows = min(sr, W - k0);
      const float *w = ring.acquire() ? s_dyn + ring.slot() * kSlabFloats : P + L.heads_W + (size_t) k0 * NH;
      if (mine)
        for (int kk = kg; kk < rows; kk += kHeadGroups) acc += s_in[(k0 + kk) * R + r] * w[kk * NH + o];
      ring.release();
    }
    s_part[kg * 128 + e] = acc;
    workers_sync();
    if (j < E) {
      float v = P[L.heads_b + o];
#pragma unroll
      for (int g = 0; g < kHeadGroups; ++g) v += s_part[g * 128 + e];
      s_heads[r][o] = v;
      if (row0 + r < a.M) a.heads[(size_t) (row0 + r) * NH + o] = v;
    }
  }
  workers_sync();
  if (j < R && row0 + j < a.M) {
    const int m = row0 + j;
    const float *o = s_heads[j];
    float4 q = make_float4(0, 0, 0, 1);
    float3 t = make_float3(o[0], o[1], o[2]);
    if (a.local_frame) {
      const float4 u = make_float4(o[10], o[11], o[12], o[13] + 1.0f);
      const float inv = 1.0f / fmaxf(sqrtf(u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w), 1e-12f);
      q = make_float4(u.x * inv, u.y * inv, u.z * inv, u.w * inv);
      const float3 c = make_float3(a.points[3 * m], a.points[3 * m + 1], a.points[3 * m + 2]);
      const float3 rc = q_rot(q, c);
      t = make_float3(t.x + c.x - rc.x, t.y + c.y - rc.y, t.z + c.z - rc.z);
    }
    a.sp_q[m] = q;
    a.sp_t[3 * m] = t.x, a.sp_t[3 * m + 1] = t.y, a.sp_t[3 * m + 2] = t.z;
    a.sp_dr[m] = make_float4(o[6], o[7], o[8], o[9]);
    a.sp_ds[m] = make_float2(o[3], o[4]);
  }
}

struct MotionBwdDev {
  MotionDev f;
  const float4 *g_sp_q;
  const float *g_sp_t;
  const float4 *g_sp_dr;
  const float2 *g_sp_ds;
  float *dpre;     // [depth, M, width] gradient of each layer's pre-activation output
  float *dheads;   // [M, NH]
  float *g_tf;     // [To] summed gradient of the time features (zeroed before the launch)
  float *wt;       // transposed copies of the layer matrices: layer i at wt_off[i], [width][in_pad(i)]
  long long wt_off[16];
  int in_pad[16];
  float *g_params;
  int accumulate;
};

// Transposed copies of the layer matrices for the backward pass (the same row-block GEMM then serves dX = dY W^T):
// wt[i][j][k] = W_i[k][j], row stride in_pad(i) (a multiple of 4, padding zero).
__global__ void __launch_bounds__(256) motion_transpose_kernel(MotionBwdDev b) {
  __shared__ float tile[32][33];
  const MotionLayout &L = b.f.L;
  const int i = blockIdx.z, W = L.width, in = L.lin_in[i], ip = b.in_pad[i];
  const int k0 = blockIdx.x * 32, j0 = blockIdx.y * 32;
  if (k0 >= ip) return;
  const float *src = b.f.params + L.lin_W[i];
  float *dst = b.wt + b.wt_off[i];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int y = ty; y < 32; y += 8) {
    const int k = k0 + y, jcol = j0 + tx;
    tile[y][tx] = (k < in && jcol < W) ? src[(size_t) k * W + jcol] : 0.0f;
  }
  __syncthreads();
  for (int y = ty; y < 32; y += 8) {
    const int jrow = j0 + y, k = k0 + tx;
    if (jrow < W && k < ip) dst[(size_t) jrow * ip + k] = tile[tx][y];
  }
}

// Backward pass 1: one block = kMotionRows rows back through the heads and the layers; leaves dpre / dheads for the
// weight-gradient kernel and sums the gradient of the time features.
__global__ void __launch_bounds__(kMotionThreads) motion_backward_rows_kernel(MotionBwdDev b) {
  constexpr int R = kMotionRows;
  extern __shared__ __align__(128) float s_dyn[];            // slabs [kSlabBufs][kSlabFloats] | partial sums
  float *s_part = s_dyn + kSlabBufs * kSlabFloats;
  __shared__ __align__(8) uint64_t s_full[kSlabBufs], s_empty[kSlabBufs];
  __shared__ int s_dead;
  __shared__ MatSeq s_seq;
  __shared__ __align__(16) float s_dy[kMotionMaxIn * R];     // [k][r]: gradient of the current layer's pre-activation
  __shared__ float s_gh[R][kHeadsMax];
  __shared__ float s_gtf[64];
  const MotionDev &a = b.f;
  const MotionLayout &L = a.L;
  const int j = threadIdx.x, nt = kWorkers, row0 = blockIdx.x * R, W = L.width, M = a.M;
  const float *P = a.params;
  if (j == 0) {
    s_seq.n = L.depth;
    for (int s = 0; s < L.depth; ++s) {  // consumed from the last layer down
      const int i = L.depth - 1 - s;
      s_seq.ptr[s] = b.wt + b.wt_off[i], s_seq.rows[s] = W, s_seq.stride[s] = b.in_pad[i];
    }
    seq_finish(s_seq);
  }
  for (int u = j; u < 64; u += nt) s_gtf[u] = 0.0f;
  SlabRing ring;
  if (ring_start(ring, s_dyn, s_full, s_empty, &s_seq, &s_dead)) return;  // the producer warp

  // the heads' matrix [W][NH] into shared memory (the partial-sum area is idle until the first layer)
  float *s_wh = s_part;
  for (int e = j; e < W * L.NH / 4; e += nt)
    reinterpret_cast<float4 *>(s_wh)[e] = reinterpret_cast<const float4 *>(P + L.heads_W)[e];
  // adjoint of the epilogue -> gradient of the raw head outputs
  if (j < R) {
    float *g = s_gh[j];
    for (int o = 0; o < kHeadsMax; ++o) g[o] = 0.0f;
    const int m = row0 + j;
    if (m < M) {
      const float3 gt = make_float3(b.g_sp_t[3 * m], b.g_sp_t[3 * m + 1], b.g_sp_t[3 * m + 2]);
      g[0] = gt.x, g[1] = gt.y, g[2] = gt.z;
      const float2 gs = b.g_sp_ds[m];
      g[3] = gs.x, g[4] = gs.y;
      const float4 gr = b.g_sp_dr[m];
      g[6] = gr.x, g[7] = gr.y, g[8] = gr.z, g[9] = gr.w;
      if (a.local_frame) {
        const float *o = a.heads + (size_t) m * L.NH;
        const float4 u = make_float4(o[10], o[11], o[12], o[13] + 1.0f);
        const float nrm = fmaxf(sqrtf(u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w), 1e-12f);
        const float inv = 1.0f / nrm;
        const float4 q = make_float4(u.x * inv, u.y * inv, u.z * inv, u.w * inv);
        const float3 c = make_float3(a.points[3 * m], a.points[3 * m + 1], a.points[3 * m + 2]);
        // t' = t + c - R(q) c  ->  dL/dR = -gt (outer) c
        float dR[9] = {-gt.x * c.x, -gt.x * c.y, -gt.x * c.z, -gt.y * c.x, -gt.y * c.y, -gt.y * c.z,
                       -gt.z * c.x, -gt.z * c.y, -gt.z * c.z};
        float4 gq = q_adjoint(q, dR);
        const float4 gq_in = b.g_sp_q[m];
        gq = make_float4(gq.x + gq_in.x, gq.y + gq_in.y, gq.z + gq_in.z, gq.w + gq_in.w);
        const float d = q.x * gq.x + q.y * gq.y + q.z * gq.z + q.w * gq.w;
        g[10] = (gq.x - q.x * d) * inv, g[11] = (gq.y - q.y * d) * inv;
        g[12] = (gq.z - q.z * d) * inv, g[13] = (gq.w - q.w * d) * inv;
      }
      for (int o = 0; o < L.NH; ++o) b.dheads[(size_t) m * L.NH + o] = g[o];
    }
  }
  workers_sync();

  // Through a ReLU: item (column n of layer i, rows 4 half ..) of the gradient dh of layer i's activations becomes the
  // gradient of its pre-activations, kept in global memory for the weight gradients and in s_dy for the next product.
  // hv = the four activations, fetched by the caller ahead of the arithmetic that produced dh.
  auto through_relu = [&](int i, int n, int half, float4 dh, const float (&hv)[4]) {
    const float4 g = make_float4(hv[0] > 0.0f ? dh.x : 0.0f, hv[1] > 0.0f ? dh.y : 0.0f, hv[2] > 0.0f ? dh.z : 0.0f,
        hv[3] > 0.0f ? dh.w : 0.0f);
    *reinterpret_cast<float4 *>(s_dy + n * R + 4 * half) = g;
    const int m = row0 + 4 * half;
    float *d = b.dpre + ((size_t) i * M + m) * W + n;
    if (m < M) d[0] = g.x;
    if (m + 1 < M) d[W] = g.y;
    if (m + 2 < M) d[2 * W] = g.z;
    if (m + 3 < M) d[3 * W] = g.w;
  };
  // the four activations of item (n, half) of layer i; rows beyond M read as 0 (their gradient stays 0)
  auto fetch_h = [&](int i, int n, int half, float (&hv)[4]) {
    const int m = row0 + 4 * half;
    const float *h = a.h + ((size_t) i * M + m) * W + n;
#pragma unroll
    for (int q = 0; q < 4; ++q) hv[q] = (m + q < M) ? h[(size_t) q * W] : 0.0f;
  };

  // gradient of the last activations: dh[n][r] = sum_o g[r][o] Wh[n][o]
  {
    for (int e = j; e < 2 * W; e += nt) {
      const int half = e >= W ? 1 : 0, n = e - half * W;
      float hv[4];
      fetch_h(L.depth - 1, n, half, hv);
      float4 dh = make_float4(0, 0, 0, 0);
      for (int o = 0; o < L.NH; ++o) {
        const float w = s_wh[n * L.NH + o];
        dh.x += s_gh[4 * half][o] * w, dh.y += s_gh[4 * half + 1][o] * w;
        dh.z += s_gh[4 * half + 2][o] * w, dh.w += s_gh[4 * half + 3][o] * w;
      }
      through_relu(L.depth - 1, n, half, dh, hv);
    }
  }
  workers_sync();  // s_dy complete, s_wh no longer needed

  for (int i = L.depth - 1, s = 0; i >= 0; --i, ++s) {
    // dX[r][k] = sum_j dY[r][j] W[k][j], as a row-block GEMM on the transposed copy.  Its columns: the encodings
    // first where the layer has them (only their time features carry a gradient on), then the previous activations.
    const int ip = b.in_pad[i];
    const int lead = (i == 0 || i == L.skip + 1) ? L.in0 : 0;
    float hv[kItemSlots][4];
#pragma unroll
    for (int slot = 0; slot < kItemSlots; ++slot) {  // the previous layer's activations for this thread's items, fetched early
      const int e = j + slot * kWorkers;
      const int half = e >= ip ? 1 : 0, n = e - half * ip - lead;
      if (i > 0 && e < 2 * ip && n >= 0 && n < W) fetch_h(i - 1, n, half, hv[slot]);
      else hv[slot][0] = hv[slot][1] = hv[slot][2] = hv[slot][3] = 0.0f;
    }
    rowblock_gemm(ring, s_dyn, s, s_dy, s_part);
    rowblock_reduce(s_part, ip, [&](int slot, int k, int half, float4 dx) {
      if (lead && k >= L.Ep && k < L.in0) atomicAdd(&s_gtf[k - L.Ep], (dx.x + dx.y) + (dx.z + dx.w));
      const int n = k - lead;
      if (i > 0 && n >= 0 && n < W) through_relu(i - 1, n, half, dx, hv[slot]);
    });
    workers_sync();
  }
  for (int u = j; u < L.To; u += nt)
    if (s_gtf[u] != 0.0f) atomicAdd(b.g_tf + u, s_gtf[u]);
}

// Backward pass 2: weight and bias gradients, one block per 32 x 128 tile of one matrix (dW = X^T dY over all M rows,
// 4 x 4 outputs per thread, the next 32 rows of X and dY fetched into registers while the current ones are
// multiplied); the last block of the grid runs the time network's backward.
constexpr int kTileK = 32, kTileJ = 128, kTileR = 32;

__device__ __forceinline__ void store_grad(float *dst, float v, int accumulate) {
  if (accumulate) *dst += v;
  else *dst = v;
}

__global__ void __launch_bounds__(256) motion_backward_weights_kernel(MotionBwdDev b, int tiles_per_layer_k,
    int tiles_j, int n_layer_blocks, int n_head_blocks) {
  __shared__ __align__(16) float s_x[kTileR][kTileK];
  __shared__ __align__(16) float s_dy[kTileR][kTileJ];
  const MotionDev &a = b.f;
  const MotionLayout &L = a.L;
  const int tid = threadIdx.x, W = L.width, M = a.M;
  int blk = blockIdx.x;
  if (blk < n_layer_blocks + n_head_blocks) {
    // which matrix, which tile
    int i, kt, jt, in, out;
    const float *dY;
    long long offW, offb;
    if (blk < n_layer_blocks) {
      const int per = tiles_per_layer_k * tiles_j;
      i = blk / per;
      const int t = blk - i * per;
      kt = t / tiles_j, jt = t - kt * tiles_j;
      in = L.lin_in[i], out = W, dY = b.dpre + (size_t) i * M * W, offW = L.lin_W[i], offb = L.lin_b[i];
    } else {
      i = L.depth;  // heads: input = last activations
      kt = blk - n_layer_blocks, jt = 0;
      in = W, out = L.NH, dY = b.dheads, offW = L.heads_W, offb = L.heads_b;
    }
    const int k0 = kt * kTileK, j0 = jt * kTileJ;
    if (k0 >= in || j0 >= out) return;
    // element (m, k) of the layer's input, assembled from the saved pieces
    auto x_at = [&](int m, int k) -> float {
      if (m >= M || k >= in) return 0.0f;
      if (i == 0) return a.x0[(size_t) m * L.in0 + k];
      if (i == L.skip + 1)
        return k < L.in0 ? a.x0[(size_t) m * L.in0 + k] : a.h[((size_t) (i - 1) * M + m) * W + (k - L.in0)];
      return a.h[((size_t) (i - 1) * M + m) * W + k];
    };
    float px[4], pdy[16];  // this thread's share of the next 32 rows
    auto fetch = [&](int r0) {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int e = tid + n * 256, r = e >> 5, kk = e & 31;
        px[n] = x_at(r0 + r, k0 + kk);
      }
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const int e = tid + n * 256, r = e >> 7, jj = e & 127, m = r0 + r, jcol = j0 + jj;
        pdy[n] = (m < M && jcol < out) ? dY[(size_t) m * out + jcol] : 0.0f;
      }
    };
    const int tk = tid >> 5, tj = tid & 31;  // 8 groups of 4 rows of the tile x 32 groups of 4 columns
    float acc[4][4], accb[4] = {0, 0, 0, 0};
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.0f;
    fetch(0);
    for (int r0 = 0; r0 < M; r0 += kTileR) {
      __syncthreads();  // the previous rows have been consumed
#pragma unroll
      for (int n = 0; n < 4; ++n) (&s_x[0][0])[tid + n * 256] = px[n];
#pragma unroll
      for (int n = 0; n < 16; ++n) (&s_dy[0][0])[tid + n * 256] = pdy[n];
      __syncthreads();
      if (r0 + kTileR < M) fetch(r0 + kTileR);
#pragma unroll 8
      for (int r = 0; r < kTileR; ++r) {
        const float4 x = *reinterpret_cast<const float4 *>(&s_x[r][4 * tk]);
        const float4 d = *reinterpret_cast<const float4 *>(&s_dy[r][4 * tj]);
        acc[0][0] += x.x * d.x, acc[0][1] += x.x * d.y, acc[0][2] += x.x * d.z, acc[0][3] += x.x * d.w;
        acc[1][0] += x.y * d.x, acc[1][1] += x.y * d.y, acc[1][2] += x.y * d.z, acc[1][3] += x.y * d.w;
        acc[2][0] += x.z * d.x, acc[2][1] += x.z * d.y, acc[2][2] += x.z * d.z, acc[2][3] += x.z * d.w;
        acc[3][0] += x.w * d.x, acc[3][1] += x.w * d.y, acc[3][2] += x.w * d.z, acc[3][3] += x.w * d.w;
        if (tk == 0) accb[0] += d.x, accb[1] += d.y, accb[2] += d.z, accb[3] += d.w;
      }
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int jcol = j0 + 4 * tj + v;
      if (jcol >= out) break;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + 4 * tk + u;
        if (k < in) store_grad(b.g_params + offW + (long long) k * out + jcol, acc[u][v], b.accumulate);
      }
      if (kt == 0 && tk == 0) store_grad(b.g_params + offb + jcol, accb[v], b.accumulate);
    }
    return;
  }
  // time network backward (single block): features = W2^T hidden + b2, hidden = relu(W0^T te + b0)
  if (L.Ht == 0) return;
  __shared__ float s_te[32], s_ghid[1024];
  if (tid == 0) freq_encode(a.t[0], (L.Et - 1) / 2, a.scale_t, 1, 0, s_te);
  for (int u = tid; u < L.Ht; u += 256) {
    float g = 0.0f;
    const float hid = a.time_hidden[u];
    for (int o = 0; o < L.To; ++o) {
      const float go = b.g_tf[o];
      g += go * a.params[L.time2_W + (long long) u * L.To + o];
      store_grad(b.g_params + L.time2_W + (long long) u * L.To + o, hid * go, b.accumulate);
    }
    s_ghid[u] = hid > 0.0f ? g : 0.0f;
  }
  for (int o = tid; o < L.To; o += 256) store_grad(b.g_params + L.time2_b + o, b.g_tf[o], b.accumulate);
  __syncthreads();
  for (int u = tid; u < L.Ht; u += 256) {
    store_grad(b.g_params + L.time0_b + u, s_ghid[u], b.accumulate);
    for (int k = 0; k < L.Et; ++k)
      store_grad(b.g_params + L.time0_W + (long long) k * L.Ht + u, s_te[k] * s_ghid[u], b.accumulate);
  }
}

// ------------------------------------------------------------------------------------------------
// kernel-weighted LBS weights
// ------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256) lbs_weights_forward_kernel(int P, int K, const float *__restrict__ d2,
    const int64_t *__restrict__ idx, const float *__restrict__ raw_radius, const float *__restrict__ raw_weight,
    float *__restrict__ w) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  float u[FSGS_KNN_MAX_K], s = 0.0f;
  for (int k = 0; k < K; ++k) {
    const int m = (int) idx[(size_t) i * K + k];
    const float r = expf(raw_radius[m]);
    float v = expf(-d2[(size_t) i * K + k] / (2.0f * r * r));
    if (raw_weight) v *= 1.0f / (1.0f + expf(-raw_weight[m]));
    u[k] = v + 1e-7f;
    s += u[k];
  }
  for (int k = 0; k < K; ++k) w[(size_t) i * K + k] = u[k] / s;
}

// Adjoint of the kernel weights in two passes.  Pass 1, one thread per Gaussian (coalesced rows, the exponentials
// once per pair): the contribution of every pair (i, k) to the gradient of its superpoint's raw radius and raw weight.
// Pass 2, one block per superpoint over its grouped pairs: sums them in a fixed order, no atomics -- a superpoint
// that owns many times the average number of pairs only costs more two-load iterations.  (Doing all of pass 1's
// arithmetic inside pass 2's loop made the most popular superpoint's block the whole kernel: 70 us at 300 k x 3.)
__global__ void __launch_bounds__(256) lbs_weights_backward_pairs_kernel(int P, int K, const float *__restrict__ d2,
    const int64_t *__restrict__ idx, const float *__restrict__ raw_radius, const float *__restrict__ raw_weight,
    const float *__restrict__ g_w, float2 *__restrict__ contrib) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  float ek[FSGS_KNN_MAX_K], uk[FSGS_KNN_MAX_K], rk[FSGS_KNN_MAX_K], sk[FSGS_KNN_MAX_K];
  float S = 0.0f, gdotw = 0.0f;
  for (int k = 0; k < K; ++k) {
    const int mk = (int) idx[(size_t) i * K + k];
    rk[k] = expf(raw_radius[mk]);
    sk[k] = raw_weight ? 1.0f / (1.0f + expf(-raw_weight[mk])) : 1.0f;
    ek[k] = expf(-d2[(size_t) i * K + k] / (2.0f * rk[k] * rk[k]));
    uk[k] = ek[k] * sk[k] + 1e-7f;
    S += uk[k];
    gdotw += g_w[(size_t) i * K + k] * uk[k];
  }
  for (int k = 0; k < K; ++k) {
    const float gu = (g_w[(size_t) i * K + k] - gdotw / S) / S;  // dL/du of this pair
    const float d = d2[(size_t) i * K + k];
    // d u / d raw_radius = e * sigma * d / r^2 ;  d u / d raw_weight = e * sigma (1 - sigma)
    contrib[(size_t) i * K + k] = make_float2(gu * ek[k] * sk[k] * d / (rk[k] * rk[k]), gu * ek[k] * sk[k] * (1.0f - sk[k]));
  }
}

__global__ void __launch_bounds__(256) lbs_weights_backward_sum_kernel(const float2 *__restrict__ contrib,
    const int32_t *__restrict__ offsets, const int32_t *__restrict__ pairs, int has_weight, float *__restrict__ g_radius,
    float *__restrict__ g_weight, int accumulate) {
  __shared__ float s_a[8], s_b[8];
  const int m = blockIdx.x;
  float ga = 0.0f, gb = 0.0f;
#pragma unroll 4
  for (int e = offsets[m] + threadIdx.x; e < offsets[m + 1]; e += blockDim.x) {
    const float2 c = contrib[pairs[e]];
    ga += c.x, gb += c.y;
  }
  for (int o = 16; o > 0; o >>= 1) ga += __shfl_xor_sync(0xffffffffu, ga, o), gb += __shfl_xor_sync(0xffffffffu, gb, o);
  if ((threadIdx.x & 31) == 0) s_a[threadIdx.x >> 5] = ga, s_b[threadIdx.x >> 5] = gb;
  __syncthreads();
  if (threadIdx.x == 0) {
    float ta = 0.0f, tb = 0.0f;
    for (int w = 0; w < 8; ++w) ta += s_a[w], tb += s_b[w];
    store_grad(g_radius + m, ta, accumulate);
    if (g_weight) store_grad(g_weight + m, has_weight ? tb : 0.0f, accumulate);
  }
}

static bool fill_motion(const fsgs_motion_args *a, MotionDev &d) {
  if (!a || !motion_layout(&a->cfg, d.L)) return false;
  d.M = a->cfg.M, d.local_frame = a->cfg.local_frame;
  d.scale_p = a->cfg.scale_p > 0 ? a->cfg.scale_p : 1.0f, d.scale_t = a->cfg.scale_t > 0 ? a->cfg.scale_t : 1.0f;
  d.points = a->sp_points, d.t = a->t, d.params = a->params;
  if (d.M <= 0 || !d.points || !d.t || !d.params || !a->workspace) return false;
  // workspace: x0 | h | heads | time_hidden | dpre | dheads | g_tf
  float *w = (float *) a->workspace;
  const size_t M = d.M;
  d.x0 = w, w += pad4(M * d.L.in0);
  d.h = w, w += pad4((size_t) d.L.depth * M * d.L.width);
  d.heads = w, w += pad4(M * d.L.NH);
  d.time_hidden = w, w += pad4(d.L.Ht > 0 ? d.L.Ht : 4);
  return true;
}

static size_t motion_wt_floats(const MotionLayout &L) {
  size_t n = 0;
  for (int i = 0; i < L.depth; ++i) n += (size_t) L.width * pad4(L.lin_in[i]);
  return n;
}

static size_t motion_ws_floats(const MotionLayout &L, size_t M) {
  return pad4(M * L.in0) + 2 * pad4((size_t) L.depth * M * L.width) + 2 * pad4(M * L.NH) + pad4(L.Ht > 0 ? L.Ht : 4) + 64 +
         motion_wt_floats(L);
}

// the opt-in above 48 KB of dynamic shared memory is a per-device attribute of each kernel
static bool motion_configure() {
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  if (configured[dev]) return true;
  const int dyn = (int) (sizeof(float) * kMotionDynFloats);
  if (cudaFuncSetAttribute(motion_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) != cudaSuccess ||
      cudaFuncSetAttribute(motion_backward_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn) != cudaSuccess)
    return false;
  configured[dev] = true;
  return true;
}

}  // namespace fsgs

using namespace fsgs;

extern "C" int64_t fsgs_motion_param_count(const fsgs_motion_cfg *cfg) {
  MotionLayout L;
  return motion_layout(cfg, L) ? (int64_t) L.total : -1;
}

// offsets[0..3] time0_W, time0_b, time2_W, time2_b; then (W, b) of every linear layer; then heads W, b
extern "C" int fsgs_motion_param_offsets(const fsgs_motion_cfg *cfg, int64_t *offsets, int32_t *inputs) {
  MotionLayout L;
  FSGS_REQUIRE(offsets && inputs && motion_layout(cfg, L));
  offsets[0] = L.time0_W, offsets[1] = L.time0_b, offsets[2] = L.time2_W, offsets[3] = L.time2_b;
  for (int i = 0; i < L.depth; ++i) offsets[4 + 2 * i] = L.lin_W[i], offsets[5 + 2 * i] = L.lin_b[i], inputs[i] = L.lin_in[i];
  offsets[4 + 2 * L.depth] = L.heads_W, offsets[5 + 2 * L.depth] = L.heads_b;
  return FSGS_OK;
}

extern "C" size_t fsgs_motion_workspace_bytes(const fsgs_motion_cfg *cfg) {
  MotionLayout L;
  if (!motion_layout(cfg, L) || cfg->M <= 0) return 0;
  return sizeof(float) * motion_ws_floats(L, (size_t) cfg->M);
}

extern "C" int fsgs_motion_forward(const fsgs_motion_args *a, fsgs_stream_t stream) {
  MotionDev d;
  FSGS_REQUIRE(fill_motion(a, d));
  FSGS_REQUIRE(a->sp_q && a->sp_t && a->sp_dr && a->sp_ds);
  if (a->workspace_bytes < fsgs_motion_workspace_bytes(&a->cfg)) return FSGS_ERR_WORKSPACE;
  d.sp_q = (float4 *) a->sp_q, d.sp_t = a->sp_t, d.sp_dr = (float4 *) a->sp_dr, d.sp_ds = (float2 *) a->sp_ds;
  if (!motion_configure()) return FSGS_ERR_LAUNCH;
  motion_forward_kernel<<<ceil_div(d.M, kMotionRows), kMotionThreads, sizeof(float) * kMotionDynFloats,
      (cudaStream_t) stream>>>(d);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_motion_backward(const fsgs_motion_args *a, fsgs_stream_t stream) {
  MotionBwdDev b;
  FSGS_REQUIRE(fill_motion(a, b.f));
  FSGS_REQUIRE(a->g_sp_q && a->g_sp_t && a->g_sp_dr && a->g_sp_ds && a->g_params);
  if (a->workspace_bytes < fsgs_motion_workspace_bytes(&a->cfg)) return FSGS_ERR_WORKSPACE;
  const MotionLayout &L = b.f.L;
  const size_t M = b.f.M;
  float *w = b.f.time_hidden + pad4(L.Ht > 0 ? L.Ht : 4);
  b.dpre = w, w += pad4((size_t) L.depth * M * L.width);
  b.dheads = w, w += pad4(M * L.NH);
  b.g_tf = w, w += 64;
  b.wt = w;
  {
    long long off = 0;
    for (int i = 0; i < L.depth; ++i) {
      b.in_pad[i] = (int) pad4(L.lin_in[i]);
      b.wt_off[i] = off;
      off += (long long) L.width * b.in_pad[i];
    }
  }
  b.g_sp_q = (const float4 *) a->g_sp_q, b.g_sp_t = a->g_sp_t, b.g_sp_dr = (const float4 *) a->g_sp_dr;
  b.g_sp_ds = (const float2 *) a->g_sp_ds;
  b.g_params = a->g_params, b.accumulate = a->accumulate;
  cudaStream_t st = (cudaStream_t) stream;
  if (!motion_configure()) return FSGS_ERR_LAUNCH;
  cudaMemsetAsync(b.g_tf, 0, sizeof(float) * 64, st);
  motion_transpose_kernel<<<dim3(ceil_div(L.in0 + L.width, 32), ceil_div(L.width, 32), L.depth), 256, 0, st>>>(b);
  FSGS_LAUNCH_CHECK();
  motion_backward_rows_kernel<<<ceil_div(b.f.M, kMotionRows), kMotionThreads, sizeof(float) * kMotionDynFloats, st>>>(b);
  FSGS_LAUNCH_CHECK();
  const int tiles_k = ceil_div(L.in0 + L.width, kTileK);  // enough for the widest input; narrower layers exit early
  const int tiles_j = ceil_div(L.width, kTileJ);
  const int n_layer = L.depth * tiles_k * tiles_j, n_head = ceil_div(L.width, kTileK);
  motion_backward_weights_kernel<<<n_layer + n_head + 1, 256, 0, st>>>(b, tiles_k, tiles_j, n_layer, n_head);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" int fsgs_lbs_weights_forward(int P, int K, const float *d2, const int64_t *idx, const float *raw_radius,
    const float *raw_weight, float *weights, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && K > 0 && K <= FSGS_KNN_MAX_K && d2 && idx && raw_radius && weights);
  if (P == 0) return FSGS_OK;
  lbs_weights_forward_kernel<<<ceil_div(P, 256), 256, 0, (cudaStream_t) stream>>>(P, K, d2, idx, raw_radius, raw_weight,
      weights);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}

extern "C" size_t fsgs_lbs_weights_backward_workspace_bytes(int P, int K) {
  return P > 0 && K > 0 ? sizeof(float2) * (size_t) P * K : 0;
}

extern "C" int fsgs_lbs_weights_backward(int P, int K, int M, const float *d2, const int64_t *idx,
    const float *raw_radius, const float *raw_weight, const float *g_weights, const int32_t *sp_pair_offsets,
    const int32_t *sp_pairs, float *g_raw_radius, float *g_raw_weight, int accumulate, void *workspace,
    size_t workspace_bytes, fsgs_stream_t stream) {
  FSGS_REQUIRE(P >= 0 && K > 0 && K <= FSGS_KNN_MAX_K && M > 0 && d2 && idx && raw_radius && g_weights);
  FSGS_REQUIRE(sp_pair_offsets && sp_pairs && g_raw_radius);
  if (workspace_bytes < fsgs_lbs_weights_backward_workspace_bytes(P, K) || (P > 0 && !workspace)) return FSGS_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t) stream;
  float2 *contrib = (float2 *) workspace;
  if (P > 0) {
    lbs_weights_backward_pairs_kernel<<<ceil_div(P, 256), 256, 0, st>>>(P, K, d2, idx, raw_radius, raw_weight, g_weights,
        contrib);
    FSGS_LAUNCH_CHECK();
  }
  lbs_weights_backward_sum_kernel<<<M, 256, 0, st>>>(contrib, sp_pair_offsets, sp_pairs, raw_weight != nullptr,
      g_raw_radius, g_raw_weight, accumulate);
  FSGS_LAUNCH_CHECK();
  return FSGS_OK;
}
