// The layer boundary of "parallel" layers on a depth-averaged stream, one kernel:
//
//   X   = x + sigmoid(g1 + b1) * d1 + sigmoid(g2 + b2) * d2       (the layer's result)
//   x'  = sum_j w[j] * X_j  (j over the earlier results, kept in `hist`) + w[last] * X
//   y   = x' / sqrt(mean(x'^2) + eps) * nw                        (what the next layer reads)
//
// Every term is optional: a contribution d may be absent, come in the activation type or
// as a stack of 32-bit partial sums (added in order), and may have no gate; without
// `hist` there is no averaging (x' = X); without `nw` y is x' itself, rounded.  All sums
// are 32-bit.  X is stored as entry `n_hist` of `hist` (unless a row list picks rows: the
// last layer's gather for the head), x' as the new stream.  A row's result depends on
// that row alone, and the order of every sum is fixed by the sizes.
//
// One block per row, x' staying in shared memory between the two passes; or, for the few rows
// of a decode step, a cluster of blocks per row (below).
#include "common.cuh"
#include <type_traits>

struct GatedTerm {
  const void* delta;        // [T, N] activation type, or null
  const float* parts;       // [n_parts][T, N] 32-bit partial sums, or null
  int n_parts;
  long long part_stride;    // floats between partial sums
  const float* gate;        // [T, gate_ld] logits, or null: the term is not gated
  long long gate_ld;
  const float* gate_bias;   // [N] or null
};

struct GatedNormArgs {
  const float* res_in;      // [T, N] or null
  GatedTerm term[2];
  float* hist;              // [n_hist + 1][T, N] or null
  long long hist_stride;    // floats between entries
  int n_hist;               // entries that hold earlier results
  const float* avg_w;       // [n_hist + 1]
  const int* rows;          // [n_rows] or null: all T rows in order
  const float* norm_w;      // [N] 32-bit, or null
  float eps;
  float* res_out;           // [n_rows, N] (may be res_in when rows is null) or null
  void* y;                  // [n_rows, N]
  int n_rows, N;
};

__device__ __forceinline__ float gn_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// V consecutive values: one 16-byte piece (8 bytes for bfloat16) where V is 4, else one value.
template <int V> __device__ __forceinline__ void gn_load(const float* p, float (&o)[V]) {
  if constexpr (V == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x, o[1] = v.y, o[2] = v.z, o[3] = v.w;
  } else {
    o[0] = p[0];
  }
}
template <int V> __device__ __forceinline__ void gn_load(const bf16* p, float (&o)[V]) {
  if constexpr (V == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    o[0] = __low2float(a), o[1] = __high2float(a), o[2] = __low2float(b), o[3] = __high2float(b);
  } else {
    o[0] = __bfloat162float(p[0]);
  }
}
template <int V> __device__ __forceinline__ void gn_store(float* p, const float (&v)[V]) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else p[0] = v[0];
}
template <int V> __device__ __forceinline__ void gn_store(bf16* p, const float (&v)[V]) {
  if constexpr (V == 4) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  } else {
    p[0] = __float2bfloat16_rn(v[0]);
  }
}

// The new stream's V values at columns n .. n + V - 1 of source row t; the layer's result is
// stored among the earlier ones on the way.  Loads that do not depend on one another (the
// partial sums, the earlier results) are requested together and used in order.
// GN_AHEAD: how many earlier results are requested at a time: many where a step has few rows (the
// time is the loads' round trips), fewer where it has many (registers decide how many rows an SM holds)
template <typename T, int V, int GN_AHEAD>
__device__ __forceinline__ void gn_values(const GatedNormArgs& a, size_t t, int n, float (&xp)[V]) {
  const int N = a.N;
  // the first earlier results depend on nothing of this layer: they are requested first and
  // are on their way while the layer's own terms are put together
  constexpr bool EARLY = GN_AHEAD > 8;
  constexpr int PARTS = EARLY ? 8 : 4;      // partial sums requested at a time
  float hv[GN_AHEAD][V];
  if (EARLY && a.hist) {
#pragma unroll
    for (int u = 0; u < GN_AHEAD; ++u) {
      const int j = u < a.n_hist ? u : (a.n_hist > 0 ? a.n_hist - 1 : 0);
      if (a.n_hist > 0) gn_load<V>(a.hist + (size_t)j * a.hist_stride + t * N + n, hv[u]);
    }
  }
  float X[V];
#pragma unroll
  for (int e = 0; e < V; ++e) X[e] = 0.f;
  if (a.res_in) gn_load<V>(a.res_in + t * N + n, X);
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const GatedTerm& g = a.term[c];
    if (!g.delta && !g.parts) continue;
    float d[V], z[V], b[V];
#pragma unroll
    for (int e = 0; e < V; ++e) d[e] = 0.f, z[e] = 0.f, b[e] = 0.f;
    if (g.gate) gn_load<V>(g.gate + t * g.gate_ld + n, z);
    if (g.gate && g.gate_bias) gn_load<V>(g.gate_bias + n, b);
    if (g.delta) {
      gn_load<V>((const T*)g.delta + t * N + n, d);
    } else {
      for (int k0 = 0; k0 < g.n_parts; k0 += PARTS) {
        float pk[PARTS][V];
#pragma unroll
        for (int u = 0; u < PARTS; ++u) {
          const int k = k0 + u < g.n_parts ? k0 + u : g.n_parts - 1;
          gn_load<V>(g.parts + (size_t)k * g.part_stride + t * N + n, pk[u]);
        }
#pragma unroll
        for (int u = 0; u < PARTS; ++u)
          if (k0 + u < g.n_parts) {
#pragma unroll
            for (int e = 0; e < V; ++e) d[e] += pk[u][e];
          }
      }
    }
    if (g.gate) {
#pragma unroll
      for (int e = 0; e < V; ++e) d[e] *= gn_sigmoid(z[e] + b[e]);
    }
#pragma unroll
    for (int e = 0; e < V; ++e) X[e] += d[e];
  }
  if (!a.hist) {
#pragma unroll
    for (int e = 0; e < V; ++e) xp[e] = X[e];
    return;
  }
  if (!a.rows) gn_store<V>(a.hist + (size_t)a.n_hist * a.hist_stride + t * N + n, X);
#pragma unroll
  for (int e = 0; e < V; ++e) xp[e] = 0.f;
  for (int j0 = 0; j0 < a.n_hist; j0 += GN_AHEAD) {
    if (j0 > 0 || !EARLY) {
#pragma unroll
      for (int u = 0; u < GN_AHEAD; ++u) {
        const int j = j0 + u < a.n_hist ? j0 + u : a.n_hist - 1;
        gn_load<V>(a.hist + (size_t)j * a.hist_stride + t * N + n, hv[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < GN_AHEAD; ++u)
      if (j0 + u < a.n_hist) {
        const float w = a.avg_w[j0 + u];
#pragma unroll
        for (int e = 0; e < V; ++e) xp[e] = fmaf(w, hv[u][e], xp[e]);
      }
  }
  const float w = a.avg_w[a.n_hist];
#pragma unroll
  for (int e = 0; e < V; ++e) xp[e] = fmaf(w, X[e], xp[e]);
}

template <typename T, int V>
__global__ void __launch_bounds__(256) gated_norm_kernel(const GatedNormArgs a) {
  extern __shared__ __align__(16) float gn_row[];        // [N]
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int r = blockIdx.x, N = a.N;
  const size_t t = a.rows ? (size_t)a.rows[r] : (size_t)r;
  float ss = 0.f;
  for (int n = threadIdx.x * V; n < N; n += blockDim.x * V) {
    float xp[V];
    gn_values<T, V, 8>(a, t, n, xp);
    gn_store<V>(gn_row + n, xp);
#pragma unroll
    for (int e = 0; e < V; ++e) ss = fmaf(xp[e], xp[e], ss);
  }
  pdl_launch_dependents_if_large();
  float inv = 1.f;
  if (a.norm_w) inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)N + a.eps);
  for (int n = threadIdx.x * V; n < N; n += blockDim.x * V) {   // a thread reads back what it wrote
    float xp[V], w[V], o[V];
    gn_load<V>(gn_row + n, xp);
    if (a.res_out) gn_store<V>(a.res_out + (size_t)r * N + n, xp);
#pragma unroll
    for (int e = 0; e < V; ++e) w[e] = 1.f;
    if (a.norm_w) gn_load<V>(a.norm_w + n, w);
#pragma unroll
    for (int e = 0; e < V; ++e) o[e] = a.norm_w ? xp[e] * inv * w[e] : xp[e];
    gn_store<V>((T*)a.y + (size_t)r * N + n, o);
  }
}

// A handful of rows (a decode step) would keep a handful of SMs busy, each walking a long row
// alone.  Here a cluster of GN_CLUSTER blocks shares a row: each block owns an eighth of the
// columns (a thread four of them, kept in registers), the sums of squares meet through
// distributed shared memory (added in rank order, so the result is a fixed sum), and every
// block scales its columns.  The cluster barrier is the hardware's; no block spins on memory.
#define GN_CLUSTER 8
#include <cooperative_groups.h>
namespace cg = cooperative_groups;
template <typename T>
__global__ void gated_norm_cluster_kernel(const GatedNormArgs a) {
  __shared__ float scratch[32];
  __shared__ float ss_all[GN_CLUSTER];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int N = a.N, cols = N / GN_CLUSTER;
  const int r = blockIdx.x / GN_CLUSTER;
  const size_t t = a.rows ? (size_t)a.rows[r] : (size_t)r;
  const int n = rank * cols + threadIdx.x * 4;
  const bool active = threadIdx.x * 4 < cols;
  float xp[4] = {0.f, 0.f, 0.f, 0.f};
  float ss = 0.f;
  if (active) {
    gn_values<T, 4, 16>(a, t, n, xp);
#pragma unroll
    for (int e = 0; e < 4; ++e) ss = fmaf(xp[e], xp[e], ss);
    if (a.res_out) gn_store<4>(a.res_out + (size_t)r * N + n, xp);
  }
  ss = block_sum(ss, scratch);
  // every block puts its sum into every block's table (thread k writes to block k), so that
  // one cluster barrier is enough: after it each block reads its own shared memory only
  if (threadIdx.x < GN_CLUSTER) cluster.map_shared_rank(ss_all, threadIdx.x)[rank] = ss;
  cluster.sync();
  float total = 0.f;
#pragma unroll
  for (int k = 0; k < GN_CLUSTER; ++k) total += ss_all[k];
  if (active) {
    float w[4] = {1.f, 1.f, 1.f, 1.f}, o[4];
    const float inv = a.norm_w ? 1.0f / sqrtf(total / (float)N + a.eps) : 1.f;
    if (a.norm_w) gn_load<4>(a.norm_w + n, w);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = a.norm_w ? xp[e] * inv * w[e] : xp[e];
    gn_store<4>((T*)a.y + (size_t)r * N + n, o);
  }
}

template <typename T, int V>
static int launch_rows(const GatedNormArgs& a, cudaStream_t s) {
  const size_t smem = (size_t)a.N * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_UNSUPPORTED;
  static size_t configured = 48 * 1024;     // per instantiation
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gated_norm_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return gb_launch(gated_norm_kernel<T, V>, dim3(a.n_rows), dim3(256), smem, s, a);
}

template <typename T>
static int launch(const GatedNormArgs& a, cudaStream_t s) {
  if (a.n_rows < 0 || a.N <= 0 || !a.y) return GB_ERR_BAD_ARG;
  if (a.hist && (!a.avg_w || a.n_hist < 0)) return GB_ERR_BAD_ARG;
  for (int c = 0; c < 2; ++c)
    if (a.term[c].parts && a.term[c].n_parts <= 0) return GB_ERR_BAD_ARG;
  if (a.n_rows == 0) return 0;
  // 16-byte pieces need every row of every tensor to start on a 16-byte boundary
  uintptr_t bits = (uintptr_t)a.res_in | (uintptr_t)a.hist | (uintptr_t)a.norm_w | (uintptr_t)a.res_out |
                   (uintptr_t)a.y | (uintptr_t)(a.hist_stride * 4);
  for (int c = 0; c < 2; ++c) {
    const GatedTerm& g = a.term[c];
    bits |= (uintptr_t)g.delta | (uintptr_t)g.parts | (uintptr_t)(g.part_stride * 4) | (uintptr_t)g.gate |
            (uintptr_t)(g.gate_ld * 4) | (uintptr_t)g.gate_bias;
  }
  const bool wide = (bits & 15) == 0 && a.N % 4 == 0;
  // The cluster kernel is chosen by the number of rows and adds the squares in another order
  // than the kernel of one block a row.  The 32-bit path never takes it: there the order of a
  // row's sums may depend on the width alone, so that a token's result is the same in a step
  // of one row and in a step of thousands.
  constexpr bool by_rows_too = !std::is_same<T, float>::value;
  if (by_rows_too && wide && a.n_rows <= 64 && a.N >= 512 && a.N % (4 * GN_CLUSTER) == 0 &&
      a.N / GN_CLUSTER / 4 <= 1024) {
    const int threads = ((a.N / GN_CLUSTER / 4 + 31) / 32) * 32;
    return gb_launch_cluster(gated_norm_cluster_kernel<T>, dim3(a.n_rows * GN_CLUSTER), dim3(threads), 0, s,
                             GN_CLUSTER, a);
  }
  return wide ? launch_rows<T, 4>(a, s) : launch_rows<T, 1>(a, s);
}

GB_EXPORT int gb_gated_norm_f32(const GatedNormArgs* a, cudaStream_t s) { return launch<float>(*a, s); }
GB_EXPORT int gb_gated_norm_bf16(const GatedNormArgs* a, cudaStream_t s) { return launch<bf16>(*a, s); }
