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
// One block per row; x' stays in shared memory between the two passes.
#include "common.cuh"

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

template <typename T>
__global__ void __launch_bounds__(256) gated_norm_kernel(const GatedNormArgs a) {
  extern __shared__ float gn_row[];        // [N]
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int r = blockIdx.x, N = a.N;
  const size_t t = a.rows ? (size_t)a.rows[r] : (size_t)r;
  float ss = 0.f;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float X = a.res_in ? a.res_in[t * N + n] : 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const GatedTerm& g = a.term[c];
      if (!g.delta && !g.parts) continue;
      float d = 0.f;
      if (g.delta) d = to_f32<T>(((const T*)g.delta)[t * N + n]);
      else
        for (int k = 0; k < g.n_parts; ++k) d += g.parts[(size_t)k * g.part_stride + t * N + n];
      if (g.gate) d *= gn_sigmoid(g.gate[t * g.gate_ld + n] + (g.gate_bias ? g.gate_bias[n] : 0.f));
      X += d;
    }
    float xp = X;
    if (a.hist) {
      if (!a.rows) a.hist[(size_t)a.n_hist * a.hist_stride + t * N + n] = X;
      xp = 0.f;
      for (int j = 0; j < a.n_hist; ++j) xp = fmaf(a.avg_w[j], a.hist[(size_t)j * a.hist_stride + t * N + n], xp);
      xp = fmaf(a.avg_w[a.n_hist], X, xp);
    }
    gn_row[n] = xp;
    ss = fmaf(xp, xp, ss);
  }
  pdl_launch_dependents_if_large();
  float inv = 1.f;
  if (a.norm_w) inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)N + a.eps);
  for (int n = threadIdx.x; n < N; n += blockDim.x) {   // a thread reads back what it wrote
    const float xp = gn_row[n];
    if (a.res_out) a.res_out[(size_t)r * N + n] = xp;
    ((T*)a.y)[(size_t)r * N + n] = from_f32<T>(a.norm_w ? xp * inv * a.norm_w[n] : xp);
  }
}

template <typename T>
static int launch(const GatedNormArgs& a, cudaStream_t s) {
  if (a.n_rows < 0 || a.N <= 0 || !a.y) return GB_ERR_BAD_ARG;
  if (a.hist && (!a.avg_w || a.n_hist < 0)) return GB_ERR_BAD_ARG;
  for (int c = 0; c < 2; ++c)
    if (a.term[c].parts && a.term[c].n_parts <= 0) return GB_ERR_BAD_ARG;
  if (a.n_rows == 0) return 0;
  const size_t smem = (size_t)a.N * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_UNSUPPORTED;
  static size_t configured = 48 * 1024;     // per instantiation
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gated_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return gb_launch(gated_norm_kernel<T>, dim3(a.n_rows), dim3(256), smem, s, a);
}

GB_EXPORT int gb_gated_norm_f32(const GatedNormArgs* a, cudaStream_t s) { return launch<float>(*a, s); }
GB_EXPORT int gb_gated_norm_bf16(const GatedNormArgs* a, cudaStream_t s) { return launch<bf16>(*a, s); }
