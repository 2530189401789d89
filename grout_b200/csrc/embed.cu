// Token embedding: out[t, :] = table[ids[t], :], a pure copy
// (the reference's embedding_batch_f16, src/kernels.rs:693-711).
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* ids,
                             T* __restrict__ out, int H, int V) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;  // an id outside the table gives a zero row
  const T* src = table + (size_t)(ok ? id : 0) * H;
  T* dst = out + (size_t)t * H;
  const int per16 = 16 / (int)sizeof(T);
  if ((H % per16) == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
    const int n = H / per16;
    for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = ok ? s4[i] : make_int4(0, 0, 0, 0);
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? src[i] : from_f32<T>(0.f);
  }
  pdl_launch_dependents_if_large();
}

template <typename T>
static int embed_launch(const void* table, const int* ids, void* out, int n_tokens, int H, int V,
                        cudaStream_t stream) {
  if (n_tokens < 0 || H <= 0 || V <= 0) return GB_ERR_BAD_ARG;
  if (n_tokens == 0) return 0;
  return gb_launch(embed_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)table, ids,
                   (T*)out, H, V);
}

GB_EXPORT int gb_embed_f32(const void* table, const int* ids, void* out, int n_tokens, int H, int V,
                           cudaStream_t s) {
  return embed_launch<float>(table, ids, out, n_tokens, H, V, s);
}
GB_EXPORT int gb_embed_bf16(const void* table, const int* ids, void* out, int n_tokens, int H,
                            int V, cudaStream_t s) {
  return embed_launch<bf16>(table, ids, out, n_tokens, H, V, s);
}

// Token embedding plus a learned position vector, then an RMS norm:
//   out[t, :] = v / sqrt(mean(v^2) + eps) * w,   v = table[ids[t], :] + positions[pos[t], :]
// The sum and the norm are 32-bit and so is `out`, which is the residual stream.
// A position outside the table (a padding row's is always 0) gives a zero vector.
template <typename T>
__global__ void embed_pos_norm_kernel(const T* __restrict__ table, const T* __restrict__ positions,
                                      const int* ids, const int* pos, const float* __restrict__ w,
                                      float eps, float* __restrict__ out, int H, int V, int P) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t], p = pos[t];
  const bool ok = id >= 0 && id < V, pok = p >= 0 && p < P;
  const T* src = table + (size_t)(ok ? id : 0) * H;
  const T* ps = positions + (size_t)(pok ? p : 0) * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = (ok ? to_f32<T>(src[i]) : 0.f) + (pok ? to_f32<T>(ps[i]) : 0.f);
    row[i] = v;
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
  pdl_launch_dependents_if_large();
  float* dst = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = row[i] * inv * w[i];
}

template <typename T>
static int embed_pos_norm_launch(const void* table, const void* positions, const int* ids,
                                 const int* pos, const float* w, float eps, float* out,
                                 int n_tokens, int H, int V, int P, cudaStream_t stream) {
  if (n_tokens < 0 || H <= 0 || V <= 0 || P <= 0 || !w) return GB_ERR_BAD_ARG;
  if (n_tokens == 0) return 0;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(embed_pos_norm_kernel<T>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = ((H + 3) / 4 + 31) / 32 * 32;   // by H only, so the sums' tree is fixed
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  return gb_launch(embed_pos_norm_kernel<T>, dim3(n_tokens), dim3(threads), smem, stream,
                   (const T*)table, (const T*)positions, ids, pos, w, eps, out, H, V, P);
}

GB_EXPORT int gb_embed_pos_norm_f32(const void* table, const void* positions, const int* ids,
                                    const int* pos, const float* w, float eps, float* out,
                                    int n_tokens, int H, int V, int P, cudaStream_t s) {
  return embed_pos_norm_launch<float>(table, positions, ids, pos, w, eps, out, n_tokens, H, V, P, s);
}
GB_EXPORT int gb_embed_pos_norm_bf16(const void* table, const void* positions, const int* ids,
                                     const int* pos, const float* w, float eps, float* out,
                                     int n_tokens, int H, int V, int P, cudaStream_t s) {
  return embed_pos_norm_launch<bf16>(table, positions, ids, pos, w, eps, out, n_tokens, H, V, P, s);
}

// Token embedding times a constant: out[t, :] = scale * table[ids[t], :] as 32-bit rows,
// which are the residual stream itself (a scaled row need not be a bfloat16 number).
template <typename T>
__global__ void embed_scaled_kernel(const T* __restrict__ table, const int* ids, float scale,
                                    float* __restrict__ out, int H, int V) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < V;  // an id outside the table gives a zero row
  const T* src = table + (size_t)(ok ? id : 0) * H;
  float* dst = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? scale * to_f32<T>(src[i]) : 0.f;
  pdl_launch_dependents_if_large();
}
template <typename T>
static int embed_scaled_launch(const void* table, const int* ids, float scale, float* out, int n_tokens,
                               int H, int V, cudaStream_t stream) {
  if (n_tokens < 0 || H <= 0 || V <= 0) return GB_ERR_BAD_ARG;
  if (n_tokens == 0) return 0;
  return gb_launch(embed_scaled_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)table, ids,
                   scale, out, H, V);
}
GB_EXPORT int gb_embed_scaled_f32(const void* table, const int* ids, float scale, float* out,
                                  int n_tokens, int H, int V, cudaStream_t s) {
  return embed_scaled_launch<float>(table, ids, scale, out, n_tokens, H, V, s);
}
GB_EXPORT int gb_embed_scaled_bf16(const void* table, const int* ids, float scale, float* out,
                                   int n_tokens, int H, int V, cudaStream_t s) {
  return embed_scaled_launch<bf16>(table, ids, scale, out, n_tokens, H, V, s);
}
