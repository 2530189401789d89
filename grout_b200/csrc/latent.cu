// Attention whose keys and values are expanded from one small latent vector per
// token.  The mixer's one projection gives, per token, the queries (per head `dn`
// plain and `dr` rotated elements), a row of R + dr numbers and a gate.  The first
// R numbers, RMS-normalised with a weight, are the latent c; the last dr, rotated,
// are a key part that all heads share.  A head's plain key is Wuk_h c and its
// value Wuv_h c, so
//
//   score = q_plain . (Wuk_h c) + q_rot . k_rot = (Wuk_h^T q_plain) . c + q_rot . k_rot
//   out   = Wuv_h (sum_j p_j c_j)
//
// and the cache holds one row [c | k_rot] per token, shared by the heads, which
// serves as key and as value: attention runs as if every query head read one kv
// head of R + dr elements, with the query [Wuk_h^T q_plain | q_rot].
//
// `prepare` does the norm and the rotations in 32-bit on the projection's 32-bit
// sums, stores the cache row and writes the queries' two parts; the rotation
// pairs element 2i with element 2i + 1.  `heads_mm` is the per-head product
// out[t, h, :] = W_h x[t, h, :] that folds Wuk into the queries and expands the
// attention's output, the latter with the gate sigmoid(g) applied to its 32-bit sums.
#include "common.cuh"

struct LatentArgs {
  const float* proj;       // [T, H (dn + dr) + R + dr + H dv] 32-bit sums: q | down | gate
  const float* norm_w;     // [R]
  const float* inv_freq;   // [dr / 2]
  const int* token_seq;    // [T]
  const int* token_pos;    // [T]
  const int* slots;        // [n_seqs]
  const int* block_table;  // [slots, max_pages]
  void* pages;             // [n_pages, 1, page, Ds]
  void* q_plain;           // [T, H, dn]
  void* q_full;            // [T, H, Ds]: columns R .. R + dr get the rotated part, columns from R + dr on zeros
  int n_tokens, H, dn, dr, R, dv, Ds, max_pages, page;
  float eps;
};

template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const LatentArgs a) {
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = a.H, dn = a.dn, dr = a.dr, R = a.R, Ds = a.Ds;
  const int C = H * (dn + dr) + R + dr + H * a.dv;
  const float* row = a.proj + (size_t)t * C;
  const float* down = row + H * (dn + dr);
  const float pos = (float)a.token_pos[t];
  float ss = 0.f;
  for (int i = tid; i < R; i += blockDim.x) ss = fmaf(down[i], down[i], ss);
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)R + a.eps);
  pdl_launch_dependents_if_large();
  const int slot = a.slots[a.token_seq[t]];
  if (slot >= 0) {
    const int p = a.token_pos[t];
    const int pg = a.block_table[(size_t)slot * a.max_pages + p / a.page];
    T* dst = (T*)a.pages + ((size_t)pg * a.page + p % a.page) * Ds;
    for (int i = tid; i < Ds; i += blockDim.x) {
      float v = 0.f;
      if (i < R) v = down[i] * inv * a.norm_w[i];
      else if (i < R + dr) {
        const int e = i - R, pair = e >> 1;
        float s, c;
        sincosf(pos * a.inv_freq[pair], &s, &c);
        const float u = down[R + 2 * pair], w = down[R + 2 * pair + 1];
        v = (e & 1) ? w * c + u * s : u * c - w * s;
      }
      dst[i] = from_f32<T>(v);
    }
  }
  for (int i = tid; i < H * (dn + dr); i += blockDim.x) {
    const int h = i / (dn + dr), e = i % (dn + dr);
    if (e < dn) {
      ((T*)a.q_plain)[((size_t)t * H + h) * dn + e] = from_f32<T>(row[i]);
    } else {
      const int r = e - dn, pair = r >> 1;
      float s, c;
      sincosf(pos * a.inv_freq[pair], &s, &c);
      const float u = row[h * (dn + dr) + dn + 2 * pair], w = row[h * (dn + dr) + dn + 2 * pair + 1];
      ((T*)a.q_full)[((size_t)t * H + h) * Ds + R + r] = from_f32<T>((r & 1) ? w * c + u * s : u * c - w * s);
    }
  }
  for (int i = tid; i < H * (Ds - R - dr); i += blockDim.x) {
    const int h = i / (Ds - R - dr), e = i % (Ds - R - dr);
    ((T*)a.q_full)[((size_t)t * H + h) * Ds + R + dr + e] = from_f32<T>(0.f);
  }
}

template <typename T>
static int latent_prepare(const LatentArgs& a, cudaStream_t s) {
  if (a.n_tokens < 0 || a.H <= 0 || a.dn <= 0 || a.dr < 0 || a.dr % 2 || a.R <= 0 || a.dv < 0 ||
      a.Ds < a.R + a.dr || a.page <= 0 || a.max_pages <= 0)
    return GB_ERR_BAD_ARG;
  if (!a.proj || !a.norm_w || !a.token_seq || !a.token_pos || !a.slots || !a.block_table || !a.pages ||
      !a.q_plain || !a.q_full || (a.dr && !a.inv_freq))
    return GB_ERR_BAD_ARG;
  if (a.n_tokens == 0) return 0;
  return gb_launch(latent_prepare_kernel<T>, dim3(a.n_tokens), dim3(256), 0, s, a);
}
GB_EXPORT int gb_latent_prepare_f32(const LatentArgs* a, cudaStream_t s) { return latent_prepare<float>(*a, s); }
GB_EXPORT int gb_latent_prepare_bf16(const LatentArgs* a, cudaStream_t s) { return latent_prepare<bf16>(*a, s); }

// out[t, h, n] = gate(t, h, n) * sum_k w[h, n, k] x[t, h, k]
//   x rows [T, H, ldx] (the first K of a head's ldx elements are read), w [H, N, K],
//   out rows [T, H, ldo] (the first N of ldo are written); gate = sigmoid(g[t * ldg + h N + n])
//   when g is given, else one.  Sums are 32-bit in a fixed order whatever T.
struct HeadsMmArgs {
  const void* x;
  const void* w;
  void* out;
  const float* g;
  int T, H, K, N, ldx, ldo, ldg;
};

#define HM_BM 16
#define HM_BN 64
#define HM_BK 32

template <typename T>
__global__ void __launch_bounds__(256) heads_mm_kernel(const HeadsMmArgs a) {
  __shared__ float As[HM_BM][HM_BK];
  __shared__ float Bs[HM_BN][HM_BK + 1];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int tid = threadIdx.x, h = blockIdx.z;
  const int t0 = blockIdx.x * HM_BM, n0 = blockIdx.y * HM_BN;
  const int K = a.K, N = a.N;
  const T* x = (const T*)a.x;
  const T* w = (const T*)a.w + (size_t)h * N * K;
  const int tx = tid & 63, ty = tid >> 6;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += HM_BK) {
    for (int i = tid; i < HM_BM * HM_BK; i += 256) {
      const int r = i / HM_BK, k = i % HM_BK;
      As[r][k] = (t0 + r < a.T && k0 + k < K)
                     ? to_f32<T>(x[((size_t)(t0 + r) * a.H + h) * a.ldx + k0 + k]) : 0.f;
    }
    for (int i = tid; i < HM_BN * HM_BK; i += 256) {
      const int n = i / HM_BK, k = i % HM_BK;
      Bs[n][k] = (n0 + n < N && k0 + k < K) ? to_f32<T>(w[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HM_BK; ++k) {
      const float b = Bs[tx][k];
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[r] = fmaf(As[ty * 4 + r][k], b, acc[r]);
    }
    __syncthreads();
  }
  pdl_launch_dependents_if_large();
  if (n0 + tx >= N) return;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = t0 + ty * 4 + r;
    if (t >= a.T) continue;
    float v = acc[r];
    if (a.g) {
      const float gv = a.g[(size_t)t * a.ldg + h * N + n0 + tx];
      v *= 1.0f / (1.0f + expf(-gv));
    }
    ((T*)a.out)[((size_t)t * a.H + h) * a.ldo + n0 + tx] = from_f32<T>(v);
  }
}

template <typename T>
static int heads_mm(const HeadsMmArgs& a, cudaStream_t s) {
  if (a.T < 0 || a.H <= 0 || a.K <= 0 || a.N <= 0 || a.ldx < a.K || a.ldo < a.N || a.H > 65535)
    return GB_ERR_BAD_ARG;
  if (!a.x || !a.w || !a.out) return GB_ERR_BAD_ARG;
  if (a.T == 0) return 0;
  return gb_launch(heads_mm_kernel<T>, dim3((a.T + HM_BM - 1) / HM_BM, (a.N + HM_BN - 1) / HM_BN, a.H),
                   dim3(256), 0, s, a);
}
GB_EXPORT int gb_heads_mm_f32(const HeadsMmArgs* a, cudaStream_t s) { return heads_mm<float>(*a, s); }
GB_EXPORT int gb_heads_mm_bf16(const HeadsMmArgs* a, cudaStream_t s) { return heads_mm<bf16>(*a, s); }
