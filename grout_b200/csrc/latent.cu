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
// attention's output, the latter with the gate sigmoid(g) applied to its 32-bit sums:
// for 32-bit tensors a plain tiled kernel, for bfloat16 on the tensor cores.
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

// A block owns one token and the heads blockIdx.y * heads_per_block ..; the block of the
// first heads also normalises the latent and stores the token's cache row.
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const LatentArgs a, const int heads_per_block) {
  __shared__ float scratch[32];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  const int H = a.H, dn = a.dn, dr = a.dr, R = a.R, Ds = a.Ds;
  const int h0 = blockIdx.y * heads_per_block, nh = min(heads_per_block, H - h0);
  const int C = H * (dn + dr) + R + dr + H * a.dv;
  const float* __restrict__ row = a.proj + (size_t)t * C;
  const float* __restrict__ down = row + H * (dn + dr);
  const float pos = (float)a.token_pos[t];
  if (blockIdx.y == 0) {
    float ss = 0.f;
    for (int i = tid; i < R; i += blockDim.x) ss = fmaf(down[i], down[i], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)R + a.eps);
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
  }
  pdl_launch_dependents_if_large();
  T* __restrict__ q_plain = (T*)a.q_plain + ((size_t)t * H + h0) * dn;
  T* __restrict__ q_full = (T*)a.q_full + ((size_t)t * H + h0) * Ds;
  const float* __restrict__ qrow = row + (size_t)h0 * (dn + dr);
  for (int i = tid; i < nh * (dn + dr); i += blockDim.x) {
    const int h = i / (dn + dr), e = i % (dn + dr);
    if (e < dn) {
      q_plain[(size_t)h * dn + e] = from_f32<T>(qrow[i]);
    } else {
      const int r = e - dn, pair = r >> 1;
      float s, c;
      sincosf(pos * a.inv_freq[pair], &s, &c);
      const float u = qrow[h * (dn + dr) + dn + 2 * pair], w = qrow[h * (dn + dr) + dn + 2 * pair + 1];
      q_full[(size_t)h * Ds + R + r] = from_f32<T>((r & 1) ? w * c + u * s : u * c - w * s);
    }
  }
  for (int i = tid; i < nh * (Ds - R - dr); i += blockDim.x) {
    const int h = i / (Ds - R - dr), e = i % (Ds - R - dr);
    q_full[(size_t)h * Ds + R + dr + e] = from_f32<T>(0.f);
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
  // few tokens: four heads a block, so that a step of a handful of rows fills more than a handful of SMs
  const int heads_per_block = a.n_tokens <= 64 ? min(a.H, 4) : a.H;
  return gb_launch(latent_prepare_kernel<T>, dim3(a.n_tokens, (a.H + heads_per_block - 1) / heads_per_block),
                   dim3(256), 0, s, a, heads_per_block);
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

// The same product for bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit sums).
// A block owns 32 MW rows and HT_BN columns of one head; its warps stand MW by 2, each
// with 32 rows and 32 columns: two row tiles by four column tiles of the instruction.
// x and w both have a head's elements side by side, which is the order the instruction
// wants its operands in, so a lane reads its pairs from the staged tiles as they are.
// Rows and elements outside the matrices are staged as zeros.  A sum's order does not
// depend on T.
#define HT_BN 64
#define HT_BK 64
#define HT_LD (HT_BK + 8)     // 36 words a row: the eight rows a lane group reads fall on different banks

// ITERS turns of eight elements (16 bytes) a thread: all of a thread's loads are asked for
// before the first is stored, so a stage costs one trip to memory, not one a turn.
template <int ITERS, int THREADS>
__device__ __forceinline__ void ht_stage(bf16 (*dst)[HT_LD], const bf16* src, size_t ld, int rows_here,
                                         int k0, int K, bool vec, int tid) {
  uint4 v[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = tid + it * THREADS;
    const int r = i / (HT_BK / 8), kv = (i % (HT_BK / 8)) * 8;
    v[it] = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows_here) {
      const bf16* p = src + (size_t)r * ld + k0 + kv;
      if (vec && k0 + kv + 8 <= K) {
        v[it] = *reinterpret_cast<const uint4*>(p);
      } else {
        __align__(16) bf16 e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = k0 + kv + j < K ? p[j] : __float2bfloat16_rn(0.f);
        v[it] = *reinterpret_cast<const uint4*>(e);
      }
    }
  }
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int i = tid + it * THREADS;
    *reinterpret_cast<uint4*>(&dst[i / (HT_BK / 8)][(i % (HT_BK / 8)) * 8]) = v[it];
  }
}

template <int MW>
__global__ void __launch_bounds__(MW * 64) heads_mm_tc_kernel(const HeadsMmArgs a, const int vec) {
  constexpr int BM = 32 * MW, THREADS = MW * 64;
  __shared__ __align__(16) bf16 As[BM][HT_LD];
  __shared__ __align__(16) bf16 Bs[HT_BN][HT_LD];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, h = blockIdx.z;
  const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, tig = lane & 3;
  const int t0 = blockIdx.x * BM, n0 = blockIdx.y * HT_BN;
  const int K = a.K, N = a.N;
  const bf16* x = (const bf16*)a.x + ((size_t)t0 * a.H + h) * a.ldx;
  const bf16* w = (const bf16*)a.w + ((size_t)h * N + n0) * K;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HT_BK) {
    if (k0) __syncthreads();
    ht_stage<BM * (HT_BK / 8) / THREADS, THREADS>(As, x, (size_t)a.H * a.ldx, min(BM, a.T - t0), k0, K, vec & 1, tid);
    ht_stage<HT_BN * (HT_BK / 8) / THREADS, THREADS>(Bs, w, (size_t)K, min(HT_BN, N - n0), k0, K, vec & 2, tid);
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HT_BK; kk += 16) {
      if (k0 + kk >= K) break;
      unsigned af[2][4], bfr[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const bf16* r0 = &As[wm * 32 + i * 16 + g][kk + 2 * tig];
        af[i][0] = *reinterpret_cast<const unsigned*>(r0);
        af[i][1] = *reinterpret_cast<const unsigned*>(r0 + 8 * HT_LD);
        af[i][2] = *reinterpret_cast<const unsigned*>(r0 + 8);
        af[i][3] = *reinterpret_cast<const unsigned*>(r0 + 8 * HT_LD + 8);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bf16* r0 = &Bs[wn * 32 + j * 8 + g][kk + 2 * tig];
        bfr[j][0] = *reinterpret_cast<const unsigned*>(r0);
        bfr[j][1] = *reinterpret_cast<const unsigned*>(r0 + 8);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          asm volatile(
              "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
              "{%0,%1,%2,%3};\n"
              : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
              : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(bfr[j][0]), "r"(bfr[j][1]));
    }
  }
  pdl_launch_dependents_if_large();
  const bool pack = vec & 4;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int t = t0 + wm * 32 + i * 16 + g + half * 8;
      if (t >= a.T) continue;
      bf16* o = (bf16*)a.out + ((size_t)t * a.H + h) * a.ldo;
      const float* gp = a.g ? a.g + (size_t)t * a.ldg + h * N : nullptr;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + wn * 32 + j * 8 + 2 * tig;
        if (n >= N) continue;
        float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
        if (gp) {
          v0 *= 1.0f / (1.0f + expf(-gp[n]));
          if (n + 1 < N) v1 *= 1.0f / (1.0f + expf(-gp[n + 1]));
        }
        if (pack && n + 1 < N) {
          *reinterpret_cast<__nv_bfloat162*>(o + n) = __floats2bfloat162_rn(v0, v1);
        } else {
          o[n] = __float2bfloat16_rn(v0);
          if (n + 1 < N) o[n + 1] = __float2bfloat16_rn(v1);
        }
      }
    }
}

template <typename T>
static int heads_mm(const HeadsMmArgs& a, cudaStream_t s) {
  if (a.T < 0 || a.H <= 0 || a.K <= 0 || a.N <= 0 || a.ldx < a.K || a.ldo < a.N || a.H > 65535)
    return GB_ERR_BAD_ARG;
  if (!a.x || !a.w || !a.out) return GB_ERR_BAD_ARG;
  if (a.T == 0) return 0;
  if (sizeof(T) == 2) {
    // bit 0: rows of x can be read 16 bytes at a time; bit 1: rows of w; bit 2: pairs of the result stored as one word
    const int vec = ((a.ldx % 8 == 0 && (uintptr_t)a.x % 16 == 0) ? 1 : 0) |
                    ((a.K % 8 == 0 && (uintptr_t)a.w % 16 == 0) ? 2 : 0) |
                    ((a.ldo % 2 == 0 && (uintptr_t)a.out % 4 == 0) ? 4 : 0);
    const unsigned ny = (a.N + HT_BN - 1) / HT_BN;
    if (a.T <= 32) return gb_launch(heads_mm_tc_kernel<1>, dim3(1, ny, a.H), dim3(64), 0, s, a, vec);
    if (a.T <= 64) return gb_launch(heads_mm_tc_kernel<2>, dim3(1, ny, a.H), dim3(128), 0, s, a, vec);
    return gb_launch(heads_mm_tc_kernel<4>, dim3((a.T + 127) / 128, ny, a.H), dim3(256), 0, s, a, vec);
  }
  return gb_launch(heads_mm_kernel<T>, dim3((a.T + HM_BM - 1) / HM_BM, (a.N + HM_BN - 1) / HM_BN, a.H),
                   dim3(256), 0, s, a);
}
GB_EXPORT int gb_heads_mm_f32(const HeadsMmArgs* a, cudaStream_t s) { return heads_mm<float>(*a, s); }
GB_EXPORT int gb_heads_mm_bf16(const HeadsMmArgs* a, cudaStream_t s) { return heads_mm<bf16>(*a, s); }
