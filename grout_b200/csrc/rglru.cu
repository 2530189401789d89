// A gated linear recurrence per channel behind a short causal convolution (the
// recurrent block of Griffin).  With xb = x + x_bias the second branch of the mixer's
// projection, per channel c and token t of a sequence
//
//   u_t   = conv_b + sum_j conv_w[c, taps-1-j] xb_(t-j)        (zeros before the start)
//   r_t   = sigmoid(Wa_b u_t,b + ba),  i_t = sigmoid(Wi_b u_t,b + bi)
//           (the channels form `blocks` equal parts; part b has square matrices of its own)
//   a_t   = exp(-factor r_t softplus(lam_c))
//   S_t   = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t                (S = 0 before the first token)
//   out_t = S_t * gelu_tanh(y + y_bias)                          (the first branch)
//
// All of it is 32-bit; the input is the 32-bit sums of the projection (columns
// y [C] | x [C]) and only `out` is rounded to the activation type.  A sequence's
// state is the last taps-1 values of xb, then S.
//
// A step of few rows (decoding) is two kernels.  `gates_few` owns a part of the
// channels, a tile of its outputs and up to RG_ROWS rows: it computes the part's u
// itself (from the rows and the kept tail), splits the sums over the part's inputs
// among eight groups of threads and adds them up in shared memory.  `scan` walks a
// sequence's rows with one thread per channel, applies the first branch and keeps
// the new tail and S for sequences whose slot is not negative.
//
// A step of many rows: `conv` computes u for every row; `gates_tile` is a 32-bit
// matrix product of 64 rows by 64 outputs of both matrices a block (a thread holds
// 4 x 4 sums of each); and where a sequence brings more than RG_CHUNK rows the scan
// goes chunk by chunk: `scan_local` reduces every chunk to the pair (product of its
// decays, what it adds to a state of zero), and `scan_apply` folds the pairs of the
// chunks before its own into the state it starts from and then walks its rows.  The
// recurrence is linear, so this is the same sum in another order.
#include "common.cuh"

struct RglruArgs {
  const float* proj;      // [T, 2 C] 32-bit sums: y | x
  const float* bias;      // [2 C] the projection's biases, y's then x's
  const float* conv_w;    // [C, taps]
  const float* conv_b;    // [C]
  const float* wa_t;      // [blocks, bw, bw] transposed: [part, in, out]
  const float* ba;        // [C]
  const float* wi_t;      // [blocks, bw, bw]
  const float* bi;        // [C]
  const float* lam;       // [C]
  const int* token_seq;   // [T]
  const int* cu_q;        // [n_seqs + 1]
  const int* slots;       // [n_seqs]
  float* state;           // [slots, state_stride]: tail [taps - 1, C], then S [C]
  long long state_stride;
  float* u;               // [T, C] scratch
  float* ab;              // [T, 2, C] scratch: decay, input
  void* out;              // [T, C]
  float* chunks;          // [T / RG_CHUNK + n_seqs, 2, C] scratch: a chunk's decay product and sum
  float* start;           // [n_seqs, C] scratch: S before the step
  int n_tokens, n_seqs, C, blocks, taps;
  float factor;
  int max_rows;           // the most rows a sequence brings (0: unknown)
};

#define RG_ROWS 8        // rows of a block of gates_few
#define RG_FEW 32        // up to this many rows the step is one of few rows
#define RG_OT 32         // outputs of a block of gates_few
#define RG_KS 8          // groups that share a sum in gates_few
#define RG_CHUNK 64      // rows of a chunk of the scan
#define RG_TM 64         // rows and outputs of a block of gates_tile
#define RG_TK 16
static_assert(RG_KS == RG_ROWS, "gates_few adds up with one thread per (row, output)");

// u of row t, channel c: this step's rows and, before them, the kept tail
__device__ __forceinline__ float rg_conv(const RglruArgs& a, int t, int c) {
  const int C = a.C, taps = a.taps;
  const int seq = a.token_seq[t];
  const int r = t - a.cu_q[seq];                          // the row's place among its sequence's rows
  const int slot = a.slots[seq];
  const float* tail = slot >= 0 ? a.state + (size_t)slot * a.state_stride : nullptr;
  float acc = a.conv_b[c];
  const float xb = a.bias[C + c];
  for (int j = 0; j < taps; ++j) {
    // the input j tokens back: a row of this step, or row (taps - 1 - (j - r)) of the tail
    float x;
    if (j <= r) x = a.proj[(size_t)(t - j) * 2 * C + C + c] + xb;
    else x = tail ? tail[(size_t)(taps - 1 - (j - r)) * C + c] : 0.f;
    acc = fmaf(a.conv_w[(size_t)c * taps + taps - 1 - j], x, acc);
  }
  return acc;
}

// decay and input of the recurrence from the two gates' sums
__device__ __forceinline__ void rg_gate(const RglruArgs& a, int t, int c, float sa, float si, float u) {
  const float lam = a.lam[c];
  const float sp = lam > 20.f ? lam : log1pf(expf(lam));          // softplus
  const float r = 1.0f / (1.0f + expf(-(sa + a.ba[c])));
  const float g = 1.0f / (1.0f + expf(-(si + a.bi[c])));
  const float log_a = -a.factor * r * sp;
  float* dst = a.ab + (size_t)t * 2 * a.C;
  dst[c] = expf(log_a);
  // 1 - a^2 = -expm1(2 log a): no cancellation when a is close to one
  dst[a.C + c] = sqrtf(-expm1f(2.0f * log_a)) * g * u;
}

__global__ void __launch_bounds__(256) rglru_conv_kernel(const RglruArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < a.C) a.u[(size_t)t * a.C + c] = rg_conv(a, t, c);
  pdl_launch_dependents_if_large();
}

__global__ void __launch_bounds__(RG_OT* RG_KS) rglru_gates_few_kernel(const RglruArgs a) {
  extern __shared__ float sm[];
  const int C = a.C, bw = C / a.blocks;
  const int otiles = (bw + RG_OT - 1) / RG_OT;
  const int part = blockIdx.x / otiles, o0 = (blockIdx.x % otiles) * RG_OT;
  const int t0 = blockIdx.y * RG_ROWS, nt = min(RG_ROWS, a.n_tokens - t0);
  float* us = sm;                               // [RG_ROWS, bw]
  float* red = sm + RG_ROWS * bw;               // [RG_KS, RG_ROWS, 2, RG_OT]
  const int tid = threadIdx.x, o = tid % RG_OT, ks = tid / RG_OT;
  const float* wa = a.wa_t + (size_t)part * bw * bw;
  const float* wi = a.wi_t + (size_t)part * bw * bw;
  pdl_launch_dependents_if_small();
  pdl_wait();
  for (int i = tid; i < RG_ROWS * bw; i += blockDim.x) {
    const int tt = i / bw, k = i % bw;
    us[i] = tt < nt ? rg_conv(a, t0 + tt, part * bw + k) : 0.f;
  }
  __syncthreads();
  float ra[RG_ROWS], ri[RG_ROWS];
#pragma unroll
  for (int tt = 0; tt < RG_ROWS; ++tt) ra[tt] = ri[tt] = 0.f;
  if (o0 + o < bw) {
#pragma unroll 4
    for (int k = ks; k < bw; k += RG_KS) {
      const float va = wa[(size_t)k * bw + o0 + o], vi = wi[(size_t)k * bw + o0 + o];
#pragma unroll
      for (int tt = 0; tt < RG_ROWS; ++tt) {
        const float x = us[tt * bw + k];
        ra[tt] = fmaf(va, x, ra[tt]);
        ri[tt] = fmaf(vi, x, ri[tt]);
      }
    }
  }
#pragma unroll
  for (int tt = 0; tt < RG_ROWS; ++tt) {
    red[((ks * RG_ROWS + tt) * 2 + 0) * RG_OT + o] = ra[tt];
    red[((ks * RG_ROWS + tt) * 2 + 1) * RG_OT + o] = ri[tt];
  }
  __syncthreads();
  pdl_launch_dependents_if_large();
  // thread (row, output): the groups' sums in a fixed order
  const int tt = tid / RG_OT;
  if (tt >= nt || o0 + o >= bw) return;
  float sa = 0.f, si = 0.f;
#pragma unroll
  for (int g = 0; g < RG_KS; ++g) {
    sa += red[((g * RG_ROWS + tt) * 2 + 0) * RG_OT + o];
    si += red[((g * RG_ROWS + tt) * 2 + 1) * RG_OT + o];
  }
  rg_gate(a, t0 + tt, part * bw + o0 + o, sa, si, us[tt * bw + o0 + o]);
}

// 64 rows by 64 outputs of one part, both matrices: thread (tx, ty) of 16 x 16 holds
// rows ty * 4 .. + 3 and outputs tx * 4 .. + 3.
__global__ void __launch_bounds__(256) rglru_gates_tile_kernel(const RglruArgs a) {
  __shared__ __align__(16) float us[RG_TK][RG_TM + 4];     // [k][row]
  __shared__ __align__(16) float was[RG_TK][RG_TM];        // [k][output]
  __shared__ __align__(16) float wis[RG_TK][RG_TM];
  const int C = a.C, bw = C / a.blocks;
  const int otiles = (bw + RG_TM - 1) / RG_TM;
  const int part = blockIdx.x / otiles, o0 = (blockIdx.x % otiles) * RG_TM;
  const int t0 = blockIdx.y * RG_TM;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const float* wa = a.wa_t + (size_t)part * bw * bw;
  const float* wi = a.wi_t + (size_t)part * bw * bw;
  float sa[4][4], si[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) sa[r][c] = si[r][c] = 0.f;
  pdl_launch_dependents_if_small();
  pdl_wait();
  for (int k0 = 0; k0 < bw; k0 += RG_TK) {
    __syncthreads();
    for (int i = tid; i < RG_TM * RG_TK; i += 256) {
      const int r = i / RG_TK, k = i % RG_TK;
      us[k][r] = (t0 + r < a.n_tokens && k0 + k < bw) ? a.u[(size_t)(t0 + r) * C + part * bw + k0 + k] : 0.f;
      const int kk = i / RG_TM, n = i % RG_TM;
      const bool in = k0 + kk < bw && o0 + n < bw;
      was[kk][n] = in ? wa[(size_t)(k0 + kk) * bw + o0 + n] : 0.f;
      wis[kk][n] = in ? wi[(size_t)(k0 + kk) * bw + o0 + n] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < RG_TK; ++k) {
      const float4 x4 = *reinterpret_cast<const float4*>(&us[k][ty * 4]);
      const float4 a4 = *reinterpret_cast<const float4*>(&was[k][tx * 4]);
      const float4 i4 = *reinterpret_cast<const float4*>(&wis[k][tx * 4]);
      const float x[4] = {x4.x, x4.y, x4.z, x4.w};
      const float va[4] = {a4.x, a4.y, a4.z, a4.w};
      const float vi[4] = {i4.x, i4.y, i4.z, i4.w};
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          sa[r][c] = fmaf(x[r], va[c], sa[r][c]);
          si[r][c] = fmaf(x[r], vi[c], si[r][c]);
        }
    }
  }
  pdl_launch_dependents_if_large();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = t0 + ty * 4 + r;
    if (t >= a.n_tokens) break;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int o = o0 + tx * 4 + c;
      if (o < bw) rg_gate(a, t, part * bw + o, sa[r][c], si[r][c], a.u[(size_t)t * C + part * bw + o]);
    }
  }
}

__device__ __forceinline__ float rg_gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The tail a sequence keeps after the step: the last taps - 1 inputs of the old tail
// followed by this step's rows.  One thread per channel reads before it writes.
__device__ __forceinline__ void rg_keep_tail(const RglruArgs& a, float* st, int first, int n, int c) {
  const int C = a.C, taps = a.taps;
  const float xb = a.bias[C + c];
  float keep[16];
  for (int j = 0; j < taps - 1; ++j) {       // j-th row of the new tail is input n - (taps - 1) + j
    const int r = n - (taps - 1) + j;
    keep[j] = r >= 0 ? a.proj[(size_t)(first + r) * 2 * C + C + c] + xb : st[(size_t)(taps - 1 + r) * C + c];
  }
  for (int j = 0; j < taps - 1; ++j) st[(size_t)j * C + c] = keep[j];
}

template <typename T>
__global__ void __launch_bounds__(128) rglru_scan_kernel(const RglruArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int seq = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int C = a.C, taps = a.taps;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  if (c >= C || n <= 0) return;
  const int slot = a.slots[seq];
  float* st = slot >= 0 ? a.state + (size_t)slot * a.state_stride : nullptr;
  float S = st ? st[(size_t)(taps - 1) * C + c] : 0.f;
  const float yb = a.bias[c];
  const float* __restrict__ ab = a.ab;
  const float* __restrict__ proj = a.proj;
  T* __restrict__ out = (T*)a.out;
  for (int r = 0; r < n; ++r) {
    const size_t t = (size_t)(first + r);
    S = fmaf(ab[t * 2 * C + c], S, ab[t * 2 * C + C + c]);
    out[t * C + c] = from_f32<T>(S * rg_gelu_tanh(proj[t * 2 * C + c] + yb));
  }
  pdl_launch_dependents_if_large();
  if (!st) return;
  st[(size_t)(taps - 1) * C + c] = S;
  rg_keep_tail(a, st, first, n, c);
}

// Chunk z of a sequence is its rows z RG_CHUNK .. ; its pair lives at entry
// (first row / RG_CHUNK + the sequence's number), which no other chunk has.
__device__ __forceinline__ size_t rg_chunk_entry(int first, int z, int seq) {
  return (size_t)((first + z * RG_CHUNK) / RG_CHUNK + seq);
}

__global__ void __launch_bounds__(128) rglru_scan_local_kernel(const RglruArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int seq = blockIdx.y, z = blockIdx.z, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int C = a.C;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  const int r0 = z * RG_CHUNK;
  if (c >= C || r0 >= n) return;
  if (z == 0) {
    const int slot = a.slots[seq];
    a.start[(size_t)seq * C + c] = slot >= 0 ? a.state[(size_t)slot * a.state_stride + (size_t)(a.taps - 1) * C + c] : 0.f;
  }
  if (r0 + RG_CHUNK >= n) return;            // nothing follows the sequence's last chunk
  const float* __restrict__ ab = a.ab;
  float A = 1.f, B = 0.f;
#pragma unroll 8
  for (int r = 0; r < RG_CHUNK; ++r) {
    const size_t t = (size_t)(first + r0 + r);
    const float av = ab[t * 2 * C + c];
    A *= av;
    B = fmaf(av, B, ab[t * 2 * C + C + c]);
  }
  float* dst = a.chunks + rg_chunk_entry(first, z, seq) * 2 * C;
  dst[c] = A;
  dst[C + c] = B;
  pdl_launch_dependents_if_large();
}

template <typename T>
__global__ void __launch_bounds__(128) rglru_scan_apply_kernel(const RglruArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int seq = blockIdx.y, z = blockIdx.z, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int C = a.C, taps = a.taps;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  const int r0 = z * RG_CHUNK;
  if (c >= C || r0 >= n) return;
  float S = a.start[(size_t)seq * C + c];
  for (int zz = 0; zz < z; ++zz) {
    const float* src = a.chunks + rg_chunk_entry(first, zz, seq) * 2 * C;
    S = fmaf(src[c], S, src[C + c]);
  }
  const float yb = a.bias[c];
  const float* __restrict__ ab = a.ab;
  const float* __restrict__ proj = a.proj;
  T* __restrict__ out = (T*)a.out;
  const int nr = min(RG_CHUNK, n - r0);
#pragma unroll 4
  for (int r = 0; r < nr; ++r) {
    const size_t t = (size_t)(first + r0 + r);
    S = fmaf(ab[t * 2 * C + c], S, ab[t * 2 * C + C + c]);
    out[t * C + c] = from_f32<T>(S * rg_gelu_tanh(proj[t * 2 * C + c] + yb));
  }
  pdl_launch_dependents_if_large();
  if (r0 + RG_CHUNK < n) return;             // the last chunk keeps the state
  const int slot = a.slots[seq];
  if (slot < 0) return;
  float* st = a.state + (size_t)slot * a.state_stride;
  st[(size_t)(taps - 1) * C + c] = S;
  rg_keep_tail(a, st, first, n, c);
}

template <typename T>
static int rglru_forward(const RglruArgs& a, cudaStream_t s) {
  if (a.n_tokens < 0 || a.n_seqs < 0 || a.C <= 0 || a.blocks <= 0 || a.C % a.blocks || a.taps < 1 ||
      a.n_seqs > 65535 || a.max_rows < 0)
    return GB_ERR_BAD_ARG;
  if (a.taps > 17) return GB_ERR_UNSUPPORTED;
  if (!a.proj || !a.bias || !a.conv_w || !a.conv_b || !a.wa_t || !a.ba || !a.wi_t || !a.bi || !a.lam ||
      !a.token_seq || !a.cu_q || !a.slots || !a.state || !a.u || !a.ab || !a.out || !a.chunks || !a.start)
    return GB_ERR_BAD_ARG;
  if (a.n_tokens == 0 || a.n_seqs == 0) return 0;
  const int bw = a.C / a.blocks;
  int e;
  if (a.n_tokens <= RG_FEW) {
    const size_t smem = ((size_t)RG_ROWS * bw + (size_t)RG_KS * RG_ROWS * 2 * RG_OT) * sizeof(float);
    if (smem > 200 * 1024) return GB_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
      cudaError_t ce = cudaFuncSetAttribute(rglru_gates_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (ce != cudaSuccess) return (int)ce;
    }
    e = gb_launch(rglru_gates_few_kernel, dim3(a.blocks * ((bw + RG_OT - 1) / RG_OT), (a.n_tokens + RG_ROWS - 1) / RG_ROWS),
                  dim3(RG_OT * RG_KS), smem, s, a);
  } else {
    if (a.n_tokens > 65535 * RG_TM) return GB_ERR_UNSUPPORTED;
    e = gb_launch(rglru_conv_kernel, dim3((a.C + 255) / 256, a.n_tokens), dim3(256), 0, s, a);
    if (e) return e;
    e = gb_launch(rglru_gates_tile_kernel, dim3(a.blocks * ((bw + RG_TM - 1) / RG_TM), (a.n_tokens + RG_TM - 1) / RG_TM),
                  dim3(256), 0, s, a);
  }
  if (e) return e;
  const int most = a.max_rows > 0 ? min(a.max_rows, a.n_tokens) : a.n_tokens;
  const dim3 grid((a.C + 127) / 128, a.n_seqs, (most + RG_CHUNK - 1) / RG_CHUNK);
  if (grid.z <= 1) return gb_launch(rglru_scan_kernel<T>, grid, dim3(128), 0, s, a);
  if (grid.z > 65535) return GB_ERR_UNSUPPORTED;
  e = gb_launch(rglru_scan_local_kernel, grid, dim3(128), 0, s, a);
  if (e) return e;
  return gb_launch(rglru_scan_apply_kernel<T>, grid, dim3(128), 0, s, a);
}

GB_EXPORT int gb_rglru_forward_f32(const RglruArgs* a, cudaStream_t s) { return rglru_forward<float>(*a, s); }
GB_EXPORT int gb_rglru_forward_bf16(const RglruArgs* a, cudaStream_t s) { return rglru_forward<bf16>(*a, s); }
