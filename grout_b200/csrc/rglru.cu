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
// Three kernels.  `conv` computes u for every row (from this step's rows and the
// kept tail).  `gates` computes a and the recurrence's input for a tile of rows
// and one part of the channels: the part's rows of u are staged in shared memory,
// a thread owns one output channel of both matrices (stored transposed, [part, in,
// out], so that a warp reads neighbours) and RG_ROWS rows.  `scan` walks a
// sequence's rows with one thread per channel, applies the first branch, and
// keeps the new tail and S for sequences whose slot is not negative.
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
  int n_tokens, n_seqs, C, blocks, taps;
  float factor;
};

#define RG_ROWS 8

__global__ void __launch_bounds__(256) rglru_conv_kernel(const RglruArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x, C = a.C, taps = a.taps;
  const int seq = a.token_seq[t];
  const int first = a.cu_q[seq], r = t - first;          // r: the row's place among its sequence's rows
  const int slot = a.slots[seq];
  const float* tail = slot >= 0 ? a.state + (size_t)slot * a.state_stride : nullptr;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = a.conv_b[c];
    const float xb = a.bias[C + c];
    for (int j = 0; j < taps; ++j) {
      // the input j tokens back: a row of this step, or row (taps - 1 - (j - r)) of the tail
      float x;
      if (j <= r) x = a.proj[(size_t)(t - j) * 2 * C + C + c] + xb;
      else x = tail ? tail[(size_t)(taps - 1 - (j - r)) * C + c] : 0.f;
      acc = fmaf(a.conv_w[(size_t)c * taps + taps - 1 - j], x, acc);
    }
    a.u[(size_t)t * C + c] = acc;
  }
  pdl_launch_dependents_if_large();
}

__global__ void __launch_bounds__(256) rglru_gates_kernel(const RglruArgs a) {
  extern __shared__ float us[];        // [RG_ROWS, bw]
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int C = a.C, bw = C / a.blocks, part = blockIdx.y;
  const int t0 = blockIdx.x * RG_ROWS, nt = min(RG_ROWS, a.n_tokens - t0);
  for (int i = threadIdx.x; i < RG_ROWS * bw; i += blockDim.x) {
    const int tt = i / bw, k = i % bw;
    us[i] = tt < nt ? a.u[(size_t)(t0 + tt) * C + part * bw + k] : 0.f;
  }
  __syncthreads();
  const float* wa = a.wa_t + (size_t)part * bw * bw;
  const float* wi = a.wi_t + (size_t)part * bw * bw;
  for (int o = threadIdx.x; o < bw; o += blockDim.x) {
    float ra[RG_ROWS], ri[RG_ROWS];
#pragma unroll
    for (int tt = 0; tt < RG_ROWS; ++tt) ra[tt] = ri[tt] = 0.f;
    for (int k = 0; k < bw; ++k) {
      const float va = wa[(size_t)k * bw + o], vi = wi[(size_t)k * bw + o];
#pragma unroll
      for (int tt = 0; tt < RG_ROWS; ++tt) {
        const float x = us[tt * bw + k];
        ra[tt] = fmaf(va, x, ra[tt]);
        ri[tt] = fmaf(vi, x, ri[tt]);
      }
    }
    const int c = part * bw + o;
    const float lam = a.lam[c];
    const float sp = lam > 20.f ? lam : log1pf(expf(lam));          // softplus
    const float ba = a.ba[c], bi = a.bi[c];
#pragma unroll
    for (int tt = 0; tt < RG_ROWS; ++tt) {
      if (tt >= nt) break;
      const float r = 1.0f / (1.0f + expf(-(ra[tt] + ba)));
      const float g = 1.0f / (1.0f + expf(-(ri[tt] + bi)));
      const float log_a = -a.factor * r * sp;
      const float av = expf(log_a);
      // 1 - a^2 = -expm1(2 log a): no cancellation when a is close to one
      const float in = sqrtf(-expm1f(2.0f * log_a)) * g * us[tt * bw + o];
      float* dst = a.ab + (size_t)(t0 + tt) * 2 * C;
      dst[c] = av;
      dst[C + c] = in;
    }
  }
  pdl_launch_dependents_if_large();
}

__device__ __forceinline__ float rg_gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
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
  for (int r = 0; r < n; ++r) {
    const size_t t = (size_t)(first + r);
    S = fmaf(a.ab[t * 2 * C + c], S, a.ab[t * 2 * C + C + c]);
    ((T*)a.out)[t * C + c] = from_f32<T>(S * rg_gelu_tanh(a.proj[t * 2 * C + c] + yb));
  }
  pdl_launch_dependents_if_large();
  if (!st) return;
  st[(size_t)(taps - 1) * C + c] = S;
  // the new tail: the last taps - 1 inputs of the old tail followed by this step's rows
  const float xb = a.bias[C + c];
  float keep[16];
  for (int j = 0; j < taps - 1; ++j) {       // j-th row of the new tail is input n - (taps - 1) + j
    const int r = n - (taps - 1) + j;
    keep[j] = r >= 0 ? a.proj[(size_t)(first + r) * 2 * C + C + c] + xb : st[(size_t)(taps - 1 + r) * C + c];
  }
  for (int j = 0; j < taps - 1; ++j) st[(size_t)j * C + c] = keep[j];
}

template <typename T>
static int rglru_forward(const RglruArgs& a, cudaStream_t s) {
  if (a.n_tokens < 0 || a.n_seqs < 0 || a.C <= 0 || a.blocks <= 0 || a.C % a.blocks || a.taps < 1 ||
      a.n_seqs > 65535)
    return GB_ERR_BAD_ARG;
  if (a.taps > 17) return GB_ERR_UNSUPPORTED;
  if (!a.proj || !a.bias || !a.conv_w || !a.conv_b || !a.wa_t || !a.ba || !a.wi_t || !a.bi || !a.lam ||
      !a.token_seq || !a.cu_q || !a.slots || !a.state || !a.u || !a.ab || !a.out)
    return GB_ERR_BAD_ARG;
  if (a.n_tokens == 0 || a.n_seqs == 0) return 0;
  const int bw = a.C / a.blocks;
  const size_t smem = (size_t)RG_ROWS * bw * sizeof(float);
  if (smem > 200 * 1024) return GB_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t ce = cudaFuncSetAttribute(rglru_gates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
  }
  int e = gb_launch(rglru_conv_kernel, dim3(a.n_tokens), dim3(256), 0, s, a);
  if (e) return e;
  const int threads = bw >= 256 ? 256 : (bw + 31) / 32 * 32;
  e = gb_launch(rglru_gates_kernel, dim3((a.n_tokens + RG_ROWS - 1) / RG_ROWS, a.blocks), dim3(threads), smem, s, a);
  if (e) return e;
  return gb_launch(rglru_scan_kernel<T>, dim3((a.C + 127) / 128, a.n_seqs), dim3(128), 0, s, a);
}

GB_EXPORT int gb_rglru_forward_f32(const RglruArgs* a, cudaStream_t s) { return rglru_forward<float>(*a, s); }
GB_EXPORT int gb_rglru_forward_bf16(const RglruArgs* a, cudaStream_t s) { return rglru_forward<bf16>(*a, s); }
