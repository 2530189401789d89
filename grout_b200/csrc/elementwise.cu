// Small elementwise kernels: SiLU(gate) * up on the fused gate|up projection,
// and conversions between 32-bit and bfloat16.
#include "common.cuh"

// in [n_rows, 2 I]; with group == 0 the gate is in columns [0, I) and up in
// [I, 2 I); with group g > 0 the columns come in runs of g gates followed by
// their g ups (the layout the decode product's fused epilogue uses).
// out[r, i] = g / (1 + exp(-g)) * u in 32-bit, one rounding at the store
// (the reference's silu_mul_2d_f16, src/kernels.rs:271-296).
// The gate's activation: 0 = silu, g / (1 + exp(-g)); 1 = the tanh form of gelu,
// 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))); 2 = relu.
template <int ACT> __device__ __forceinline__ float gate_act(float g) {
  if (ACT == 2) return fmaxf(g, 0.f);
  if (ACT == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return g / (1.0f + expf(-g));
}

template <typename T, int ACT>
__global__ void silu_mul_kernel(const T* in, T* __restrict__ out, int I, int group) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t r = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= I) return;
  const int gi = group ? (i / group) * 2 * group + (i % group) : i;
  const int ui = group ? gi + group : I + i;
  const float g = to_f32<T>(in[r * 2 * I + gi]);
  const float u = to_f32<T>(in[r * 2 * I + ui]);
  pdl_launch_dependents_if_large();
  out[r * I + i] = from_f32<T>(gate_act<ACT>(g) * u);
}

// bf16, eight outputs per thread in 16-byte pieces: for the plain layout and for
// groups of 8 a thread's gates are 16 contiguous bytes and so are its ups.
template <int ACT>
__global__ void silu_mul_vec8_kernel(const bf16* in, bf16* __restrict__ out, int I, int group) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t r = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;   // which run of 8 outputs
  if (v * 8 >= I) return;
  const bf16* row = in + r * 2 * (size_t)I;
  const bf16* gp = group ? row + (size_t)v * 16 : row + (size_t)v * 8;
  const bf16* up = group ? gp + 8 : row + I + (size_t)v * 8;
  const uint4 g4 = *reinterpret_cast<const uint4*>(gp);
  const uint4 u4 = *reinterpret_cast<const uint4*>(up);
  pdl_launch_dependents_if_large();
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
  uint4 o4;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float ga = __low2float(g2[k]), gb = __high2float(g2[k]);
    const float ua = __low2float(u2[k]), ub = __high2float(u2[k]);
    o2[k] = __floats2bfloat162_rn(gate_act<ACT>(ga) * ua, gate_act<ACT>(gb) * ub);
  }
  *reinterpret_cast<uint4*>(out + r * (size_t)I + (size_t)v * 8) = o4;
}

template <typename T, int ACT = 0>
static int silu_mul(const void* in, void* out, int n_rows, int I, int group, cudaStream_t s) {
  if (n_rows < 0 || I <= 0 || group < 0 || (group && I % group)) return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  if (n_rows > 65535) {
    // rows go to grid.y; split very long steps
    for (int r0 = 0; r0 < n_rows; r0 += 65535) {
      const int n = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
      int e = silu_mul<T, ACT>((const T*)in + (size_t)r0 * 2 * I, (T*)out + (size_t)r0 * I, n, I, group, s);
      if (e) return e;
    }
    return 0;
  }
  if (sizeof(T) == 2 && I % 8 == 0 && (group == 0 || group == 8) &&
      ((((uintptr_t)in) | ((uintptr_t)out)) & 15) == 0)
    return gb_launch(silu_mul_vec8_kernel<ACT>, dim3((I / 8 + 127) / 128, n_rows), dim3(128), 0, s,
                     (const bf16*)in, (bf16*)out, I, group);
  return gb_launch(silu_mul_kernel<T, ACT>, dim3((I + 255) / 256, n_rows), dim3(256), 0, s,
                   (const T*)in, (T*)out, I, group);
}
GB_EXPORT int gb_silu_mul_f32(const void* in, void* out, int n_rows, int I, int group,
                              cudaStream_t s) {
  return silu_mul<float>(in, out, n_rows, I, group, s);
}
GB_EXPORT int gb_silu_mul_bf16(const void* in, void* out, int n_rows, int I, int group,
                               cudaStream_t s) {
  return silu_mul<bf16>(in, out, n_rows, I, group, s);
}
// The same with the tanh form of gelu as the gate's activation.
GB_EXPORT int gb_gelu_tanh_mul_f32(const void* in, void* out, int n_rows, int I, int group,
                                   cudaStream_t s) {
  return silu_mul<float, 1>(in, out, n_rows, I, group, s);
}
GB_EXPORT int gb_gelu_tanh_mul_bf16(const void* in, void* out, int n_rows, int I, int group,
                                    cudaStream_t s) {
  return silu_mul<bf16, 1>(in, out, n_rows, I, group, s);
}
// The same with relu as the gate's activation.
GB_EXPORT int gb_relu_mul_f32(const void* in, void* out, int n_rows, int I, int group, cudaStream_t s) {
  return silu_mul<float, 2>(in, out, n_rows, I, group, s);
}
GB_EXPORT int gb_relu_mul_bf16(const void* in, void* out, int n_rows, int I, int group, cudaStream_t s) {
  return silu_mul<bf16, 2>(in, out, n_rows, I, group, s);
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = from_f32<TO>(to_f32<TI>(in[i]));
}
template <typename TI, typename TO>
static int cast(const void* in, void* out, long long n, cudaStream_t s) {
  if (n < 0) return GB_ERR_BAD_ARG;
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  cast_kernel<TI, TO><<<(int)blocks, 256, 0, s>>>((const TI*)in, (TO*)out, (size_t)n);
  return gb_status();
}
GB_EXPORT int gb_cast_f32_to_bf16(const void* in, void* out, long long n, cudaStream_t s) {
  return cast<float, bf16>(in, out, n, s);
}
GB_EXPORT int gb_cast_bf16_to_f32(const void* in, void* out, long long n, cudaStream_t s) {
  return cast<bf16, float>(in, out, n, s);
}

// Keeps the stream busy for `ns` nanoseconds (at most a millisecond): one thread
// reads the global timer until the time is up and waits for nothing else.  The
// per-operation profile queues it in front of each timed call so that the host
// has queued the call and its two events before the device reaches them;
// otherwise the time between the events of a short kernel is the host's, not
// the kernel's.
__global__ void delay_kernel(unsigned long long ns) {
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (int i = 0; i < (1 << 20); ++i) {          // bounded whatever the timer does
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    if (t - t0 >= ns) break;
    __nanosleep(200);
  }
}
GB_EXPORT int gb_delay_ns(long long ns, cudaStream_t s) {
  if (ns < 0 || ns > 1000000) return GB_ERR_BAD_ARG;
  delay_kernel<<<1, 1, 0, s>>>((unsigned long long)ns);
  return gb_status();
}

// out[i] = max(in[i], 0)^2: the activation of a feed-forward without a gate.  The
// square is taken in 32-bit and rounded once.
template <typename T>
__global__ void relu_squared_kernel(const T* in, T* __restrict__ out, size_t n) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = fmaxf(to_f32<T>(in[i]), 0.f);
  pdl_launch_dependents_if_large();
  out[i] = from_f32<T>(v * v);
}
__global__ void relu_squared_vec8_kernel(const bf16* in, bf16* __restrict__ out, size_t n8) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 x4 = reinterpret_cast<const uint4*>(in)[i];
  pdl_launch_dependents_if_large();
  const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x4);
  uint4 o4;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float a = fmaxf(__low2float(x2[k]), 0.f), b = fmaxf(__high2float(x2[k]), 0.f);
    o2[k] = __floats2bfloat162_rn(a * a, b * b);
  }
  reinterpret_cast<uint4*>(out)[i] = o4;
}
template <typename T>
static int relu_squared(const void* in, void* out, long long n, cudaStream_t s) {
  if (n < 0 || !in || !out) return GB_ERR_BAD_ARG;
  if (n == 0) return 0;
  if (sizeof(T) == 2 && n % 8 == 0 && ((((uintptr_t)in) | ((uintptr_t)out)) & 15) == 0)
    return gb_launch(relu_squared_vec8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, s,
                     (const bf16*)in, (bf16*)out, (size_t)(n / 8));
  return gb_launch(relu_squared_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s,
                   (const T*)in, (T*)out, (size_t)n);
}
GB_EXPORT int gb_relu_squared_f32(const void* in, void* out, long long n, cudaStream_t s) {
  return relu_squared<float>(in, out, n, s);
}
GB_EXPORT int gb_relu_squared_bf16(const void* in, void* out, long long n, cudaStream_t s) {
  return relu_squared<bf16>(in, out, n, s);
}

// x[i] <- cap * tanh(x[i] * scale / cap) in place on 32-bit values (cap <= 0: only
// the scaling): what an output head with a scaled and capped logit does.
__global__ void scale_softcap_kernel(float* x, size_t n, float scale, float cap) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i] * scale;
  if (cap > 0.f) v = cap * tanhf(v / cap);
  x[i] = v;
}
GB_EXPORT int gb_scale_softcap_f32(float* x, long long n, float scale, float cap, cudaStream_t s) {
  if (n < 0 || !x) return GB_ERR_BAD_ARG;
  if (n == 0) return 0;
  return gb_launch(scale_softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x,
                   (size_t)n, scale, cap);
}

// A gated feed-forward's inner step with biases, on the 32-bit sums of the fused gate|up
// product: out[r, i] = act(g + bias_g) * (u + bias_u), rounded once.  `in` [n_rows, 2 I] and
// `bias` [2 I] have the same layout (plain or in groups, as silu_mul's).
template <typename T, int ACT>
__global__ void bias_gate_mul_kernel(const float* in, const float* __restrict__ bias, T* __restrict__ out,
                                     int I, int group) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t r = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= I) return;
  const int gi = group ? (i / group) * 2 * group + (i % group) : i;
  const int ui = group ? gi + group : I + i;
  const float g = in[r * 2 * I + gi] + bias[gi];
  const float u = in[r * 2 * I + ui] + bias[ui];
  pdl_launch_dependents_if_large();
  out[r * I + i] = from_f32<T>(gate_act<ACT>(g) * u);
}
template <typename T>
static int bias_gate_mul(const float* in, const float* bias, void* out, int n_rows, int I, int group,
                         int act, cudaStream_t s) {
  if (n_rows < 0 || I <= 0 || group < 0 || (group && I % group) || act < 0 || act > 2 || !in || !bias || !out)
    return GB_ERR_BAD_ARG;
  for (int r0 = 0; r0 < n_rows; r0 += 65535) {      // rows go to grid.y
    const int n = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
    const dim3 grid((I + 255) / 256, n);
    const float* src = in + (size_t)r0 * 2 * I;
    T* dst = (T*)out + (size_t)r0 * I;
    int e = act == 0 ? gb_launch(bias_gate_mul_kernel<T, 0>, grid, dim3(256), 0, s, src, bias, dst, I, group)
          : act == 1 ? gb_launch(bias_gate_mul_kernel<T, 1>, grid, dim3(256), 0, s, src, bias, dst, I, group)
                     : gb_launch(bias_gate_mul_kernel<T, 2>, grid, dim3(256), 0, s, src, bias, dst, I, group);
    if (e) return e;
  }
  return 0;
}
GB_EXPORT int gb_bias_gate_mul_f32(const float* in, const float* bias, void* out, int n_rows, int I,
                                   int group, int act, cudaStream_t s) {
  return bias_gate_mul<float>(in, bias, out, n_rows, I, group, act, s);
}
GB_EXPORT int gb_bias_gate_mul_bf16(const float* in, const float* bias, void* out, int n_rows, int I,
                                    int group, int act, cudaStream_t s) {
  return bias_gate_mul<bf16>(in, bias, out, n_rows, I, group, act, s);
}

// x[r, :] += bias in place on 32-bit rows: a projection's bias added to its 32-bit sums.
__global__ void add_bias_kernel(float* x, const float* __restrict__ bias, size_t n, int N) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  x[i] += bias[i % N];
}
GB_EXPORT int gb_add_bias_f32(float* x, const float* bias, long long n_rows, int N, cudaStream_t s) {
  if (n_rows < 0 || N <= 0 || !x || !bias) return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  const size_t n = (size_t)n_rows * N;
  return gb_launch(add_bias_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, x, bias, n, N);
}

// A sigmoid gate per (row, head) on an attention's output, with a constant factor:
// out[t, h * Dv + d] = x[t, h, d] * sigmoid(gate[t, h]) * mult for d < Dv.  x's heads are
// Ds wide (Ds >= Dv: what lies beyond Dv is dropped); the gates' logits are 32-bit with a
// row pitch of their own, and so has out, which may be part of a wider row.
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ x, const float* __restrict__ gate, long long gate_ld,
                                 T* __restrict__ out, long long out_ld, int nq, int Ds, int Dv, float mult) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nq * Dv) return;
  const int h = i / Dv, d = i % Dv;
  const float g = gate ? 1.0f / (1.0f + expf(-gate[t * gate_ld + h])) : 1.0f;
  pdl_launch_dependents_if_large();
  out[t * out_ld + i] = from_f32<T>(to_f32<T>(x[(t * nq + h) * Ds + d]) * g * mult);
}
// The same in 16-byte pieces (a thread takes 16 / sizeof(T) neighbours of one head), two rows a
// block where a row has few pieces.
template <typename T>
__global__ void __launch_bounds__(256) head_gate_vec_kernel(const T* __restrict__ x, const float* __restrict__ gate,
                                                            long long gate_ld, T* __restrict__ out, long long out_ld,
                                                            int n_rows, int nq, int Ds, int Dv, float mult) {
  constexpr int V = 16 / (int)sizeof(T);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int per_row = nq * Dv / V;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_rows * per_row) return;
  const size_t t = (size_t)(i / per_row);
  const int p = (int)(i % per_row), h = p / (Dv / V), d = (p % (Dv / V)) * V;
  const float g = (gate ? 1.0f / (1.0f + expf(-gate[t * gate_ld + h])) : 1.0f) * mult;
  const uint4 raw = *reinterpret_cast<const uint4*>(x + (t * nq + h) * Ds + d);
  const T* v = reinterpret_cast<const T*>(&raw);
  uint4 res;
  T* o = reinterpret_cast<T*>(&res);
#pragma unroll
  for (int e = 0; e < V; ++e) o[e] = from_f32<T>(to_f32<T>(v[e]) * g);
  pdl_launch_dependents_if_large();
  *reinterpret_cast<uint4*>(out + t * out_ld + (size_t)h * Dv + d) = res;
}
template <typename T>
static int head_gate(const void* x, const float* gate, long long gate_ld, void* out, long long out_ld,
                     int n_rows, int nq, int Ds, int Dv, float mult, cudaStream_t s) {
  if (n_rows < 0 || nq <= 0 || Dv <= 0 || Ds < Dv || !x || !out || out_ld < (long long)nq * Dv ||
      (gate && gate_ld < nq))
    return GB_ERR_BAD_ARG;
  if (n_rows == 0) return 0;
  constexpr int V = 16 / (int)sizeof(T);
  if (Dv % V == 0 && Ds % V == 0 && out_ld % V == 0 && ((((uintptr_t)x) | ((uintptr_t)out)) & 15) == 0) {
    const long long pieces = (long long)n_rows * (nq * Dv / V);
    return gb_launch(head_gate_vec_kernel<T>, dim3((unsigned)((pieces + 255) / 256)), dim3(256), 0, s,
                     (const T*)x, gate, gate_ld, (T*)out, out_ld, n_rows, nq, Ds, Dv, mult);
  }
  for (int r0 = 0; r0 < n_rows; r0 += 65535) {      // rows go to grid.y
    const int n = n_rows - r0 < 65535 ? n_rows - r0 : 65535;
    int e = gb_launch(head_gate_kernel<T>, dim3((nq * Dv + 255) / 256, n), dim3(256), 0, s,
                      (const T*)x + (size_t)r0 * nq * Ds, gate ? gate + (size_t)r0 * gate_ld : gate, gate_ld,
                      (T*)out + (size_t)r0 * out_ld, out_ld, nq, Ds, Dv, mult);
    if (e) return e;
  }
  return 0;
}
GB_EXPORT int gb_head_gate_f32(const void* x, const float* gate, long long gate_ld, void* out, long long out_ld,
                               int n_rows, int nq, int Ds, int Dv, float mult, cudaStream_t s) {
  return head_gate<float>(x, gate, gate_ld, out, out_ld, n_rows, nq, Ds, Dv, mult, s);
}
GB_EXPORT int gb_head_gate_bf16(const void* x, const float* gate, long long gate_ld, void* out, long long out_ld,
                                int n_rows, int nq, int Ds, int Dv, float mult, cudaStream_t s) {
  return head_gate<bf16>(x, gate, gate_ld, out, out_ld, n_rows, nq, Ds, Dv, mult, s);
}
