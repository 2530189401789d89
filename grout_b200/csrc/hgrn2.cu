// Linear attention whose forget gate also decides what is written (HGRN2).  Per head,
// with q, f [dk] and v [dv] of a token,
//
//   q = silu(zq),   f = low + (1 - low) * sigmoid(zf + bias)        (low: a learned floor per channel)
//   S <- diag(f) S + (1 - f) v^T      (S [dk, dv], 32-bit, zero when the sequence starts)
//   o  = S^T q
//   y  = o / sqrt(mean(o^2) + eps) * w * out_scale                  (w [dv] shared by the heads)
//
// There is no key: 1 - f stands where a key would.  Everything here is 32-bit: the input
// is the 32-bit sums of a projection (row pitch `ld`; zq, zf [H dk] and v [H dv] start at
// the columns q_col, f_col, v_col), and only y is rounded to the activation type.  y's row
// pitch is `y_ld`, so a head's read-out can be written into a wider row that another
// kernel fills up (the input of an output projection that serves two mixers).
//
// Two kernels.  `scan` walks a sequence's rows in order: a block owns one (sequence,
// head) and HG_COLS columns of S; a column's dk elements live in the registers of eight
// lanes; the rows' q and f are computed from the sums HG_STAGE rows at a time into shared
// memory, and the eight partial read-outs of a column meet by shuffles.  The state is read
// once and written once per step, for sequences whose slot is not negative (padding rows
// start from zeros and store nothing).  `finish` normalises a head's read-out.  The order
// of a column's sums does not depend on how a sequence's rows are cut into steps, so a
// prompt in portions of fewer than HG_CHUNK_MIN rows or row by row leaves the same state bit
// for bit.
//
// A step in which a sequence brings HG_CHUNK_MIN rows or more goes chunk by chunk, since one
// block per (sequence, head, columns) would walk thousands of rows alone.  The recurrence is
// linear in S: with b_t the product of the gates from a chunk's first row to row t,
// S_t = diag(b_t) S_start + (the state that the chunk's rows build from zeros), so
// `scan` takes every chunk of HG_CHUNK rows at the same time, each from zeros, and leaves the
// chunk's read-outs, what it adds to the state, the product of its gates and q_t * b_t;
// `prefix` turns those into the states at the chunks' starts (S <- diag(product) S + added,
// in the chunks' order) and stores the last; `cross` adds S_start^T (q_t * b_t) to the
// read-outs, a tiled 32-bit product.  The products of gates are taken directly (no
// logarithms), so this is the same arithmetic in another order.
#include "common.cuh"

struct Hgrn2Args {
  const float* proj;      // [T, ld]
  long long ld;
  int q_col, f_col, v_col;
  const float* f_bias;    // [H dk]
  const float* lower;     // [H dk]
  const float* norm_w;    // [dv]
  const int* cu_q;        // [n_seqs + 1]
  const int* slots;       // [n_seqs]
  float* state;           // [slots, state_stride], a sequence's H matrices [dk, dv]
  long long state_stride;
  float* o;               // [T, H, dv] scratch: the read-outs
  void* y;                // [T, y_ld]: H dv columns are written
  long long y_ld;
  int n_tokens, n_seqs, H, dk, dv;
  float norm_eps, out_scale;
  float* qb;              // [T, H, dk] scratch of a step that goes chunk by chunk: q_t * b_t
  float* chunk_state;     // [T / HG_CHUNK + n_seqs, H, dk, dv] scratch: what a chunk adds, then its start state
  float* chunk_decay;     // [T / HG_CHUNK + n_seqs, H, dk] scratch: the product of a chunk's gates
  int max_rows;           // the most rows a sequence brings (0: unknown)
};

#define HG_LANES 8      // lanes that share a column of the state
#define HG_COLS 16      // columns a block owns
#define HG_STAGE 16     // rows staged at a time
#define HG_CHUNK 64     // rows of a chunk where a sequence brings many
#define HG_CHUNK_MIN 256  // a step goes chunk by chunk when a sequence brings this many rows

// Chunk z of a sequence is its rows z HG_CHUNK .. ; its scratch lies at entry
// (first row / HG_CHUNK + the sequence's number), which no other chunk has.
__device__ __forceinline__ size_t hg_entry(int first, int z, int seq) {
  return (size_t)((first + z * HG_CHUNK) / HG_CHUNK + seq);
}

__device__ __forceinline__ float hg_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// Row r of a lane's share of a column is element hg_row(lane, r) of the head: runs of four
// neighbours per lane where a lane has a multiple of four, else every eighth element.
template <int KPL>
__device__ __forceinline__ int hg_row(int lane, int r) {
  return (KPL % 4 == 0) ? (r >> 2) * 32 + lane * 4 + (r & 3) : r * HG_LANES + lane;
}

// CPT: columns of S a thread owns (the rows' q and f are read from shared memory once for all
// of them).  CHUNKED: the block owns one chunk of its sequence, starts from zeros and leaves
// what the chunk adds to the state in the chunk's entry instead of the sequence's state.
template <int KPL, int CPT, bool CHUNKED>
__global__ void __launch_bounds__(HG_COLS* HG_LANES) hgrn2_scan_kernel(const Hgrn2Args a) {
  constexpr int DKP = KPL * HG_LANES;            // dk rounded up; the rest is q = 0, f = 1
  constexpr int BC = HG_COLS * CPT;              // columns a block owns
  __shared__ __align__(16) float qs[HG_STAGE][DKP];
  __shared__ __align__(16) float fs[HG_STAGE][DKP];
  __shared__ float vs[HG_STAGE][BC];
  __shared__ float bs[CHUNKED ? DKP : 1];        // the product of the chunk's gates so far
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int col_tiles = (a.dv + BC - 1) / BC;
  const int h = blockIdx.x, seq = blockIdx.y, c0 = (blockIdx.z % col_tiles) * BC;
  const int z = blockIdx.z / col_tiles;          // the chunk (0 unless CHUNKED)
  const int dk = a.dk, dv = a.dv;
  const int seq_first = a.cu_q[seq], seq_n = a.cu_q[seq + 1] - seq_first;
  const int first = seq_first + z * HG_CHUNK;
  const int n = CHUNKED ? min(HG_CHUNK, seq_n - z * HG_CHUNK) : seq_n;
  if (n <= 0) return;
  const int tid = threadIdx.x, lane = tid % HG_LANES, cb = c0 + (tid / HG_LANES) * CPT;
  const int slot = a.slots[seq];
  float* sp = CHUNKED ? a.chunk_state + (hg_entry(seq_first, z, seq) * a.H + h) * (size_t)dk * dv
                      : (slot >= 0 ? a.state + (size_t)slot * a.state_stride + (size_t)h * dk * dv : nullptr);
  float S[CPT][KPL];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int r = 0; r < KPL; ++r) {
      const int i = hg_row<KPL>(lane, r);
      S[c][r] = (!CHUNKED && sp && cb + c < dv && i < dk) ? sp[(size_t)i * dv + cb + c] : 0.f;
    }
  if (CHUNKED)
    for (int e = tid; e < DKP; e += blockDim.x) bs[e] = 1.f;
  for (int t0 = 0; t0 < n; t0 += HG_STAGE) {
    const int nt = min(HG_STAGE, n - t0);
    __syncthreads();
    for (int i = tid; i < nt * DKP; i += blockDim.x) {
      const int tt = i / DKP, e = i % DKP;
      float q = 0.f, f = 1.f;
      if (e < dk) {
        const float* row = a.proj + (size_t)(first + t0 + tt) * a.ld;
        const int c = h * dk + e;
        const float zq = row[a.q_col + c], low = a.lower[c];
        q = zq * hg_sigmoid(zq);
        f = low + (1.0f - low) * hg_sigmoid(row[a.f_col + c] + a.f_bias[c]);
      }
      qs[tt][e] = q;
      fs[tt][e] = f;
    }
    for (int i = tid; i < nt * BC; i += blockDim.x) {
      const int tt = i / BC, c = c0 + i % BC;
      vs[tt][i % BC] = c < dv ? a.proj[(size_t)(first + t0 + tt) * a.ld + a.v_col + h * dv + c] : 0.f;
    }
    __syncthreads();
    if (CHUNKED) {
      // a thread walks a channel's staged rows in order and carries the product of its gates
      for (int e = tid; e < dk; e += blockDim.x) {
        float b = bs[e];
        for (int tt = 0; tt < nt; ++tt) {
          b *= fs[tt][e];
          if (c0 == 0) a.qb[((size_t)(first + t0 + tt) * a.H + h) * dk + e] = qs[tt][e] * b;
        }
        bs[e] = b;
      }
    }
    for (int tt = 0; tt < nt; ++tt) {
      float v[CPT], acc[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) v[c] = vs[tt][(tid / HG_LANES) * CPT + c], acc[c] = 0.f;
      if (KPL % 4 == 0) {
#pragma unroll
        for (int r = 0; r < KPL; r += 4) {
          const float4 f4 = *reinterpret_cast<const float4*>(&fs[tt][hg_row<KPL>(lane, r)]);
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][hg_row<KPL>(lane, r)]);
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            S[c][r] = fmaf(f4.x, S[c][r], (1.0f - f4.x) * v[c]);
            S[c][r + 1] = fmaf(f4.y, S[c][r + 1], (1.0f - f4.y) * v[c]);
            S[c][r + 2] = fmaf(f4.z, S[c][r + 2], (1.0f - f4.z) * v[c]);
            S[c][r + 3] = fmaf(f4.w, S[c][r + 3], (1.0f - f4.w) * v[c]);
            acc[c] = fmaf(S[c][r], q4.x, acc[c]);
            acc[c] = fmaf(S[c][r + 1], q4.y, acc[c]);
            acc[c] = fmaf(S[c][r + 2], q4.z, acc[c]);
            acc[c] = fmaf(S[c][r + 3], q4.w, acc[c]);
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
          const int i = hg_row<KPL>(lane, r);
          const float f = fs[tt][i], q = qs[tt][i];
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            S[c][r] = fmaf(f, S[c][r], (1.0f - f) * v[c]);
            acc[c] = fmaf(S[c][r], q, acc[c]);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
        acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
        acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 4);
        if (lane == 0 && cb + c < dv) a.o[((size_t)(first + t0 + tt) * a.H + h) * dv + cb + c] = acc[c];
      }
    }
  }
  pdl_launch_dependents_if_large();
  if (sp) {
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
      for (int r = 0; r < KPL; ++r) {
        const int i = hg_row<KPL>(lane, r);
        if (i < dk && cb + c < dv) sp[(size_t)i * dv + cb + c] = S[c][r];
      }
  }
  if (CHUNKED && c0 == 0) {
    __syncthreads();            // (the last stage's products are in bs)
    for (int e = tid; e < dk; e += blockDim.x)
      a.chunk_decay[(hg_entry(seq_first, z, seq) * a.H + h) * (size_t)dk + e] = bs[e];
  }
}

// The states at the chunks' starts: a thread owns one element of a (sequence, head)'s matrix,
// walks the chunks in order, leaves in every chunk's entry the state the chunk starts from in
// place of what the chunk adds, and stores the state after the last.
__global__ void __launch_bounds__(256) hgrn2_prefix_kernel(const Hgrn2Args a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int h = blockIdx.y, seq = blockIdx.z, H = a.H;
  const size_t per = (size_t)a.dk * a.dv;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  if (e >= per || n <= 0) return;
  const int i = (int)(e / a.dv);
  const int slot = a.slots[seq];
  float* sp = slot >= 0 ? a.state + (size_t)slot * a.state_stride + (size_t)h * per : nullptr;
  float S = sp ? sp[e] : 0.f;
  const int chunks = (n + HG_CHUNK - 1) / HG_CHUNK;
  for (int z0 = 0; z0 < chunks; z0 += 8) {      // eight chunks' loads at a time, used in order
    float add[8], dec[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int z = z0 + u < chunks ? z0 + u : chunks - 1;
      const size_t en = hg_entry(first, z, seq) * H + h;
      add[u] = a.chunk_state[en * per + e];
      dec[u] = a.chunk_decay[en * a.dk + i];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (z0 + u < chunks) {
        a.chunk_state[(hg_entry(first, z0 + u, seq) * H + h) * per + e] = S;
        S = fmaf(dec[u], S, add[u]);
      }
    }
  }
  if (sp) sp[e] = S;
}

// o[t, h, :] += S_start^T (q_t * b_t) for every row of every chunk: a tile of 64 rows and 64
// columns a block, a thread owns 4 x 4 sums, the head's elements staged 16 at a time.
#define HG_TK 16
__global__ void __launch_bounds__(256) hgrn2_cross_kernel(const Hgrn2Args a) {
  __shared__ __align__(16) float As[HG_TK][HG_CHUNK];     // [element][row]
  __shared__ __align__(16) float Bs[HG_TK][64];           // [element][column]
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int H = a.H, dk = a.dk, dv = a.dv;
  const int col_tiles = (dv + 63) / 64;
  const int h = blockIdx.x, seq = blockIdx.y, z = blockIdx.z / col_tiles, c0 = (blockIdx.z % col_tiles) * 64;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  if (z * HG_CHUNK >= n) return;
  const int rows = min(HG_CHUNK, n - z * HG_CHUNK), r0 = first + z * HG_CHUNK;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const float* st = a.chunk_state + (hg_entry(first, z, seq) * H + h) * (size_t)dk * dv;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < dk; k0 += HG_TK) {
    __syncthreads();
    {
      const int m = tid / 4, kk = (tid % 4) * 4;          // 64 rows x 16 elements
      const float* src = a.qb + ((size_t)(r0 + m) * H + h) * dk + k0 + kk;
#pragma unroll
      for (int i = 0; i < 4; ++i) As[kk + i][m] = (m < rows && k0 + kk + i < dk) ? src[i] : 0.f;
      const int kr = tid / 16, cc = (tid % 16) * 4;       // 16 elements x 64 columns
#pragma unroll
      for (int j = 0; j < 4; ++j)
        Bs[kr][cc + j] = (k0 + kr < dk && c0 + cc + j < dv) ? st[(size_t)(k0 + kr) * dv + c0 + cc + j] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HG_TK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }
  pdl_launch_dependents_if_large();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= rows) continue;
    float* o = a.o + ((size_t)(r0 + m) * H + h) * dv + c0 + tx * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (c0 + tx * 4 + j < dv) o[j] += acc[i][j];
  }
}

// One warp per (row, head): the read-out's root mean square, the weight, the factor.
template <typename T>
__global__ void __launch_bounds__(128) hgrn2_finish_kernel(const Hgrn2Args a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + warp;
  if (unit >= (long long)a.n_tokens * a.H) return;
  const int t = (int)(unit / a.H), h = (int)(unit % a.H), dv = a.dv;
  const float* o = a.o + (size_t)unit * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss = fmaf(o[d], o[d], ss);
  ss = warp_sum(ss);
  const float inv = a.out_scale / sqrtf(ss / (float)dv + a.norm_eps);
  T* y = (T*)a.y + (size_t)t * a.y_ld + (size_t)h * dv;
  for (int d = lane; d < dv; d += 32) y[d] = from_f32<T>(o[d] * a.norm_w[d] * inv);
  pdl_launch_dependents_if_large();
}

static bool hg_chunked(const Hgrn2Args& a) {
  return a.max_rows >= HG_CHUNK_MIN && a.qb && a.chunk_state && a.chunk_decay;
}

template <int KPL, int CPT>
static int launch_scan_cols(const Hgrn2Args& a, cudaStream_t s) {
  const int col_tiles = (a.dv + HG_COLS * CPT - 1) / (HG_COLS * CPT);
  if (!hg_chunked(a))
    return gb_launch(hgrn2_scan_kernel<KPL, CPT, false>, dim3(a.H, a.n_seqs, col_tiles),
                     dim3(HG_COLS * HG_LANES), 0, s, a);
  const int chunks = (a.max_rows + HG_CHUNK - 1) / HG_CHUNK;
  if ((long long)col_tiles * chunks > 65535) return GB_ERR_UNSUPPORTED;
  int e = gb_launch(hgrn2_scan_kernel<KPL, CPT, true>, dim3(a.H, a.n_seqs, col_tiles * chunks),
                    dim3(HG_COLS * HG_LANES), 0, s, a);
  if (e) return e;
  const size_t per = (size_t)a.dk * a.dv;
  e = gb_launch(hgrn2_prefix_kernel, dim3((unsigned)((per + 255) / 256), a.H, a.n_seqs), dim3(256), 0, s, a);
  if (e) return e;
  return gb_launch(hgrn2_cross_kernel, dim3(a.H, a.n_seqs, chunks * ((a.dv + 63) / 64)), dim3(256), 0, s, a);
}

// A thread owns several columns of S where a head is wide enough for that to leave blocks for
// every SM (four columns of heads up to 128 elements, two of longer ones); a column's sums are
// the same in every case.
template <int KPL>
static int launch_scan(const Hgrn2Args& a, cudaStream_t s) {
  constexpr int WIDE = KPL <= 16 ? 4 : 2;
  // (a step of few rows is the time to bring the state in and out: many small blocks do that best)
  if (a.dv >= HG_COLS * WIDE && a.max_rows >= HG_STAGE) return launch_scan_cols<KPL, WIDE>(a, s);
  return launch_scan_cols<KPL, 1>(a, s);
}

template <typename T>
static int launch(const Hgrn2Args& a, cudaStream_t s) {
  if (a.n_tokens < 0 || a.n_seqs <= 0 || a.H <= 0 || a.dk <= 0 || a.dv <= 0 || !a.proj || !a.state ||
      !a.o || !a.y || !a.f_bias || !a.lower || !a.norm_w || !a.cu_q || !a.slots)
    return GB_ERR_BAD_ARG;
  if (a.dk > 256 || a.n_seqs > 65535 || a.H > 65535) return GB_ERR_UNSUPPORTED;
  if (a.n_tokens == 0) return 0;
  const int kpl = (a.dk + HG_LANES - 1) / HG_LANES;
  int e;
  if (kpl <= 1) e = launch_scan<1>(a, s);
  else if (kpl <= 2) e = launch_scan<2>(a, s);
  else if (kpl <= 3) e = launch_scan<3>(a, s);
  else if (kpl <= 4) e = launch_scan<4>(a, s);
  else if (kpl <= 6) e = launch_scan<6>(a, s);
  else if (kpl <= 8) e = launch_scan<8>(a, s);
  else if (kpl <= 12) e = launch_scan<12>(a, s);
  else if (kpl <= 16) e = launch_scan<16>(a, s);
  else if (kpl <= 24) e = launch_scan<24>(a, s);
  else e = launch_scan<32>(a, s);
  if (e) return e;
  const long long units = (long long)a.n_tokens * a.H;
  return gb_launch(hgrn2_finish_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, s, a);
}

GB_EXPORT int gb_hgrn2_f32(const Hgrn2Args* a, cudaStream_t s) { return launch<float>(*a, s); }
GB_EXPORT int gb_hgrn2_bf16(const Hgrn2Args* a, cudaStream_t s) { return launch<bf16>(*a, s); }
