// Retention: linear attention with a fixed decay per head and neither softmax nor
// denominator.  Per head, with q, k [dk] and v [dv] of a token,
//
//   S <- decay_h S + k v^T          (S [dk, dv], 32-bit, zero when the sequence starts)
//   o  = S^T q
//   y  = o / sqrt(mean(o^2) + eps) * silu(gate)
//
// q and k are rotated first: of every head's first `rot_dim` elements, element i
// and element i + rot_dim/2 turn by pos * inv_freq[i]; k is then multiplied by
// `k_scale`.  Everything here is 32-bit: the input is the 32-bit sums of the
// mixer's one projection (columns q [H dk] | k [H dk] | v [H dv] | gate [H dv]),
// and only y is rounded to the activation type.
//
// Three kernels.  `rotate` writes the turned q and scaled k of every row.  `scan`
// walks a sequence's rows in order: a block owns one (sequence, head) and RT_COLS
// columns of S; a column's dk elements live in the registers of eight lanes, the
// rows' q, k and v are staged in shared memory RT_STAGE rows at a time, and the
// eight partial read-outs of a column meet by shuffles.  The state is read once
// and written once per step, for sequences whose slot is not negative (padding
// rows read zeros and store nothing).  `finish` normalises a head's read-out and
// applies the gate.
//
// A step in which a sequence brings RT_CHUNK_MIN rows or more goes chunk by chunk, five
// kernels.  `chunk` takes every chunk of RT_CHUNK rows at the same time, each from zeros,
// as three tiled 32-bit products: P = (Q K^T) under the mask decay^(i-j) (j <= i), the
// read-outs within the chunk P V, and what the chunk adds to the state,
// sum_t decay^(rows-1-t) k_t v_t^T.  `prefix` turns those into the states at the chunks'
// starts (S <- decay^rows S + added, in the chunks' order) and stores the last; `cross`
// adds decay^(j+1) S_start^T q to row j of every chunk, a tiled 32-bit product too.  The
// recurrence is linear, so this is the same sum in another order.
//
// A step in which every sequence brings one row (decoding) is one kernel, `step`:
// a block owns one (sequence, head), turns the row's q and k itself, streams the
// head's whole state through once (a warp reads and writes whole rows of S), adds
// up the warps' partial read-outs in shared memory and finishes the head.
#include "common.cuh"

struct RetentionArgs {
  const float* proj;      // [T, 2 H dk + 2 H dv]
  const float* decay;     // [H]
  const float* inv_freq;  // [rot_dim / 2]
  const int* token_pos;   // [T]
  const int* cu_q;        // [n_seqs + 1]
  const int* slots;       // [n_seqs]
  float* state;           // [slots, state_stride], a sequence's H matrices [dk, dv]
  long long state_stride;
  float* qk;              // [T, 2, H, dk] scratch: turned q, turned and scaled k
  float* o;               // [T, H, dv] scratch: the read-outs
  float* chunk_state;     // [T / RT_CHUNK + n_seqs, H, dk, dv] scratch of a step that goes chunk by chunk
  void* y;                // [T, H dv]
  int n_tokens, n_seqs, H, dk, dv, rot_dim;
  float k_scale, norm_eps;
  int max_rows;           // the most rows a sequence brings (0: unknown)
};

#define RT_LANES 8      // lanes that share a column of the state
#define RT_COLS 16      // columns a block owns
#define RT_STAGE 16     // rows staged at a time
#define RT_CHUNK 64     // rows of a chunk where a sequence brings more than that
#define RT_TM 64        // rows of a block of the chunks' second pass
#define RT_TN 128       // columns of its tile
#define RT_TK 16        // elements of a head it stages at a time
#define RT_CHUNK_MIN 256  // a step goes chunk by chunk when a sequence brings this many rows

__global__ void __launch_bounds__(256) retention_rotate_kernel(const RetentionArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x;
  const int H = a.H, dk = a.dk, half = a.rot_dim / 2;
  const int C = 2 * H * dk + 2 * H * a.dv;
  const float* row = a.proj + (size_t)t * C;
  float* out = a.qk + (size_t)t * 2 * H * dk;
  const float pos = (float)a.token_pos[t];
  // one thread per (q or k, head, element below dk - half): an element outside the
  // rotated part passes, a rotated pair is written by the thread of its first element
  for (int i = threadIdx.x; i < 2 * H * dk; i += blockDim.x) {
    const int e = i % dk;
    const float mul = i >= H * dk ? a.k_scale : 1.0f;
    if (e >= a.rot_dim) { out[i] = row[i] * mul; continue; }
    if (e >= half) continue;
    float s, c;
    sincosf(pos * a.inv_freq[e], &s, &c);
    const float u = row[i], v = row[i + half];
    out[i] = (u * c - v * s) * mul;
    out[i + half] = (v * c + u * s) * mul;
  }
  pdl_launch_dependents_if_large();
}

// Row r of a lane's share of a column is element rt_row(lane, r) of the head: runs of four
// neighbours per lane where a lane has a multiple of four (16-byte shared-memory reads
// that the eight lanes of a column make side by side), else every eighth element.
template <int KPL>
__device__ __forceinline__ int rt_row(int lane, int r) {
  return (KPL % 4 == 0) ? (r >> 2) * 32 + lane * 4 + (r & 3) : r * RT_LANES + lane;
}

// Chunk z of a sequence is its rows z RT_CHUNK .. ; its matrices live at entry
// (first row / RT_CHUNK + the sequence's number), which no other chunk has.
__device__ __forceinline__ size_t rt_entry(int first, int z, int seq) {
  return (size_t)((first + z * RT_CHUNK) / RT_CHUNK + seq);
}

template <int KPL>
__global__ void __launch_bounds__(RT_COLS* RT_LANES) retention_scan_kernel(const RetentionArgs a) {
  constexpr int DKP = KPL * RT_LANES;            // dk rounded up; the rest is zeros
  __shared__ __align__(16) float qs[RT_STAGE][DKP];
  __shared__ __align__(16) float ks[RT_STAGE][DKP];
  __shared__ float vs[RT_STAGE][RT_COLS];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int h = blockIdx.x, seq = blockIdx.y, c0 = blockIdx.z * RT_COLS;
  const int H = a.H, dk = a.dk, dv = a.dv;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  if (n <= 0) return;
  const int tid = threadIdx.x, lane = tid % RT_LANES, col = c0 + tid / RT_LANES;
  const bool live = col < dv;
  const int slot = a.slots[seq];
  float* sp = slot >= 0 ? a.state + (size_t)slot * a.state_stride + (size_t)h * dk * dv : nullptr;
  const float decay = a.decay[h];
  float S[KPL];
#pragma unroll
  for (int r = 0; r < KPL; ++r) {
    const int i = rt_row<KPL>(lane, r);
    S[r] = (sp && live && i < dk) ? sp[(size_t)i * dv + col] : 0.f;
  }
  const int C = 2 * H * dk + 2 * H * dv;
  for (int t0 = 0; t0 < n; t0 += RT_STAGE) {
    const int nt = min(RT_STAGE, n - t0);
    __syncthreads();
    for (int i = tid; i < nt * DKP; i += blockDim.x) {
      const int tt = i / DKP, e = i % DKP;
      const float* src = a.qk + ((size_t)(first + t0 + tt) * 2 * H + h) * dk;
      qs[tt][e] = e < dk ? src[e] : 0.f;
      ks[tt][e] = e < dk ? src[(size_t)H * dk + e] : 0.f;
    }
    for (int i = tid; i < nt * RT_COLS; i += blockDim.x) {
      const int tt = i / RT_COLS, c = c0 + i % RT_COLS;
      vs[tt][i % RT_COLS] = c < dv ? a.proj[(size_t)(first + t0 + tt) * C + 2 * H * dk + h * dv + c] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float v = vs[tt][tid / RT_LANES];
      float acc = 0.f;
      if (KPL % 4 == 0) {
#pragma unroll
        for (int r = 0; r < KPL; r += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(&ks[tt][rt_row<KPL>(lane, r)]);
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][rt_row<KPL>(lane, r)]);
          S[r] = fmaf(decay, S[r], k4.x * v);
          S[r + 1] = fmaf(decay, S[r + 1], k4.y * v);
          S[r + 2] = fmaf(decay, S[r + 2], k4.z * v);
          S[r + 3] = fmaf(decay, S[r + 3], k4.w * v);
          acc = fmaf(S[r], q4.x, acc);
          acc = fmaf(S[r + 1], q4.y, acc);
          acc = fmaf(S[r + 2], q4.z, acc);
          acc = fmaf(S[r + 3], q4.w, acc);
        }
      } else {
#pragma unroll
        for (int r = 0; r < KPL; ++r) {
          const int i = rt_row<KPL>(lane, r);
          S[r] = fmaf(decay, S[r], ks[tt][i] * v);
          acc = fmaf(S[r], qs[tt][i], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (lane == 0 && live) a.o[((size_t)(first + t0 + tt) * H + h) * dv + col] = acc;
    }
  }
  pdl_launch_dependents_if_large();
  if (sp && live) {
#pragma unroll
    for (int r = 0; r < KPL; ++r) {
      const int i = rt_row<KPL>(lane, r);
      if (i < dk) sp[(size_t)i * dv + col] = S[r];
    }
  }
}

// One chunk of one head, from a state of zeros, as three 32-bit products of 64 x 64 tiles
// (a thread owns 4 x 4 sums): P = (Q K^T) * D with D[i][j] = decay^(i-j) for j <= i and 0
// above; the chunk's read-outs O = P V; and what the chunk adds to the state,
// sum_t decay^(rows-1-t) k_t v_t^T, left in the chunk's entry.
#define RT_CT 64
__global__ void __launch_bounds__(256) retention_chunk_kernel(const RetentionArgs a) {
  extern __shared__ __align__(16) float rc_sm[];
  float (*PsT)[RT_CT] = reinterpret_cast<float (*)[RT_CT]>(rc_sm);                     // [key row j][query row i]
  float (*Vs)[RT_CT] = reinterpret_cast<float (*)[RT_CT]>(rc_sm + RT_CT * RT_CT);      // [row t][column]
  float (*Kt)[RT_CT] = reinterpret_cast<float (*)[RT_CT]>(rc_sm + 2 * RT_CT * RT_CT);  // [row t][element], weighted
  float (*Qs)[RT_CT] = reinterpret_cast<float (*)[RT_CT]>(rc_sm + 3 * RT_CT * RT_CT);  // [RT_TK][row]
  float (*Ks)[RT_CT] = Qs + RT_TK;
  float* dpow = rc_sm + 3 * RT_CT * RT_CT + 2 * RT_TK * RT_CT;                         // decay^0 .. decay^RT_CT
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int H = a.H, dk = a.dk, dv = a.dv;
  const int h = blockIdx.x, seq = blockIdx.y, z = blockIdx.z;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  if (z * RT_CHUNK >= n) return;
  const int rows = min(RT_CHUNK, n - z * RT_CHUNK), r0 = first + z * RT_CHUNK;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int C = 2 * H * dk + 2 * H * dv;
  const float decay = a.decay[h];
  if (tid <= RT_CT) dpow[tid] = powf(decay, (float)tid);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < dk; k0 += RT_TK) {
    __syncthreads();
    {
      const int m = tid / 4, kk = (tid % 4) * 4;
      const float* src = a.qk + ((size_t)(r0 + m) * 2 * H + h) * dk + k0 + kk;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool in = m < rows && k0 + kk + i < dk;
        Qs[kk + i][m] = in ? src[i] : 0.f;
        Ks[kk + i][m] = in ? src[(size_t)H * dk + i] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < RT_TK; ++kk) {
      const float4 q4 = *reinterpret_cast<const float4*>(&Qs[kk][ty * 4]);
      const float4 k4 = *reinterpret_cast<const float4*>(&Ks[kk][tx * 4]);
      const float qv[4] = {q4.x, q4.y, q4.z, q4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
    }
  }
  // P under the decay mask, stored with the key row first
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float pv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = ty * 4 + i, kj = tx * 4 + j;
      pv[i] = kj <= qi ? acc[i][j] * dpow[qi - kj] : 0.f;
    }
    *reinterpret_cast<float4*>(&PsT[tx * 4 + j][ty * 4]) = make_float4(pv[0], pv[1], pv[2], pv[3]);
  }
  float* sp = a.chunk_state + (rt_entry(first, z, seq) * H + h) * (size_t)dk * dv;
  for (int c0 = 0; c0 < dv; c0 += RT_CT) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RT_CT * RT_CT / 256; ++i) {
      const int idx = tid + i * 256, t = idx / RT_CT, c = idx % RT_CT;
      Vs[t][c] = (t < rows && c0 + c < dv) ? a.proj[(size_t)(r0 + t) * C + 2 * H * dk + h * dv + c0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 8
    for (int t = 0; t < RT_CT; ++t) {
      const float4 p4 = *reinterpret_cast<const float4*>(&PsT[t][ty * 4]);
      const float4 v4 = *reinterpret_cast<const float4*>(&Vs[t][tx * 4]);
      const float pv[4] = {p4.x, p4.y, p4.z, p4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(pv[i], vv[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = ty * 4 + i;
      if (m >= rows) continue;
      float* o = a.o + ((size_t)(r0 + m) * H + h) * dv + c0 + tx * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c0 + tx * 4 + j < dv) o[j] = acc[i][j];
    }
    for (int i0 = 0; i0 < dk; i0 += RT_CT) {
      __syncthreads();
#pragma unroll
      for (int i = 0; i < RT_CT * RT_CT / 256; ++i) {
        const int idx = tid + i * 256, t = idx / RT_CT, e = idx % RT_CT;
        Kt[t][e] = (t < rows && i0 + e < dk)
                       ? a.qk[((size_t)(r0 + t) * 2 * H + H + h) * dk + i0 + e] * dpow[rows - 1 - t] : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 8
      for (int t = 0; t < RT_CT; ++t) {
        const float4 k4 = *reinterpret_cast<const float4*>(&Kt[t][ty * 4]);
        const float4 v4 = *reinterpret_cast<const float4*>(&Vs[t][tx * 4]);
        const float kv[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(kv[i], vv[j], acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = i0 + ty * 4 + i;
        if (e >= dk) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c0 + tx * 4 + j < dv) sp[(size_t)e * dv + c0 + tx * 4 + j] = acc[i][j];
      }
    }
  }
  pdl_launch_dependents_if_large();
}

// The states at the chunks' starts: a thread owns one element of a (sequence, head)'s
// matrix, walks the chunks in order, leaves in every chunk's entry the state the chunk
// starts from in place of what the chunk adds, and stores the state after the last.
__global__ void __launch_bounds__(256) retention_prefix_kernel(const RetentionArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int h = blockIdx.y, seq = blockIdx.z, H = a.H;
  const size_t per = (size_t)a.dk * a.dv;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  if (e >= per || n <= 0) return;
  const int slot = a.slots[seq];
  float* sp = slot >= 0 ? a.state + (size_t)slot * a.state_stride + (size_t)h * per : nullptr;
  const float decay = a.decay[h];
  const float whole = powf(decay, (float)RT_CHUNK);
  float S = sp ? sp[e] : 0.f;
  const int nz = (n + RT_CHUNK - 1) / RT_CHUNK;
  const float last = powf(decay, (float)(n - (nz - 1) * RT_CHUNK));
  // eight chunks a turn: their loads are all asked for before the first is used
  for (int z0 = 0; z0 < nz; z0 += 8) {
    float add[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      add[j] = z0 + j < nz ? __ldcs(a.chunk_state + (rt_entry(first, z0 + j, seq) * H + h) * per + e) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (z0 + j >= nz) break;
      a.chunk_state[(rt_entry(first, z0 + j, seq) * H + h) * per + e] = S;
      S = fmaf(z0 + j == nz - 1 ? last : whole, S, add[j]);
    }
  }
  pdl_launch_dependents_if_large();
  if (sp) sp[e] = S;
}

// What the state at a chunk's start adds to the chunk's read-outs: row j of the chunk
// gets decay^(j+1) S^T q.  A block owns RT_TM rows of one chunk and RT_TN columns of one
// head; a thread owns 4 rows and 8 columns; the head's elements come RT_TK at a time.
__global__ void __launch_bounds__(256) retention_cross_kernel(const RetentionArgs a) {
  __shared__ __align__(16) float qs[RT_TK][RT_TM];
  __shared__ __align__(16) float ss[RT_TK][RT_TN];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int H = a.H, dk = a.dk, dv = a.dv;
  const int col_tiles = (dv + RT_TN - 1) / RT_TN;
  const int h = blockIdx.y, seq = blockIdx.z;
  const int c0 = (blockIdx.x % col_tiles) * RT_TN;
  const int tile = blockIdx.x / col_tiles;
  const int z = tile / (RT_CHUNK / RT_TM), j0 = (tile % (RT_CHUNK / RT_TM)) * RT_TM;
  const int first = a.cu_q[seq], n = a.cu_q[seq + 1] - first;
  if (z * RT_CHUNK + j0 >= n) return;
  const int rows = min(RT_TM, n - z * RT_CHUNK - j0);
  const int r0 = first + z * RT_CHUNK + j0;
  const float* S = a.chunk_state + (rt_entry(first, z, seq) * H + h) * (size_t)dk * dv;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < dk; k0 += RT_TK) {
    __syncthreads();
    {
      const int m = tid / 4, kk = (tid % 4) * 4;
      const float* src = a.qk + ((size_t)(r0 + m) * 2 * H + h) * dk + k0 + kk;
#pragma unroll
      for (int i = 0; i < 4; ++i) qs[kk + i][m] = (m < rows && k0 + kk + i < dk) ? src[i] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < RT_TK * RT_TN / 256; ++i) {
      const int idx = tid + i * 256, kk = idx / RT_TN, c = idx % RT_TN;
      ss[kk][c] = (k0 + kk < dk && c0 + c < dv) ? S[(size_t)(k0 + kk) * dv + c0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < RT_TK; ++kk) {
      const float4 q4 = *reinterpret_cast<const float4*>(&qs[kk][ty * 4]);
      const float4 s0 = *reinterpret_cast<const float4*>(&ss[kk][tx * 4]);
      const float4 s1 = *reinterpret_cast<const float4*>(&ss[kk][64 + tx * 4]);
      const float qv[4] = {q4.x, q4.y, q4.z, q4.w};
      const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(qv[i], sv[j], acc[i][j]);
    }
  }
  pdl_launch_dependents_if_large();
  const float decay = a.decay[h];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= rows) continue;
    const float f = powf(decay, (float)(j0 + m + 1));
    float* o = a.o + ((size_t)(r0 + m) * H + h) * dv;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (c < dv) o[c] = fmaf(f, acc[i][j], o[c]);
    }
  }
}

// y[t, h, :] = o / sqrt(mean(o^2) + eps) * silu(gate): one warp per (row, head)
template <typename T>
__global__ void __launch_bounds__(128) retention_finish_kernel(const RetentionArgs a) {
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)a.n_tokens * a.H) return;
  const int t = (int)(w / a.H), h = (int)(w % a.H), dv = a.dv;
  const int C = 2 * a.H * a.dk + 2 * a.H * dv;
  const float* o = a.o + ((size_t)t * a.H + h) * dv;
  const float* g = a.proj + (size_t)t * C + 2 * a.H * a.dk + a.H * dv + h * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(o[i], o[i], ss);
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + a.norm_eps);
  pdl_launch_dependents_if_large();
  T* y = (T*)a.y + ((size_t)t * a.H + h) * dv;
  for (int i = lane; i < dv; i += 32) {
    const float gv = g[i];
    y[i] = from_f32<T>(o[i] * inv * (gv / (1.0f + expf(-gv))));
  }
}

#define RT_STEP_WARPS 8

// One row per sequence.  DVJ: columns a lane holds (dv <= 32 DVJ).
template <typename T, int DVJ>
__global__ void __launch_bounds__(RT_STEP_WARPS * 32) retention_step_kernel(const RetentionArgs a) {
  extern __shared__ float sm[];
  __shared__ float scratch[32];
  const int h = blockIdx.x, seq = blockIdx.y;
  const int H = a.H, dk = a.dk, dv = a.dv, half = a.rot_dim / 2;
  float* qs = sm;                      // [dk]
  float* ks = qs + dk;                 // [dk]
  float* vs = ks + dk;                 // [dv]
  float* part = vs + dv;               // [RT_STEP_WARPS, dv]
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const float decay = a.decay[h];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = a.cu_q[seq];
  if (a.cu_q[seq + 1] - t <= 0) return;
  const int C = 2 * H * dk + 2 * H * dv;
  const float* row = a.proj + (size_t)t * C;
  const float pos = (float)a.token_pos[t];
  for (int e = tid; e < dk; e += blockDim.x) {
    const float* q = row + h * dk;
    const float* k = row + H * dk + h * dk;
    if (e >= a.rot_dim) { qs[e] = q[e]; ks[e] = k[e] * a.k_scale; continue; }
    if (e >= half) continue;
    float sn, cs;
    sincosf(pos * a.inv_freq[e], &sn, &cs);
    qs[e] = q[e] * cs - q[e + half] * sn;
    qs[e + half] = q[e + half] * cs + q[e] * sn;
    ks[e] = (k[e] * cs - k[e + half] * sn) * a.k_scale;
    ks[e + half] = (k[e + half] * cs + k[e] * sn) * a.k_scale;
  }
  for (int c = tid; c < dv; c += blockDim.x) vs[c] = row[2 * H * dk + h * dv + c];
  __syncthreads();
  const int slot = a.slots[seq];
  float* sp = slot >= 0 ? a.state + (size_t)slot * a.state_stride + (size_t)h * dk * dv : nullptr;
  float v[DVJ], acc[DVJ];
#pragma unroll
  for (int j = 0; j < DVJ; ++j) {
    v[j] = lane + 32 * j < dv ? vs[lane + 32 * j] : 0.f;
    acc[j] = 0.f;
  }
  // four rows of S a pass: all their loads are issued before the first is used
  for (int i0 = w; i0 < dk; i0 += 4 * RT_STEP_WARPS) {
    float S[4][DVJ];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + r * RT_STEP_WARPS;
#pragma unroll
      for (int j = 0; j < DVJ; ++j) {
        const int c = lane + 32 * j;
        S[r][j] = (sp && i < dk && c < dv) ? sp[(size_t)i * dv + c] : 0.f;
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + r * RT_STEP_WARPS;
      if (i >= dk) break;
      const float ki = ks[i], qi = qs[i];
#pragma unroll
      for (int j = 0; j < DVJ; ++j) {
        const int c = lane + 32 * j;
        const float Sn = fmaf(decay, S[r][j], ki * v[j]);
        if (sp && c < dv) sp[(size_t)i * dv + c] = Sn;
        acc[j] = fmaf(Sn, qi, acc[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < DVJ; ++j)
    if (lane + 32 * j < dv) part[w * dv + lane + 32 * j] = acc[j];
  __syncthreads();
  pdl_launch_dependents_if_large();
  // thread c finishes column c (and c + 256, ...): the warps' parts in a fixed order
  float o[(DVJ * 32 + RT_STEP_WARPS * 32 - 1) / (RT_STEP_WARPS * 32)];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < (int)(sizeof(o) / sizeof(float)); ++j) {
    const int c = tid + j * RT_STEP_WARPS * 32;
    o[j] = 0.f;
    if (c < dv) {
      for (int ww = 0; ww < RT_STEP_WARPS; ++ww) o[j] += part[ww * dv + c];
      ss = fmaf(o[j], o[j], ss);
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dv + a.norm_eps);
  const float* g = row + 2 * H * dk + H * dv + h * dv;
  T* y = (T*)a.y + ((size_t)t * H + h) * dv;
#pragma unroll
  for (int j = 0; j < (int)(sizeof(o) / sizeof(float)); ++j) {
    const int c = tid + j * RT_STEP_WARPS * 32;
    if (c < dv) {
      const float gv = g[c];
      y[c] = from_f32<T>(o[j] * inv * (gv / (1.0f + expf(-gv))));
    }
  }
}

template <typename T, int DVJ>
static int retention_step_launch(const RetentionArgs& a, cudaStream_t s) {
  const size_t smem = (size_t)(2 * a.dk + a.dv + RT_STEP_WARPS * a.dv) * sizeof(float);
  return gb_launch(retention_step_kernel<T, DVJ>, dim3(a.H, a.n_seqs), dim3(RT_STEP_WARPS * 32), smem, s, a);
}

template <int KPL>
static int retention_scan_launch(const RetentionArgs& a, cudaStream_t s) {
  return gb_launch(retention_scan_kernel<KPL>, dim3(a.H, a.n_seqs, (a.dv + RT_COLS - 1) / RT_COLS),
                   dim3(RT_COLS * RT_LANES), 0, s, a);
}

static int retention_chunk_launch(const RetentionArgs& a, cudaStream_t s, int chunks) {
  const size_t smem = (size_t)(3 * RT_CT * RT_CT + 2 * RT_TK * RT_CT + RT_CT + 1) * sizeof(float);
  static bool raised = false;    // more than the 48 KB a kernel gets without asking
  if (!raised) {
    cudaError_t ce = cudaFuncSetAttribute(retention_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    raised = true;
  }
  return gb_launch(retention_chunk_kernel, dim3(a.H, a.n_seqs, chunks), dim3(256), smem, s, a);
}

template <typename T>
static int retention_forward(const RetentionArgs& a, cudaStream_t s) {
  if (a.n_tokens < 0 || a.n_seqs < 0 || a.H <= 0 || a.dk <= 0 || a.dv <= 0 || a.rot_dim < 0 ||
      a.rot_dim > a.dk || a.rot_dim % 2 || a.n_seqs > 65535)
    return GB_ERR_BAD_ARG;
  if (!a.proj || !a.decay || !a.token_pos || !a.cu_q || !a.slots || !a.state || !a.qk || !a.o ||
      !a.y || (a.rot_dim && !a.inv_freq))
    return GB_ERR_BAD_ARG;
  if (a.dk > 256) return GB_ERR_UNSUPPORTED;
  if (a.n_tokens == 0 || a.n_seqs == 0) return 0;
  if (a.max_rows == 1 && a.dv <= 256 && a.H <= 65535) {
    if (a.dv <= 32) return retention_step_launch<T, 1>(a, s);
    if (a.dv <= 64) return retention_step_launch<T, 2>(a, s);
    if (a.dv <= 128) return retention_step_launch<T, 4>(a, s);
    return retention_step_launch<T, 8>(a, s);
  }
  int e = gb_launch(retention_rotate_kernel, dim3(a.n_tokens), dim3(256), 0, s, a);
  if (e) return e;
  // a sequence of many rows goes chunk by chunk: every chunk alone from zeros and all at
  // once, then the states at the chunks' starts, then what those add to the read-outs
  int chunks = a.max_rows >= RT_CHUNK_MIN && a.chunk_state ? (a.max_rows + RT_CHUNK - 1) / RT_CHUNK : 0;
  if (chunks > 65535 || (long long)chunks * (RT_CHUNK / RT_TM) * ((a.dv + RT_TN - 1) / RT_TN) > 0x7fffffffLL) chunks = 0;
  const int kpl = (a.dk + RT_LANES - 1) / RT_LANES;
  if (chunks) e = retention_chunk_launch(a, s, chunks);
  else if (kpl <= 1) e = retention_scan_launch<1>(a, s);
  else if (kpl <= 2) e = retention_scan_launch<2>(a, s);
  else if (kpl <= 4) e = retention_scan_launch<4>(a, s);
  else if (kpl <= 8) e = retention_scan_launch<8>(a, s);
  else if (kpl <= 16) e = retention_scan_launch<16>(a, s);
  else e = retention_scan_launch<32>(a, s);
  if (e) return e;
  if (chunks) {
    e = gb_launch(retention_prefix_kernel, dim3((a.dk * a.dv + 255) / 256, a.H, a.n_seqs), dim3(256), 0, s, a);
    if (e) return e;
    e = gb_launch(retention_cross_kernel,
                  dim3(chunks * (RT_CHUNK / RT_TM) * ((a.dv + RT_TN - 1) / RT_TN), a.H, a.n_seqs), dim3(256), 0, s, a);
    if (e) return e;
  }
  const long long warps = (long long)a.n_tokens * a.H;
  return gb_launch(retention_finish_kernel<T>, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, s, a);
}

GB_EXPORT int gb_retention_forward_f32(const RetentionArgs* a, cudaStream_t s) {
  return retention_forward<float>(*a, s);
}
GB_EXPORT int gb_retention_forward_bf16(const RetentionArgs* a, cudaStream_t s) {
  return retention_forward<bf16>(*a, s);
}
