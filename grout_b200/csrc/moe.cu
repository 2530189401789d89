// A feed-forward made of many small experts, of which every token uses a few.
//
//   z = x Wr^T (32-bit);  s = softmax(z) over all router outputs
//   choice score c = s + correction;  the outputs form n_groups equal groups of
//   neighbours, a group's score is its largest c, and only outputs of the
//   keep_groups best groups can be chosen (the others count as -inf);  the `top`
//   outputs with the largest c are chosen and weigh in with their s, as it is
//   expert e < E:   g = min(x Wg_e^T, limit), u = clamp(x Wu_e^T, -limit, limit),
//                   y = (g sigmoid(slope g) (u + 1)) Wd_e^T
//   output >= E:    an expert that hands its input on, y = x
//   out = sum over the chosen of s * y
//
// Each of these terms is an argument.  `score_fn` 1 takes s = sigmoid(z), every output
// by itself, instead of the softmax; `score_fn` 2 lets the logits z choose and takes the
// softmax over the chosen logits alone as the weights; `router_bias` is added to z; `correction` may be null (no correction); a limit
// of +inf clamps nothing; `up_offset` is the 1 in (u + 1) and may be 0; with
// `weigh_input` the weight multiplies the expert's input instead of its result,
// y = expert(s x): gate and up have no bias, so their 32-bit sums are multiplied by s
// before the activation, and the second product is stored as it is.
//
// Nothing here needs the host to know how many tokens an expert got, so a step
// can be captured: `route` chooses and counts, and its last block turns the counts into a
// list of (token, choice) pairs ordered by expert; the two products walk
// tiles of that list; a block finds its expert from the counts, and blocks
// beyond the last tile return.  A pair's row is computed the same way wherever it
// lands in the list, so a token's result does not depend on the batch.  The
// weighted results are left as `top` 32-bit partial sums [top, T, W]
// (choice j of token t in out[j, t, :]), which the norm that follows adds in
// order.
#include "attn_mma.cuh"

struct MoeArgs {
  const void* x;            // [T, W] activations
  const float* router_w;    // [E + n_identity, W]
  const float* correction;  // [E + n_identity]
  const void* w_gate;       // [E, F, W]
  const void* w_up;         // [E, F, W]
  const void* w_down;       // [E, W, F]
  int* ids;                 // [T, top] chosen outputs
  float* wts;               // [T, top] their scores
  int* rank;                // [T, top] place of the pair among its expert's pairs
  int* counts;              // [E + 1] pairs per expert, and the tickets of `route`'s blocks; zero on entry
  int* offsets;             // [E + 1]
  int* perm;                // [T top] pairs (t * top + j) ordered by expert
  void* act;                // [T top, F] activations of the experts' inner layer, in list order
  float* out;               // [top, T, W]
  int T, W, F, E, n_identity, top, n_groups, keep_groups;
  float limit, slope;
  int score_fn;              // 0: softmax over the outputs, 1: sigmoid of each, 2: softmax over the chosen
  int weigh_input;           // the weight multiplies the expert's input, not its result
  float up_offset;           // y = act(g) (u + up_offset)
  const float* router_bias;  // [E + n_identity] added to z, or null
};

#define MOE_MAX_OUTPUTS 1024

#define MOE_ROUTE_THREADS 256
#define MOE_ROUTE_CHUNK 8     // router outputs whose sums a thread carries side by side

template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_THREADS) moe_route_kernel(const MoeArgs a) {
  extern __shared__ float sm[];   // z [n_all], c [n_all]
  __shared__ float part[MOE_ROUTE_THREADS / 32][MOE_ROUTE_CHUNK];
  __shared__ float gbest[MOE_MAX_OUTPUTS];
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nwarps = blockDim.x >> 5;
  const int n_all = a.E + a.n_identity, W = a.W;
  float* z = sm;
  float* c = sm + n_all;
  const T* x = (const T*)a.x + (size_t)t * W;
  // every thread takes a slice of the row against a few router rows at a time, so that
  // all of a slice's loads are under way together; the sums are put together in a fixed
  // order (lanes by the shuffle tree, then warp after warp)
  for (int e0 = 0; e0 < n_all; e0 += MOE_ROUTE_CHUNK) {
    float acc[MOE_ROUTE_CHUNK];
#pragma unroll
    for (int u = 0; u < MOE_ROUTE_CHUNK; ++u) acc[u] = 0.f;
    const int nu = min(MOE_ROUTE_CHUNK, n_all - e0);
#pragma unroll 4
    for (int i = tid; i < W; i += MOE_ROUTE_THREADS) {
      const float xv = to_f32<T>(x[i]);
#pragma unroll
      for (int u = 0; u < MOE_ROUTE_CHUNK; ++u)
        if (u < nu) acc[u] = fmaf(xv, a.router_w[(size_t)(e0 + u) * W + i], acc[u]);
    }
#pragma unroll
    for (int u = 0; u < MOE_ROUTE_CHUNK; ++u) {
      const float v = warp_sum(acc[u]);
      if (lane == 0) part[warp][u] = v;
    }
    __syncthreads();
    if (tid < MOE_ROUTE_CHUNK && e0 + tid < n_all) {
      float v = 0.f;
      for (int w = 0; w < nwarps; ++w) v += part[w][tid];
      z[e0 + tid] = v + (a.router_bias ? a.router_bias[e0 + tid] : 0.f);
    }
    __syncthreads();
  }
  if (tid == 0) {
    float mx = -INFINITY, sum = 0.f;
    if (a.score_fn == 1) {
      for (int e = 0; e < n_all; ++e) z[e] = 1.0f / (1.0f + expf(-z[e]));
    } else if (a.score_fn == 2) {
      // the logits themselves choose; the chosen ones' weights are worked out below
    } else {
      for (int e = 0; e < n_all; ++e) mx = fmaxf(mx, z[e]);
      for (int e = 0; e < n_all; ++e) { z[e] = expf(z[e] - mx); sum += z[e]; }
      for (int e = 0; e < n_all; ++e) z[e] = z[e] / sum;
    }
    for (int e = 0; e < n_all; ++e) c[e] = z[e] + (a.correction ? a.correction[e] : 0.f);
    if (a.n_groups > 1 && a.keep_groups < a.n_groups) {
      const int per = n_all / a.n_groups;
      // drop the groups that are not among the best: n_groups - keep_groups times the worst
      // remaining one (of equal groups the later one goes first)
      float* best = gbest;                       // a group's best choice score; NaN once dropped
      for (int g = 0; g < a.n_groups; ++g) {
        float b = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, c[e]);
        best[g] = b;
      }
      for (int d = 0; d < a.n_groups - a.keep_groups; ++d) {
        int worst = -1;
        float worst_v = INFINITY;
        for (int g = 0; g < a.n_groups; ++g)
          if (!isnan(best[g]) && best[g] <= worst_v) { worst_v = best[g]; worst = g; }
        best[worst] = NAN;
        for (int e = worst * per; e < (worst + 1) * per; ++e) c[e] = -INFINITY;
      }
    }
    for (int j = 0; j < a.top; ++j) {   // the largest first; of equal ones the earlier
      int best = 0;
      float best_v = -INFINITY;
      bool found = false;
      for (int e = 0; e < n_all; ++e)
        if (!isnan(c[e]) && (!found || c[e] > best_v)) { best = e; best_v = c[e]; found = true; }
      c[best] = NAN;                    // taken
      a.ids[(size_t)t * a.top + j] = best;
      a.wts[(size_t)t * a.top + j] = z[best];
    }
    if (a.score_fn == 2) {              // softmax over the chosen logits alone; the first is the largest
      float* w = a.wts + (size_t)t * a.top;
      const float top_z = w[0];
      float sum = 0.f;
      for (int j = 0; j < a.top; ++j) { w[j] = expf(w[j] - top_z); sum += w[j]; }
      for (int j = 0; j < a.top; ++j) w[j] = w[j] / sum;
    }
  }
  __syncthreads();
  for (int j = tid; j < a.top; j += blockDim.x) {   // the choices' places among their experts' pairs
    const int e = a.ids[(size_t)t * a.top + j];
    a.rank[(size_t)t * a.top + j] = e < a.E ? atomicAdd(&a.counts[e], 1) : -1;
  }
  pdl_launch_dependents_if_large();
  for (int j = 0; j < a.top; ++j) {     // experts that hand their input on
    if (a.ids[(size_t)t * a.top + j] < a.E) continue;
    const float w = a.wts[(size_t)t * a.top + j];
    float* o = a.out + ((size_t)j * a.T + t) * W;
    for (int i = tid; i < W; i += blockDim.x) o[i] = w * to_f32<T>(x[i]);
  }
  // The block that finishes last turns the counts into the list of pairs ordered by expert:
  // every block publishes its choices, then draws a ticket (counts[E]); the one that draws
  // the last ticket sees all of them.  It leaves the counts and the ticket at zero for the
  // next call.
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = atomicAdd(&a.counts[a.E], 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (tid == 0) {          // few experts: a serial scan is shorter than its set-up
    int run = 0;
    for (int e = 0; e < a.E; ++e) { a.offsets[e] = run; run += __ldcg(&a.counts[e]); }
    a.offsets[a.E] = run;
  }
  __syncthreads();
  const int n_pairs = a.T * a.top;
  for (int p = tid; p < n_pairs; p += blockDim.x) {
    const int e = __ldcg(&a.ids[p]);
    if (e < a.E) a.perm[a.offsets[e] + __ldcg(&a.rank[p])] = p;
  }
  __syncthreads();
  for (int e = tid; e <= a.E; e += blockDim.x) a.counts[e] = 0;
}

#define MOE_BM 16
#define MOE_BN 64
#define MOE_BK 32

// Which expert and which of its tiles of BM pairs block `b` has; false beyond the last.
template <int BM = MOE_BM>
__device__ __forceinline__ bool moe_find_tile(const int* offsets, int E, int b, int& e_out,
                                              int& first, int& n_rows) {
  int tiles = 0;
  for (int e = 0; e < E; ++e) {
    const int cnt = offsets[e + 1] - offsets[e];
    const int nt = (cnt + BM - 1) / BM;
    if (b < tiles + nt) {
      e_out = e;
      first = offsets[e] + (b - tiles) * BM;
      n_rows = min(BM, offsets[e + 1] - first);
      return true;
    }
    tiles += nt;
  }
  return false;
}

// act[p, f] = fn(x[token(p)] . Wg_e[f], x[token(p)] . Wu_e[f]) for the pairs p of a tile
template <typename T>
__global__ void __launch_bounds__(256) moe_up_kernel(const MoeArgs a) {
  __shared__ float As[MOE_BM][MOE_BK];
  __shared__ float Gs[MOE_BN][MOE_BK + 1];
  __shared__ float Us[MOE_BN][MOE_BK + 1];
  __shared__ int tok[MOE_BM];
  pdl_launch_dependents_if_small();
  pdl_wait();
  int e, first, n_rows;
  if (!moe_find_tile(a.offsets, a.E, blockIdx.x, e, first, n_rows)) return;
  const int tid = threadIdx.x, W = a.W, F = a.F;
  const int f0 = blockIdx.y * MOE_BN;
  if (tid < MOE_BM) tok[tid] = tid < n_rows ? a.perm[first + tid] / a.top : -1;
  __syncthreads();
  const T* wg = (const T*)a.w_gate + (size_t)e * F * W;
  const T* wu = (const T*)a.w_up + (size_t)e * F * W;
  const int tx = tid & 63, ty = tid >> 6;      // column, group of four rows
  float accg[4] = {0.f, 0.f, 0.f, 0.f}, accu[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < W; k0 += MOE_BK) {
    for (int i = tid; i < MOE_BM * MOE_BK; i += 256) {
      const int r = i / MOE_BK, k = i % MOE_BK;
      As[r][k] = (tok[r] >= 0 && k0 + k < W) ? to_f32<T>(((const T*)a.x)[(size_t)tok[r] * W + k0 + k]) : 0.f;
    }
    for (int i = tid; i < MOE_BN * MOE_BK; i += 256) {
      const int n = i / MOE_BK, k = i % MOE_BK;
      const bool ok = f0 + n < F && k0 + k < W;
      Gs[n][k] = ok ? to_f32<T>(wg[(size_t)(f0 + n) * W + k0 + k]) : 0.f;
      Us[n][k] = ok ? to_f32<T>(wu[(size_t)(f0 + n) * W + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_BK; ++k) {
      const float g = Gs[tx][k], u = Us[tx][k];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float x = As[ty * 4 + r][k];
        accg[r] = fmaf(x, g, accg[r]);
        accu[r] = fmaf(x, u, accu[r]);
      }
    }
    __syncthreads();
  }
  pdl_launch_dependents_if_large();
  if (f0 + tx >= F) return;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = ty * 4 + r;
    if (row >= n_rows) continue;
    float g = accg[r], u = accu[r];
    if (a.weigh_input) { const float w = a.wts[a.perm[first + row]]; g *= w; u *= w; }
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    const float y = g / (1.0f + expf(-a.slope * g)) * (u + a.up_offset);
    ((T*)a.act)[(size_t)(first + row) * F + f0 + tx] = from_f32<T>(y);
  }
}

// out[j, t, :] = s * (act[p] . Wd_e^T) for the pairs p = t * top + j of a tile
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(const MoeArgs a) {
  __shared__ float As[MOE_BM][MOE_BK];
  __shared__ float Bs[MOE_BN][MOE_BK + 1];
  __shared__ int pair[MOE_BM];
  pdl_launch_dependents_if_small();
  pdl_wait();
  int e, first, n_rows;
  if (!moe_find_tile(a.offsets, a.E, blockIdx.x, e, first, n_rows)) return;
  const int tid = threadIdx.x, W = a.W, F = a.F;
  const int n0 = blockIdx.y * MOE_BN;
  if (tid < MOE_BM) pair[tid] = tid < n_rows ? a.perm[first + tid] : -1;
  __syncthreads();
  const T* wd = (const T*)a.w_down + (size_t)e * W * F;
  const int tx = tid & 63, ty = tid >> 6;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < F; k0 += MOE_BK) {
    for (int i = tid; i < MOE_BM * MOE_BK; i += 256) {
      const int r = i / MOE_BK, k = i % MOE_BK;
      As[r][k] = (r < n_rows && k0 + k < F) ? to_f32<T>(((const T*)a.act)[(size_t)(first + r) * F + k0 + k]) : 0.f;
    }
    for (int i = tid; i < MOE_BN * MOE_BK; i += 256) {
      const int n = i / MOE_BK, k = i % MOE_BK;
      Bs[n][k] = (n0 + n < W && k0 + k < F) ? to_f32<T>(wd[(size_t)(n0 + n) * F + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_BK; ++k) {
      const float b = Bs[tx][k];
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[r] = fmaf(As[ty * 4 + r][k], b, acc[r]);
    }
    __syncthreads();
  }
  pdl_launch_dependents_if_large();
  if (n0 + tx >= W) return;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = ty * 4 + r;
    if (row >= n_rows) continue;
    const int p = pair[row], t = p / a.top, j = p % a.top;
    a.out[((size_t)j * a.T + t) * W + n0 + tx] = (a.weigh_input ? 1.0f : a.wts[p]) * acc[r];
  }
}


// ---- the two products on the tensor cores (bfloat16, widths that are multiples of 8) ----
// A block of four warps takes a tile of BM pairs and 64 output columns (mma.sync m16n8k16,
// 32-bit sums).  With BM = 128 or 64 (many tokens) the warps are two by two, each with half
// the rows and 32 columns;
// with BM = 16 (a decode step: a handful of pairs per expert, the weights' bytes are the
// cost) the tile is 32 columns wide, so that more blocks stream weights at once, and the
// warps share the 16 rows and take 8 columns each.  Rows of the activations
// (gathered by token for the first product, in list order for the second) and rows of the
// expert's weight reach shared memory by 16-byte asynchronous copies, STAGES chunks of 64
// columns of the inner size in flight; rows and columns beyond the tile's end are filled
// with zeros.  The first product runs gate and up side by side and applies the expert's
// activation to its 32-bit sums; the second multiplies by the pair's weight and stores 32-bit.
#define MT_BN 64
#define MT_BK 64
#define MT_LD (MT_BK + 8)

__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}

template <bool UP, int BM>
struct MoeTile {
  static constexpr int NB = UP ? 2 : 1;
  static constexpr int BN = BM >= 64 ? MT_BN : 32;
  static constexpr int THREADS = 128;
  // a warp's share of the tile: MI pieces of 16 rows by NJ pieces of 8 columns.  Many rows:
  // the four warps are two by two, each with half the rows and 32 columns, so that a
  // fragment read from shared memory feeds several MMAs.  16 rows: the warps share them
  // and take 8 columns each.
  static constexpr int MI = BM >= 64 ? BM / 32 : 1;
  static constexpr int NJ = BM >= 64 ? 4 : 1;
  static constexpr int STAGES = BM >= 64 ? 3 : 4;
  static constexpr int STAGE_ELEMS = (BM + NB * BN) * MT_LD;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_ELEMS * sizeof(bf16);
};

template <bool UP, int BM>
__global__ void __launch_bounds__(128) moe_tc_kernel(const MoeArgs a) {
  using Tile = MoeTile<UP, BM>;
  constexpr int NB = Tile::NB, STAGES = Tile::STAGES, BN = Tile::BN, NT = Tile::THREADS;
  constexpr int MI = Tile::MI, NJ = Tile::NJ;
  extern __shared__ __align__(16) bf16 tiles[];
  __shared__ int src_row[BM];
  pdl_launch_dependents_if_small();
  pdl_wait();
  int e, first, n_rows;
  if (!moe_find_tile<BM>(a.offsets, a.E, blockIdx.x, e, first, n_rows)) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = UP ? a.W : a.F, N = UP ? a.F : a.W;
  const int n0 = blockIdx.y * BN;
  for (int i = tid; i < BM; i += NT) {
    int r = -1;
    if (i < n_rows) r = UP ? a.perm[first + i] / a.top : first + i;
    src_row[i] = r;
  }
  __syncthreads();
  const bf16* A = (const bf16*)(UP ? a.x : a.act);
  const bf16* B0 = (const bf16*)(UP ? a.w_gate : a.w_down) + (size_t)e * N * K;
  const bf16* B1 = UP ? (const bf16*)a.w_up + (size_t)e * N * K : nullptr;
  auto load = [&](int stage, int k0) {
    bf16* As = tiles + stage * Tile::STAGE_ELEMS;
    bf16* Bs = As + BM * MT_LD;
    for (int c = tid; c < BM * 8; c += NT) {             // rows x 8 pieces of 8 elements
      const int r = c >> 3, pc = (c & 7) * 8, kc = k0 + pc;
      const bool ok = src_row[r] >= 0 && kc < K;
      cp_async16(As + r * MT_LD + pc, ok ? A + (size_t)src_row[r] * K + kc : A, ok);
    }
#pragma unroll
    for (int i = 0; i < BN * 8 / NT; ++i) {
      const int c = tid + i * NT, r = c >> 3, pc = (c & 7) * 8, kc = k0 + pc;
      const bool ok = n0 + r < N && kc < K;
      cp_async16(Bs + r * MT_LD + pc, ok ? B0 + (size_t)(n0 + r) * K + kc : B0, ok);
      if (UP) cp_async16(Bs + (BN + r) * MT_LD + pc, ok ? B1 + (size_t)(n0 + r) * K + kc : B1, ok);
    }
  };
  float acc[NB][MI][NJ][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int m = 0; m < MI; ++m)
#pragma unroll
      for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[b][m][j][x] = 0.f;
  const int row_w = BM >= 64 ? (warp >> 1) * (BM / 2) : 0;
  const int col_w = BM >= 64 ? (warp & 1) * 32 : warp * 8;
  const int arow = row_w + (lane & 7) + ((lane >> 3) & 1) * 8, acol = (lane >> 4) * 8;
  // two 8-column pieces at a time (four 8 x 8 blocks), or one (two blocks: lanes 0-15 give the rows)
  const int brow = col_w + (lane & 7) + (NJ > 1 ? (lane >> 4) * 8 : 0), bcol = ((lane >> 3) & 1) * 8;
  const int nk = (K + MT_BK - 1) / MT_BK;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {      // a group per stage, empty beyond the end
    if (st < nk) load(st, st * MT_BK);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<STAGES - 2>();                  // chunk kt has landed
    __syncthreads();                              // ... for every thread; chunk kt - 1 is done with
    if (kt + STAGES - 1 < nk) load((kt + STAGES - 1) % STAGES, (kt + STAGES - 1) * MT_BK);
    cp_async_commit();
    const bf16* As = tiles + (kt % STAGES) * Tile::STAGE_ELEMS;
    const bf16* Bs = As + BM * MT_LD;
#pragma unroll
    for (int k = 0; k < MT_BK / 16; ++k) {
      uint32_t af[MI][4];
#pragma unroll
      for (int m = 0; m < MI; ++m) ldmatrix_x4(af[m], As + (arow + m * 16) * MT_LD + k * 16 + acol);
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        if (NJ == 1) {
          uint32_t bf[2];
          ldmatrix_x2(bf, Bs + (b * BN + brow) * MT_LD + k * 16 + bcol);
#pragma unroll
          for (int m = 0; m < MI; ++m) mma_16816(acc[b][m][0], af[m], bf[0], bf[1]);
        } else {
#pragma unroll
          for (int j = 0; j + 1 < NJ; j += 2) {
            uint32_t bf[4];
            ldmatrix_x4(bf, Bs + (b * BN + j * 8 + brow) * MT_LD + k * 16 + bcol);
#pragma unroll
            for (int m = 0; m < MI; ++m) {
              mma_16816(acc[b][m][j], af[m], bf[0], bf[1]);
              mma_16816(acc[b][m][j + 1], af[m], bf[2], bf[3]);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  pdl_launch_dependents_if_large();
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int m = 0; m < MI; ++m)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = row_w + m * 16 + g + half * 8;
      if (row >= n_rows) continue;
      if (UP) {
        bf16* dst = (bf16*)a.act + (size_t)(first + row) * N;
        const float wi = a.weigh_input ? a.wts[a.perm[first + row]] : 1.0f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const int col = n0 + col_w + j * 8 + t * 2;
          float y[2];
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const float gt = fminf(wi * acc[0][m][j][half * 2 + x], a.limit);
            const float up = fminf(fmaxf(wi * acc[NB - 1][m][j][half * 2 + x], -a.limit), a.limit);
            y[x] = gt / (1.0f + expf(-a.slope * gt)) * (up + a.up_offset);
          }
          if (col + 1 < N) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(y[0], y[1]);
          else if (col < N) dst[col] = from_f32<bf16>(y[0]);
        }
      } else {
        const int p = a.perm[first + row], tok = p / a.top, jc = p % a.top;
        const float w = a.weigh_input ? 1.0f : a.wts[p];
        float* dst = a.out + ((size_t)jc * a.T + tok) * N;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const int col = n0 + col_w + j * 8 + t * 2;
          if (col + 1 < N)
            *reinterpret_cast<float2*>(dst + col) = make_float2(w * acc[0][m][j][half * 2], w * acc[0][m][j][half * 2 + 1]);
          else if (col < N) dst[col] = w * acc[0][m][j][half * 2];
        }
      }
    }
}

template <bool UP, int BM>
static int moe_tc_launch(const MoeArgs& a, long long pairs, cudaStream_t s) {
  const long long tiles = pairs / BM + (pairs < a.E ? pairs : a.E);
  if (tiles > 0x7fffffffLL) return GB_ERR_UNSUPPORTED;
  const size_t smem = MoeTile<UP, BM>::SMEM;
  cudaError_t ce = cudaFuncSetAttribute(moe_tc_kernel<UP, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (ce != cudaSuccess) return (int)ce;
  const int N = UP ? a.F : a.W, BN = MoeTile<UP, BM>::BN;
  return gb_launch(moe_tc_kernel<UP, BM>, dim3((unsigned)tiles, (N + BN - 1) / BN),
                   dim3(MoeTile<UP, BM>::THREADS), smem, s, a);
}

static int moe_check(const MoeArgs& a) {
  if (a.T < 0 || a.W <= 0 || a.F <= 0 || a.E <= 0 || a.n_identity < 0 || a.top <= 0 ||
      a.n_groups <= 0 || a.keep_groups <= 0 || a.keep_groups > a.n_groups)
    return GB_ERR_BAD_ARG;
  const int n_all = a.E + a.n_identity;
  if (n_all % a.n_groups || a.top > n_all) return GB_ERR_BAD_ARG;
  if (n_all > MOE_MAX_OUTPUTS) return GB_ERR_UNSUPPORTED;
  if (a.score_fn < 0 || a.score_fn > 2) return GB_ERR_BAD_ARG;
  if (!a.x || !a.router_w || !a.w_gate || !a.w_up || !a.w_down || !a.ids || !a.wts ||
      !a.rank || !a.counts || !a.offsets || !a.perm || !a.act || !a.out)
    return GB_ERR_BAD_ARG;
  return 0;
}

template <typename T>
static int moe_forward(const MoeArgs& a, cudaStream_t s) {
  int e = moe_check(a);
  if (e) return e;
  if (a.T == 0) return 0;
  const int n_all = a.E + a.n_identity;
  e = gb_launch(moe_route_kernel<T>, dim3(a.T), dim3(MOE_ROUTE_THREADS), (size_t)2 * n_all * sizeof(float), s, a);
  if (e) return e;
  // the most tiles the pairs can make: every expert may end in a tile that is not full
  const long long pairs = (long long)a.T * a.top;
  if (sizeof(T) == 2 && a.W % 8 == 0 && a.F % 8 == 0 &&
      ((((uintptr_t)a.x) | ((uintptr_t)a.act) | ((uintptr_t)a.w_gate) | ((uintptr_t)a.w_up) |
        ((uintptr_t)a.w_down) | ((uintptr_t)a.out)) & 15) == 0) {
    // few pairs per expert (a decode step): narrow tiles, deeper pipeline
    if (pairs <= 4LL * a.E) {
      e = moe_tc_launch<true, 16>(a, pairs, s);
      if (e) return e;
      return moe_tc_launch<false, 16>(a, pairs, s);
    }
    if (pairs >= 64LL * a.E) {      // 64 pairs an expert and more: tiles of 128 rows
      e = moe_tc_launch<true, 128>(a, pairs, s);
      if (e) return e;
      return moe_tc_launch<false, 128>(a, pairs, s);
    }
    e = moe_tc_launch<true, 64>(a, pairs, s);
    if (e) return e;
    return moe_tc_launch<false, 64>(a, pairs, s);
  }
  const long long tiles = pairs / MOE_BM + (pairs < a.E ? pairs : a.E);
  if (tiles > 0x7fffffffLL) return GB_ERR_UNSUPPORTED;
  e = gb_launch(moe_up_kernel<T>, dim3((unsigned)tiles, (a.F + MOE_BN - 1) / MOE_BN), dim3(256), 0, s, a);
  if (e) return e;
  return gb_launch(moe_down_kernel<T>, dim3((unsigned)tiles, (a.W + MOE_BN - 1) / MOE_BN), dim3(256), 0, s, a);
}

// Three launches: route (with the ordering of the pairs), the experts' first products with
// their activation, their second products with the weights.
GB_EXPORT int gb_moe_forward_f32(const MoeArgs* a, cudaStream_t s) { return moe_forward<float>(*a, s); }
GB_EXPORT int gb_moe_forward_bf16(const MoeArgs* a, cudaStream_t s) { return moe_forward<bf16>(*a, s); }
