// A feed-forward of routed experts: every token goes through `top` of E small gated feed-forwards.
//
//   1. sb_moe_route: from float router logits [T, E], the `top` largest scores of every token (sigmoid or softmax
//      scores; lowest index on ties) and their weights, as float.
//   2. sb_moe_sort: the (token, choice) pairs grouped by expert: offsets[E + 1] and the pairs in that order, plus
//      the list of row tiles (expert, first row) the products run over. Which place a pair gets inside its
//      expert's group depends on timing, but nothing computed from it does: a pair's result is a function of its
//      own row alone.
//   3. sb_moe_gate_up: act[row] = f( w * (x W_gate^T), w * (x W_up^T) ) for the rows of every tile, x the pair's
//      token. The weight multiplies the expert's input; a product is linear, so it is applied to the float sums.
//   4. sb_moe_down: out[pair] = act[row] W_down^T, written at the pair's own place; with top == 1 that is the result,
//      otherwise sb_moe_combine adds a token's `top` rows in order.
// Experts without a gate (sb_moe_up: act[row] = f(x W_up^T), f = relu squared) and a choice that is read from a table
// over token ids instead of router logits (sb_moe_route_table) go through the same grouping and the same down product.
// Products accumulate in float over k in ascending order, whatever else is in the step.
#include "common.cuh"

using namespace sb;

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

constexpr int ROUTE_MAX_TOP = 16;

// A warp per token: lane l holds the logits of experts l, l + 32, ... (at most ROUTE_PER_LANE of them); the best of
// what is left is found `top` times by a shuffle tree over (logit, index), lower index first on equal logits.
constexpr int ROUTE_PER_LANE = 32;      // so at most 1024 experts

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int E, int top, int score_kind, int renorm,
                                                        int n_tokens, int* __restrict__ idx, float* __restrict__ wts) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * E;
  float mine[ROUTE_PER_LANE];
  float zmax = -INFINITY;
#pragma unroll
  for (int u = 0; u < ROUTE_PER_LANE; ++u) {
    const int e = lane + 32 * u;
    mine[u] = e < E ? z[e] : -INFINITY;
    zmax = fmaxf(zmax, mine[u]);
  }
  float denom = 1.f;
  if (score_kind == 1) {                        // softmax over all experts
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
    float part = 0.f;
#pragma unroll
    for (int u = 0; u < ROUTE_PER_LANE; ++u)
      if (lane + 32 * u < E) part += expf(mine[u] - zmax);
    denom = warp_sum(part);
  }
  float val = 0.f, total = 0.f;                 // lane s keeps the s-th choice
  int chosen = -1;
  for (int s = 0; s < top; ++s) {
    float m = -INFINITY;
    int arg = 0x7fffffff;
#pragma unroll
    for (int u = 0; u < ROUTE_PER_LANE; ++u) {
      const int e = lane + 32 * u;
      if (e < E && (mine[u] > m || (mine[u] == m && e < arg)) && mine[u] != -INFINITY) { m = mine[u]; arg = e; }
    }
    if (arg == 0x7fffffff) {                     // nothing left in this lane (or only minus infinity): offer its first free slot last
      m = -INFINITY;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (om > m || (om == m && oa < arg)) { m = om; arg = oa; }
    }
    if (arg != 0x7fffffff && (arg & 31) == lane) {
#pragma unroll
      for (int u = 0; u < ROUTE_PER_LANE; ++u)
        if (u == (arg >> 5)) mine[u] = -INFINITY;    // taken
    }
    const float v = score_kind == 1 ? expf(m - zmax) / denom : sigmoid_f(m);
    total += v;
    if (lane == s) { val = v; chosen = arg == 0x7fffffff ? 0 : arg; }
  }
  if (lane < top) {
    idx[(size_t)t * top + lane] = chosen;
    wts[(size_t)t * top + lane] = renorm ? val / total : val;
  }
}

// As moe_route_kernel, for a router with a bias on the choice: the scores (softmax over the first E of a row's ``stride``
// logits, or sigmoid) choose through score + bias[e], lowest index first on ties, while the weights are the scores
// themselves, divided by (their sum + sum_eps) if asked. A lane holds PER_LANE outputs (E <= 32 * PER_LANE): few for the
// usual counts, so the loops over them are short. E counts every output the router scores; an index at or beyond
// the number of real experts means "the token itself" to the kernels after this one.
template <int PER_LANE>
__global__ void __launch_bounds__(128) moe_route_bias_kernel(const float* __restrict__ logits, int stride, int E, int top, int score_kind,
                                                             int renorm, float sum_eps, const float* __restrict__ bias, int n_tokens,
                                                             int* __restrict__ idx, float* __restrict__ wts, float weight_scale) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * stride;
  float score[PER_LANE], pick[PER_LANE];
  float zmax = -INFINITY;
#pragma unroll
  for (int u = 0; u < PER_LANE; ++u) {
    const int e = lane + 32 * u;
    score[u] = e < E ? z[e] : -INFINITY;
    zmax = fmaxf(zmax, score[u]);
  }
  if (score_kind == 1) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
    float part = 0.f;
#pragma unroll
    for (int u = 0; u < PER_LANE; ++u)
      if (lane + 32 * u < E) { score[u] = expf(score[u] - zmax); part += score[u]; }
    const float denom = warp_sum(part);
#pragma unroll
    for (int u = 0; u < PER_LANE; ++u)
      if (lane + 32 * u < E) score[u] /= denom;
  } else {
#pragma unroll
    for (int u = 0; u < PER_LANE; ++u)
      if (lane + 32 * u < E) score[u] = sigmoid_f(score[u]);
  }
#pragma unroll
  for (int u = 0; u < PER_LANE; ++u) {
    const int e = lane + 32 * u;
    pick[u] = e < E ? score[u] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float val = 0.f, total = 0.f;                 // lane s keeps the s-th choice
  int chosen = 0;
  for (int s = 0; s < top; ++s) {
    float m = -INFINITY, sc = 0.f;
    int arg = 0x7fffffff;
#pragma unroll
    for (int u = 0; u < PER_LANE; ++u) {
      const int e = lane + 32 * u;
      if (e < E && pick[u] != -INFINITY && (pick[u] > m || (pick[u] == m && e < arg))) { m = pick[u]; arg = e; sc = score[u]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      const float os = __shfl_xor_sync(0xffffffffu, sc, o);
      if (om > m || (om == m && oa < arg)) { m = om; arg = oa; sc = os; }
    }
    if (arg != 0x7fffffff && (arg & 31) == lane) {
#pragma unroll
      for (int u = 0; u < PER_LANE; ++u)
        if (u == (arg >> 5)) pick[u] = -INFINITY;    // taken
    }
    total += sc;
    if (lane == s) { val = sc; chosen = arg == 0x7fffffff ? 0 : arg; }
  }
  if (lane < top) {
    idx[(size_t)t * top + lane] = chosen;
    wts[(size_t)t * top + lane] = (renorm ? val / (total + sum_eps) : val) * weight_scale;
  }
}

constexpr int TM = 32;            // rows of a tile of the plain-arithmetic products (the tensor-core ones take MB_M)

// One block. order[offsets[e] .. offsets[e+1]) = the pairs of expert e; tiles: (expert, first row) for every TM rows
// of an expert's group, n_tiles[0] of them.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int E, int tile_rows,
                                                        int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ tiles,
                                                        int* __restrict__ n_tiles) {
  extern __shared__ int sh[];
  int* count = sh;            // [E]
  int* start = sh + E;        // [E + 1]
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      offsets[e] = at;
      for (int r0 = 0; r0 < count[e]; r0 += tile_rows) {
        tiles[2 * nt] = e;
        tiles[2 * nt + 1] = at + r0;
        ++nt;
      }
      at += count[e];
    }
    start[E] = at;
    offsets[E] = at;
    n_tiles[0] = nt;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < E) order[start[e] + atomicAdd(&count[e], 1)] = p;
  }
}

// The experts of a token from a table over token ids: idx[t, j] = table[token[t], j], every weight 1 / top. A token id
// below zero, -(s + 1), stands for the token last sampled for state slot s (as in the embedding kernel).
__global__ void __launch_bounds__(256) moe_route_table_kernel(const int* __restrict__ tokens, const int* __restrict__ last_token,
                                                              int n_slots, const int* __restrict__ table, int vocab, int E, int top,
                                                              int n_tokens, int* __restrict__ idx, float* __restrict__ wts,
                                                              int* __restrict__ errors) {
  const int w = blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= n_tokens * top) return;
  const int t = w / top, j = w - t * top;
  int tok = tokens[t];
  if (tok < 0 && last_token != nullptr && -tok - 1 < n_slots) tok = last_token[-tok - 1];
  int e = (tok >= 0 && tok < vocab) ? table[(size_t)tok * top + j] : -1;
  if (e < 0 || e >= E) {
    atomicAdd(errors, 1);        // a token outside the table or an entry outside the experts: counted, expert 0 stands in
    e = 0;
  }
  idx[w] = e;
  wts[w] = 1.0f / (float)top;
}

constexpr int TK = 32;
constexpr int GU_COLS = 32;       // gate columns of a tile (and as many up columns)
constexpr int DN_COLS = 64;
constexpr int MOE_THREADS = 256;

// grid (column tiles of ff, row tiles). x [T, K] with row stride; w_gu [E, 2 ff, K] (gate rows, then up rows).
// act kinds: 0 = silu(g) * u; 1 = the clamped form: g <- min(g, limit), u <- clamp(u, -limit, limit), g * sigmoid(alpha g) * (u + 1);
// 2 = no gate: w_gu is [E, ff, K] and the output is relu(x W^T)^2.
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS) moe_gate_up_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ w_gu,
                                                                  const int* __restrict__ order, const int* __restrict__ offsets,
                                                                  const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                                  const float* __restrict__ wts, int top, int K, int ff, int scale_input,
                                                                  int act_kind, float limit, float alpha, T* __restrict__ act) {
  if ((int)blockIdx.y >= n_tiles[0]) return;
  __shared__ float As[TK][TM + 1];
  __shared__ float Bg[TK][GU_COLS + 1];
  __shared__ float Bu[TK][GU_COLS + 1];
  __shared__ int tok[TM];
  __shared__ float rw[TM];
  const int e = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
  const int rows = min(TM, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * GU_COLS;
  const int tid = threadIdx.x;
  if (tid < TM) {
    const int pair = tid < rows ? order[row0 + tid] : -1;
    tok[tid] = pair >= 0 ? pair / top : -1;
    rw[tid] = pair >= 0 ? wts[pair] : 0.f;
  }
  __syncthreads();
  const bool gated = act_kind != 2;
  const T* wg = w_gu + (size_t)e * (gated ? 2 : 1) * ff * K;
  const T* wu = wg + (size_t)ff * K;
  const int ty = tid >> 4, tx = tid & 15;               // rows 2 ty, 2 ty + 1; columns 2 tx, 2 tx + 1
  float ag[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, au[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int w = tid; w < TM * TK; w += MOE_THREADS) {
      const int m = w / TK, kk = w - m * TK;
      const int tk = tok[m];
      As[kk][m] = (tk >= 0 && k0 + kk < K) ? to_float(x[(size_t)tk * x_stride + k0 + kk]) : 0.f;
    }
    for (int w = tid; w < GU_COLS * TK; w += MOE_THREADS) {
      const int nn = w / TK, kk = w - nn * TK;
      const bool ok = n0 + nn < ff && k0 + kk < K;
      Bg[kk][nn] = ok ? to_float(wg[(size_t)(n0 + nn) * K + k0 + kk]) : 0.f;
      Bu[kk][nn] = (ok && gated) ? to_float(wu[(size_t)(n0 + nn) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = As[kk][2 * ty], a1 = As[kk][2 * ty + 1];
      const float g0 = Bg[kk][2 * tx], g1 = Bg[kk][2 * tx + 1], u0 = Bu[kk][2 * tx], u1 = Bu[kk][2 * tx + 1];
      ag[0][0] += a0 * g0; ag[0][1] += a0 * g1; ag[1][0] += a1 * g0; ag[1][1] += a1 * g1;
      au[0][0] += a0 * u0; au[0][1] += a0 * u1; au[1][0] += a1 * u0; au[1][1] += a1 * u1;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = 2 * ty + i;
    if (m >= rows) continue;
    const float sc = scale_input ? rw[m] : 1.f;
#pragma unroll
    for (int jx = 0; jx < 2; ++jx) {
      const int nn = n0 + 2 * tx + jx;
      if (nn >= ff) continue;
      float g = ag[i][jx] * sc, u = au[i][jx] * sc, yv;
      if (act_kind == 2) {
        g = fmaxf(g, 0.f);
        yv = g * g;
      } else if (act_kind == 1) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        yv = g * sigmoid_f(alpha * g) * (u + 1.f);
      } else {
        yv = g * sigmoid_f(g) * u;
      }
      act[(size_t)(row0 + m) * ff + nn] = from_float<T>(yv);
    }
  }
}

// grid (column tiles of N, row tiles). act [rows, ff]; w_down [E, N, ff]; out [pairs, N] at the pair's own place, each
// row times its weight unless the weight already went into the input.
template <typename T, typename O>
__global__ void __launch_bounds__(MOE_THREADS) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down,
                                                               const int* __restrict__ order, const int* __restrict__ offsets,
                                                               const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                               const float* __restrict__ wts, int ff, int N, int scale_output,
                                                               O* __restrict__ out) {
  if ((int)blockIdx.y >= n_tiles[0]) return;
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][DN_COLS + 1];
  __shared__ int pair_of[TM];
  const int e = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
  const int rows = min(TM, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * DN_COLS;
  const int tid = threadIdx.x;
  if (tid < TM) pair_of[tid] = tid < rows ? order[row0 + tid] : -1;
  __syncthreads();
  const T* w = w_down + (size_t)e * N * ff;
  const int ty = tid >> 4, tx = tid & 15;               // rows 2 ty, 2 ty + 1; columns tx, tx + 16, tx + 32, tx + 48
  float acc[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int jx = 0; jx < 4; ++jx) acc[i][jx] = 0.f;
  for (int k0 = 0; k0 < ff; k0 += TK) {
    for (int v = tid; v < TM * TK; v += MOE_THREADS) {
      const int m = v / TK, kk = v - m * TK;
      As[kk][m] = (m < rows && k0 + kk < ff) ? to_float(act[(size_t)(row0 + m) * ff + k0 + kk]) : 0.f;
    }
    for (int v = tid; v < DN_COLS * TK; v += MOE_THREADS) {
      const int nn = v / TK, kk = v - nn * TK;
      Bs[kk][nn] = (n0 + nn < N && k0 + kk < ff) ? to_float(w[(size_t)(n0 + nn) * ff + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = As[kk][2 * ty], a1 = As[kk][2 * ty + 1];
#pragma unroll
      for (int jx = 0; jx < 4; ++jx) {
        const float b = Bs[kk][tx + 16 * jx];
        acc[0][jx] += a0 * b;
        acc[1][jx] += a1 * b;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = 2 * ty + i;
    if (m >= rows) continue;
    const int pair = pair_of[m];
    const float sc = scale_output ? wts[pair] : 1.f;
#pragma unroll
    for (int jx = 0; jx < 4; ++jx) {
      const int nn = n0 + tx + 16 * jx;
      if (nn < N) out[(size_t)pair * N + nn] = from_float<O>(acc[i][jx] * sc);
    }
  }
}


// ------------------------------------------------------------------------------------------ bfloat16 on tensor cores
// The same two products with mma.sync m16n8k16 (bfloat16 in, float accumulators): tiles of MB_M rows x 64 columns,
// k in steps of 32 through a three-stage cp.async ring, four warps as 2 x 2, each 32 rows x 32 columns. Rows of the
// shared tiles are 80 bytes apart, so the eight 16-byte rows an ldmatrix reads fall into different banks. For
// gate/up a block's 64 columns are 32 gate columns and the 32 up columns of the same outputs, and a warp takes 16 of
// each, so a thread holds the gate and the up sum of the same output and applies the activation itself.
constexpr int MB_M = 64, MB_N = 64, MB_K = 32, MB_STAGES = 3, MB_LD = MB_K + 8, MB_THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;                       // 0: nothing is read, the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One k-loop for both products. a_row(m): global pointer of row m of the A tile at k = 0 (null: a row of zeros);
// b_row(n): the same for row n of the B tile (a weight row); any_global: an address in global memory for the copies that
// read nothing. acc[i][j]: rows wm * 32 + i * 16 (+8), columns wn * 32 + j * 8.
template <typename ARow, typename BRow>
__device__ __forceinline__ void mma_tile_loop(ARow a_row, BRow b_row, const __nv_bfloat16* any_global, int K, __nv_bfloat16* smem,
                                              float (&acc)[2][4][4]) {
  typedef __nv_bfloat16 B;
  B* As = smem;                                     // [stages][MB_M][MB_LD]
  B* Bs = smem + MB_STAGES * MB_M * MB_LD;          // [stages][MB_N][MB_LD]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;
  // this thread's two 16-byte pieces of each tile: rows r0 and r0 + 32, piece (tid & 3) of the row's four
  const int r0 = tid >> 2, piece = (tid & 3) * 8;
  const B* a_src[2] = {a_row(r0), a_row(r0 + 32)};
  const B* b_src[2] = {b_row(r0), b_row(r0 + 32)};
  auto load = [&](int stage, int k0) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int row = r0 + 32 * u;
      cp_async16(As + ((size_t)stage * MB_M + row) * MB_LD + piece, a_src[u] ? a_src[u] + k0 + piece : any_global, a_src[u] != nullptr);
      cp_async16(Bs + ((size_t)stage * MB_N + row) * MB_LD + piece, b_src[u] ? b_src[u] + k0 + piece : any_global, b_src[u] != nullptr);
    }
  };
  const int nk = K / MB_K;
#pragma unroll
  for (int s = 0; s < MB_STAGES - 1; ++s) {
    if (s < nk) load(s, s * MB_K);
    cp_async_commit();
  }
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<MB_STAGES - 2>();
    __syncthreads();                                 // tile kt is there, and every warp is done with tile kt - 1
    const int nxt = kt + MB_STAGES - 1;
    if (nxt < nk) load(nxt % MB_STAGES, nxt * MB_K);
    cp_async_commit();
    const B* at = As + (size_t)(kt % MB_STAGES) * MB_M * MB_LD;
    const B* bt = Bs + (size_t)(kt % MB_STAGES) * MB_N * MB_LD;
#pragma unroll
    for (int kk = 0; kk < MB_K; kk += 16) {
      unsigned af[2][4], bf[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)      // 16 x 16 of A: lanes 0-15 rows 0-15 at k, lanes 16-31 the same rows at k + 8
        ldmatrix_x4(af[i], at + (size_t)(wm * 32 + i * 16 + (lane & 15)) * MB_LD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < 2; ++j)      // 16 columns x 16 of k: matrices (n 0-7, k), (n 0-7, k + 8), (n 8-15, k), (n 8-15, k + 8)
        ldmatrix_x4(bf[j], bt + (size_t)(wn * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3)) * MB_LD + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
    }
  }
  cp_async_wait<0>();
}

constexpr size_t MB_SMEM = (size_t)MB_STAGES * (MB_M + MB_N) * MB_LD * sizeof(__nv_bfloat16);

// grid (ceil(ff / 32), row tiles of MB_M rows). Tile rows of the B tile: warp column wn takes rows wn * 32 .. + 31 =
// 16 gate rows (outputs n0 + wn * 16 ..) and then the 16 up rows of the same outputs.
__global__ void __launch_bounds__(MB_THREADS) moe_gate_up_mma_kernel(
    const __nv_bfloat16* __restrict__ x, int x_stride, const __nv_bfloat16* __restrict__ w_gu, const int* __restrict__ order,
    const int* __restrict__ offsets, const int* __restrict__ tiles, const int* __restrict__ n_tiles, const float* __restrict__ wts,
    int top, int K, int ff, int scale_input, int act_kind, float limit, float alpha, __nv_bfloat16* __restrict__ act) {
  if ((int)blockIdx.y >= n_tiles[0]) return;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* smem = (__nv_bfloat16*)raw;
  __shared__ int tok[MB_M];
  __shared__ float rw[MB_M];
  const int e = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
  const int rows = min(MB_M, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * 32;
  const int tid = threadIdx.x;
  if (tid < MB_M) {
    const int pair = tid < rows ? order[row0 + tid] : -1;
    tok[tid] = pair >= 0 ? pair / top : -1;
    rw[tid] = pair >= 0 ? wts[pair] : 0.f;
  }
  __syncthreads();
  const __nv_bfloat16* wg = w_gu + (size_t)e * 2 * ff * K;
  float acc[2][4][4] = {};
  mma_tile_loop(
      [&](int m) -> const __nv_bfloat16* { return tok[m] >= 0 ? x + (size_t)tok[m] * x_stride : nullptr; },
      [&](int n) -> const __nv_bfloat16* {
        const int wn = n >> 5, within = n & 31;
        const int col = n0 + wn * 16 + (within & 15);
        if (col >= ff) return nullptr;
        return wg + ((size_t)(within >> 4) * ff + col) * K;           // within >= 16: the up row of that output
      },
      wg, K, smem, acc);
  const int lane = tid & 31, warp = tid >> 5, wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = wm * 32 + i * 16 + (lane >> 2) + half * 8;
      if (m >= rows) continue;
      const float sc = scale_input ? rw[m] : 1.f;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = n0 + wn * 16 + j * 8 + (lane & 3) * 2 + c;
          if (col >= ff) continue;
          float g = acc[i][j][half * 2 + c] * sc, u = acc[i][j + 2][half * 2 + c] * sc, yv;
          if (act_kind == 1) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            yv = g * sigmoid_f(alpha * g) * (u + 1.f);
          } else {
            yv = g * sigmoid_f(g) * u;
          }
          act[(size_t)(row0 + m) * ff + col] = __float2bfloat16_rn(yv);
        }
    }
}

// The product without a gate: grid (ceil(ff / 64), row tiles of MB_M rows); w_up [E, ff, K]; act = relu(x W^T)^2.
__global__ void __launch_bounds__(MB_THREADS) moe_up_mma_kernel(
    const __nv_bfloat16* __restrict__ x, int x_stride, const __nv_bfloat16* __restrict__ w_up, const int* __restrict__ order,
    const int* __restrict__ offsets, const int* __restrict__ tiles, const int* __restrict__ n_tiles, int top, int K, int ff,
    __nv_bfloat16* __restrict__ act) {
  if ((int)blockIdx.y >= n_tiles[0]) return;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* smem = (__nv_bfloat16*)raw;
  __shared__ int tok[MB_M];
  const int e = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
  const int rows = min(MB_M, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * MB_N;
  const int tid = threadIdx.x;
  if (tid < MB_M) {
    const int pair = tid < rows ? order[row0 + tid] : -1;
    tok[tid] = pair >= 0 ? pair / top : -1;
  }
  __syncthreads();
  const __nv_bfloat16* w = w_up + (size_t)e * ff * K;
  float acc[2][4][4] = {};
  mma_tile_loop([&](int m) -> const __nv_bfloat16* { return tok[m] >= 0 ? x + (size_t)tok[m] * x_stride : nullptr; },
                [&](int n) -> const __nv_bfloat16* { return n0 + n < ff ? w + (size_t)(n0 + n) * K : nullptr; }, w, K, smem, acc);
  const int lane = tid & 31, warp = tid >> 5, wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = wm * 32 + i * 16 + (lane >> 2) + half * 8;
      if (m >= rows) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = n0 + wn * 32 + j * 8 + (lane & 3) * 2 + c;
          if (col >= ff) continue;
          const float g = fmaxf(acc[i][j][half * 2 + c], 0.f);
          act[(size_t)(row0 + m) * ff + col] = __float2bfloat16_rn(g * g);
        }
    }
}

// grid (ceil(N / 64), row tiles).
template <typename O>
__global__ void __launch_bounds__(MB_THREADS) moe_down_mma_kernel(const __nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ w_down,
                                                                  const int* __restrict__ order, const int* __restrict__ offsets,
                                                                  const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                                  const float* __restrict__ wts, int ff, int N, int scale_output,
                                                                  O* __restrict__ out) {
  if ((int)blockIdx.y >= n_tiles[0]) return;
  extern __shared__ __align__(16) unsigned char raw[];
  __nv_bfloat16* smem = (__nv_bfloat16*)raw;
  __shared__ int pair_of[MB_M];
  const int e = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
  const int rows = min(MB_M, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * MB_N;
  const int tid = threadIdx.x;
  if (tid < MB_M) pair_of[tid] = tid < rows ? order[row0 + tid] : -1;
  __syncthreads();
  const __nv_bfloat16* w = w_down + (size_t)e * N * ff;
  float acc[2][4][4] = {};
  mma_tile_loop([&](int m) -> const __nv_bfloat16* { return m < rows ? act + (size_t)(row0 + m) * ff : nullptr; },
                [&](int n) -> const __nv_bfloat16* { return n0 + n < N ? w + (size_t)(n0 + n) * ff : nullptr; }, w, ff, smem, acc);
  const int lane = tid & 31, warp = tid >> 5, wm = warp >> 1, wn = warp & 1;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = wm * 32 + i * 16 + (lane >> 2) + half * 8;
      if (m >= rows) continue;
      const int pair = pair_of[m];
      const float sc = scale_output ? wts[pair] : 1.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = n0 + wn * 32 + j * 8 + (lane & 3) * 2 + c;
          if (col < N) out[(size_t)pair * N + col] = from_float<O>(acc[i][j][half * 2 + c] * sc);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ parts, int top, int N, long long total,
                                                          T* __restrict__ out) {
  for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
    const long long t = w / N;
    const int c = (int)(w - t * N);
    float s = 0.f;
    for (int k = 0; k < top; ++k) s += parts[((size_t)t * top + k) * N + c];
    out[w] = from_float<T>(s);
  }
}


// The sum over a token's choices when some of them are not experts, plus what every token gets:
//   out[t] = sum_k ( idx[t, k] < E_real ? parts[t * top + k] : wts[t * top + k] * x[t] )  +  g_t * shared[t]
// with g_t = sigmoid(gate[t * gate_stride]) if a gate is given, else 1; shared may be null.
template <typename T> __device__ __forceinline__ float4 moe_load4(const T* p);
template <> __device__ __forceinline__ float4 moe_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 moe_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void moe_store4(T* p, float4 v);
template <> __device__ __forceinline__ void moe_store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void moe_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// VEC elements a thread (4: N and x_stride multiples of 4, every pointer 16-byte aligned; else 1).
template <typename T, int VEC>
__global__ void __launch_bounds__(256) moe_combine_more_kernel(const float* __restrict__ parts, const int* __restrict__ idx,
                                                               const float* __restrict__ wts, int E_real, const T* __restrict__ x,
                                                               int x_stride, const T* __restrict__ shared, const float* __restrict__ gate,
                                                               int gate_stride, int top, int N, long long total, T* __restrict__ out) {
  const int nv = N / VEC;
  for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(w / nv);
    const int c = (int)(w - (long long)t * nv) * VEC;
    float s[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) s[v] = 0.f;
    for (int k = 0; k < top; ++k) {
      const size_t pair = (size_t)t * top + k;
      if (idx[pair] < E_real) {
        if (VEC == 4) {
          const float4 p4 = *reinterpret_cast<const float4*>(parts + pair * N + c);
          s[0] += p4.x; s[1 % VEC] += p4.y; s[2 % VEC] += p4.z; s[3 % VEC] += p4.w;
        } else {
          s[0] += parts[pair * N + c];
        }
      } else {
        const float wt = wts[pair];
        if (VEC == 4) {
          const float4 x4 = moe_load4<T>(x + (size_t)t * x_stride + c);
          s[0] += wt * x4.x; s[1 % VEC] += wt * x4.y; s[2 % VEC] += wt * x4.z; s[3 % VEC] += wt * x4.w;
        } else {
          s[0] += wt * to_float(x[(size_t)t * x_stride + c]);
        }
      }
    }
    if (shared) {
      const float g = gate ? sigmoid_f(gate[(size_t)t * gate_stride]) : 1.f;
      if (VEC == 4) {
        const float4 h4 = moe_load4<T>(shared + (size_t)t * N + c);
        s[0] += g * h4.x; s[1 % VEC] += g * h4.y; s[2 % VEC] += g * h4.z; s[3 % VEC] += g * h4.w;
      } else {
        s[0] += g * to_float(shared[(size_t)t * N + c]);
      }
    }
    if (VEC == 4) moe_store4<T>(out + (size_t)t * N + c, make_float4(s[0], s[1 % VEC], s[2 % VEC], s[3 % VEC]));
    else out[(size_t)t * N + c] = from_float<T>(s[0]);
  }
}

}  // namespace

// Rows of a tile for a step's products: the tensor-core kernels (bfloat16, k a multiple of 32 and rows 16-byte aligned on
// both products) take 64, the plain ones 32. The grouping (sb_moe_sort) and both products must be given the same answer.
SB_EXPORT int sb_moe_tile_rows(int dtype, int K, int ff, int x_stride) {
  const bool mma = dtype == SB_DTYPE_BF16 && K % MB_K == 0 && ff % MB_K == 0 && x_stride % 8 == 0;
  return mma ? MB_M : TM;
}

// logits float [T, E] -> idx int32 [T, top], wts float [T, top]. score_kind 0: sigmoid of the logit, 1: softmax over the
// experts; renorm: the chosen weights divided by their sum.
SB_EXPORT int sb_moe_route(const float* logits, int E, int top, int score_kind, int renorm, int n_tokens, int* idx, float* wts,
                           cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || top > ROUTE_MAX_TOP || E > 32 * ROUTE_PER_LANE) return SB_ERR_LIMIT;
  moe_route_kernel<<<(n_tokens + 3) / 4, 128, 0, stream>>>(logits, E, top, score_kind, renorm, n_tokens, idx, wts);
  SB_LAUNCH_CHECK();
  return 0;
}

// idx int32 [n_pairs] -> offsets [E + 1], order [n_pairs], tiles [2 * (n_pairs / tile_rows + E)], n_tiles [1].
SB_EXPORT int sb_moe_sort(const int* idx, int n_pairs, int E, int tile_rows, int* offsets, int* order, int* tiles, int* n_tiles,
                          cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (E <= 0 || E > 4096 || tile_rows <= 0) return SB_ERR_LIMIT;
  moe_sort_kernel<<<1, 1024, (size_t)(2 * E + 1) * sizeof(int), stream>>>(idx, n_pairs, E, tile_rows, offsets, order, tiles, n_tiles);
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_moe_gate_up(const void* x, int x_stride, const void* w_gu, const int* order, const int* offsets, const int* tiles,
                             const int* n_tiles, const float* wts, int top, int n_pairs, int E, int K, int ff, int scale_input,
                             int act_kind, float limit, float alpha, void* act, int dtype, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  const int tile_rows = sb_moe_tile_rows(dtype, K, ff, x_stride);
  const int max_tiles = n_pairs / tile_rows + (E < n_pairs ? E : n_pairs);
  if (max_tiles > 65535) return SB_ERR_LIMIT;
  if (tile_rows == MB_M) {
    if (!aligned16(x) || !aligned16(w_gu)) return SB_ERR_ALIGN;
    cudaFuncSetAttribute(moe_gate_up_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MB_SMEM);
    moe_gate_up_mma_kernel<<<dim3((ff + 31) / 32, max_tiles), MB_THREADS, MB_SMEM, stream>>>(
        (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)w_gu, order, offsets, tiles, n_tiles, wts, top, K, ff, scale_input,
        act_kind, limit, alpha, (__nv_bfloat16*)act);
    SB_LAUNCH_CHECK();
    return 0;
  }
  dim3 grid((ff + GU_COLS - 1) / GU_COLS, max_tiles);
  if (dtype == SB_DTYPE_F32)
    moe_gate_up_kernel<float><<<grid, MOE_THREADS, 0, stream>>>((const float*)x, x_stride, (const float*)w_gu, order, offsets, tiles,
                                                                 n_tiles, wts, top, K, ff, scale_input, act_kind, limit, alpha, (float*)act);
  else if (dtype == SB_DTYPE_BF16)
    moe_gate_up_kernel<__nv_bfloat16><<<grid, MOE_THREADS, 0, stream>>>((const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)w_gu,
                                                                         order, offsets, tiles, n_tiles, wts, top, K, ff, scale_input,
                                                                         act_kind, limit, alpha, (__nv_bfloat16*)act);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// tokens int32 [T] -> idx int32 [T, top], wts float [T, top] from table int32 [vocab, top]; ``errors``: a counter that
// receives tokens outside the table and entries outside 0 .. E-1.
SB_EXPORT int sb_moe_route_table(const int* tokens, const int* last_token, int n_slots, const int* table, int vocab, int E, int top,
                                 int n_tokens, int* idx, float* wts, int* errors, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || vocab <= 0 || !errors) return SB_ERR_SHAPE;
  const int total = n_tokens * top;
  moe_route_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(tokens, last_token, n_slots, table, vocab, E, top, n_tokens, idx, wts,
                                                                  errors);
  SB_LAUNCH_CHECK();
  return 0;
}

// The experts' first product without a gate: act [n_pairs rows in grouped order, ff] = relu(x W_up^T)^2, w_up [E, ff, K].
SB_EXPORT int sb_moe_up(const void* x, int x_stride, const void* w_up, const int* order, const int* offsets, const int* tiles,
                        const int* n_tiles, const float* wts, int top, int n_pairs, int E, int K, int ff, void* act, int dtype,
                        cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  const int tile_rows = sb_moe_tile_rows(dtype, K, ff, x_stride);
  const int max_tiles = n_pairs / tile_rows + (E < n_pairs ? E : n_pairs);
  if (max_tiles > 65535) return SB_ERR_LIMIT;
  if (tile_rows == MB_M) {
    if (!aligned16(x) || !aligned16(w_up)) return SB_ERR_ALIGN;
    cudaFuncSetAttribute(moe_up_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MB_SMEM);
    moe_up_mma_kernel<<<dim3((ff + MB_N - 1) / MB_N, max_tiles), MB_THREADS, MB_SMEM, stream>>>(
        (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)w_up, order, offsets, tiles, n_tiles, top, K, ff, (__nv_bfloat16*)act);
    SB_LAUNCH_CHECK();
    return 0;
  }
  dim3 grid((ff + GU_COLS - 1) / GU_COLS, max_tiles);
  if (dtype == SB_DTYPE_F32)
    moe_gate_up_kernel<float><<<grid, MOE_THREADS, 0, stream>>>((const float*)x, x_stride, (const float*)w_up, order, offsets, tiles,
                                                                 n_tiles, wts, top, K, ff, 0, 2, 0.f, 0.f, (float*)act);
  else if (dtype == SB_DTYPE_BF16)
    moe_gate_up_kernel<__nv_bfloat16><<<grid, MOE_THREADS, 0, stream>>>((const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)w_up,
                                                                         order, offsets, tiles, n_tiles, wts, top, K, ff, 0, 2, 0.f, 0.f,
                                                                         (__nv_bfloat16*)act);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// out: [n_pairs, N] of dtype out_dtype (float for rows that are still to be added up).
SB_EXPORT int sb_moe_down(const void* act, const void* w_down, const int* order, const int* offsets, const int* tiles, const int* n_tiles,
                          const float* wts, int n_pairs, int E, int ff, int N, int scale_output, void* out, int dtype, int out_dtype,
                          int tile_rows, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (tile_rows != TM && tile_rows != MB_M) return SB_ERR_SHAPE;
  const int max_tiles = n_pairs / tile_rows + (E < n_pairs ? E : n_pairs);
  if (max_tiles > 65535) return SB_ERR_LIMIT;
  if (tile_rows == MB_M) {
    if (dtype != SB_DTYPE_BF16 || ff % MB_K) return SB_ERR_SHAPE;
    if (!aligned16(act) || !aligned16(w_down)) return SB_ERR_ALIGN;
    dim3 mgrid((N + MB_N - 1) / MB_N, max_tiles);
    if (out_dtype == SB_DTYPE_BF16) {
      cudaFuncSetAttribute(moe_down_mma_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MB_SMEM);
      moe_down_mma_kernel<__nv_bfloat16><<<mgrid, MB_THREADS, MB_SMEM, stream>>>(
          (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, order, offsets, tiles, n_tiles, wts, ff, N, scale_output,
          (__nv_bfloat16*)out);
    } else if (out_dtype == SB_DTYPE_F32) {
      cudaFuncSetAttribute(moe_down_mma_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MB_SMEM);
      moe_down_mma_kernel<float><<<mgrid, MB_THREADS, MB_SMEM, stream>>>((const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, order,
                                                                          offsets, tiles, n_tiles, wts, ff, N, scale_output, (float*)out);
    } else {
      return SB_ERR_DTYPE;
    }
    SB_LAUNCH_CHECK();
    return 0;
  }
  dim3 grid((N + DN_COLS - 1) / DN_COLS, max_tiles);
  if (dtype == SB_DTYPE_F32 && out_dtype == SB_DTYPE_F32)
    moe_down_kernel<float, float><<<grid, MOE_THREADS, 0, stream>>>((const float*)act, (const float*)w_down, order, offsets, tiles, n_tiles,
                                                                     wts, ff, N, scale_output, (float*)out);
  else if (dtype == SB_DTYPE_BF16 && out_dtype == SB_DTYPE_BF16)
    moe_down_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, MOE_THREADS, 0, stream>>>(
        (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, order, offsets, tiles, n_tiles, wts, ff, N, scale_output,
        (__nv_bfloat16*)out);
  else if (dtype == SB_DTYPE_BF16 && out_dtype == SB_DTYPE_F32)
    moe_down_kernel<__nv_bfloat16, float><<<grid, MOE_THREADS, 0, stream>>>((const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, order,
                                                                             offsets, tiles, n_tiles, wts, ff, N, scale_output, (float*)out);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// parts float [T * top, N] -> out [T, N]: a token's rows added in the order of its choices.
SB_EXPORT int sb_moe_combine(const float* parts, int top, int n_tokens, int N, void* out, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const long long total = (long long)n_tokens * N;
  const long long want = (total + 255) / 256;
  const int blocks = (int)(want < sm_count() * 8 ? want : sm_count() * 8);
  if (dtype == SB_DTYPE_F32) moe_combine_kernel<float><<<blocks, 256, 0, stream>>>(parts, top, N, total, (float*)out);
  else if (dtype == SB_DTYPE_BF16) moe_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(parts, top, N, total, (__nv_bfloat16*)out);
  else return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// As sb_moe_route with more: the row stride of the logits (columns beyond E are not the router's), a float bias [E] or
// null that joins the scores for the choice only, sum_eps, added to the sum the chosen scores are divided by, and
// weight_scale, a constant every weight is multiplied by.
SB_EXPORT int sb_moe_route_bias(const float* logits, int stride, int E, int top, int score_kind, int renorm, float sum_eps,
                                const float* bias, int n_tokens, int* idx, float* wts, float weight_scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || top > ROUTE_MAX_TOP || E > 32 * ROUTE_PER_LANE) return SB_ERR_LIMIT;
  if (stride < E) return SB_ERR_SHAPE;
  auto k = E <= 64 ? moe_route_bias_kernel<2> : E <= 128 ? moe_route_bias_kernel<4> : E <= 256 ? moe_route_bias_kernel<8>
                                                                                               : moe_route_bias_kernel<ROUTE_PER_LANE>;
  k<<<(n_tokens + 3) / 4, 128, 0, stream>>>(logits, stride, E, top, score_kind, renorm, sum_eps, bias, n_tokens, idx, wts, weight_scale);
  SB_LAUNCH_CHECK();
  return 0;
}

// out [T, N] = the sum of a token's rows of parts (float [T * top, N]) where idx names one of the E_real experts, and
// wts * x[t] where it names none (N must then be x's width); plus shared [T, N] (or null), times sigmoid(gate[t]) if a
// gate (float, rows gate_stride apart) is given.
SB_EXPORT int sb_moe_combine_more(const float* parts, const int* idx, const float* wts, int E_real, const void* x, int x_stride,
                                  const void* shared, const float* gate, int gate_stride, int top, int n_tokens, int N, void* out,
                                  int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (!parts || !idx || !wts || !x || top <= 0 || x_stride < N) return SB_ERR_SHAPE;
  const bool vec = N % 4 == 0 && x_stride % 4 == 0 && aligned16(parts) && aligned16(x) && aligned16(out) && (!shared || aligned16(shared));
  const long long total = (long long)n_tokens * (vec ? N / 4 : N);
  const long long want = (total + 255) / 256;
  const int blocks = (int)(want < sm_count() * 16 ? want : sm_count() * 16);
  if (dtype == SB_DTYPE_F32) {
    auto k = vec ? moe_combine_more_kernel<float, 4> : moe_combine_more_kernel<float, 1>;
    k<<<blocks, 256, 0, stream>>>(parts, idx, wts, E_real, (const float*)x, x_stride, (const float*)shared, gate, gate_stride, top, N, total,
                                  (float*)out);
  } else if (dtype == SB_DTYPE_BF16) {
    auto k = vec ? moe_combine_more_kernel<__nv_bfloat16, 4> : moe_combine_more_kernel<__nv_bfloat16, 1>;
    k<<<blocks, 256, 0, stream>>>(parts, idx, wts, E_real, (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)shared, gate, gate_stride,
                                  top, N, total, (__nv_bfloat16*)out);
  } else return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}
