// Kernels of mixers that carry a state of fixed size from token to token instead of (or beside) cached keys:
// short causal convolutions over time, the blends of a token's input with its predecessor's (token shift), linear
// recurrences over a matrix state per head (fixed decay, selective state space, gated delta rule, a decay per key
// channel with a bonus for the current token), the normalisation-and-gate that follows them, and the cache write of
// an attention whose values are normalised and whose queries and keys are not rotated.
//
// A step is ragged: row r brings the tokens cu_q[r] .. cu_q[r+1]-1 and owns state slot slots[r]. State tensors
// are float [max_slots, ...] and are zero when a slot is handed out, so "zeros before the start" needs no
// special case: a request's first portion reads the zeros, every later portion what the one before left.
// Everything that enters a recurrence is float, in both dtypes; activations read and written are T.
#include "common.cuh"

using namespace sb;

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float load_w(const void* p, int dtype, size_t i) {
  return dtype == SB_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// ------------------------------------------------------------------------------------------ short convolution
// out[t, c] = act( bias[c] + sum_j w[c, j] * in[t - taps + 1 + j, c]  (+ in[t, c] if residual) ), in[-1], in[-2], ...
// of a row's first token being the inputs the state holds: state[slot, m, c] is the input taps - 1 - m tokens
// before the portion's start (slots are slot_stride floats apart: the states of a slot may lie in one row of a pool). With inline_state (every row brings one token) the thread also shifts the state.
constexpr int CONV_THREADS = 128;
constexpr int CONV_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS) causal_conv_kernel(
    const T* __restrict__ x, int x_stride, const T* __restrict__ w, const T* __restrict__ bias, float* __restrict__ state,
    const int* __restrict__ slots, const int* __restrict__ cu_q, const int* __restrict__ token_row, T* __restrict__ out,
    int out_stride, int C, int taps, int act, int residual, int inline_state, long long slot_stride) {
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  const int t = blockIdx.y;
  if (c >= C) return;
  const int r = token_row[t];
  const int i = t - cu_q[r];
  const int K = taps - 1;
  float* st = state + (size_t)slots[r] * slot_stride + c;
  float acc = bias ? to_float(bias[c]) : 0.f;
  float cur = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = i - K + j;
    const float v = src >= 0 ? to_float(x[(size_t)(t - K + j) * x_stride + c]) : st[(size_t)(K + src) * C];
    acc += to_float(w[(size_t)c * taps + j]) * v;
    cur = v;
  }
  if (residual) acc += cur;
  if (act == 1) acc = silu_f(acc);
  out[(size_t)t * out_stride + c] = from_float<T>(acc);
  if (inline_state) {
    for (int m = 0; m + 1 < K; ++m) st[(size_t)m * C] = st[(size_t)(m + 1) * C];
    if (K > 0) st[(size_t)(K - 1) * C] = cur;
  }
}

// The same for eight neighbouring channels a thread, fetched 16 bytes at a time (bfloat16 with every row start and the
// channel count a multiple of eight); the arithmetic per channel is the one above, in the same order.
template <int TAPS>      // the number of taps when it is 2, 3 or 4 (the eight filters are then fetched 16 bytes at a time); 0: any
__global__ void __launch_bounds__(CONV_THREADS) causal_conv8_kernel(
    const __nv_bfloat16* __restrict__ x, int x_stride, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
    float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu_q, const int* __restrict__ token_row,
    __nv_bfloat16* __restrict__ out, int out_stride, int C, int taps, int act, int residual, int inline_state, long long slot_stride) {
  const int c = (blockIdx.x * CONV_THREADS + threadIdx.x) * 8;
  const int t = blockIdx.y;
  if (c >= C) return;
  const int r = token_row[t];
  const int i = t - cu_q[r];
  if (TAPS > 0) taps = TAPS;
  const int K = taps - 1;
  float* st = state + (size_t)slots[r] * slot_stride + c;
  float acc[8], cur[8];
  uint4 wraw[TAPS > 0 ? TAPS : 1];                  // the filters of channels c .. c + 7 lie together: 8 * taps values
  if (TAPS > 0) {
#pragma unroll
    for (int u = 0; u < TAPS; ++u) wraw[u] = *reinterpret_cast<const uint4*>(w + (size_t)c * TAPS + u * 8);
  }
  const __nv_bfloat16* wl = reinterpret_cast<const __nv_bfloat16*>(wraw);
#pragma unroll
  for (int e = 0; e < 8; ++e) { acc[e] = bias ? to_float(bias[c + e]) : 0.f; cur[e] = 0.f; }
#pragma unroll
  for (int j = 0; j < (TAPS > 0 ? TAPS : taps); ++j) {
    const int src = i - K + j;
    if (src >= 0) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(t - K + j) * x_stride + c);
      const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int e = 0; e < 8; ++e) cur[e] = to_float(v[e]);
    } else {
      const float4 a = *reinterpret_cast<const float4*>(st + (size_t)(K + src) * C), b = *reinterpret_cast<const float4*>(st + (size_t)(K + src) * C + 4);
      cur[0] = a.x; cur[1] = a.y; cur[2] = a.z; cur[3] = a.w; cur[4] = b.x; cur[5] = b.y; cur[6] = b.z; cur[7] = b.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += (TAPS > 0 ? to_float(wl[e * TAPS + j]) : to_float(w[(size_t)(c + e) * taps + j])) * cur[e];
  }
  uint4 packed;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float v = acc[e];
    if (residual) v += cur[e];
    if (act == 1) v = silu_f(v);
    o[e] = __float2bfloat16_rn(v);
  }
  *reinterpret_cast<uint4*>(out + (size_t)t * out_stride + c) = packed;
  if (inline_state) {
    for (int m = 0; m + 1 < K; ++m)
#pragma unroll
      for (int e = 0; e < 8; ++e) st[(size_t)m * C + e] = st[(size_t)(m + 1) * C + e];
    if (K > 0)
#pragma unroll
      for (int e = 0; e < 8; ++e) st[(size_t)(K - 1) * C + e] = cur[e];
  }
}

// After a step: the state of row r becomes its last taps - 1 inputs (older ones come from the old state when the
// portion is shorter than that). One thread per (row, channel) reads all it needs before it writes.
template <typename T>
__global__ void __launch_bounds__(CONV_THREADS) conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                                                   const int* __restrict__ slots, const int* __restrict__ cu_q, int C,
                                                                   int taps, long long slot_stride) {
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  const int r = blockIdx.y;
  if (c >= C) return;
  const int q0 = cu_q[r], n = cu_q[r + 1] - q0;
  const int K = taps - 1;
  float* st = state + (size_t)slots[r] * slot_stride + c;
  float keep[CONV_MAX_TAPS];
#pragma unroll
  for (int m = 0; m < CONV_MAX_TAPS; ++m) {
    if (m < K) {
      const int src = n - K + m;                        // index among the portion's tokens
      keep[m] = src >= 0 ? to_float(x[(size_t)(q0 + src) * x_stride + c]) : st[(size_t)(m + n) * C];
    }
  }
#pragma unroll
  for (int m = 0; m < CONV_MAX_TAPS; ++m)
    if (m < K) st[(size_t)m * C] = keep[m];
}

// ------------------------------------------------------------------------------------------ linear recurrences
// One state matrix S [dk, dv] per (request, head); per token, with a decay a (a number, or one per row of S):
//   S <- a * S;   u = v                      (MODE_DECAY, MODE_SSM: u = dt * x)
//                 u = beta * (v - S^T k)     (MODE_DELTA)
//   S <- S + k u^T;   o = S^T q  (+ D * x for MODE_SSM)
// MODE_WKV reads out first: o = S^T q + (sum_i q_i b_i k_i) v with a bonus b per (head, row) for the token's own
// k v^T; then S <- diag(a) S + k v^T with a decay a = exp(-exp(rate + bias)) per row of S.
// Two kernels. The first works on every (token, head) at once and leaves, as float, what the walk over the tokens
// reads: q and k (after silu, or as unit vectors), the decays (after softplus and the exponentials), the values and
// the per-token factor (dt or beta). The second walks: the columns of S never meet, so a block takes (request, head, a
// slice of columns) and goes through the row's tokens in order. A thread keeps REC_RPT rows of one column in
// registers; P lanes share a column and add their parts by shuffles, so dk <= 32 * REC_RPT. Rows are padded to
// dkp = REC_RPT * P with k = q = 0, which leaves the padded rows of S at zero and the inner loops free of tests. The
// tokens' vectors come through a two-stage cp.async ring, REC_TS tokens a stage, so the next tokens arrive while
// these are worked on; a thread's rows are 4 P apart in fours, so it reads them 16 bytes at a time and the lanes of
// a column read neighbouring 16 bytes.
constexpr int MODE_DECAY = 0, MODE_SSM = 1, MODE_DELTA = 2, MODE_WKV = 3, MODE_GLA = 4;
// MODE_GLA: S <- diag(a) S + k v^T, o = S^T q (read out after the update), a = sigmoid(rate + bias)^rate_scale per row of S,
// formed as exp(-softplus(-(rate + bias)) * rate_scale); q times q_scale.
constexpr int REC_RPT = 16;
constexpr int REC_THREADS = 128;
constexpr int REC_TS = 16;

struct RecArgs {
  const void* q; const void* k; const void* v;      // [T, *] activations: row strides below, head h at h * dk (dv)
  int q_stride, k_stride, v_stride;
  const void* aux;  int aux_stride;                  // SSM: dt before softplus [T, H]; DELTA: beta before the sigmoid [T, H]
  const void* rate; int rate_stride;                 // DELTA: decay rate before softplus [T, H * dk], or [T, H] with rate_per_head;
  int rate_dtype, rate_per_head;                     // WKV: the exponent's variable part [T, H * dk] (dt_bias [H * dk] is added)
  const float* bonus;                                // WKV: [H, dk] float
  const void* decay;                                 // DECAY: [H] float decays
  const void* a_log; const void* dt_bias; const void* d_skip;   // parameters (dtype par_dtype)
  int par_dtype;
  float* state;                                      // [slots, H, dk, dv], slots state_stride floats apart
  long long state_stride;
  const int* slots; const int* cu_q;
  float* out; int out_stride;                        // [T, H * dv] float
  int H, Hqk, dk, dv, P, dkp, dvp, n_tokens;
  float q_scale;
  float rate_scale;                                  // GLA: the exponent of the sigmoid (one over the temperature)
  // float work space, made by the first kernel: qf, kf [T, Hqk, dkp]; af [T, H, dkp] (DELTA, WKV, GLA); vf [T, H, dvp]; sc, dec [T, H]
  float *qf, *kf, *af, *vf, *sc, *dec;
};

// A warp per (token, head) of max(H, Hqk) heads, four warps a block: a head has a few dozen to a few hundred elements.
template <typename T, int MODE>
__global__ void __launch_bounds__(REC_THREADS) recurrence_prep_kernel(RecArgs a) {
  const int heads = a.H > a.Hqk ? a.H : a.Hqk;
  const long long wid = (long long)blockIdx.x * (REC_THREADS / 32) + (threadIdx.x >> 5);
  if (wid >= (long long)a.n_tokens * heads) return;      // (a whole warp leaves together; nothing below waits for the block)
  const int t = (int)(wid / heads), h = (int)(wid - (long long)t * heads), tid = threadIdx.x & 31;
  const int dk = a.dk, dkp = a.dkp, dv = a.dv, dvp = a.dvp;
  if (h < a.Hqk) {
    const T* qr = (const T*)a.q + (size_t)t * a.q_stride + (size_t)h * dk;
    const T* kr = (const T*)a.k + (size_t)t * a.k_stride + (size_t)h * dk;
    float* qo = a.qf + ((size_t)t * a.Hqk + h) * dkp;
    float* ko = a.kf + ((size_t)t * a.Hqk + h) * dkp;
    float fq = 1.f, fk = 1.f;
    if (MODE == MODE_DELTA) {
      float sq = 0.f, sk = 0.f;
      for (int i = tid; i < dk; i += 32) {
        const float x = to_float(qr[i]), y = to_float(kr[i]);
        sq += x * x;
        sk += y * y;
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      fq = a.q_scale / sqrtf(sq + 1e-6f);
      fk = 1.f / sqrtf(sk + 1e-6f);
    }
    if (MODE == MODE_GLA) fq = a.q_scale;
    for (int i = tid; i < dkp; i += 32) {
      float x = 0.f, y = 0.f;
      if (i < dk) {
        x = to_float(qr[i]);
        y = to_float(kr[i]);
        if (MODE == MODE_DECAY) { x = silu_f(x); y = silu_f(y); }
        x *= fq;
        y *= fk;
      }
      qo[i] = x;
      ko[i] = y;
    }
  }
  if (h < a.H) {
    const T* vr = (const T*)a.v + (size_t)t * a.v_stride + (size_t)h * dv;
    float* vo = a.vf + ((size_t)t * a.H + h) * dvp;
    for (int j = tid; j < dvp; j += 32) {
      float x = j < dv ? to_float(vr[j]) : 0.f;
      if (MODE == MODE_DECAY) x = silu_f(x);
      vo[j] = x;
    }
    if (MODE == MODE_DELTA) {
      const float neg_a = -expf(load_w(a.a_log, a.par_dtype, h));
      float* ao = a.af + ((size_t)t * a.H + h) * dkp;
      if (a.rate_per_head) {                   // one decay for all rows of the head's state
        const float g = expf(neg_a * softplus_f(load_w(a.rate, a.rate_dtype, (size_t)t * a.rate_stride + h) + load_w(a.dt_bias, a.par_dtype, h)));
        for (int i = tid; i < dkp; i += 32) ao[i] = i < dk ? g : 1.f;
      } else {
        const size_t r0 = (size_t)t * a.rate_stride + (size_t)h * dk;
        for (int i = tid; i < dkp; i += 32)
          ao[i] = i < dk ? expf(neg_a * softplus_f(load_w(a.rate, a.rate_dtype, r0 + i) + load_w(a.dt_bias, a.par_dtype, (size_t)h * dk + i))) : 1.f;
      }
    }
    if (MODE == MODE_GLA) {
      const size_t r0 = (size_t)t * a.rate_stride + (size_t)h * dk;
      float* ao = a.af + ((size_t)t * a.H + h) * dkp;
      for (int i = tid; i < dkp; i += 32)
        ao[i] = i < dk ? expf(-softplus_f(-(load_w(a.rate, a.rate_dtype, r0 + i) + load_w(a.dt_bias, a.par_dtype, (size_t)h * dk + i))) * a.rate_scale)
                       : 1.f;
    }
    float bonus_dot = 0.f;
    if (MODE == MODE_WKV) {
      // (H == Hqk here: every head has a receptance and a key of its own)
      const size_t r0 = (size_t)t * a.rate_stride + (size_t)h * dk;
      const T* qr = (const T*)a.q + (size_t)t * a.q_stride + (size_t)h * dk;
      const T* kr = (const T*)a.k + (size_t)t * a.k_stride + (size_t)h * dk;
      float* ao = a.af + ((size_t)t * a.H + h) * dkp;
      for (int i = tid; i < dkp; i += 32) {
        ao[i] = i < dk ? expf(-expf(load_w(a.rate, a.rate_dtype, r0 + i) + load_w(a.dt_bias, a.par_dtype, (size_t)h * dk + i))) : 1.f;
        if (i < dk) bonus_dot += to_float(qr[i]) * a.bonus[(size_t)h * dk + i] * to_float(kr[i]);
      }
      bonus_dot = warp_sum(bonus_dot);
    }
    if (tid == 0) {
      float sc = 1.f, dec = 1.f;
      if (MODE == MODE_DECAY) dec = ((const float*)a.decay)[h];
      if (MODE == MODE_SSM) {
        sc = softplus_f(to_float(((const T*)a.aux)[(size_t)t * a.aux_stride + h]) + load_w(a.dt_bias, a.par_dtype, h));
        dec = expf(-expf(load_w(a.a_log, a.par_dtype, h)) * sc);
      }
      if (MODE == MODE_DELTA) sc = sigmoid_f(to_float(((const T*)a.aux)[(size_t)t * a.aux_stride + h]));
      if (MODE == MODE_WKV) sc = bonus_dot;
      a.sc[(size_t)t * a.H + h] = sc;
      a.dec[(size_t)t * a.H + h] = dec;
    }
  }
}

__device__ __forceinline__ void rec_cp16(float* smem, const float* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(g));
}
__device__ __forceinline__ void rec_cp4(float* smem, const float* g) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(g));
}

// grid (dvp / VC, H, rows); 128 threads; VC = 128 / P columns a block.
template <int MODE>
__global__ void __launch_bounds__(REC_THREADS) recurrence_scan_kernel(RecArgs a) {
  constexpr bool DELTA = MODE == MODE_DELTA, SKIP = MODE == MODE_SSM, WKV = MODE == MODE_WKV, GLA = MODE == MODE_GLA;
  constexpr bool ROWS = DELTA || WKV || GLA;                               // a decay per row of S comes with every token
  extern __shared__ __align__(16) float smem[];
  const int dk = a.dk, dv = a.dv, P = a.P, dkp = a.dkp, dvp = a.dvp, H = a.H;
  const int VC = REC_THREADS / P;
  const int per_tok = (ROWS ? 3 : 2) * dkp + VC;                     // floats of a token's vectors in a stage
  const int stage_floats = REC_TS * per_tok + 2 * REC_TS;             // + sc, dec
  const int r = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * VC;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int part = lane % P, col = warp * (32 / P) + lane / P;
  const int j = j0 + col;
  const bool col_ok = j < dv;
  const int q0 = a.cu_q[r], n = a.cu_q[r + 1] - q0;
  const int hq = h / (H / a.Hqk);
  float* S = a.state + (size_t)a.slots[r] * a.state_stride + ((size_t)h * dk) * dv;
  float s[REC_RPT];
#pragma unroll
  for (int x = 0; x < REC_RPT; ++x) {
    const int i = (x >> 2) * 4 * P + part * 4 + (x & 3);
    s[x] = (col_ok && i < dk) ? S[(size_t)i * dv + j] : 0.f;
  }
  float d_skip = 0.f;
  if (SKIP) d_skip = load_w(a.d_skip, a.par_dtype, h);

  auto fetch = [&](int stage, int t0) {
    float* base = smem + (size_t)stage * stage_floats;
    const int nt = min(REC_TS, n - t0);
    const int row16 = dkp / 4;                                        // 16-byte pieces of a q (k, a) row
    for (int w = tid; w < nt * row16; w += REC_THREADS) {
      const int tt = w / row16, c = (w - tt * row16) * 4;
      const size_t tok = (size_t)(q0 + t0 + tt);
      float* dst = base + (size_t)tt * per_tok;
      rec_cp16(dst + c, a.qf + (tok * a.Hqk + hq) * dkp + c);
      rec_cp16(dst + dkp + c, a.kf + (tok * a.Hqk + hq) * dkp + c);
      if (ROWS) rec_cp16(dst + 2 * dkp + c, a.af + (tok * H + h) * dkp + c);
    }
    const int v16 = VC / 4;
    for (int w = tid; w < nt * v16; w += REC_THREADS) {
      const int tt = w / v16, c = (w - tt * v16) * 4;
      rec_cp16(base + (size_t)tt * per_tok + (ROWS ? 3 : 2) * dkp + c, a.vf + ((size_t)(q0 + t0 + tt) * H + h) * dvp + j0 + c);
    }
    for (int w = tid; w < 2 * nt; w += REC_THREADS) {
      const int tt = w >> 1;
      rec_cp4(base + REC_TS * per_tok + w, ((w & 1) ? a.dec : a.sc) + (size_t)(q0 + t0 + tt) * H + h);
    }
  };

  if (n > 0) fetch(0, 0);
  asm volatile("cp.async.commit_group;");
  int stage = 0;
  for (int t0 = 0; t0 < n; t0 += REC_TS, stage ^= 1) {
    if (t0 + REC_TS < n) fetch(stage ^ 1, t0 + REC_TS);
    asm volatile("cp.async.commit_group;");
    asm volatile("cp.async.wait_group 1;");
    __syncthreads();                                                  // this stage has arrived for every thread
    const float* base = smem + (size_t)stage * stage_floats;
    const int nt = min(REC_TS, n - t0);
#pragma unroll 2      // the sums of one token's read-out overlap with the next token's update
    for (int tt = 0; tt < nt; ++tt) {
      const float4* q4 = reinterpret_cast<const float4*>(base + (size_t)tt * per_tok);
      const float4* k4 = q4 + dkp / 4;
      const float4* a4 = k4 + dkp / 4;
      const float vv = base[(size_t)tt * per_tok + (ROWS ? 3 : 2) * dkp + col];
      const float sc = base[REC_TS * per_tok + 2 * tt], dec = base[REC_TS * per_tok + 2 * tt + 1];
      float4 kk[4], qq[4];
#pragma unroll
      for (int x4 = 0; x4 < 4; ++x4) {
        kk[x4] = k4[x4 * P + part];
        qq[x4] = q4[x4 * P + part];
      }
      if (WKV) {
        // the read-out sees the state the tokens before left, and this token's own k v^T through the bonus (sc)
        float oo[4];
#pragma unroll
        for (int x4 = 0; x4 < 4; ++x4) {
          const float4 aa = a4[x4 * P + part];
          oo[x4] = s[4 * x4] * qq[x4].x + s[4 * x4 + 1] * qq[x4].y + s[4 * x4 + 2] * qq[x4].z + s[4 * x4 + 3] * qq[x4].w;
          s[4 * x4] = s[4 * x4] * aa.x + kk[x4].x * vv; s[4 * x4 + 1] = s[4 * x4 + 1] * aa.y + kk[x4].y * vv;
          s[4 * x4 + 2] = s[4 * x4 + 2] * aa.z + kk[x4].z * vv; s[4 * x4 + 3] = s[4 * x4 + 3] * aa.w + kk[x4].w * vv;
        }
        float o_acc = (oo[0] + oo[1]) + (oo[2] + oo[3]);
        for (int o = P >> 1; o > 0; o >>= 1) o_acc += __shfl_xor_sync(0xffffffffu, o_acc, o);
        o_acc += sc * vv;
        if (part == 0 && col_ok) a.out[(size_t)(q0 + t0 + tt) * a.out_stride + (size_t)h * dv + j] = o_acc;
        continue;
      }
      float u;
      if (DELTA) {
        float dot[4];
#pragma unroll
        for (int x4 = 0; x4 < 4; ++x4) {
          const float4 aa = a4[x4 * P + part];
          s[4 * x4] *= aa.x; s[4 * x4 + 1] *= aa.y; s[4 * x4 + 2] *= aa.z; s[4 * x4 + 3] *= aa.w;
          dot[x4] = s[4 * x4] * kk[x4].x + s[4 * x4 + 1] * kk[x4].y + s[4 * x4 + 2] * kk[x4].z + s[4 * x4 + 3] * kk[x4].w;
        }
        float d = (dot[0] + dot[1]) + (dot[2] + dot[3]);
        for (int o = P >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        u = sc * (vv - d);
      } else if (GLA) {
#pragma unroll
        for (int x4 = 0; x4 < 4; ++x4) {
          const float4 aa = a4[x4 * P + part];
          s[4 * x4] *= aa.x; s[4 * x4 + 1] *= aa.y; s[4 * x4 + 2] *= aa.z; s[4 * x4 + 3] *= aa.w;
        }
        u = vv;
      } else {
#pragma unroll
        for (int x = 0; x < REC_RPT; ++x) s[x] *= dec;
        u = sc * vv;
      }
      float oo[4];
#pragma unroll
      for (int x4 = 0; x4 < 4; ++x4) {
        s[4 * x4] += kk[x4].x * u; s[4 * x4 + 1] += kk[x4].y * u; s[4 * x4 + 2] += kk[x4].z * u; s[4 * x4 + 3] += kk[x4].w * u;
        oo[x4] = s[4 * x4] * qq[x4].x + s[4 * x4 + 1] * qq[x4].y + s[4 * x4 + 2] * qq[x4].z + s[4 * x4 + 3] * qq[x4].w;
      }
      float o_acc = (oo[0] + oo[1]) + (oo[2] + oo[3]);
      for (int o = P >> 1; o > 0; o >>= 1) o_acc += __shfl_xor_sync(0xffffffffu, o_acc, o);
      if (SKIP) o_acc += d_skip * vv;
      if (part == 0 && col_ok) a.out[(size_t)(q0 + t0 + tt) * a.out_stride + (size_t)h * dv + j] = o_acc;
    }
    __syncthreads();                                                  // before the stage after next overwrites this one
  }
  asm volatile("cp.async.wait_group 0;");
#pragma unroll
  for (int x = 0; x < REC_RPT; ++x) {
    const int i = (x >> 2) * 4 * P + part * 4 + (x & 3);
    if (col_ok && i < dk) S[(size_t)i * dv + j] = s[x];
  }
}

static inline int rec_lanes(int dk) {
  int P = 1;
  while (P * REC_RPT < dk) P <<= 1;
  return P;
}

static inline long long rec_work_floats(int mode, int n_tokens, int H, int Hqk, int dk, int dv) {
  const int P = rec_lanes(dk), dkp = P * REC_RPT, VC = REC_THREADS / P, dvp = (dv + VC - 1) / VC * VC;
  return (long long)n_tokens * ((long long)2 * Hqk * dkp + ((mode == MODE_DELTA || mode == MODE_WKV || mode == MODE_GLA) ? (long long)H * dkp : 0) + (long long)H * dvp + 2 * H) + 16;
}

template <typename T, int MODE>
int launch_recurrence(RecArgs a, float* work, int n_rows, cudaStream_t stream) {
  const int P = rec_lanes(a.dk);
  if (P > 32) return SB_ERR_LIMIT;
  a.P = P;
  a.dkp = P * REC_RPT;
  const int VC = REC_THREADS / P;
  a.dvp = (a.dv + VC - 1) / VC * VC;
  const size_t T_ = (size_t)a.n_tokens;
  a.qf = work;
  a.kf = a.qf + T_ * a.Hqk * a.dkp;
  a.af = a.kf + T_ * a.Hqk * a.dkp;
  a.vf = a.af + ((MODE == MODE_DELTA || MODE == MODE_WKV || MODE == MODE_GLA) ? T_ * a.H * a.dkp : 0);
  a.sc = a.vf + T_ * a.H * a.dvp;
  a.dec = a.sc + T_ * a.H;
  if (a.n_tokens > 0x7fffffff / 1 || a.H > 65535 || a.Hqk > 65535) return SB_ERR_LIMIT;
  const long long prep_warps = (long long)a.n_tokens * (a.H > a.Hqk ? a.H : a.Hqk);
  const long long prep_blocks = (prep_warps + REC_THREADS / 32 - 1) / (REC_THREADS / 32);
  if (prep_blocks > 0x7fffffffLL) return SB_ERR_LIMIT;
  recurrence_prep_kernel<T, MODE><<<(unsigned)prep_blocks, REC_THREADS, 0, stream>>>(a);
  SB_LAUNCH_CHECK();
  const int per_tok = ((MODE == MODE_DELTA || MODE == MODE_WKV || MODE == MODE_GLA) ? 3 : 2) * a.dkp + VC;
  const size_t smem = (size_t)2 * (REC_TS * per_tok + 2 * REC_TS) * sizeof(float);
  dim3 grid(a.dvp / VC, a.H, n_rows);
  auto kernel = recurrence_scan_kernel<MODE>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return SB_ERR_LIMIT;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  kernel<<<grid, REC_THREADS, smem, stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------ norm and gate
// out[t, c] = scale * post( rms_g( pre(y[t, c]) ) * w[c mod w_size] ), a warp per (token, group), or the whole block of 128
// threads for a group of more than 512 values (TPG threads a group):
// (y is float, or of the activations' type)
//   pre:  times act(gate[t, c']) if the gate comes first; rms_g: divided by the root mean square of the group's
//   values (+ eps inside the root; no division with groups == 0, where a group is just a warp's share of the row);
//   post: times act(gate[t, c']) if the gate comes last. c' = c, or c / (C / gate_cols) for a gate per head.
template <typename T, int TPG>
__global__ void __launch_bounds__(128) gated_norm_kernel(const void* __restrict__ y, int y_dtype, int y_stride, const T* __restrict__ gate,
                                                         int gate_stride, int gate_cols, int gate_act, int gate_first,
                                                         const void* __restrict__ weight, int w_dtype, int w_size, T* __restrict__ out,
                                                         int out_stride, int n_tokens, int C, int groups, int normalise, float eps,
                                                         float scale) {
  __shared__ float red[32];
  const int lane = TPG == 32 ? (threadIdx.x & 31) : threadIdx.x;
  const long long wid = TPG == 32 ? (long long)blockIdx.x * 4 + (threadIdx.x >> 5) : (long long)blockIdx.x;
  if (wid >= (long long)n_tokens * groups) return;      // (a whole warp, or the whole block, leaves together)
  const int t = (int)(wid / groups), g = (int)(wid - (long long)t * groups);
  const int gs = C / groups, c0 = g * gs;
  const int per_gate = gate ? C / gate_cols : 1;
  const size_t yr = (size_t)t * y_stride;
  const T* gr = gate ? gate + (size_t)t * gate_stride : nullptr;
  auto gate_of = [&](int c) {
    const float z = to_float(gr[c / per_gate]);
    return gate_act == 1 ? silu_f(z) : sigmoid_f(z);
  };
  float inv = 1.f;
  if (normalise) {
    float ss = 0.f;
    for (int c = c0 + lane; c < c0 + gs; c += TPG) {
      float v = load_w(y, y_dtype, yr + c);
      if (gr && gate_first) v *= gate_of(c);
      ss += v * v;
    }
    ss = TPG == 32 ? warp_sum(ss) : block_sum(ss, red);
    inv = 1.f / sqrtf(ss / (float)gs + eps);
  }
  for (int c = c0 + lane; c < c0 + gs; c += TPG) {
    float v = load_w(y, y_dtype, yr + c);
    if (gr && gate_first) v *= gate_of(c);
    v *= inv;
    if (weight) v *= load_w(weight, w_dtype, c % w_size);
    if (gr && !gate_first) v *= gate_of(c);
    out[(size_t)t * out_stride + c] = from_float<T>(v * scale);
  }
}

// The same for the shape the recurrent read-outs have: float y, groups of a multiple of 4 up to 512 values that are all
// normalised, the gate (one value an element, applied last) and the weight optional. A warp per (token, group); a lane
// loads four neighbours at a time and keeps its share of the group in registers, so y and the gate are read once.
template <typename T> struct Vec4 { };
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[4]) { const float4 x = *(const float4*)p; o[0] = x.x; o[1] = x.y; o[2] = x.z; o[3] = x.w; }
  static __device__ __forceinline__ void store(float* p, const float (&o)[4]) { *(float4*)p = make_float4(o[0], o[1], o[2], o[3]); }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&o)[4]) {
    const uint2 x = *(const uint2*)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162*)&x.x, b = *(const __nv_bfloat162*)&x.y;
    o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&o)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
    uint2 x;
    x.x = *(const unsigned*)&a; x.y = *(const unsigned*)&b;
    *(uint2*)p = x;
  }
};

// LPG lanes a group (a power of two, at least gs / 16), so a warp takes 32 / LPG groups at once when they are short.
template <typename T, typename W>
__global__ void __launch_bounds__(128) gated_norm_vec_kernel(const float* __restrict__ y, int y_stride, const T* __restrict__ gate, int gate_stride,
                                                             int gate_act, const W* __restrict__ weight, int w_size, T* __restrict__ out,
                                                             int out_stride, int n_groups, int gs, int groups, int lpg, float eps, float scale) {
  const int lane = threadIdx.x & 31, sub = lane & (lpg - 1);
  const int gid = (blockIdx.x * 4 + (threadIdx.x >> 5)) * (32 / lpg) + lane / lpg;      // (token, group), groups fastest
  const bool live = gid < n_groups;                                   // (idle lanes still take part in the shuffles)
  const int t = live ? gid / groups : 0, c0 = live ? (gid - t * groups) * gs : 0;
  const float* yr = y + (size_t)t * y_stride + c0;
  float v[4][4];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int c = (r * lpg + sub) * 4;
    if (live && c < gs) {
      Vec4<float>::load(yr + c, v[r]);
      ss += v[r][0] * v[r][0] + v[r][1] * v[r][1] + v[r][2] * v[r][2] + v[r][3] * v[r][3];
    }
  }
  for (int o = lpg >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!live) return;
  const float inv = scale / sqrtf(ss / (float)gs + eps);
  const int w0 = weight ? c0 % w_size : 0;                            // (the weight's period is a multiple of the group)
  const T* gr = gate ? gate + (size_t)t * gate_stride + c0 : nullptr;
  T* orow = out + (size_t)t * out_stride + c0;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int c = (r * lpg + sub) * 4;
    if (c < gs) {
      float w[4] = {1.f, 1.f, 1.f, 1.f}, z[4];
      if (weight) Vec4<W>::load(weight + w0 + c, w);
      if (gr) {
        Vec4<T>::load(gr + c, z);
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] *= gate_act == 1 ? silu_f(z[i]) : sigmoid_f(z[i]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) z[i] = v[r][i] * inv * w[i];
      Vec4<T>::store(orow + c, z);
    }
  }
}

// ------------------------------------------------------------------------------------------ cache write, values normalised
// Keys and values of a step go to their pages, unrotated; with norm_dim > 0 every value head is first divided by
// the root mean square of its first norm_dim elements (what lies beyond them is padding and stays as it is).
// A warp per (token, kv head). Row layout of qkv: H query heads, Hkv key heads, Hkv value heads, D apart.
template <typename T>
__global__ void __launch_bounds__(128) kv_norm_cache_write_kernel(const T* __restrict__ qkv, int stride, const int* __restrict__ positions,
                                                                  const int* __restrict__ token_row, int H, int Hkv, int D, int norm_dim,
                                                                  float eps, T* __restrict__ kc, T* __restrict__ vc,
                                                                  const int* __restrict__ block_table, int bt_width, int ps, int num_pages,
                                                                  int n_tokens, int* __restrict__ errors) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (wid >= (long long)n_tokens * Hkv) return;
  const int t = (int)(wid / Hkv), hk = (int)(wid - (long long)t * Hkv);
  const int pos = positions[t], blk = pos / ps;
  const int page = (blk < bt_width && pos >= 0) ? block_table[(size_t)token_row[t] * bt_width + blk] : -1;
  if (page < 0 || page >= num_pages) {
    if (lane == 0) atomicAdd(errors, 1);
    return;
  }
  const T* krow = qkv + (size_t)t * stride + (size_t)(H + hk) * D;
  const T* vrow = qkv + (size_t)t * stride + (size_t)(H + Hkv + hk) * D;
  const size_t dst = (((size_t)page * Hkv + hk) * ps + (pos - blk * ps)) * D;
  float inv = 1.f;
  if (norm_dim > 0) {
    float ss = 0.f;
    for (int d = lane; d < norm_dim; d += 32) {
      const float v = to_float(vrow[d]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)norm_dim + eps);
  }
  for (int d = lane; d < D; d += 32) {
    kc[dst + d] = krow[d];
    vc[dst + d] = from_float<T>(to_float(vrow[d]) * inv);
  }
}

// ------------------------------------------------------------------------------------------ token shift
// out[m, t, c] = x[t, c] + (x[t - 1, c] - x[t, c]) * mu[m, c] for each of n_mix blends; before a row's first token stands
// the row's state (float [slots, C]: the input of the request's last token so far, zeros at the start). A thread per
// (token, channel) computes every blend of it. With one token a row (pure_decode) the same thread then stores its
// input as the new state; otherwise token_shift_state_kernel does, in a launch of its own after every read.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) token_shift_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ mu, int n_mix,
                                                          float* __restrict__ state, long long slot_stride, const int* __restrict__ slots,
                                                          const int* __restrict__ cu_q, const int* __restrict__ token_row,
                                                          T* __restrict__ out, long long mix_stride, int out_stride, int C, int pure_decode) {
  // VEC neighbouring channels a thread (16 bytes of activations at a time when VEC > 1; the launcher checks the alignment)
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= C) return;
  const int r = token_row[t];
  float* st = state + (size_t)slots[r] * slot_stride + c;
  const bool first = t <= cu_q[r];
  float cur[VEC], d[VEC];
  if (VEC > 1) {
    __align__(16) T a[VEC];
    __align__(16) T b[VEC];
    *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(x + (size_t)t * x_stride + c);
    if (!first) *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(x + (size_t)(t - 1) * x_stride + c);
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      cur[v] = to_float(a[v]);
      d[v] = (first ? st[v] : to_float(b[v])) - cur[v];
    }
  } else {
    cur[0] = to_float(x[(size_t)t * x_stride + c]);
    d[0] = (first ? st[0] : to_float(x[(size_t)(t - 1) * x_stride + c])) - cur[0];
  }
  for (int m = 0; m < n_mix; ++m) {
    __align__(16) T o[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) o[v] = from_float<T>(cur[v] + d[v] * mu[(size_t)m * C + c + v]);
    T* dst = out + (size_t)m * mix_stride + (size_t)t * out_stride + c;
    if (VEC > 1) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
    else dst[0] = o[0];
  }
  if (pure_decode) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) st[v] = cur[v];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) token_shift_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                                                long long slot_stride, const int* __restrict__ slots,
                                                                const int* __restrict__ cu_q, int C) {
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int last = cu_q[r + 1] - 1;
  if (c >= C || last < cu_q[r]) return;
  state[(size_t)slots[r] * slot_stride + c] = to_float(x[(size_t)last * x_stride + c]);
}

}  // namespace

// x [T, C] (row stride x_stride), mu float [n_mix, C], state float [slots, C] (slots slot_stride floats apart), out
// [n_mix, T, C] (blends mix_stride apart, rows out_stride apart).
SB_EXPORT int sb_token_shift(const void* x, int x_stride, const float* mu, int n_mix, float* state, long long slot_stride, const int* slots,
                             const int* cu_q, const int* token_row, void* out, long long mix_stride, int out_stride, int C, int n_tokens,
                             int n_rows, int pure_decode, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0) return 0;
  if (n_mix <= 0 || !state || x == out) return SB_ERR_SHAPE;
  if (n_tokens > 65535 || n_rows > 65535 || n_rows <= 0) return SB_ERR_LIMIT;
  const int esz = dtype == SB_DTYPE_F32 ? 4 : 2, per = 16 / esz;
  const bool vec = C % per == 0 && x_stride % per == 0 && out_stride % per == 0 && mix_stride % per == 0 && aligned16(x) && aligned16(out);
  dim3 sgrid((C + 255) / 256, n_rows), grid(vec ? (C / per + 255) / 256 : (C + 255) / 256, n_tokens);
  if (dtype == SB_DTYPE_F32) {
    auto k = vec ? token_shift_kernel<float, 4> : token_shift_kernel<float, 1>;
    k<<<grid, 256, 0, stream>>>((const float*)x, x_stride, mu, n_mix, state, slot_stride, slots, cu_q, token_row, (float*)out, mix_stride,
                                out_stride, C, pure_decode);
    SB_LAUNCH_CHECK();
    if (!pure_decode) token_shift_state_kernel<float><<<sgrid, 256, 0, stream>>>((const float*)x, x_stride, state, slot_stride, slots, cu_q, C);
  } else if (dtype == SB_DTYPE_BF16) {
    typedef __nv_bfloat16 B;
    auto k = vec ? token_shift_kernel<B, 8> : token_shift_kernel<B, 1>;
    k<<<grid, 256, 0, stream>>>((const B*)x, x_stride, mu, n_mix, state, slot_stride, slots, cu_q, token_row, (B*)out, mix_stride, out_stride,
                                C, pure_decode);
    SB_LAUNCH_CHECK();
    if (!pure_decode) token_shift_state_kernel<B><<<sgrid, 256, 0, stream>>>((const B*)x, x_stride, state, slot_stride, slots, cu_q, C);
  } else {
    return SB_ERR_DTYPE;
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// x [T, C] (row stride x_stride), w [C, taps], bias [C] or null, state float [slots, taps - 1, C], out [T, C].
// act: 0 none, 1 silu. residual: the input itself is added before the activation. A step in which every row brings one
// token (pure_decode) moves the state in the same launch; otherwise a second launch does, after every read.
SB_EXPORT int sb_causal_conv(const void* x, int x_stride, const void* w, const void* bias, float* state, const int* slots,
                             const int* cu_q, const int* token_row, void* out, int out_stride, int C, int taps, int act, int residual,
                             int n_tokens, int n_rows, int pure_decode, long long slot_stride, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS || n_rows <= 0 || n_rows > 65535 || n_tokens > 65535 * 32) return SB_ERR_LIMIT;
  if (x == out) return SB_ERR_SHAPE;
  dim3 grid((C + CONV_THREADS - 1) / CONV_THREADS, n_tokens), sgrid(grid.x, n_rows);
  if (grid.y > 65535) return SB_ERR_LIMIT;
  if (dtype == SB_DTYPE_F32) {
    causal_conv_kernel<float><<<grid, CONV_THREADS, 0, stream>>>((const float*)x, x_stride, (const float*)w, (const float*)bias, state,
                                                                  slots, cu_q, token_row, (float*)out, out_stride, C, taps, act, residual,
                                                                  pure_decode, slot_stride);
    SB_LAUNCH_CHECK();
    if (!pure_decode && taps > 1)
      conv_state_kernel<float><<<sgrid, CONV_THREADS, 0, stream>>>((const float*)x, x_stride, state, slots, cu_q, C, taps, slot_stride);
  } else if (dtype == SB_DTYPE_BF16) {
    typedef __nv_bfloat16 B;
    const bool by8 = C % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 && aligned16(x) && aligned16(out) &&
                     (!state || (aligned16(state) && slot_stride % 4 == 0));
    if (by8) {
      auto k8 = causal_conv8_kernel<0>;
      if (aligned16(w)) k8 = taps == 2 ? causal_conv8_kernel<2> : taps == 3 ? causal_conv8_kernel<3> : taps == 4 ? causal_conv8_kernel<4> : k8;
      k8<<<dim3((C / 8 + CONV_THREADS - 1) / CONV_THREADS, n_tokens), CONV_THREADS, 0, stream>>>(
          (const B*)x, x_stride, (const B*)w, (const B*)bias, state, slots, cu_q, token_row, (B*)out, out_stride, C, taps, act, residual,
          pure_decode, slot_stride);
    } else
      causal_conv_kernel<B><<<grid, CONV_THREADS, 0, stream>>>((const B*)x, x_stride, (const B*)w, (const B*)bias, state, slots, cu_q,
                                                                token_row, (B*)out, out_stride, C, taps, act, residual, pure_decode, slot_stride);
    SB_LAUNCH_CHECK();
    if (!pure_decode && taps > 1)
      conv_state_kernel<B><<<sgrid, CONV_THREADS, 0, stream>>>((const B*)x, x_stride, state, slots, cu_q, C, taps, slot_stride);
  } else {
    return SB_ERR_DTYPE;
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// Floats of work space sb_linear_recurrence needs for a step of n_tokens tokens.
SB_EXPORT long long sb_linear_recurrence_work_floats(int mode, int n_tokens, int H, int Hqk, int dk, int dv) {
  if (dk <= 0 || dk > 32 * REC_RPT) return -1;
  return rec_work_floats(mode, n_tokens, H, Hqk, dk, dv);
}

// The recurrences (mode 0: fixed decay per head with silu on q, k, v; 1: selective state space; 2: gated delta rule, its
// rate per row of the state or, with rate_per_head, per head; 3: decay per key channel with a bonus [H, dk] for the
// current token, read out before the update). See RecArgs for what each pointer is; unused ones are null. ``rate`` has a
// dtype of its own (rate_dtype). out is float [T, H * dv]; work: 16-byte aligned floats,
// as many as sb_linear_recurrence_work_floats says.
SB_EXPORT int sb_linear_recurrence(int mode, const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                                   const void* aux, int aux_stride, const void* rate, int rate_stride, int rate_dtype, int rate_per_head,
                                   const float* bonus, const float* decay, const void* a_log, const void* dt_bias, const void* d_skip, int par_dtype, float* state,
                                   const int* slots, const int* cu_q, float* out, int out_stride, int H, int Hqk, int dk, int dv,
                                   float q_scale, int n_rows, int n_tokens, float* work, long long state_stride, int dtype, float rate_scale,
                                   cudaStream_t stream) {
  if (n_rows <= 0 || n_tokens <= 0) return 0;
  if (!work || !aligned16(work)) return SB_ERR_ALIGN;
  if (H <= 0 || Hqk <= 0 || H % Hqk || dk <= 0 || dv <= 0) return SB_ERR_SHAPE;
  if (n_rows > 65535 || H > 65535 || dk > 32 * REC_RPT) return SB_ERR_LIMIT;
  if (mode == MODE_WKV && (H != Hqk || !rate || !dt_bias || !bonus)) return SB_ERR_SHAPE;
  if (mode == MODE_GLA && (!rate || !dt_bias)) return SB_ERR_SHAPE;
  if (rate && rate_dtype != SB_DTYPE_F32 && rate_dtype != SB_DTYPE_BF16) return SB_ERR_DTYPE;
  RecArgs a;
  a.q = q; a.k = k; a.v = v; a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.aux = aux; a.aux_stride = aux_stride; a.rate = rate; a.rate_stride = rate_stride; a.rate_dtype = rate_dtype;
  a.rate_per_head = rate_per_head; a.bonus = bonus; a.decay = decay;
  a.a_log = a_log; a.dt_bias = dt_bias; a.d_skip = d_skip; a.par_dtype = par_dtype; a.state = state; a.state_stride = state_stride; a.slots = slots; a.cu_q = cu_q;
  a.out = out; a.out_stride = out_stride; a.H = H; a.Hqk = Hqk; a.dk = dk; a.dv = dv; a.P = 1; a.dkp = a.dvp = 0; a.n_tokens = n_tokens;
  a.q_scale = q_scale; a.rate_scale = rate_scale; a.qf = a.kf = a.af = a.vf = a.sc = a.dec = nullptr;
  if (dtype == SB_DTYPE_F32) {
    if (mode == MODE_DECAY) return launch_recurrence<float, MODE_DECAY>(a, work, n_rows, stream);
    if (mode == MODE_SSM) return launch_recurrence<float, MODE_SSM>(a, work, n_rows, stream);
    if (mode == MODE_DELTA) return launch_recurrence<float, MODE_DELTA>(a, work, n_rows, stream);
    if (mode == MODE_WKV) return launch_recurrence<float, MODE_WKV>(a, work, n_rows, stream);
    if (mode == MODE_GLA) return launch_recurrence<float, MODE_GLA>(a, work, n_rows, stream);
  } else if (dtype == SB_DTYPE_BF16) {
    if (mode == MODE_DECAY) return launch_recurrence<__nv_bfloat16, MODE_DECAY>(a, work, n_rows, stream);
    if (mode == MODE_SSM) return launch_recurrence<__nv_bfloat16, MODE_SSM>(a, work, n_rows, stream);
    if (mode == MODE_DELTA) return launch_recurrence<__nv_bfloat16, MODE_DELTA>(a, work, n_rows, stream);
    if (mode == MODE_WKV) return launch_recurrence<__nv_bfloat16, MODE_WKV>(a, work, n_rows, stream);
    if (mode == MODE_GLA) return launch_recurrence<__nv_bfloat16, MODE_GLA>(a, work, n_rows, stream);
  } else {
    return SB_ERR_DTYPE;
  }
  return SB_ERR_SHAPE;
}

// y [T, C], float or the activations' type (y_dtype); gate [T, gate_cols] or null (gate_act 0 sigmoid, 1 silu; gate_first: before the norm); weight [w_size]
// or null (w_size divides C); groups > 0: each of the groups equal parts of a row is divided by its own root mean square.
SB_EXPORT int sb_gated_norm(const void* y, int y_dtype, int y_stride, const void* gate, int gate_stride, int gate_cols, int gate_act, int gate_first,
                            const void* weight, int w_dtype, int w_size, void* out, int out_stride, int n_tokens, int C, int groups,
                            float eps, float scale, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0) return 0;
  const int normalise = groups > 0 ? 1 : 0;
  if (groups <= 0) groups = gate ? gate_cols : 1;
  if (C % groups || (gate && (gate_cols <= 0 || C % gate_cols)) || (weight && (w_size <= 0 || C % w_size))) return SB_ERR_SHAPE;
  const long long warps = (long long)n_tokens * groups;
  {   // the recurrent read-outs' shape on the kernel that moves 16 bytes a lane
    const int gs = C / groups, esz = dtype == SB_DTYPE_F32 ? 4 : 2, wsz = w_dtype == SB_DTYPE_F32 ? 4 : 2;
    const bool fits = normalise && y_dtype == SB_DTYPE_F32 && gs <= 512 && gs % 4 == 0 && y_stride % 4 == 0 && out_stride % 4 == 0 &&
                      aligned16(y) && (reinterpret_cast<uintptr_t>(out) % (4 * esz)) == 0 &&
                      (!gate || (!gate_first && gate_cols == C && gate_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(gate) % (4 * esz)) == 0)) &&
                      (!weight || (w_size % gs == 0 && (reinterpret_cast<uintptr_t>(weight) % (4 * wsz)) == 0 &&
                                   (w_dtype == SB_DTYPE_F32 || w_dtype == SB_DTYPE_BF16))) &&
                      (dtype == SB_DTYPE_F32 || dtype == SB_DTYPE_BF16) && warps <= 0x7fff0000LL;
    if (fits) {
      int lpg = 1;
      while (lpg * 16 < gs) lpg <<= 1;                                // four rounds of four values a lane cover the group
      const int per_block = 4 * (32 / lpg);
      const unsigned nb = (unsigned)((warps + per_block - 1) / per_block);
#define SB_GNV(T, W)                                                                                                            \
  gated_norm_vec_kernel<T, W><<<nb, 128, 0, stream>>>((const float*)y, y_stride, (const T*)gate, gate_stride, gate_act, (const W*)weight, \
                                                      weight ? w_size : gs, (T*)out, out_stride, (int)warps, gs, groups, lpg, eps, scale)
      if (dtype == SB_DTYPE_F32) {
        if (w_dtype == SB_DTYPE_F32) SB_GNV(float, float); else SB_GNV(float, __nv_bfloat16);
      } else {
        if (w_dtype == SB_DTYPE_F32) SB_GNV(__nv_bfloat16, float); else SB_GNV(__nv_bfloat16, __nv_bfloat16);
      }
#undef SB_GNV
      SB_LAUNCH_CHECK();
      return 0;
    }
  }
  const bool wide = C / groups > 512;                     // a block per group
  const long long blocks = wide ? warps : (warps + 3) / 4;
  if (blocks > 0x7fffffffLL) return SB_ERR_LIMIT;
  if (wide) {
    if (dtype == SB_DTYPE_F32)
      gated_norm_kernel<float, 128><<<(unsigned)blocks, 128, 0, stream>>>(y, y_dtype, y_stride, (const float*)gate, gate_stride, gate_cols,
                                                                           gate_act, gate_first, weight, w_dtype, w_size, (float*)out,
                                                                           out_stride, n_tokens, C, groups, normalise, eps, scale);
    else if (dtype == SB_DTYPE_BF16)
      gated_norm_kernel<__nv_bfloat16, 128><<<(unsigned)blocks, 128, 0, stream>>>(
          y, y_dtype, y_stride, (const __nv_bfloat16*)gate, gate_stride, gate_cols, gate_act, gate_first, weight, w_dtype, w_size,
          (__nv_bfloat16*)out, out_stride, n_tokens, C, groups, normalise, eps, scale);
    else
      return SB_ERR_DTYPE;
    SB_LAUNCH_CHECK();
    return 0;
  }
  if (dtype == SB_DTYPE_F32)
    gated_norm_kernel<float, 32><<<(unsigned)blocks, 128, 0, stream>>>(y, y_dtype, y_stride, (const float*)gate, gate_stride, gate_cols, gate_act,
                                                                    gate_first, weight, w_dtype, w_size, (float*)out, out_stride, n_tokens,
                                                                    C, groups, normalise, eps, scale);
  else if (dtype == SB_DTYPE_BF16)
    gated_norm_kernel<__nv_bfloat16, 32><<<(unsigned)blocks, 128, 0, stream>>>(y, y_dtype, y_stride, (const __nv_bfloat16*)gate, gate_stride, gate_cols,
                                                                            gate_act, gate_first, weight, w_dtype, w_size,
                                                                            (__nv_bfloat16*)out, out_stride, n_tokens, C, groups, normalise,
                                                                            eps, scale);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_kv_norm_cache_write(const void* qkv, int stride, const int* positions, const int* token_row, int H, int Hkv, int D,
                                     int norm_dim, float eps, void* kc, void* vc, const int* block_table, int bt_width, int ps,
                                     int num_pages, int n_tokens, int* errors, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H < 0 || Hkv <= 0 || D <= 0 || norm_dim < 0 || norm_dim > D || ps <= 0 || bt_width <= 0) return SB_ERR_SHAPE;
  const long long blocks = ((long long)n_tokens * Hkv + 3) / 4;
  if (blocks > 0x7fffffffLL) return SB_ERR_LIMIT;
  if (dtype == SB_DTYPE_F32)
    kv_norm_cache_write_kernel<float><<<(unsigned)blocks, 128, 0, stream>>>((const float*)qkv, stride, positions, token_row, H, Hkv, D,
                                                                             norm_dim, eps, (float*)kc, (float*)vc, block_table, bt_width,
                                                                             ps, num_pages, n_tokens, errors);
  else if (dtype == SB_DTYPE_BF16)
    kv_norm_cache_write_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, stream>>>(
        (const __nv_bfloat16*)qkv, stride, positions, token_row, H, Hkv, D, norm_dim, eps, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc,
        block_table, bt_width, ps, num_pages, n_tokens, errors);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}
