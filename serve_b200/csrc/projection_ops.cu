// What sits between a mixer's input projection and its attention, for mixers that do not rotate all of every head:
//
//   sb_add_layernorm          x += delta; out = (x - mean) / sqrt(var + eps) * weight   (float residual stream)
//   sb_normed_qk_cache_write  queries and keys divided by the root mean square of the token's whole projection (all
//                             heads at once) and multiplied by a weight, queries also by a temperature that grows
//                             with the logarithm of the position; keys and values into their cache pages
//   sb_latent_prepare         latent attention: the latent vector normalised, the shared key part and every head's
//                             rotated query part turned by position; one cache row per token
//   sb_gated_activation       act(gate, up) of a fused gate/up product: silu(g) * u, the clamped form
//                             g <- min(g, limit), u <- clamp(u, -limit, limit), g * sigmoid(alpha g) * (u + 1), or
//                             gelu(g) * u with the tanh form of gelu
//   sb_embedding_pair         x = table[token] * scale + pair_table[row], the row a hash of the token and the one before
//                             it; a request's last token is kept per state slot for its next portion
//   sb_bias_round             float sums + bias, rounded once to the activations' type
//   sb_softcap                l <- c * tanh(l / c) on float logits
//
// All arithmetic is float: sums of squares, means, the logarithm, angles (float(position) * frequency, full-precision
// sincosf) and the activation; T is the storage type of activations and cache pages. Reductions run in a fixed order
// that depends on the block size only, never on the batch.
#include "common.cuh"

using namespace sb;

namespace {

template <typename T> __device__ __forceinline__ float4 load4f(const T* p);
template <> __device__ __forceinline__ float4 load4f<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4f<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void store4f(T* p, float4 v);
template <> __device__ __forceinline__ void store4f<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4f<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// ------------------------------------------------------------------------------------------- add + layer norm
// One block per row; the row (after the addition) is kept in shared memory between the three passes: mean, mean of
// squared deviations, output. With rows != nullptr, row b of the output comes from x[rows[b]] and x is not written.
// VEC: four elements at a time (dim a multiple of 4, aligned pointers).
template <typename T, typename W, bool VEC>
__global__ void add_layernorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const int* __restrict__ rows,
                                     const W* __restrict__ weight, T* __restrict__ out, int dim, float eps) {
  __shared__ float red[32];
  extern __shared__ __align__(16) float rowbuf[];
  const int b = blockIdx.x;
  const int src_row = rows ? rows[b] : b;
  float* xr = x + (size_t)src_row * dim;
  const T* dr = delta ? delta + (size_t)src_row * dim : nullptr;
  const bool write_x = !rows && dr;
  float s = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + i);
      if (dr) {
        const float4 d = load4f<T>(dr + i);
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
      }
      *reinterpret_cast<float4*>(rowbuf + i) = v;
      if (write_x) *reinterpret_cast<float4*>(xr + i) = v;
      s += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      float v = xr[i];
      if (dr) v += to_float(dr[i]);
      rowbuf[i] = v;
      if (write_x) xr[i] = v;
      s += v;
    }
  }
  const float mean = block_sum(s, red) / (float)dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {      // (the barriers inside block_sum have published the row)
    const float d = rowbuf[i] - mean;
    ss += d * d;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)dim + eps);
  T* orow = out + (size_t)b * dim;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(rowbuf + i);
      const float4 w = load4f<W>(weight + i);
      store4f<T>(orow + i, make_float4((v.x - mean) * inv * w.x, (v.y - mean) * inv * w.y, (v.z - mean) * inv * w.z, (v.w - mean) * inv * w.w));
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) orow[i] = from_float<T>((rowbuf[i] - mean) * inv * to_float(weight[i]));
  }
}

template <typename T, typename W>
int launch_add_layernorm(float* x, const void* delta, const int* rows, const void* weight, void* out, int n_rows, int dim, float eps,
                         cudaStream_t stream) {
  const size_t smem = (size_t)dim * sizeof(float);
  if (smem > 200 * 1024) return SB_ERR_LIMIT;
  const bool vec = (dim % 4) == 0 && aligned16(x) && aligned16(out) && aligned16(weight) && (!delta || aligned16(delta));
  const int threads = dim >= 4096 ? 512 : (dim >= 1024 ? 256 : 128);
  auto k = vec ? add_layernorm_kernel<T, W, true> : add_layernorm_kernel<T, W, false>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  k<<<n_rows, threads, smem, stream>>>(x, (const T*)delta, rows, (const W*)weight, (T*)out, dim, eps);
  SB_LAUNCH_CHECK();
  return 0;
}

// --------------------------------------------------------------------- whole-projection norm, temperature, cache write
// proj [T, (H + 2 G) * D] (row stride given): H query heads, G key heads, G value heads, each padded to D elements (the
// padding holds zeros). One block per token.
template <typename T>
__global__ void __launch_bounds__(256) normed_qk_cache_write_kernel(
    T* __restrict__ proj, int stride, const int* __restrict__ positions, const int* __restrict__ token_row, int H, int G, int D,
    int dim, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps, float temp_coef, int temp_every,
    T* __restrict__ kc, T* __restrict__ vc, const int* __restrict__ block_table, int bt_width, int ps, int num_pages, int write_cache,
    int* __restrict__ errors) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  T* row = proj + (size_t)t * stride;
  const int nq = H * D, nk = G * D;
  const int pos = positions[t];
  float inv_q = 1.f, inv_k = 1.f;
  if (q_weight != nullptr) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = to_float(row[i]); sq += v * v; }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = to_float(row[nq + i]); sk += v * v; }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    inv_q = 1.0f / sqrtf(sq / (float)(H * dim) + eps);
    inv_k = 1.0f / sqrtf(sk / (float)(G * dim) + eps);
  }
  float temp = 1.f;
  if (temp_coef != 0.f) temp = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
  for (int i = threadIdx.x; i < nq; i += blockDim.x) {
    float v = to_float(row[i]);
    if (q_weight != nullptr) v = v * inv_q * q_weight[i];
    row[i] = from_float<T>(v * temp);
  }
  if (!write_cache) return;
  const int blk = pos / ps;
  const int page = (pos >= 0 && blk < bt_width) ? block_table[(size_t)token_row[t] * bt_width + blk] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicAdd(errors, 1);
    return;
  }
  const int within = pos - blk * ps;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    const size_t off = (((size_t)page * G + g) * ps + within) * D + d;
    float kv = to_float(row[nq + i]);
    if (k_weight != nullptr) kv = kv * inv_k * k_weight[i];
    kc[off] = from_float<T>(kv);
    vc[off] = row[nq + nk + i];
  }
}

// ------------------------------------------------------------------------------------------------ latent attention
// proj [T, stride]: columns [0, n_q) are H query heads of (dim + rd) each, [n_q, n_q + rank) the latent vector, then rd
// of the shared key part. Writes, per token: the row [c * inv_rms * weight | rotated key part | zeros] of D elements into
// the cache (one key/value head) and, if asked, into row_out [T, row_stride] (its first rank + rd columns); and for every
// head columns [q_off, D) of q_lat (rows q_stride apart, heads D apart): the rotated query part, then zeros (columns
// [0, q_off) are made elsewhere: the product of the plain query part with the keys' read-out matrix when q_off = rank,
// the plain query part itself when q_off = dim). With ``lat`` the latent vector and the shared key part come from a buffer
// of their own [T, lat_stride] (its first rank + rd columns) instead of the columns after the queries.
// Rotation: pairs (2 i, 2 i + 1), or with half_pairs (i, i + rot_dims / 2), i < rot_dims / 2, angle = float(position) *
// inv_freq[i]; the rest passes unchanged.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(
    const T* __restrict__ proj, int stride, int n_q, const int* __restrict__ positions, const int* __restrict__ token_row,
    const float* __restrict__ c_weight, float eps, const float* __restrict__ inv_freq, int rot_dims, int H, int dim, int rd, int rank,
    int D, T* __restrict__ q_lat, int q_stride, int q_off, T* __restrict__ row_out, int row_stride, T* __restrict__ kc,
    const int* __restrict__ block_table, int bt_width, int ps, int num_pages, int write_cache, int* __restrict__ errors, int half_pairs,
    const T* __restrict__ lat, int lat_stride) {
  __shared__ float red[32];
  extern __shared__ float cs[];            // [rot_dims / 2][2]: cosine and sine of the token's angles
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * stride;
  // the latent vector and the shared key part: columns n_q .. of proj, or a buffer of their own
  const T* lrow = lat ? lat + (size_t)t * lat_stride : row + n_q;
  const int pos = positions[t];
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cs[2 * i] = c;
    cs[2 * i + 1] = s;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_float(lrow[i]); ss += v * v; }
  ss = block_sum(ss, red);                 // (its barriers also publish cs)
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  // element j of a rotated part whose plain values start at src
  auto rotated = [&](const T* src, int j) -> float {
    if (j >= rot_dims) return to_float(src[j]);
    if (half_pairs) {
      const int i = j < half ? j : j - half;
      const float u = to_float(src[i]), v = to_float(src[i + half]);
      return j < half ? u * cs[2 * i] - v * cs[2 * i + 1] : v * cs[2 * i] + u * cs[2 * i + 1];
    }
    const int i = j >> 1;
    const float u = to_float(src[2 * i]), v = to_float(src[2 * i + 1]);
    return (j & 1) ? v * cs[2 * i] + u * cs[2 * i + 1] : u * cs[2 * i] - v * cs[2 * i + 1];
  };
  const int tail = D - q_off;              // columns of a head from the rotated part on
  for (int w = threadIdx.x; w < H * tail; w += blockDim.x) {
    const int h = w / tail, j = w - h * tail;
    const float v = j < rd ? rotated(row + (size_t)h * (dim + rd) + dim, j) : 0.f;
    q_lat[(size_t)t * q_stride + (size_t)h * D + q_off + j] = from_float<T>(v);
  }
  if (row_out != nullptr) {
    for (int i = threadIdx.x; i < rank + rd; i += blockDim.x) {
      const float v = i < rank ? to_float(lrow[i]) * inv * c_weight[i] : rotated(lrow + rank, i - rank);
      row_out[(size_t)t * row_stride + i] = from_float<T>(v);
    }
  }
  if (!write_cache) return;
  const int blk = pos / ps;
  const int page = (pos >= 0 && blk < bt_width) ? block_table[(size_t)token_row[t] * bt_width + blk] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicAdd(errors, 1);
    return;
  }
  const int Dc = rank + rd <= D ? D : 0;   // (a cache row is written only where it fits: the caller checks)
  T* dst = kc + ((size_t)page * ps + (pos - blk * ps)) * Dc;
  for (int i = threadIdx.x; i < Dc; i += blockDim.x) {
    float v = 0.f;
    if (i < rank) v = to_float(lrow[i]) * inv * c_weight[i];
    else if (i < rank + rd) v = rotated(lrow + rank, i - rank);
    dst[i] = from_float<T>(v);
  }
}

// ------------------------------------------------------------------------------------------------ gated activation
__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

// gate_up [T, 2 I] (gate columns, then up columns) -> out [T, I]. kind 0: silu(g) * u; 1: the clamped form; 2: gelu(g) * u.
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total, int kind, float limit,
                                        float alpha) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    float g = to_float(gate_up[t * 2 * inter + i]);
    float u = to_float(gate_up[t * 2 * inter + inter + i]);
    float y;
    if (kind == 1) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      y = g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
    } else if (kind == 2) {
      y = gelu_tanh_f(g) * u;
    } else {
      y = g / (1.0f + expf(-g)) * u;
    }
    out[idx] = from_float<T>(y);
  }
}

// bfloat16, 8 outputs a thread (16 bytes of gate, 16 of up)
__global__ void gated_activation_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter8,
                                                 size_t total8, int kind, float limit, float alpha) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter8;
    const int i = (int)(idx - t * inter8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + (t * 2 * inter8 + i) * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + (t * 2 * inter8 + inter8 + i) * 8);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
      float y0, y1;
      if (kind == 1) {
        g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
        u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
        y0 = g.x / (1.0f + expf(-alpha * g.x)) * (u.x + 1.0f);
        y1 = g.y / (1.0f + expf(-alpha * g.y)) * (u.y + 1.0f);
      } else if (kind == 2) {
        y0 = gelu_tanh_f(g.x) * u.x;
        y1 = gelu_tanh_f(g.y) * u.y;
      } else {
        y0 = g.x / (1.0f + expf(-g.x)) * u.x;
        y1 = g.y / (1.0f + expf(-g.y)) * u.y;
      }
      o2[k] = __floats2bfloat162_rn(y0, y1);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = ov;
  }
}

// ------------------------------------------------------------------------------------------------ dynamic tanh
// A norm without statistics: y = tanh(alpha * x) * w + b, every element on its own; par = [w (dim) | b (dim) | alpha].
//   x given:  v = x[row] (+ d), d = delta[row] or, with ``through`` (the parameters of the norm the delta still has to
//             pass), tanh(alpha' delta[row]) w' + b'; x[row] = v unless rows are picked; out = dyt(v)
//   x null:   out = dyt(delta)
// Float arithmetic throughout; delta and out have dtypes of their own.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256) dynamic_tanh_kernel(float* __restrict__ x, const TD* __restrict__ delta, const float* __restrict__ through,
                                                           const int* __restrict__ rows, const float* __restrict__ par, TO* __restrict__ out,
                                                           int n_rows, int dim) {
  const float alpha = par[2 * dim];
  const float alpha_d = through ? through[2 * dim] : 0.f;
  const size_t total = (size_t)n_rows * dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / dim), c = (int)(i - (size_t)r * dim);
    const size_t src = (size_t)(rows ? rows[r] : r) * dim + c;
    float v;
    if (x) {
      v = x[src];
      if (delta) {
        float d = to_float(delta[src]);
        if (through) d = tanhf(alpha_d * d) * through[c] + through[dim + c];
        v += d;
        if (!rows) x[src] = v;
      }
    } else {
      v = to_float(delta[src]);
    }
    out[i] = from_float<TO>(tanhf(alpha * v) * par[c] + par[dim + c]);
  }
}

// The same, four elements a thread with 16-byte (8-byte for bfloat16) loads and stores: dim a multiple of 4 and every
// pointer aligned to 16 bytes.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256) dynamic_tanh_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                                               const float* __restrict__ through, const int* __restrict__ rows,
                                                               const float* __restrict__ par, TO* __restrict__ out, int n_rows, int dim) {
  const float alpha = par[2 * dim];
  const float alpha_d = through ? through[2 * dim] : 0.f;
  const int dim4 = dim >> 2;
  const size_t total4 = (size_t)n_rows * dim4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / dim4), c = (int)(i - (size_t)r * dim4) * 4;
    const size_t src = (size_t)(rows ? rows[r] : r) * dim + c;
    float4 v;
    if (x) {
      v = *reinterpret_cast<const float4*>(x + src);
      if (delta) {
        float4 d = load4f<TD>(delta + src);
        if (through) {
          const float4 w = *reinterpret_cast<const float4*>(through + c), b = *reinterpret_cast<const float4*>(through + dim + c);
          d.x = tanhf(alpha_d * d.x) * w.x + b.x; d.y = tanhf(alpha_d * d.y) * w.y + b.y;
          d.z = tanhf(alpha_d * d.z) * w.z + b.z; d.w = tanhf(alpha_d * d.w) * w.w + b.w;
        }
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        if (!rows) *reinterpret_cast<float4*>(x + src) = v;
      }
    } else {
      v = load4f<TD>(delta + src);
    }
    const float4 w = *reinterpret_cast<const float4*>(par + c), b = *reinterpret_cast<const float4*>(par + dim + c);
    float4 o;
    o.x = tanhf(alpha * v.x) * w.x + b.x; o.y = tanhf(alpha * v.y) * w.y + b.y;
    o.z = tanhf(alpha * v.z) * w.z + b.z; o.w = tanhf(alpha * v.w) * w.w + b.w;
    store4f<TO>(out + (size_t)r * dim + c, o);
  }
}

// ------------------------------------------------------------------------------------- activations, bias, on their own
constexpr int ACT_RELU_SQUARED = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_TANH = 3;

__device__ __forceinline__ float activate(float z, int kind) {
  if (kind == ACT_RELU_SQUARED) { const float r = fmaxf(z, 0.f); return r * r; }
  if (kind == ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  if (kind == ACT_SILU) return z / (1.f + expf(-z));
  return kind == ACT_TANH ? tanhf(z) : z;
}

// out = act(x [+ bias per column]), computed in float, rounded once; x and out may be the same buffer.
template <typename T>
__global__ void __launch_bounds__(256) activation_kernel(const T* x, const float* __restrict__ bias, T* out, size_t total, int cols, int kind) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float z = to_float(x[i]);
    if (bias) z += bias[i % cols];
    out[i] = from_float<T>(activate(z, kind));
  }
}

__global__ void __launch_bounds__(256) add_bias_kernel(float* __restrict__ x, const float* __restrict__ bias, size_t total, int cols) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) x[i] += bias[i % cols];
}

// ------------------------------------------------------------- bias, whole-projection norm, partial rotation, cache write
// sums float [T, (H + 2 G) * D] (row stride given): the float sums of the fused query | key | value projection, heads padded
// to D with zeros (G = 0: queries only). Per token, one block: add the bias; divide all queries together (and all keys
// together) by the root mean square over their H * dim (G * dim) true elements and multiply by a float weight laid out
// like the padded projection; rotate the first ``rot`` elements of every query and key head, element i with i + rot / 2,
// by the angle position * inv_freq[i]; queries to q_out [T, H * D], keys and values to their page. Everything is float
// until the one rounding at the store. The row (with its bias) and the token's cosines and sines are kept in shared
// memory, so the sums are read from memory once (rows of up to 200 KB). With head_norm every query and key head is
// instead divided, after its rotation, by its own root mean square over its dim true elements, without a weight.
template <typename T>
__global__ void __launch_bounds__(512) qk_prepare_kernel(
    const float* __restrict__ sums, int stride, const float* __restrict__ bias, const int* __restrict__ positions,
    const int* __restrict__ token_row, int H, int G, int D, int dim, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    float eps, const float* __restrict__ inv_freq, int rot, T* __restrict__ q_out, int q_stride, T* __restrict__ kc, T* __restrict__ vc,
    const int* __restrict__ block_table, int bt_width, int ps, int num_pages, int* __restrict__ errors, int head_norm) {
  __shared__ float red[32];
  extern __shared__ float dyn[];            // [half] cosines, [half] sines of this token's angles, then the token's row with its bias
  const int t = blockIdx.x;
  const float* row = sums + (size_t)t * stride;
  const int nq = H * D, nk = G * D, half = rot >> 1;
  const int n_all = nq + 2 * nk;
  float* cs_table = dyn;
  float* vals = dyn + (rot > 0 ? rot : 2);
  const int pos = positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &cs_table[half + j], &cs_table[j]);
  // one pass over the row: bias added, kept in shared memory, the squares of the query and of the key columns summed
  float sq = 0.f, sk = 0.f;
#pragma unroll 4      // (the loads of several rounds are in flight together: a decoding step has few blocks and waits on each)
  for (int i = threadIdx.x; i < n_all; i += blockDim.x) {
    const float v = row[i] + (bias ? bias[i] : 0.f);
    vals[i] = v;
    if (i < nq) sq += v * v;
    else if (i < nq + nk) sk += v * v;
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (q_weight != nullptr) inv_q = 1.0f / sqrtf(block_sum(sq, red) / (float)(H * dim) + eps);
  if (k_weight != nullptr && G > 0) inv_k = 1.0f / sqrtf(block_sum(sk, red) / (float)(G * dim) + eps);
  __syncthreads();                          // the table and the row are whole
  // A warp takes a head at a time, a lane an element; an element below rot / 2 is turned together with its partner rot / 2
  // further on, so every value is normalised once. Heads 0 .. H-1 are queries, the G after them keys.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int blk = ps > 0 ? pos / ps : 0;
  const int page = (G > 0 && pos >= 0 && blk < bt_width) ? block_table[(size_t)token_row[t] * bt_width + blk] : -1;
  const bool page_ok = page >= 0 && page < num_pages;
  if (G > 0 && !page_ok && threadIdx.x == 0) atomicAdd(errors, 1);
  const int within = pos - blk * ps;
  for (int head = warp; head < H + G; head += n_warps) {
    const bool is_q = head < H;
    if (!is_q && !page_ok) continue;
    const float* w = is_q ? q_weight : k_weight;
    const float inv = is_q ? inv_q : inv_k;
    const int base = head * D, w_base = is_q ? base : base - nq;
    T* dst = is_q ? q_out + (size_t)t * q_stride + base : kc + (((size_t)page * G + (head - H)) * ps + within) * D;
    if (head_norm) {
      // the head is turned in place in shared memory (a lane turns an element together with its partner), its squares are
      // summed over the warp, and the quotient is stored
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) {
        if (d >= half && d < rot) continue;
        float v = vals[base + d];
        if (d < half) {
          const float o = vals[base + d + half], cs = cs_table[d], sn = cs_table[half + d];
          const float a = v * cs - o * sn, b = o * cs + v * sn;
          vals[base + d] = a;
          vals[base + d + half] = b;
          ss += a * a + b * b;
        } else {
          ss += v * v;                                        // (zero beyond the head's true size)
        }
      }
      ss = warp_sum(ss);
      __syncwarp();
      const float inv_h = 1.0f / sqrtf(ss / (float)dim + eps);
      for (int d = lane; d < D; d += 32) dst[d] = from_float<T>(vals[base + d] * inv_h);
      continue;
    }
    for (int d = lane; d < D; d += 32) {
      if (d >= half && d < rot) continue;                    // written by its partner
      float v = vals[base + d];
      if (w) v *= inv * w[w_base + d];
      if (d < half) {
        float o = vals[base + d + half];
        if (w) o *= inv * w[w_base + d + half];
        const float cs = cs_table[d], sn = cs_table[half + d];
        dst[d] = from_float<T>(v * cs - o * sn);
        dst[d + half] = from_float<T>(o * cs + v * sn);
      } else {
        dst[d] = from_float<T>(v);
      }
    }
  }
  if (!page_ok) return;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    vc[(((size_t)page * G + g) * ps + within) * D + d] = from_float<T>(vals[nq + nk + i]);
  }
}

}  // namespace

template <typename TD, typename TO>
static int launch_dynamic_tanh(float* x, const void* delta, const float* through, const int* rows, const float* par, void* out, int n_rows,
                               int dim, cudaStream_t stream) {
  const bool vec = dim % 4 == 0 && (!x || aligned16(x)) && (!delta || aligned16(delta)) && (!through || aligned16(through)) &&
                   aligned16(par) && aligned16(out);
  const size_t total = (size_t)n_rows * (vec ? dim / 4 : dim), want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
  if (vec) dynamic_tanh_vec_kernel<TD, TO><<<blocks, 256, 0, stream>>>(x, (const TD*)delta, through, rows, par, (TO*)out, n_rows, dim);
  else dynamic_tanh_kernel<TD, TO><<<blocks, 256, 0, stream>>>(x, (const TD*)delta, through, rows, par, (TO*)out, n_rows, dim);
  SB_LAUNCH_CHECK();
  return 0;
}

// x float [*, dim] or null; delta [*, dim] of delta_dtype or null; through, par float [2 dim + 1]; rows int [n_rows] or null;
// out [n_rows, dim] of out_dtype.
SB_EXPORT int sb_add_dynamic_tanh(float* x, const void* delta, int delta_dtype, const float* through, const int* rows, const float* par,
                                  void* out, int out_dtype, int n_rows, int dim, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0 || !par || !out || (!x && !delta)) return SB_ERR_SHAPE;
  const bool df = delta == nullptr || delta_dtype == SB_DTYPE_F32;
  if (!df && delta_dtype != SB_DTYPE_BF16) return SB_ERR_DTYPE;
  if (out_dtype == SB_DTYPE_F32)
    return df ? launch_dynamic_tanh<float, float>(x, delta, through, rows, par, out, n_rows, dim, stream)
              : launch_dynamic_tanh<__nv_bfloat16, float>(x, delta, through, rows, par, out, n_rows, dim, stream);
  if (out_dtype == SB_DTYPE_BF16)
    return df ? launch_dynamic_tanh<float, __nv_bfloat16>(x, delta, through, rows, par, out, n_rows, dim, stream)
              : launch_dynamic_tanh<__nv_bfloat16, __nv_bfloat16>(x, delta, through, rows, par, out, n_rows, dim, stream);
  return SB_ERR_DTYPE;
}

// out = act(x + bias): x, out [n_rows, cols] (contiguous, may be the same buffer), bias float [cols] or null.
// kind: 0 relu squared, 1 gelu (tanh form), 2 silu, 3 tanh.
SB_EXPORT int sb_activation(const void* x, const float* bias, void* out, int n_rows, int cols, int kind, int dtype, cudaStream_t stream) {
  if (n_rows <= 0 || cols <= 0) return 0;
  if (kind < 0 || kind > 3) return SB_ERR_SHAPE;
  const size_t total = (size_t)n_rows * cols, want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
  if (dtype == SB_DTYPE_F32)
    activation_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, bias, (float*)out, total, cols, kind);
  else if (dtype == SB_DTYPE_BF16)
    activation_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, bias, (__nv_bfloat16*)out, total, cols, kind);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_add_bias(float* x, const float* bias, int n_rows, int cols, cudaStream_t stream) {
  if (n_rows <= 0 || cols <= 0) return 0;
  const size_t total = (size_t)n_rows * cols, want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
  add_bias_kernel<<<blocks, 256, 0, stream>>>(x, bias, total, cols);
  SB_LAUNCH_CHECK();
  return 0;
}

// bias float [(H + 2 G) * D] or null; q_weight float [H * D], k_weight float [G * D] or null (no norm of that side);
// inv_freq float [>= rot / 2]; G = 0 writes no cache.
SB_EXPORT int sb_qk_prepare(const float* sums, int stride, const float* bias, const int* positions, const int* token_row, int H, int G, int D,
                            int dim, const float* q_weight, const float* k_weight, float eps, const float* inv_freq, int rot, void* q_out,
                            int q_stride, void* kc, void* vc, const int* block_table, int bt_width, int ps, int num_pages, int* errors,
                            int n_tokens, int dtype, int head_norm, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G < 0 || D <= 0 || dim <= 0 || dim > D || stride < (H + 2 * G) * D || q_stride < H * D) return SB_ERR_SHAPE;
  if (rot < 0 || (rot & 1) || rot > dim || (rot > 0 && !inv_freq)) return SB_ERR_SHAPE;
  if (G > 0 && (ps <= 0 || bt_width <= 0 || !kc || !vc || !errors)) return SB_ERR_SHAPE;
  const size_t smem = ((size_t)(rot > 0 ? rot : 2) + (size_t)(H + 2 * G) * D) * sizeof(float);
  if (smem > 200 * 1024) return SB_ERR_LIMIT;
  const int threads = (H + 2 * G) * D >= 2048 ? 512 : 256;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(qk_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(qk_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  if (dtype == SB_DTYPE_F32)
    qk_prepare_kernel<float><<<n_tokens, threads, smem, stream>>>(sums, stride, bias, positions, token_row, H, G, D, dim, q_weight, k_weight, eps,
                                                            inv_freq, rot, (float*)q_out, q_stride, (float*)kc, (float*)vc, block_table,
                                                            bt_width, ps, num_pages, errors, head_norm);
  else if (dtype == SB_DTYPE_BF16)
    qk_prepare_kernel<__nv_bfloat16><<<n_tokens, threads, smem, stream>>>(sums, stride, bias, positions, token_row, H, G, D, dim, q_weight, k_weight,
                                                                    eps, inv_freq, rot, (__nv_bfloat16*)q_out, q_stride, (__nv_bfloat16*)kc,
                                                                    (__nv_bfloat16*)vc, block_table, bt_width, ps, num_pages, errors, head_norm);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_add_layernorm(float* x, const void* delta, const int* rows, const void* weight, int weight_dtype, void* out, int n_rows,
                               int dim, float eps, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (dim <= 0) return SB_ERR_SHAPE;
  if (dtype == SB_DTYPE_F32) {
    if (weight_dtype != SB_DTYPE_F32) return SB_ERR_DTYPE;
    return launch_add_layernorm<float, float>(x, delta, rows, weight, out, n_rows, dim, eps, stream);
  }
  if (dtype == SB_DTYPE_BF16) {
    if (weight_dtype == SB_DTYPE_F32) return launch_add_layernorm<__nv_bfloat16, float>(x, delta, rows, weight, out, n_rows, dim, eps, stream);
    if (weight_dtype == SB_DTYPE_BF16)
      return launch_add_layernorm<__nv_bfloat16, __nv_bfloat16>(x, delta, rows, weight, out, n_rows, dim, eps, stream);
  }
  return SB_ERR_DTYPE;
}

// q_weight, k_weight: float [H * D], [G * D] laid out like the padded projection, or both null (no norm).
SB_EXPORT int sb_normed_qk_cache_write(void* proj, int stride, const int* positions, const int* token_row, int H, int G, int D, int dim,
                                       const float* q_weight, const float* k_weight, float eps, float temp_coef, int temp_every, void* kc,
                                       void* vc, const int* block_table, int bt_width, int ps, int num_pages, int write_cache, int* errors,
                                       int n_tokens, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || D <= 0 || dim <= 0 || dim > D || temp_every <= 0 || stride < (H + 2 * G) * D) return SB_ERR_SHAPE;
  if ((q_weight == nullptr) != (k_weight == nullptr)) return SB_ERR_SHAPE;
  if (write_cache && (ps <= 0 || bt_width <= 0 || !kc || !vc || !errors)) return SB_ERR_SHAPE;
  if (dtype == SB_DTYPE_F32)
    normed_qk_cache_write_kernel<float><<<n_tokens, 256, 0, stream>>>((float*)proj, stride, positions, token_row, H, G, D, dim, q_weight,
                                                                       k_weight, eps, temp_coef, temp_every, (float*)kc, (float*)vc,
                                                                       block_table, bt_width, ps, num_pages, write_cache, errors);
  else if (dtype == SB_DTYPE_BF16)
    normed_qk_cache_write_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>(
        (__nv_bfloat16*)proj, stride, positions, token_row, H, G, D, dim, q_weight, k_weight, eps, temp_coef, temp_every, (__nv_bfloat16*)kc,
        (__nv_bfloat16*)vc, block_table, bt_width, ps, num_pages, write_cache, errors);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_latent_prepare(const void* proj, int stride, int n_q, const int* positions, const int* token_row, const float* c_weight,
                                float eps, const float* inv_freq, int rot_dims, int H, int dim, int rd, int rank, int D, void* q_lat,
                                int q_stride, int q_off, void* row_out, int row_stride, void* kc, const int* block_table, int bt_width,
                                int ps, int num_pages, int write_cache, int* errors, int n_tokens, int dtype, int half_pairs,
                                const void* lat, int lat_stride, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || dim <= 0 || rd <= 0 || rank <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > rd || q_off < 0 || D < q_off + rd ||
      q_stride < H * D || n_q != H * (dim + rd) || stride < n_q + (lat ? 0 : rank + rd) || (lat && lat_stride < rank + rd))
    return SB_ERR_SHAPE;
  if (write_cache && D < rank + rd) return SB_ERR_SHAPE;
  if (row_out != nullptr && row_stride < rank + rd) return SB_ERR_SHAPE;
  if (write_cache && (ps <= 0 || bt_width <= 0 || !kc || !errors)) return SB_ERR_SHAPE;
  const size_t smem = (size_t)(rot_dims > 0 ? rot_dims : 2) * sizeof(float);
  if (smem > 48 * 1024) return SB_ERR_LIMIT;
  if (dtype == SB_DTYPE_F32)
    latent_prepare_kernel<float><<<n_tokens, 128, smem, stream>>>((const float*)proj, stride, n_q, positions, token_row, c_weight, eps,
                                                                   inv_freq, rot_dims, H, dim, rd, rank, D, (float*)q_lat, q_stride, q_off,
                                                                   (float*)row_out, row_stride, (float*)kc, block_table, bt_width, ps,
                                                                   num_pages, write_cache, errors, half_pairs, (const float*)lat, lat_stride);
  else if (dtype == SB_DTYPE_BF16)
    latent_prepare_kernel<__nv_bfloat16><<<n_tokens, 128, smem, stream>>>(
        (const __nv_bfloat16*)proj, stride, n_q, positions, token_row, c_weight, eps, inv_freq, rot_dims, H, dim, rd, rank, D,
        (__nv_bfloat16*)q_lat, q_stride, q_off, (__nv_bfloat16*)row_out, row_stride, (__nv_bfloat16*)kc, block_table, bt_width, ps, num_pages,
        write_cache, errors, half_pairs, (const __nv_bfloat16*)lat, lat_stride);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_gated_activation(const void* gate_up, void* out, int n_tokens, int inter, int kind, float limit, float alpha, int dtype,
                                  cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (inter <= 0 || kind < 0 || kind > 2) return SB_ERR_SHAPE;
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  if (dtype == SB_DTYPE_BF16 && (inter % 8) == 0 && aligned16(gate_up) && aligned16(out)) {
    const size_t total8 = total / 8;
    const size_t want = (total8 + threads - 1) / threads;
    const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
    gated_activation_bf16_vec_kernel<<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter / 8, total8,
                                                                     kind, limit, alpha);
    SB_LAUNCH_CHECK();
    return 0;
  }
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
  if (dtype == SB_DTYPE_F32)
    gated_activation_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, inter, total, kind, limit, alpha);
  else if (dtype == SB_DTYPE_BF16)
    gated_activation_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total,
                                                                           kind, limit, alpha);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------- embedding with a pair table
namespace {

// One thread per token: the id itself (an id -(s+1) stands for last_token[s]) and the row of the pair table,
// (previous id * mul_prev + id * mul_cur) mod buckets in 64-bit integers; the sequence's first token (position 0) takes
// row ``buckets``. The id before a portion's first token is what the request's state slot holds.
__global__ void __launch_bounds__(128) pair_rows_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                                        const int* __restrict__ token_row, const int* __restrict__ cu_q,
                                                        const int* __restrict__ slots, const int* __restrict__ prev_state,
                                                        long long state_stride, const int* __restrict__ last_token, int n_slots, int vocab,
                                                        long long mul_prev, long long mul_cur, int buckets, int n_tokens,
                                                        int* __restrict__ ids, int* __restrict__ rows) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  auto resolve = [&](int tok) {
    if (tok < 0 && last_token != nullptr && -tok - 1 < n_slots) tok = last_token[-tok - 1];
    return tok;
  };
  const int r = token_row[t];
  const int cur = resolve(tokens[t]);
  ids[t] = cur;
  int row = buckets;
  if (positions[t] > 0) {
    const int prev = t > cu_q[r] ? resolve(tokens[t - 1]) : prev_state[(size_t)slots[r] * state_stride];
    const bool ok = cur >= 0 && cur < vocab && prev >= 0 && prev < vocab;
    row = ok ? (int)(((long long)prev * mul_prev + (long long)cur * mul_cur) % (long long)buckets) : buckets;
  }
  rows[t] = row;
}

// One block per token: out = table[id] * scale + pairs[row], both products and the sum in float. The block of a row's last
// token leaves its id in the request's state slot (every read of the slot happened in the launch before).
template <typename T>
__global__ void __launch_bounds__(256) embedding_pair_kernel(const int* __restrict__ ids, const int* __restrict__ rows,
                                                             const T* __restrict__ table, const T* __restrict__ pairs,
                                                             float* __restrict__ out, int dim, int vocab, float scale,
                                                             const int* __restrict__ token_row, const int* __restrict__ cu_q,
                                                             const int* __restrict__ slots, int* __restrict__ prev_state,
                                                             long long state_stride) {
  const int t = blockIdx.x;
  const int tok = ids[t];
  const bool ok = tok >= 0 && tok < vocab;
  const T* src = table + (size_t)(ok ? tok : 0) * dim;
  const T* add = pairs + (size_t)rows[t] * dim;
  float* dst = out + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = ok ? to_float(src[i]) * scale + to_float(add[i]) : 0.f;
  if (threadIdx.x == 0) {
    const int r = token_row[t];
    if (t == cu_q[r + 1] - 1) prev_state[(size_t)slots[r] * state_stride] = tok;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bias_round_kernel(const float* __restrict__ sums, int stride, const float* __restrict__ bias,
                                                         T* __restrict__ out, int out_stride, int cols, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols;
    const int c = (int)(i - r * cols);
    out[r * out_stride + c] = from_float<T>(sums[r * stride + c] + (bias ? bias[c] : 0.f));
  }
}

// float sums + bias -> bfloat16, four columns a thread.
__global__ void __launch_bounds__(256) bias_round_vec_kernel(const float* __restrict__ sums, int stride, const float* __restrict__ bias,
                                                             __nv_bfloat16* __restrict__ out, int out_stride, int cols4, size_t total4) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols4;
    const int c = (int)(i - r * cols4) * 4;
    float4 v = *reinterpret_cast<const float4*>(sums + r * stride + c);
    if (bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias + c);
      v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    }
    store4f<__nv_bfloat16>(out + r * out_stride + c, v);
  }
}

__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ x, size_t total, float cap, float inv_cap) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv_cap);
}

}  // namespace

// tokens, positions, token_row [T]; cu_q [R + 1]; slots [R]; prev_state: int32 view of a float state, one value per slot,
// slots state_stride ints apart; table [vocab, dim], pairs [buckets + 1, dim] of ``dtype``; work: 2 T ints; out float [T, dim].
SB_EXPORT int sb_embedding_pair(const int* tokens, const int* positions, const int* token_row, const int* cu_q, const int* slots,
                                int* prev_state, long long state_stride, const int* last_token, int n_slots, const void* table,
                                const void* pairs, int vocab, int dim, int buckets, long long mul_prev, long long mul_cur, float scale,
                                int* work, float* out, int n_tokens, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || vocab <= 0 || buckets <= 0 || !prev_state || !work) return SB_ERR_SHAPE;
  if (mul_prev < 0 || mul_cur < 0 || mul_prev > (1LL << 31) || mul_cur > (1LL << 31)) return SB_ERR_LIMIT;
  int* ids = work;
  int* rows = work + n_tokens;
  pair_rows_kernel<<<(n_tokens + 127) / 128, 128, 0, stream>>>(tokens, positions, token_row, cu_q, slots, prev_state, state_stride,
                                                               last_token, n_slots, vocab, mul_prev, mul_cur, buckets, n_tokens, ids, rows);
  SB_LAUNCH_CHECK();
  const int threads = dim >= 1024 ? 256 : 128;
  if (dtype == SB_DTYPE_F32)
    embedding_pair_kernel<float><<<n_tokens, threads, 0, stream>>>(ids, rows, (const float*)table, (const float*)pairs, out, dim, vocab, scale,
                                                                  token_row, cu_q, slots, prev_state, state_stride);
  else if (dtype == SB_DTYPE_BF16)
    embedding_pair_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(ids, rows, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs,
                                                                          out, dim, vocab, scale, token_row, cu_q, slots, prev_state,
                                                                          state_stride);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// out [n_rows, cols] (rows out_stride apart) = sums (float, rows stride apart) + bias (float [cols] or null), rounded once.
SB_EXPORT int sb_bias_round(const float* sums, int stride, const float* bias, void* out, int out_stride, int n_rows, int cols, int dtype,
                            cudaStream_t stream) {
  if (n_rows <= 0 || cols <= 0) return 0;
  if (stride < cols || out_stride < cols) return SB_ERR_SHAPE;
  if (dtype == SB_DTYPE_BF16 && cols % 4 == 0 && stride % 4 == 0 && out_stride % 4 == 0 && aligned16(sums) && (!bias || aligned16(bias)) &&
      (reinterpret_cast<uintptr_t>(out) % 8) == 0) {
    const size_t total4 = (size_t)n_rows * (cols / 4), want4 = (total4 + 255) / 256;
    const int blocks4 = (int)(want4 < (size_t)sm_count() * 16 ? want4 : (size_t)sm_count() * 16);
    bias_round_vec_kernel<<<blocks4, 256, 0, stream>>>(sums, stride, bias, (__nv_bfloat16*)out, out_stride, cols / 4, total4);
    SB_LAUNCH_CHECK();
    return 0;
  }
  const size_t total = (size_t)n_rows * cols, want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
  if (dtype == SB_DTYPE_F32) bias_round_kernel<float><<<blocks, 256, 0, stream>>>(sums, stride, bias, (float*)out, out_stride, cols, total);
  else if (dtype == SB_DTYPE_BF16)
    bias_round_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(sums, stride, bias, (__nv_bfloat16*)out, out_stride, cols, total);
  else return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// x (float, contiguous) <- cap * tanh(x / cap).
SB_EXPORT int sb_softcap(float* x, long long total, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return SB_ERR_SHAPE;
  const size_t want = ((size_t)total + 255) / 256;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
  softcap_kernel<<<blocks, 256, 0, stream>>>(x, (size_t)total, cap, 1.0f / cap);
  SB_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------- sigmoid gate
namespace {

// out[t, c] = scale * a[t, c] * sigmoid(gate[t, c / per_gate]) (gate null: scale * a), the product in float, rounded once.
template <typename T, typename TG>
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(const T* __restrict__ a, int a_stride, const TG* __restrict__ gate, int gate_stride,
                                                           int per_gate, T* __restrict__ out, int out_stride, int cols, size_t total,
                                                           float scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols;
    const int c = (int)(i - r * cols);
    float v = to_float(a[r * a_stride + c]) * scale;
    if (gate) v *= 1.f / (1.f + expf(-to_float(gate[r * gate_stride + c / per_gate])));
    out[r * out_stride + c] = from_float<T>(v);
  }
}

// The same for bfloat16 operands, eight neighbouring columns a thread (16-byte loads and stores): cols, the row strides and, for a
// gate per run of columns, the run's length are multiples of 8. PER_ELEMENT: a gate value per column, else one per run.
template <typename TG, bool PER_ELEMENT>
__global__ void __launch_bounds__(256) sigmoid_gate_vec_kernel(const __nv_bfloat16* __restrict__ a, int a_stride, const TG* __restrict__ gate,
                                                               int gate_stride, int per_gate, __nv_bfloat16* __restrict__ out, int out_stride,
                                                               int cols8, size_t total8, float scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols8;
    const int c = (int)(i - r * cols8) * 8;
    const uint4 av = *reinterpret_cast<const uint4*>(a + r * a_stride + c);
    const __nv_bfloat16* ae = reinterpret_cast<const __nv_bfloat16*>(&av);
    float g[8];
    if (gate == nullptr) {
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] = 1.f;
    } else if (PER_ELEMENT) {
#pragma unroll
      for (int e = 0; e < 8; e += 4) {
        const float4 gv = load4f<TG>(gate + r * gate_stride + c + e);
        g[e] = 1.f / (1.f + expf(-gv.x)); g[e + 1] = 1.f / (1.f + expf(-gv.y));
        g[e + 2] = 1.f / (1.f + expf(-gv.z)); g[e + 3] = 1.f / (1.f + expf(-gv.w));
      }
    } else {
      const float one = 1.f / (1.f + expf(-to_float(gate[r * gate_stride + c / per_gate])));
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] = one;
    }
    uint4 ov;
    __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
    for (int e = 0; e < 8; ++e) oe[e] = __float2bfloat16_rn(to_float(ae[e]) * scale * g[e]);
    *reinterpret_cast<uint4*>(out + r * out_stride + c) = ov;
  }
}

}  // namespace

// a, out [n_rows, cols] (row strides given; may be the same buffer), gate [n_rows, gate_cols] or null, of the operands' type or
// (gate_f32) float; gate_cols divides cols.
SB_EXPORT int sb_sigmoid_gate(const void* a, int a_stride, const void* gate, int gate_stride, int gate_cols, void* out, int out_stride,
                              int n_rows, int cols, float scale, int dtype, int gate_f32, cudaStream_t stream) {
  if (n_rows <= 0 || cols <= 0) return 0;
  if (a_stride < cols || out_stride < cols || (gate && (gate_cols <= 0 || cols % gate_cols || gate_stride < gate_cols))) return SB_ERR_SHAPE;
  const int per_gate = gate ? cols / gate_cols : 1;
  if (dtype == SB_DTYPE_BF16 && cols % 8 == 0 && a_stride % 8 == 0 && out_stride % 8 == 0 && aligned16(a) && aligned16(out) &&
      (!gate || (per_gate == 1 ? (gate_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(gate) % (gate_f32 ? 16 : 8)) == 0) : per_gate % 8 == 0))) {
    typedef __nv_bfloat16 B;
    const size_t total8 = (size_t)n_rows * (cols / 8), want8 = (total8 + 255) / 256;
    const int blocks8 = (int)(want8 < (size_t)sm_count() * 16 ? want8 : (size_t)sm_count() * 16);
#define SB_GATE_VEC(TG, PE)                                                                                                           \
  sigmoid_gate_vec_kernel<TG, PE><<<blocks8, 256, 0, stream>>>((const B*)a, a_stride, (const TG*)gate, gate_stride, per_gate, (B*)out, \
                                                              out_stride, cols / 8, total8, scale)
    if (gate_f32) { if (per_gate == 1) SB_GATE_VEC(float, true); else SB_GATE_VEC(float, false); }
    else { if (per_gate == 1) SB_GATE_VEC(B, true); else SB_GATE_VEC(B, false); }
#undef SB_GATE_VEC
    SB_LAUNCH_CHECK();
    return 0;
  }
  const size_t total = (size_t)n_rows * cols, want = (total + 255) / 256;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? want : (size_t)sm_count() * 16);
  if (dtype == SB_DTYPE_F32)
    sigmoid_gate_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)a, a_stride, (const float*)gate, gate_stride, per_gate,
                                                                  (float*)out, out_stride, cols, total, scale);
  else if (dtype == SB_DTYPE_BF16 && gate_f32)
    sigmoid_gate_kernel<__nv_bfloat16, float><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)a, a_stride, (const float*)gate, gate_stride,
                                                                          per_gate, (__nv_bfloat16*)out, out_stride, cols, total, scale);
  else if (dtype == SB_DTYPE_BF16)
    sigmoid_gate_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)a, a_stride, (const __nv_bfloat16*)gate,
                                                                                  gate_stride, per_gate, (__nv_bfloat16*)out, out_stride, cols,
                                                                                  total, scale);
  else return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}
