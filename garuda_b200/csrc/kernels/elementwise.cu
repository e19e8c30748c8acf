// Embedding, RMS norm, rotary positions with the write into the paged cache,
// SiLU-gate and the residual add. All arithmetic is 32-bit; only what is stored
// may be bfloat16. Formulas: garuda/src/simd/mod.rs (rmsnorm :166-173, rope
// :196-206, silu :161-163, add_assign :176-179) and garuda/src/llama/mod.rs
// (embedding row copy :198-200, :1078-1085; norm weight multiply :733-738;
// rotate then store :784-791).
#include "common.cuh"

GB_DEFINE_LAST_ERROR()

namespace {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                                 float* __restrict__ out, int d, int vocab, float scale, int copies) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * d * copies;       // a token's row `copies` times in a row (a residual of several streams)
  if (id < 0 || id >= vocab) {  // refused on the host before any launch; never read out of range
    for (int c = threadIdx.x; c < d * copies; c += blockDim.x) o[c] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = gb::to_float<T>(row[c]) * scale;
    for (int k = 0; k < copies; ++k) o[(size_t)k * d + c] = v;
  }
}

// logits <- logits * scale, then (cap > 0) cap * tanh(logits / cap); in place, 32-bit
__global__ void scale_softcap_kernel(float* __restrict__ x, long long n, float scale, float cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i] * scale;
  if (cap > 0.f) v = cap * tanhf(v / cap);
  x[i] = v;
}

// ------------------------------------------------------------------ rmsnorm
// One block per row. sum of squares in 32-bit: per-thread partial sums over a
// strided walk, then a fixed-order tree, so a row's result does not depend on
// which other rows are in the batch.
template <typename WT, typename OT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const WT* __restrict__ w, float eps,
                               OT* __restrict__ out, const int32_t* __restrict__ rows, int d) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float* xr = x + (size_t)src * d;
  OT* o = out + (size_t)r * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = xr[c];
    ss = fmaf(v, v, ss);
  }
  __shared__ float warp_part[32];
  __shared__ float scale_s;
  ss = gb::warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_part[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    float v = lane < (blockDim.x >> 5) ? warp_part[lane] : 0.f;
    v = gb::warp_sum(v);
    if (lane == 0) scale_s = 1.0f / sqrtf(v / (float)d + eps);
  }
  __syncthreads();
  const float scale = scale_s;
  for (int c = threadIdx.x; c < d; c += blockDim.x)
    o[c] = gb::from_float<OT>((xr[c] * scale) * gb::to_float<WT>(w[c]));
}

template <typename OT>
__device__ __forceinline__ void store4(OT* p, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}

// Rows of up to 4096 values whose length is a multiple of 4: the row is read once, 16 bytes per
// load, and kept in registers between the sum of squares and the scaling.
template <typename WT, typename OT>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, const WT* __restrict__ w, float eps, OT* __restrict__ out,
                   const int32_t* __restrict__ rows, int d) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * d);
  const int nvec = d >> 2;
  float4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = threadIdx.x + i * 256;
    v[i] = c < nvec ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  __shared__ float warp_part[8];
  __shared__ float scale_s;
  ss = gb::warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_part[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    float t = lane < 8 ? warp_part[lane] : 0.f;
    t = gb::warp_sum(t);
    if (lane == 0) scale_s = 1.0f / sqrtf(t / (float)d + eps);
  }
  __syncthreads();
  const float scale = scale_s;
  OT* o = out + (size_t)r * d;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c >= nvec) continue;
    const float w0 = gb::to_float<WT>(w[4 * c]), w1 = gb::to_float<WT>(w[4 * c + 1]);
    const float w2 = gb::to_float<WT>(w[4 * c + 2]), w3 = gb::to_float<WT>(w[4 * c + 3]);
    store4<OT>(o + 4 * c, (v[i].x * scale) * w0, (v[i].y * scale) * w1, (v[i].z * scale) * w2,
               (v[i].w * scale) * w3);
  }
}

// ------------------------------------------------- rotary + cache write
// One block per token. Heads [0, Hq) are queries, [Hq, Hq+Hkv) keys, [Hq+Hkv, Hq+2Hkv) values.
// Angle = (float)pos * inv_freq[i], in 32-bit; sine and cosine are computed once per token and pair.
template <typename IT, typename OT>
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(const IT* __restrict__ qkv, int row_stride, OT* __restrict__ q_out,
                      OT* __restrict__ k_pool, OT* __restrict__ v_pool,
                      const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                      const int32_t* __restrict__ block_table, int table_width, int Hq, int Hkv, int hd,
                      const float* __restrict__ inv_freq, int interleaved, int page_size) {
  __shared__ float sin_s[128], cos_s[128];   // head_dim / 2 <= 128
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = hd >> 1;
  const bool rotate = inv_freq != nullptr;
  if (rotate) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
  }
  long long cache_row = -1;   // row of this token in the pools, in units of one head's page_size * hd block
  if (Hkv > 0) {
    const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
    // no page behind this position: the host refuses such a step; nothing is stored
    if (page >= 0) cache_row = (long long)page * Hkv;
  }
  __syncthreads();
  const IT* src = qkv + (size_t)t * row_stride;
  // queries and keys: pairs
  const int rot_heads = Hq + Hkv;
  for (int e = threadIdx.x; e < rot_heads * half; e += blockDim.x) {
    const int head = e / half, i = e % half;
    const int ia = interleaved ? 2 * i : i;
    const int ib = interleaved ? 2 * i + 1 : i + half;
    const IT* s = src + (size_t)head * hd;
    OT* dst;
    if (head < Hq) {
      dst = q_out + ((size_t)t * Hq + head) * hd;
    } else {
      if (cache_row < 0) continue;
      dst = k_pool + ((cache_row + (head - Hq)) * page_size + (pos % page_size)) * hd;
    }
    const float a = gb::to_float<IT>(s[ia]), b = gb::to_float<IT>(s[ib]);
    if (rotate) {
      dst[ia] = gb::from_float<OT>(a * cos_s[i] - b * sin_s[i]);
      dst[ib] = gb::from_float<OT>(a * sin_s[i] + b * cos_s[i]);
    } else {
      dst[ia] = gb::from_float<OT>(a);
      dst[ib] = gb::from_float<OT>(b);
    }
  }
  // values: a copy
  if (cache_row >= 0) {
    const IT* vs = src + (size_t)(Hq + Hkv) * hd;
    for (int e = threadIdx.x; e < Hkv * hd; e += blockDim.x) {
      const int head = e / hd, c = e % hd;
      v_pool[((cache_row + head) * page_size + (pos % page_size)) * hd + c] =
          gb::from_float<OT>(gb::to_float<IT>(vs[e]));
    }
  }
}

// hd: the rotated width (pairs lie within it); head_stride: the distance between heads, which is
// larger than hd when only the first channels of every head are rotated.
__global__ void rope_inplace_kernel(float* __restrict__ x, int row_stride, int head_stride, int H, int hd,
                                    const int32_t* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int interleaved) {
  const int t = blockIdx.x, head = blockIdx.y;
  float* v = x + (size_t)t * row_stride + (size_t)head * head_stride;
  const int pos = positions[t];
  const int half = hd >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float ang = (float)pos * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    const int ia = interleaved ? 2 * i : i;
    const int ib = interleaved ? 2 * i + 1 : i + half;
    const float a = v[ia], b = v[ib];
    v[ia] = a * c - b * s;
    v[ib] = a * s + b * c;
  }
}

// ------------------------------------------------------------ SiLU-gate
// gate_up rows hold either [gate(F) | up(F)] (group 0), or gate and up packed in groups of 64:
// columns [128 q, 128 q + 64) gate features 64 q .., the next 64 their up values (group 64).
// kind: GB_ACT_SILU  silu(g) * u;  GB_ACT_GELU_TANH  gelu_tanh(g) * u;
// GB_ACT_CLAMPED_SWISH  g' = min(g, limit), u' = clamp(u, -limit, limit): g' * sigmoid(1.702 g') * (u' + 1).
enum GbGateAct : int { GB_ACT_SILU = 0, GB_ACT_GELU_TANH = 1, GB_ACT_CLAMPED_SWISH = 2 };

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ float gate_act(int kind, float limit, float g, float u) {
  if (kind == GB_ACT_GELU_TANH) return gelu_tanh(g) * u;
  if (kind == GB_ACT_CLAMPED_SWISH) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return (g / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
  }
  return (g / (1.0f + expf(-g))) * u;
}

template <typename IT, typename OT>
__global__ void silu_mul_kernel(const IT* __restrict__ gate_up, OT* __restrict__ out, int M, int F, int group,
                                int row_stride, int kind, float limit) {
  const size_t n = (size_t)M * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / F, f = i % F;
    const size_t gi = group ? (f / group) * 2 * group + f % group : f;
    const size_t ui = group ? gi + group : F + f;
    const float g = gb::to_float<IT>(gate_up[m * row_stride + gi]);
    const float u = gb::to_float<IT>(gate_up[m * row_stride + ui]);
    out[i] = gb::from_float<OT>(gate_act(kind, limit, g, u));
  }
}

template <typename YT>
__global__ void residual_add_kernel(float* __restrict__ x, const YT* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] += gb::to_float<YT>(y[i]);
}

int grid_for(size_t n, int block);

// ---------------------------------------------------------------- layer norm
// Sum of a value over the block in a fixed order (warps, then the warps' sums): a row's result
// does not depend on which other rows are in the batch.
__device__ __forceinline__ float block_sum(float v, float* part) {
  v = gb::warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // `part` may still be read from the call before
  if (lane == 0) part[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? part[lane] : 0.f;
  return gb::warp_sum(t);
}

// out = (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations (taken in a
// second pass over the row, not as mean(x^2) - mean^2). One block per row, 32-bit throughout.
template <typename WT, typename OT>
__global__ void __launch_bounds__(256)
layernorm_kernel(const float* __restrict__ x, const WT* __restrict__ w, const WT* __restrict__ b, float eps,
                 OT* __restrict__ out, const int32_t* __restrict__ rows, int d) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  __shared__ float part[32];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * d;
  float s = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) s += xr[c];
  const float mean = block_sum(s, part) / (float)d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float dv = xr[c] - mean;
    ss = fmaf(dv, dv, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, part) / (float)d + eps);
  OT* o = out + (size_t)r * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float bias = b ? gb::to_float<WT>(b[c]) : 0.f;
    o[c] = gb::from_float<OT>(((xr[c] - mean) * inv) * gb::to_float<WT>(w[c]) + bias);
  }
}

// Rows of up to 4096 values whose length is a multiple of 4: the row is read once, 16 bytes per
// load, and stays in registers between the mean, the variance and the scaling.
template <typename WT, typename OT>
__global__ void __launch_bounds__(256)
layernorm_vec_kernel(const float* __restrict__ x, const WT* __restrict__ w, const WT* __restrict__ b, float eps,
                     OT* __restrict__ out, const int32_t* __restrict__ rows, int d) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  __shared__ float part[32];
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
  const int nvec = d >> 2;
  float4 v[4];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = threadIdx.x + i * 256;
    v[i] = c < nvec ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float mean = block_sum(s, part) / (float)d;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (threadIdx.x + i * 256 >= nvec) continue;
    const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
    ss = fmaf(a0, a0, ss); ss = fmaf(a1, a1, ss); ss = fmaf(a2, a2, ss); ss = fmaf(a3, a3, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, part) / (float)d + eps);
  OT* o = out + (size_t)r * d;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c >= nvec) continue;
    float y[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      y[j] = ((y[j] - mean) * inv) * gb::to_float<WT>(w[4 * c + j]) + (b ? gb::to_float<WT>(b[4 * c + j]) : 0.f);
    store4<OT>(o + 4 * c, y[0], y[1], y[2], y[3]);
  }
}

// x[t][c] += alpha * y[t][c] + row[c]; y or row may be absent
template <typename YT, typename RT>
__global__ void residual_axpy_kernel(float* __restrict__ x, const YT* __restrict__ y, float alpha,
                                     const RT* __restrict__ row, size_t n, int d) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = x[i];
    if (y) v = fmaf(alpha, gb::to_float<YT>(y[i]), v);
    if (row) v += gb::to_float<RT>(row[i % d]);
    x[i] = v;
  }
}

// x[t] += alpha * y[t] / sqrt(mean(y[t]^2) + eps) * w: an RMS-normed branch added to the residual
template <typename WT>
__global__ void __launch_bounds__(256)
rms_add_kernel(float* __restrict__ x, const float* __restrict__ y, const WT* __restrict__ w, float eps,
               float alpha, int d) {
  __shared__ float part[32];
  const float* yr = y + (size_t)blockIdx.x * d;
  float* xr = x + (size_t)blockIdx.x * d;
  // up to 16 values a thread stay in registers between the sum and the scaling (rows of up to 4096
  // with 256 threads); a longer row's other values are read again
  float keep[16];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    keep[i] = c < d ? yr[c] : 0.f;
    ss = fmaf(keep[i], keep[i], ss);
  }
  for (int c = threadIdx.x + 16 * blockDim.x; c < d; c += blockDim.x) ss = fmaf(yr[c], yr[c], ss);
  const float inv = 1.0f / sqrtf(block_sum(ss, part) / (float)d + eps);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < d) xr[c] = fmaf(alpha, (keep[i] * inv) * gb::to_float<WT>(w[c]), xr[c]);
  }
  for (int c = threadIdx.x + 16 * blockDim.x; c < d; c += blockDim.x)
    xr[c] = fmaf(alpha, (yr[c] * inv) * gb::to_float<WT>(w[c]), xr[c]);
}

// out[t][j] = gelu_tanh(z[t][j]) * table[ids[t]][col0 + j]: a gate on a per-token table row
template <typename IT, typename TT, typename OT>
__global__ void gelu_gather_mul_kernel(const IT* __restrict__ z, const TT* __restrict__ table, int table_ld,
                                       int col0, const int32_t* __restrict__ ids, OT* __restrict__ out, int T,
                                       int dim, int vocab) {
  const size_t n = (size_t)T * dim;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / dim), j = (int)(i % dim);
    const int id = ids[t];
    const float e = (id >= 0 && id < vocab) ? gb::to_float<TT>(table[(size_t)id * table_ld + col0 + j]) : 0.f;
    out[i] = gb::from_float<OT>(gelu_tanh(gb::to_float<IT>(z[i])) * e);
  }
}

template <typename OT>
__global__ void cast_kernel(const float* __restrict__ x, OT* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = gb::from_float<OT>(x[i]);
}

int grid_for(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  return (int)(g > 148 * 16 ? 148 * 16 : (g ? g : 1));
}

}  // namespace

// out[t] = table[ids[t]] * scale (a model without an embedding multiplier passes 1)
// out [T, copies, d]: every token's row, scaled, `copies` times
GB_EXPORT int gb_embedding_copies(const void* table, int table_dtype, const int32_t* ids, float* out, int T,
                                  int d, int vocab, float scale, int copies, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (copies < 1) return gb::fail(GB_BAD_ARGUMENT, "embedding: %d copies", copies);
  return GB_DISPATCH_DTYPE(table_dtype, TT, [&]() -> int {
    return gb::check_pdl_launch(gb::launch_pdl(embedding_kernel<TT>, dim3(T), dim3(256), 0, stream, dim3(1, 1, 1),
                                               (const TT*)table, ids, out, d, vocab, scale, copies), "embedding");
  });
}

GB_EXPORT int gb_embedding(const void* table, int table_dtype, const int32_t* ids, float* out, int T,
                           int d, int vocab, float scale, cudaStream_t stream) {
  return gb_embedding_copies(table, table_dtype, ids, out, T, d, vocab, scale, 1, stream);
}

GB_EXPORT int gb_scale_softcap(float* x, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return GB_OK;
  scale_softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, n, scale, cap);
  return gb::check_launch("scale_softcap");
}

GB_EXPORT int gb_rmsnorm(const float* x, const void* w, int w_dtype, float eps, void* out, int out_dtype,
                         const int32_t* rows, int n_rows, int d, cudaStream_t stream) {
  if (n_rows <= 0) return GB_OK;
  const int block = d >= 1024 ? 256 : 128;
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      if (d % 4 == 0 && d <= 4096 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0)
        return gb::check_pdl_launch(gb::launch_pdl(rmsnorm_vec_kernel<WT, OT>, dim3(n_rows), dim3(256), 0, stream, dim3(1, 1, 1),
                                                   x, (const WT*)w, eps, (OT*)out, rows, d), "rmsnorm");
      return gb::check_pdl_launch(gb::launch_pdl(rmsnorm_kernel<WT, OT>, dim3(n_rows), dim3(block), 0, stream, dim3(1, 1, 1),
                                                 x, (const WT*)w, eps, (OT*)out, rows, d), "rmsnorm");
    });
  });
}

GB_EXPORT int gb_rope_kv_append(const void* qkv, int in_dtype, int row_stride, void* q_out, void* k_pool,
                                void* v_pool, int out_dtype, const int32_t* positions,
                                const int32_t* token_req, const int32_t* block_table, int table_width,
                                int T, int Hq, int Hkv, int hd, const float* inv_freq, int interleaved,
                                int page_size, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (hd % 2) return gb::fail(GB_UNSUPPORTED, "rope_kv_append: head_dim %d is odd", hd);
  if (Hkv > 0 && (!k_pool || !v_pool || !block_table || page_size < 1))
    return gb::fail(GB_BAD_ARGUMENT, "rope_kv_append: kv heads given without a cache to store them in");
  if (hd > 256) return gb::fail(GB_UNSUPPORTED, "rope_kv_append: head_dim %d is larger than 256", hd);
  const int work = (Hq + Hkv) * (hd / 2);
  const int block = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(
          gb::launch_pdl(rope_kv_append_kernel<IT, OT>, dim3(T), dim3(block), 0, stream, dim3(1, 1, 1), (const IT*)qkv,
                         row_stride, (OT*)q_out, (OT*)k_pool, (OT*)v_pool, positions, token_req, block_table,
                         table_width, Hq, Hkv, hd, inv_freq, interleaved, page_size),
          "rope_kv_append");
    });
  });
}

// out[t][i] = (cos, sin)((float)positions[t] * inv_freq[i]) for i < half: the rotation's angles
// (garuda/src/simd/mod.rs:196-206) once per step, for every layer's fused epilogue to read.
__global__ void rope_table_kernel(const int32_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ out, int T, int half) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, i = idx % half;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
  out[idx] = make_float2(cs, sn);
}

// A plain launch on purpose: kernels after it that start early (programmatic dependent launch) may
// read the table before their dependency wait, which is safe only because this kernel gives no
// early start signal, so that they cannot begin before it has finished.
GB_EXPORT int gb_rope_table(const int32_t* positions, const float* inv_freq, float* out, int T, int half,
                            cudaStream_t stream) {
  if (T <= 0 || half <= 0) return GB_OK;
  const int n = T * half;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(positions, inv_freq, reinterpret_cast<float2*>(out), T, half);
  return gb::check_launch("rope_table");
}

GB_EXPORT int gb_rope_inplace(float* x, int row_stride, int head_stride, int T, int H, int hd,
                              const int32_t* positions, const float* inv_freq, int interleaved,
                              cudaStream_t stream) {
  if (T <= 0 || H <= 0) return GB_OK;
  if (hd % 2) return gb::fail(GB_UNSUPPORTED, "rope_inplace: the rotated width %d is odd", hd);
  if (head_stride < hd) return gb::fail(GB_BAD_ARGUMENT, "rope_inplace: heads %d apart are narrower than %d", head_stride, hd);
  dim3 grid(T, H);
  rope_inplace_kernel<<<grid, 32, 0, stream>>>(x, row_stride, head_stride, H, hd, positions, inv_freq, interleaved);
  return gb::check_launch("rope_inplace");
}

GB_EXPORT int gb_gated_act(const void* gate_up, int in_dtype, void* out, int out_dtype, int M, int F, int group,
                           int row_stride, int kind, float limit, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return GB_OK;
  if (kind < GB_ACT_SILU || kind > GB_ACT_CLAMPED_SWISH) return gb::fail(GB_BAD_ARGUMENT, "gated_act: kind %d", kind);
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      silu_mul_kernel<IT, OT><<<grid_for((size_t)M * F, 256), 256, 0, stream>>>(
          (const IT*)gate_up, (OT*)out, M, F, group, row_stride, kind, limit);
      return gb::check_launch("gated_act");
    });
  });
}

GB_EXPORT int gb_silu_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, int M, int F, int group,
                          int row_stride, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      silu_mul_kernel<IT, OT><<<grid_for((size_t)M * F, 256), 256, 0, stream>>>(
          (const IT*)gate_up, (OT*)out, M, F, group, row_stride, GB_ACT_SILU, 0.f);
      return gb::check_launch("silu_mul");
    });
  });
}

GB_EXPORT int gb_residual_add(float* x, const void* y, int y_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(y_dtype, YT, [&]() -> int {
    residual_add_kernel<YT><<<grid_for((size_t)n, 256), 256, 0, stream>>>(x, (const YT*)y, (size_t)n);
    return gb::check_launch("residual_add");
  });
}

GB_EXPORT int gb_layernorm(const float* x, const void* w, const void* b, int w_dtype, float eps, void* out,
                           int out_dtype, const int32_t* rows, int n_rows, int d, cudaStream_t stream) {
  if (n_rows <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      if (d % 4 == 0 && d <= 4096 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0)
        return gb::check_pdl_launch(gb::launch_pdl(layernorm_vec_kernel<WT, OT>, dim3(n_rows), dim3(256), 0, stream,
                                                   dim3(1, 1, 1), x, (const WT*)w, (const WT*)b, eps, (OT*)out, rows, d),
                                    "layernorm");
      return gb::check_pdl_launch(gb::launch_pdl(layernorm_kernel<WT, OT>, dim3(n_rows), dim3(d >= 1024 ? 256 : 128), 0,
                                                 stream, dim3(1, 1, 1), x, (const WT*)w, (const WT*)b, eps, (OT*)out,
                                                 rows, d), "layernorm");
    });
  });
}

GB_EXPORT int gb_residual_axpy(float* x, const void* y, int y_dtype, float alpha, const void* row, int row_dtype,
                               int T, int d, cudaStream_t stream) {
  if (T <= 0 || d <= 0) return GB_OK;
  const size_t n = (size_t)T * d;
  return GB_DISPATCH_DTYPE(y_dtype, YT, [&]() -> int {
    return GB_DISPATCH_DTYPE(row_dtype, RT, [&]() -> int {
      residual_axpy_kernel<YT, RT><<<grid_for(n, 256), 256, 0, stream>>>(x, (const YT*)y, alpha, (const RT*)row, n, d);
      return gb::check_launch("residual_axpy");
    });
  });
}

GB_EXPORT int gb_rms_add(float* x, const float* y, const void* w, int w_dtype, float eps, float alpha, int T, int d,
                         cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    rms_add_kernel<WT><<<T, 256, 0, stream>>>(x, y, (const WT*)w, eps, alpha, d);
    return gb::check_launch("rms_add");
  });
}

GB_EXPORT int gb_gelu_gather_mul(const void* z, int z_dtype, const void* table, int table_dtype, int table_ld,
                                 int col0, const int32_t* ids, void* out, int out_dtype, int T, int dim, int vocab,
                                 cudaStream_t stream) {
  if (T <= 0 || dim <= 0) return GB_OK;
  if (col0 < 0 || col0 + dim > table_ld) return gb::fail(GB_BAD_ARGUMENT, "gelu_gather_mul: columns %d..%d of %d", col0, col0 + dim, table_ld);
  return GB_DISPATCH_DTYPE(z_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(table_dtype, TT, [&]() -> int {
      return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
        gelu_gather_mul_kernel<IT, TT, OT><<<grid_for((size_t)T * dim, 256), 256, 0, stream>>>(
            (const IT*)z, (const TT*)table, table_ld, col0, ids, (OT*)out, T, dim, vocab);
        return gb::check_launch("gelu_gather_mul");
      });
    });
  });
}

GB_EXPORT int gb_cast(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
    cast_kernel<OT><<<grid_for((size_t)n, 256), 256, 0, stream>>>(x, (OT*)out, (size_t)n);
    return gb::check_launch("cast");
  });
}
