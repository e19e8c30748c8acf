// A residual kept as S streams x [T, S, d] (32-bit): the weighted sum of the streams with the RMS
// norm behind it, and the update of all streams from a sublayer's output,
//     x_t' = sum_s mix[s][t] x_s + out_w[t] y,
// optionally followed in the same pass by the next sublayer's read (weighted sum and norm of the
// new streams). One block per token; sums of squares per thread over a strided walk, then a tree
// in a fixed order, so a token's result does not depend on the batch.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 16;
constexpr int THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = gb::warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = lane < (blockDim.x >> 5) ? scratch[lane] : 0.f;
  total = gb::warp_sum(total);
  __syncthreads();
  return total;
}

// out[r] = rms(sum_s in_w[s] x[row][s]) * w, row = rows ? rows[r] : r. NS: the number of streams
// where it is one of the usual few (the weights then live in registers), 0: any, read at run time.
template <int NS, typename WT, typename OT>
__global__ void __launch_bounds__(THREADS)
streams_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ in_w, const WT* __restrict__ w, float eps,
                       OT* __restrict__ out, const int32_t* __restrict__ rows, int S_any, int d) {
  const int S = NS > 0 ? NS : S_any;
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  extern __shared__ float u_s[];        // [d]
  __shared__ float scratch[32];
  __shared__ float a_s[MAX_STREAMS];
  if (threadIdx.x < S) a_s[threadIdx.x] = in_w[threadIdx.x];
  __syncthreads();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float* xr = x + (size_t)src * S * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < (NS > 0 ? NS : MAX_STREAMS); ++s)
      if (s < S) u = fmaf(a_s[s], xr[(size_t)s * d + c], u);
    u_s[c] = u;
    ss = fmaf(u, u, ss);
  }
  const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
  OT* o = out + (size_t)r * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = gb::from_float<OT>((u_s[c] * scale) * gb::to_float<WT>(w[c]));
}

// NEXT: also normed[t] = rms(sum_s next_in[s] x_s') * w
template <int NS, bool NEXT, typename WT, typename OT>
__global__ void __launch_bounds__(THREADS)
streams_update_kernel(float* __restrict__ x, const float* __restrict__ mix, const float* __restrict__ out_w,
                      const float* __restrict__ y, int S_any, int d, const float* __restrict__ next_in,
                      const WT* __restrict__ w, float eps, OT* __restrict__ normed) {
  constexpr int LIM = NS > 0 ? NS : MAX_STREAMS;
  const int S = NS > 0 ? NS : S_any;
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  extern __shared__ float u_s[];        // [d] (NEXT only)
  __shared__ float scratch[32];
  __shared__ float m_s[MAX_STREAMS * MAX_STREAMS], b_s[MAX_STREAMS], a_s[MAX_STREAMS];
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) m_s[i] = mix[i];
  if (threadIdx.x < S) {
    b_s[threadIdx.x] = out_w[threadIdx.x];
    a_s[threadIdx.x] = NEXT ? next_in[threadIdx.x] : 0.f;
  }
  __syncthreads();
  // with a known number of streams the weights are read once, into registers
  float m_r[NS > 0 ? NS * NS : 1], b_r[NS > 0 ? NS : 1];
  if (NS > 0) {
#pragma unroll
    for (int i = 0; i < NS * NS; ++i) m_r[NS > 0 ? i : 0] = m_s[i];
#pragma unroll
    for (int i = 0; i < NS; ++i) b_r[NS > 0 ? i : 0] = b_s[i];
  }
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * S * d;
  const float* yr = y + (size_t)t * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float old[LIM];
#pragma unroll
    for (int s = 0; s < LIM; ++s) old[s] = s < S ? xr[(size_t)s * d + c] : 0.f;
    const float yv = yr[c];
    float u = 0.f;
#pragma unroll
    for (int to = 0; to < LIM; ++to) {
      if (to < S) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < LIM; ++s)
          if (s < S) v = fmaf(NS > 0 ? m_r[NS > 0 ? s * NS + to : 0] : m_s[s * S + to], old[s], v);
        v = fmaf(NS > 0 ? b_r[NS > 0 ? to : 0] : b_s[to], yv, v);
        xr[(size_t)to * d + c] = v;
        if (NEXT) u = fmaf(a_s[to], v, u);
      }
    }
    if (NEXT) {
      u_s[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!NEXT) return;
  const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
  OT* o = normed + (size_t)t * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = gb::from_float<OT>((u_s[c] * scale) * gb::to_float<WT>(w[c]));
}

// One block per token: qkv [T, Hq hd + Hkv hd + Hkv vd] (+ bias) split into queries (to q_out
// [T, Hq, hd]) and keys and values, which go to the token's place in its pages; key rows are hd
// wide, value rows vd wide. Nothing is rotated.
template <typename IT, typename BT, typename OT>
__global__ void __launch_bounds__(THREADS)
qkv_bias_append_kernel(const IT* __restrict__ qkv, const BT* __restrict__ bias, OT* __restrict__ q_out,
                       OT* __restrict__ k_pool, OT* __restrict__ v_pool, const int32_t* __restrict__ positions,
                       const int32_t* __restrict__ token_req, const int32_t* __restrict__ block_table, int table_width,
                       int Hq, int Hkv, int hd, int vd, int page_size) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int t = blockIdx.x;
  const int nq = Hq * hd, nk = Hkv * hd, nv = Hkv * vd;
  const IT* row = qkv + (size_t)t * (nq + nk + nv);
  const int pos = positions[t];
  const int page = Hkv > 0 ? block_table[(size_t)token_req[t] * table_width + pos / page_size] : -1;
  const int at = pos % page_size;
  for (int c = threadIdx.x; c < nq + nk + nv; c += blockDim.x) {
    float v = gb::to_float<IT>(row[c]);
    if (bias != nullptr) v += gb::to_float<BT>(bias[c]);
    if (c < nq) {
      q_out[(size_t)t * nq + c] = gb::from_float<OT>(v);
    } else if (page >= 0) {         // a padding row of a replayed step has no page
      if (c < nq + nk) {
        const int h = (c - nq) / hd, ch = (c - nq) % hd;
        k_pool[(((size_t)page * Hkv + h) * page_size + at) * hd + ch] = gb::from_float<OT>(v);
      } else {
        const int h = (c - nq - nk) / vd, ch = (c - nq - nk) % vd;
        v_pool[(((size_t)page * Hkv + h) * page_size + at) * vd + ch] = gb::from_float<OT>(v);
      }
    }
  }
}

}  // namespace

GB_DEFINE_LAST_ERROR()

GB_EXPORT int gb_streams_rmsnorm(const float* x, const float* in_w, const void* w, int w_dtype, float eps, void* out,
                                 int out_dtype, const int32_t* rows, int n_rows, int S, int d, cudaStream_t stream) {
  if (n_rows <= 0) return GB_OK;
  if (S < 1 || S > MAX_STREAMS) return gb::fail(GB_UNSUPPORTED, "streams_rmsnorm: %d streams (at most %d)", S, MAX_STREAMS);
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "streams_rmsnorm: width %d", d);
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      auto kernel = S == 1 ? streams_rmsnorm_kernel<1, WT, OT> : S == 2 ? streams_rmsnorm_kernel<2, WT, OT>
                  : S == 3 ? streams_rmsnorm_kernel<3, WT, OT> : S == 4 ? streams_rmsnorm_kernel<4, WT, OT>
                  : streams_rmsnorm_kernel<0, WT, OT>;
      return gb::check_pdl_launch(gb::launch_pdl(kernel, dim3(n_rows), dim3(THREADS), smem, stream,
                                                 dim3(1, 1, 1), x, in_w, (const WT*)w, eps, (OT*)out, rows, S, d),
                                  "streams_rmsnorm");
    });
  });
}

// next_in == nullptr: the update alone.
GB_EXPORT int gb_streams_update(float* x, const float* mix, const float* out_w, const float* y, int T, int S, int d,
                                const float* next_in, const void* w, int w_dtype, float eps, void* normed,
                                int out_dtype, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (S < 1 || S > MAX_STREAMS) return gb::fail(GB_UNSUPPORTED, "streams_update: %d streams (at most %d)", S, MAX_STREAMS);
  if (next_in == nullptr) {
    auto kernel = S == 1 ? streams_update_kernel<1, false, float, float> : S == 2 ? streams_update_kernel<2, false, float, float>
                : S == 3 ? streams_update_kernel<3, false, float, float> : S == 4 ? streams_update_kernel<4, false, float, float>
                : streams_update_kernel<0, false, float, float>;
    return gb::check_pdl_launch(
        gb::launch_pdl(kernel, dim3(T), dim3(THREADS), 0, stream, dim3(1, 1, 1), x, mix,
                       out_w, y, S, d, (const float*)nullptr, (const float*)nullptr, 0.f, (float*)nullptr),
        "streams_update");
  }
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 40 * 1024) return gb::fail(GB_UNSUPPORTED, "streams_update: width %d", d);
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      auto kernel = S == 1 ? streams_update_kernel<1, true, WT, OT> : S == 2 ? streams_update_kernel<2, true, WT, OT>
                  : S == 3 ? streams_update_kernel<3, true, WT, OT> : S == 4 ? streams_update_kernel<4, true, WT, OT>
                  : streams_update_kernel<0, true, WT, OT>;
      return gb::check_pdl_launch(
          gb::launch_pdl(kernel, dim3(T), dim3(THREADS), smem, stream, dim3(1, 1, 1), x, mix,
                         out_w, y, S, d, next_in, (const WT*)w, eps, (OT*)normed),
          "streams_update");
    });
  });
}

GB_EXPORT int gb_qkv_bias_append(const void* qkv, int in_dtype, const void* bias, int bias_dtype, void* q_out,
                                 void* k_pool, void* v_pool, int out_dtype, const int32_t* positions,
                                 const int32_t* token_req, const int32_t* block_table, int table_width, int T, int Hq,
                                 int Hkv, int hd, int vd, int page_size, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (Hkv > 0 && (!k_pool || !v_pool || !block_table || page_size < 1))
    return gb::fail(GB_BAD_ARGUMENT, "qkv_bias_append: kv heads given without a cache to store them in");
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(bias_dtype, BT, [&]() -> int {
      return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
        return gb::check_pdl_launch(
            gb::launch_pdl(qkv_bias_append_kernel<IT, BT, OT>, dim3(T), dim3(THREADS), 0, stream, dim3(1, 1, 1),
                           (const IT*)qkv, (const BT*)bias, (OT*)q_out, (OT*)k_pool, (OT*)v_pool, positions, token_req,
                           block_table, table_width, Hq, Hkv, hd, vd, page_size),
            "qkv_bias_append");
      });
    });
  });
}
