// Kernels of attention over a cached latent vector: one vector per position,
// shared by all heads, from which every head's keys and values are linear maps.
//
//   c_j   = rms(W_down h_j)[0:rank] * g          (the latent, normed)
//   r_j   = rotate(W_down h_j [rank:rank+rot], j) (one rotated key part for all heads)
//   s_ij  = (q_i^nope . W_uk,h c_j + q_i^rot . r_j) * scale
//         = ((W_uk,h^T q_i^nope) . c_j + q_i^rot . r_j) * scale
//   o_i,h = W_uv,h sum_j p_ij c_j
//
// so with the query mapped through W_uk^T first, attention runs over the cached rows [c_j | r_j]
// with every head reading the same row (keys: the whole row; values: its first `rank` channels),
// and W_uv is applied to the result. Three kernels here: the write of a step's rows into the
// pages (norm and rotation included), and a product with one small matrix per head, used for both
// maps. The attention itself is the paged attention kernel with one key/value head.
// All arithmetic is 32-bit; what is stored may be bfloat16.
#include "common.cuh"

GB_DEFINE_LAST_ERROR()

namespace {

// One block per token. src row: [latent(rank) | rot part(rot)] in 32-bit, `row_stride` apart.
// The first `rot_dims` channels of the rot part are turned in pairs (2i, 2i + 1) by pos * inv_freq[i].
template <typename WT, typename OT>
__device__ __forceinline__ void append_row(const float* __restrict__ src, int row_stride, const WT* __restrict__ norm_w,
                                           float eps, int rank, int rot, int rot_dims, const float* __restrict__ inv_freq,
                                           const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                                           const int32_t* __restrict__ block_table, int table_width, int page_size,
                                           OT* __restrict__ pool) {
  __shared__ float part[8];
  __shared__ float inv_s;
  const int t = blockIdx.x;
  const float* s = src + (size_t)t * row_stride;
  const int pos = positions[t];
  const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
  float ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) ss = fmaf(s[c], s[c], ss);
  ss = gb::warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += part[w];      // the warps' sums in a fixed order
    inv_s = 1.0f / sqrtf(total / (float)rank + eps);
  }
  __syncthreads();
  if (page < 0) return;      // a padding row, or a step the host should have refused: nothing is stored
  const float inv = inv_s;
  OT* dst = pool + ((size_t)page * page_size + (pos % page_size)) * (rank + rot);
  for (int c = threadIdx.x; c < rank; c += blockDim.x)
    dst[c] = gb::from_float<OT>((s[c] * inv) * gb::to_float<WT>(norm_w[c]));
  const float* r = s + rank;
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    const float a = r[2 * i], b = r[2 * i + 1];
    dst[rank + 2 * i] = gb::from_float<OT>(a * cs - b * sn);
    dst[rank + 2 * i + 1] = gb::from_float<OT>(b * cs + a * sn);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = gb::from_float<OT>(r[c]);
}

template <typename WT, typename OT>
__global__ void __launch_bounds__(128)
latent_append_kernel(const float* __restrict__ src, int row_stride, const WT* __restrict__ norm_w, float eps,
                     int rank, int rot, int rot_dims, const float* __restrict__ inv_freq,
                     const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                     const int32_t* __restrict__ block_table, int table_width, int page_size,
                     OT* __restrict__ pool) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  append_row<WT, OT>(src, row_stride, norm_w, eps, rank, rot, rot_dims, inv_freq, positions, token_req, block_table,
                     table_width, page_size, pool);
}

// One block per token. src row: H heads of [unrotated (dn) | rotated part (rot)] in 32-bit. The
// unrotated parts go to q_nope [T, H, dn]; the rotated parts, turned like the keys' (pairs
// (2i, 2i + 1) of the first rot_dims channels by pos * inv_freq[i]), go to the last `rot` channels of
// q_lat's rows [T, H, lat_row], whose first channels a product fills afterwards.
template <typename OT>
__device__ __forceinline__ void prepare_query(const float* __restrict__ src, int row_stride, int H, int dn, int rot,
                                              int rot_dims, const float* __restrict__ inv_freq,
                                              const int32_t* __restrict__ positions, OT* __restrict__ q_nope,
                                              OT* __restrict__ q_lat, int lat_row) {
  const int t = blockIdx.x;
  const float* s = src + (size_t)t * row_stride;
  const int pos = positions[t];
  const int hw = dn + rot;
  for (int e = threadIdx.x; e < H * dn; e += blockDim.x) {
    const int h = e / dn, c = e % dn;
    q_nope[(size_t)t * H * dn + e] = gb::from_float<OT>(s[h * hw + c]);
  }
  const int half = rot_dims / 2;
  for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
    const int h = e / half, i = e % half;
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    const float a = s[h * hw + dn + 2 * i], b = s[h * hw + dn + 2 * i + 1];
    OT* dst = q_lat + ((size_t)t * H + h) * lat_row + (lat_row - rot);
    dst[2 * i] = gb::from_float<OT>(a * cs - b * sn);
    dst[2 * i + 1] = gb::from_float<OT>(b * cs + a * sn);
  }
  const int rest = rot - rot_dims;
  for (int e = threadIdx.x; e < H * rest; e += blockDim.x) {
    const int h = e / rest, c = rot_dims + e % rest;
    q_lat[((size_t)t * H + h) * lat_row + (lat_row - rot) + c] = gb::from_float<OT>(s[h * hw + dn + c]);
  }
}

template <typename OT>
__global__ void __launch_bounds__(256)
latent_query_prepare_kernel(const float* __restrict__ src, int row_stride, int H, int dn, int rot, int rot_dims,
                            const float* __restrict__ inv_freq, const int32_t* __restrict__ positions,
                            OT* __restrict__ q_nope, OT* __restrict__ q_lat, int lat_row) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  prepare_query<OT>(src, row_stride, H, dn, rot, rot_dims, inv_freq, positions, q_nope, q_lat, lat_row);
}

// Both at once for a step's rows [queries (H * (dn + rot)) | latent (rank) | key part (rot)]: the
// queries prepared and the cache row written by one block per token.
template <typename WT, typename OT>
__global__ void __launch_bounds__(256)
latent_rows_kernel(const float* __restrict__ src, int row_stride, int H, int dn, int rot, int rot_dims,
                   const float* __restrict__ inv_freq, const int32_t* __restrict__ positions, OT* __restrict__ q_nope,
                   OT* __restrict__ q_lat, const WT* __restrict__ norm_w, float eps, int rank,
                   const int32_t* __restrict__ token_req, const int32_t* __restrict__ block_table, int table_width,
                   int page_size, OT* __restrict__ pool) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  prepare_query<OT>(src, row_stride, H, dn, rot, rot_dims, inv_freq, positions, q_nope, q_lat, rank + rot);
  append_row<WT, OT>(src + (size_t)H * (dn + rot), row_stride, norm_w, eps, rank, rot, rot_dims, inv_freq, positions,
                     token_req, block_table, table_width, page_size, pool);
}

// out[t][h][n] = sum_k a[t][h][k] * w_h[n][k], n < N, and out[t][h][N + j] = a[t][h][K + j], j < tail.
// w_h[n][k] lies at w[h * w_head + n * w_n + k * w_k]: either w_n == 1 (consecutive n are adjacent:
// a thread per n) or w_k == 1 (a warp per n, lanes over k). TOK tokens share one pass over the
// weights; every output is one fixed-order sum whatever else is in the batch.
constexpr int TOK = 8;

template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(256)
head_gemm_kernel(const AT* __restrict__ a, int a_row, int a_head, const WT* __restrict__ w, long long w_head,
                 int w_n, int w_k, OT* __restrict__ out, int out_row, int out_head, int T, int N, int K, int tail) {
  extern __shared__ float a_s[];        // [TOK][K + tail]
  const int h = blockIdx.y, t0 = blockIdx.x * TOK;
  const int width = K + tail;
  for (int e = threadIdx.x; e < TOK * width; e += blockDim.x) {
    const int i = e / width, c = e % width;
    a_s[e] = t0 + i < T ? gb::to_float<AT>(a[(size_t)(t0 + i) * a_row + (size_t)h * a_head + c]) : 0.f;
  }
  __syncthreads();
  const WT* wh = w + (size_t)h * w_head;
  if (w_n == 1) {
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
      float acc[TOK];
#pragma unroll
      for (int i = 0; i < TOK; ++i) acc[i] = 0.f;
      for (int k = 0; k < K; ++k) {
        const float wv = gb::to_float<WT>(wh[(size_t)k * w_k + n]);
#pragma unroll
        for (int i = 0; i < TOK; ++i) acc[i] = fmaf(a_s[i * width + k], wv, acc[i]);
      }
#pragma unroll
      for (int i = 0; i < TOK; ++i)
        if (t0 + i < T) out[(size_t)(t0 + i) * out_row + (size_t)h * out_head + n] = gb::from_float<OT>(acc[i]);
    }
  } else {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int n = warp; n < N; n += warps) {
      float acc[TOK];
#pragma unroll
      for (int i = 0; i < TOK; ++i) acc[i] = 0.f;
      for (int k = lane; k < K; k += 32) {
        const float wv = gb::to_float<WT>(wh[(size_t)n * w_n + k]);
#pragma unroll
        for (int i = 0; i < TOK; ++i) acc[i] = fmaf(a_s[i * width + k], wv, acc[i]);
      }
#pragma unroll
      for (int i = 0; i < TOK; ++i) {
        const float v = gb::warp_sum(acc[i]);
        if (lane == 0 && t0 + i < T) out[(size_t)(t0 + i) * out_row + (size_t)h * out_head + n] = gb::from_float<OT>(v);
      }
    }
  }
  for (int e = threadIdx.x; e < TOK * tail; e += blockDim.x) {
    const int i = e / tail, j = e % tail;
    if (t0 + i < T) out[(size_t)(t0 + i) * out_row + (size_t)h * out_head + N + j] = gb::from_float<OT>(a_s[i * width + K + j]);
  }
}

}  // namespace

GB_EXPORT int gb_latent_append(const float* src, int row_stride, const void* norm_w, int w_dtype, float eps,
                               int rank, int rot, int rot_dims, const float* inv_freq, const int32_t* positions,
                               const int32_t* token_req, const int32_t* block_table, int table_width,
                               int page_size, void* pool, int pool_dtype, int T, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (rank < 1 || rot < 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2)
    return gb::fail(GB_BAD_ARGUMENT, "latent_append: rank %d, rotated part %d of which %d turned", rank, rot, rot_dims);
  if (rot_dims > 0 && !inv_freq) return gb::fail(GB_BAD_ARGUMENT, "latent_append: a rotation without frequencies");
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(pool_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(
          gb::launch_pdl(latent_append_kernel<WT, OT>, dim3(T), dim3(128), 0, stream, dim3(1, 1, 1), src, row_stride,
                         (const WT*)norm_w, eps, rank, rot, rot_dims, inv_freq, positions, token_req, block_table,
                         table_width, page_size, (OT*)pool),
          "latent_append");
    });
  });
}

GB_EXPORT int gb_latent_query_prepare(const float* src, int row_stride, int H, int dn, int rot, int rot_dims,
                                      const float* inv_freq, const int32_t* positions, void* q_nope, void* q_lat,
                                      int out_dtype, int lat_row, int T, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (H < 1 || dn < 1 || rot < 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 || lat_row < rot)
    return gb::fail(GB_BAD_ARGUMENT, "latent_query_prepare: heads %d, %d + %d channels of which %d turned", H, dn, rot, rot_dims);
  if (rot_dims > 0 && !inv_freq) return gb::fail(GB_BAD_ARGUMENT, "latent_query_prepare: a rotation without frequencies");
  return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
    return gb::check_pdl_launch(
        gb::launch_pdl(latent_query_prepare_kernel<OT>, dim3(T), dim3(256), 0, stream, dim3(1, 1, 1), src, row_stride, H, dn,
                       rot, rot_dims, inv_freq, positions, (OT*)q_nope, (OT*)q_lat, lat_row),
        "latent_query_prepare");
  });
}

GB_EXPORT int gb_latent_rows(const float* src, int row_stride, int H, int dn, int rot, int rot_dims,
                             const float* inv_freq, const int32_t* positions, void* q_nope, void* q_lat,
                             const void* norm_w, int w_dtype, float eps, int rank, const int32_t* token_req,
                             const int32_t* block_table, int table_width, int page_size, void* pool, int out_dtype,
                             int T, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (H < 1 || dn < 1 || rank < 1 || rot < 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2)
    return gb::fail(GB_BAD_ARGUMENT, "latent_rows: heads %d, %d + %d channels of which %d turned, rank %d", H, dn, rot, rot_dims, rank);
  if (rot_dims > 0 && !inv_freq) return gb::fail(GB_BAD_ARGUMENT, "latent_rows: a rotation without frequencies");
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(
          gb::launch_pdl(latent_rows_kernel<WT, OT>, dim3(T), dim3(256), 0, stream, dim3(1, 1, 1), src, row_stride, H, dn, rot,
                         rot_dims, inv_freq, positions, (OT*)q_nope, (OT*)q_lat, (const WT*)norm_w, eps, rank, token_req,
                         block_table, table_width, page_size, (OT*)pool),
          "latent_rows");
    });
  });
}

GB_EXPORT int gb_head_gemm(const void* a, int a_dtype, int a_row, int a_head, const void* w, int w_dtype,
                           long long w_head, int w_n, int w_k, void* out, int out_dtype, int out_row,
                           int out_head, int T, int H, int N, int K, int tail, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return GB_OK;
  if (N < 1 || K < 1 || tail < 0) return gb::fail(GB_BAD_ARGUMENT, "head_gemm: N %d, K %d, tail %d", N, K, tail);
  if (w_n != 1 && w_k != 1) return gb::fail(GB_UNSUPPORTED, "head_gemm: one of the weight's strides must be 1");
  const size_t smem = (size_t)TOK * (K + tail) * sizeof(float);
  if (smem > 48 * 1024) return gb::fail(GB_UNSUPPORTED, "head_gemm: rows of %d values are too wide", K + tail);
  dim3 grid((T + TOK - 1) / TOK, H);
  return GB_DISPATCH_DTYPE(a_dtype, AT, [&]() -> int {
    return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
      return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
        head_gemm_kernel<AT, WT, OT><<<grid, 256, smem, stream>>>((const AT*)a, a_row, a_head, (const WT*)w, w_head,
                                                                  w_n, w_k, (OT*)out, out_row, out_head, T, N, K, tail);
        return gb::check_launch("head_gemm");
      });
    });
  });
}
