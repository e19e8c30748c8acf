// Routed experts on the tensor cores (bfloat16, mma.sync.m16n8k16, 32-bit accumulators): the
// (token, choice) pairs of a step are sorted by expert on the device, every expert's rows are cut
// into tiles of 64, and two grouped products run over the tiles, each CTA reading its tile's
// expert from a list: gate/up with the activation in the epilogue, then down into one 32-bit row
// per pair; a last kernel adds a token's rows into the residual stream, weighted, in the
// router's order. Nothing comes back to the host in between, and the launches are the same
// whatever the router chose, so the step can be captured in a graph. An expert's weights are
// read once per 64 of its rows. A row's result does not depend on where the sort put it: its
// sums run over k in a fixed order, and the pairs of a token are added in a fixed order.
#include "attention_mma_core.cuh"
#include "common.cuh"

namespace {

using attn_mma::ldmatrix_x4;
using attn_mma::mma_16816;

constexpr int GM = 64, GN = 64, GK = 32;
constexpr int GPITCH = GK * 2 + 16;          // bytes per row of a tile in shared memory (an odd number of 16-byte chunks)
constexpr int SORT_THREADS = 1024;

// One block. pair p = t * top + j goes to expert ids[p]. Out: row_pair[R] (sorted row -> pair),
// pair_row[R] (pair -> sorted row), and the tiles: expert, first sorted row and number of rows.
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int32_t* __restrict__ ids, int R, int E, int32_t* __restrict__ row_pair,
                int32_t* __restrict__ pair_row, int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_row0,
                int32_t* __restrict__ tile_rows, int32_t* __restrict__ num_tiles) {
  extern __shared__ int32_t sm[];            // counts[E], cursor[E]
  int32_t* counts = sm;
  int32_t* cursor = sm + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < R; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      const int c = counts[e];
      cursor[e] = run;
      for (int r0 = 0; r0 < c; r0 += GM) {
        tile_expert[nt] = e;
        tile_row0[nt] = run + r0;
        tile_rows[nt] = min(GM, c - r0);
        ++nt;
      }
      run += c;
    }
    *num_tiles = nt;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < R; p += blockDim.x) {
    const int e = ids[p];
    if (e < 0 || e >= E) { pair_row[p] = -1; continue; }
    const int pos = atomicAdd(&cursor[e], 1);
    row_pair[pos] = p;
    pair_row[p] = pos;
  }
}

__device__ __forceinline__ void cp16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

__device__ __forceinline__ float gate_act(int kind, float limit, float g, float u) {
  if (kind == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  if (kind == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return (g / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
  }
  return (g / (1.0f + expf(-g))) * u;
}

// out[row0 + r][n] = sum_k A[r][k] * W_e[n][k] for the tile's rows r and columns n0 .. n0 + 63.
// A's row r is a[(gather ? gather[row0 + r] / gather_div : row0 + r) * lda ..]. GATED: W_e has
// N gate rows followed by N up rows, and out (bfloat16) is act(gate, up); else out is 32-bit.
template <bool GATED, typename OT>
__global__ void __launch_bounds__(128)
moe_gemm_kernel(const __nv_bfloat16* __restrict__ a, int lda, const int32_t* __restrict__ gather, int gather_div,
                const __nv_bfloat16* __restrict__ w, long long w_expert, OT* __restrict__ out, int ldo, int N, int K,
                const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ tile_row0,
                const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ num_tiles, int kind, float limit) {
  constexpr int BROWS = GATED ? 2 * GN : GN;
  __shared__ __align__(16) unsigned char a_s[2][GM * GPITCH];
  __shared__ __align__(16) unsigned char b_s[2][BROWS * GPITCH];
  __shared__ int32_t src_row[GM];
  const int tile = blockIdx.y;
  if (tile >= *num_tiles) return;
  const int e = tile_expert[tile], row0 = tile_row0[tile], rows = tile_rows[tile];
  const int n0 = blockIdx.x * GN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < GM) {
    int r = -1;
    if (tid < rows) r = gather ? gather[row0 + tid] / gather_div : row0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)e * w_expert;
  auto load = [&](int k0, int stage) {
#pragma unroll
    for (int i = 0; i < GM * 4 / 128; ++i) {
      const int idx = tid + i * 128, r = idx >> 2, c = idx & 3;
      const int k = k0 + c * 8;
      const bool valid = src_row[r] >= 0 && k < K;
      cp16(a_s[stage] + r * GPITCH + c * 16, a + (size_t)(valid ? src_row[r] : 0) * lda + (valid ? k : 0), valid);
    }
#pragma unroll
    for (int i = 0; i < BROWS * 4 / 128; ++i) {
      const int idx = tid + i * 128, r = idx >> 2, c = idx & 3;
      const int k = k0 + c * 8;
      const int n = n0 + (r % GN);
      const bool valid = n < N && k < K;
      const size_t wrow = (size_t)(r < GN ? n : N + n);
      cp16(b_s[stage] + r * GPITCH + c * 16, we + (valid ? wrow * K + k : 0), valid);
    }
  };
  const int wm = warp >> 1, wn = warp & 1;
  float acc[2][4][4], acc_u[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        acc[i][j][x] = 0.f;
        if (GATED) acc_u[GATED ? i : 0][j][x] = 0.f;
      }
  const int k_tiles = (K + GK - 1) / GK;
  load(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int kt = 0; kt < k_tiles; ++kt) {
    if (kt + 1 < k_tiles) load((kt + 1) * GK, (kt + 1) & 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const unsigned char* as = a_s[kt & 1];
    const unsigned char* bs = b_s[kt & 1];
#pragma unroll
    for (int kk = 0; kk < GK; kk += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
        ldmatrix_x4(af[mi], as + (wm * 32 + mi * 16 + (lane & 15)) * GPITCH + (kk + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b[4];
        const int brow = wn * 32 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldmatrix_x4(b, bs + brow * GPITCH + (kk + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
          mma_16816(acc[mi][2 * np], af[mi], b[0], b[1]);
          mma_16816(acc[mi][2 * np + 1], af[mi], b[2], b[3]);
        }
        if (GATED) {
          ldmatrix_x4(b, bs + (GN + brow) * GPITCH + (kk + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) {
            mma_16816(acc_u[GATED ? mi : 0][2 * np], af[mi], b[0], b[1]);
            mma_16816(acc_u[GATED ? mi : 0][2 * np + 1], af[mi], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
  }
  const int g = lane >> 2, tig = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int r = wm * 32 + mi * 16 + g + (x >> 1) * 8;
        const int n = n0 + wn * 32 + nt * 8 + 2 * tig + (x & 1);
        if (r >= rows || n >= N) continue;
        float v = acc[mi][nt][x];
        if (GATED) v = gate_act(kind, limit, v, acc_u[GATED ? mi : 0][nt][x]);
        out[(size_t)(row0 + r) * ldo + n] = gb::from_float<OT>(v);
      }
}

// x[t][n] += alpha * sum_j weights[t][j] * y[pair_row[t * top + j]][n], j in the router's order
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ pair_row, const float* __restrict__ weights,
                   float* __restrict__ x, int top, int N, float alpha) {
  const int t = blockIdx.x;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
      const int row = pair_row[(size_t)t * top + j];
      if (row >= 0) total = fmaf(weights[(size_t)t * top + j], y[(size_t)row * N + n], total);
    }
    x[(size_t)t * N + n] = fmaf(alpha, total, x[(size_t)t * N + n]);
  }
}

}  // namespace

// Words of int32 work space for R = T * top pairs over E experts.
GB_EXPORT long long gb_moe_grouped_index_words(long long R, int E) {
  const long long tiles = (R + GM - 1) / GM + E;
  return 2 * R + 3 * tiles + 4;
}

// h [T, K], w_gate_up [E, 2F, K], w_down [E, N, F] bfloat16; ids [T, top], weights [T, top]; x [T, N] 32-bit.
// index: gb_moe_grouped_index_words int32; act: [T * top, F] bfloat16; y: [T * top, N] 32-bit.
GB_EXPORT int gb_moe_grouped(const void* h, const void* w_gate_up, const void* w_down, const int32_t* ids,
                             const float* weights, float* x, int T, int top, int E, int F, int K, int N, int kind,
                             float limit, float alpha, int32_t* index, void* act, float* y, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (K % 8 || F % 8) return gb::fail(GB_UNSUPPORTED, "moe_grouped: widths %d and %d must be multiples of 8", K, F);
  if (E < 1 || (size_t)E * 2 * sizeof(int32_t) > 40 * 1024) return gb::fail(GB_UNSUPPORTED, "moe_grouped: %d experts", E);
  const long long R = (long long)T * top;
  const int max_tiles = (int)((R + GM - 1) / GM + E);
  int32_t* row_pair = index;
  int32_t* pair_row = index + R;
  int32_t* tile_expert = index + 2 * R;
  int32_t* tile_row0 = tile_expert + max_tiles;
  int32_t* tile_rows = tile_row0 + max_tiles;
  int32_t* num_tiles = tile_rows + max_tiles;
  moe_sort_kernel<<<1, SORT_THREADS, (size_t)E * 2 * sizeof(int32_t), stream>>>(ids, (int)R, E, row_pair, pair_row,
                                                                               tile_expert, tile_row0, tile_rows, num_tiles);
  int rc = gb::check_launch("moe_sort");
  if (rc != GB_OK) return rc;
  moe_gemm_kernel<true, __nv_bfloat16><<<dim3((F + GN - 1) / GN, max_tiles), 128, 0, stream>>>(
      (const __nv_bfloat16*)h, K, row_pair, top, (const __nv_bfloat16*)w_gate_up, (long long)2 * F * K,
      (__nv_bfloat16*)act, F, F, K, tile_expert, tile_row0, tile_rows, num_tiles, kind, limit);
  if ((rc = gb::check_launch("moe_gate_up_grouped")) != GB_OK) return rc;
  moe_gemm_kernel<false, float><<<dim3((N + GN - 1) / GN, max_tiles), 128, 0, stream>>>(
      (const __nv_bfloat16*)act, F, nullptr, 1, (const __nv_bfloat16*)w_down, (long long)N * F, y, N, N, F,
      tile_expert, tile_row0, tile_rows, num_tiles, 0, 0.f);
  if ((rc = gb::check_launch("moe_down_grouped")) != GB_OK) return rc;
  moe_combine_kernel<<<T, 256, 0, stream>>>(y, pair_row, weights, x, top, N, alpha);
  return gb::check_launch("moe_combine");
}
