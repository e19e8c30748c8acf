// Routed experts on the tensor cores (bfloat16, mma.sync.m16n8k16, 32-bit accumulators): the
// (token, choice) pairs of a step are sorted by expert on the device, every expert's rows are cut
// into tiles (of 128 rows, or of 16 where an expert has few), and two grouped products run over the tiles, each CTA reading its tile's
// expert from a list: gate/up with the activation in the epilogue, then down into one 32-bit row
// per pair; a last kernel adds a token's rows into the residual stream, weighted, in the
// router's order. Nothing comes back to the host in between, and the launches are the same
// whatever the router chose, so the step can be captured in a graph. An expert's weights are
// read once per tile of its rows. A row's result does not depend on where the sort put it: its
// sums run over k in a fixed order, and the pairs of a token are added in a fixed order.
#include "attention_mma_core.cuh"
#include "common.cuh"

namespace {

using attn_mma::ldmatrix_x4;
using attn_mma::mma_16816;

constexpr int GN = 64, GK = 64, STAGES = 3;
constexpr int TALL = 128, SHORT = 16;       // rows of a tile: groups of many rows, of a few
constexpr int GPITCH = GK * 2 + 16;          // bytes per row of a tile in shared memory (an odd number of 16-byte chunks)
constexpr int SORT_THREADS = 1024;

// One block. pair p = t * top + j goes to expert ids[p]. Out: row_pair[R] (sorted row -> pair),
// pair_row[R] (pair -> sorted row), and the tiles: expert, first sorted row and number of rows.
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int32_t* __restrict__ ids, int R, int E, int gm, int32_t* __restrict__ row_pair,
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
      for (int r0 = 0; r0 < c; r0 += gm) {
        tile_expert[nt] = e;
        tile_row0[nt] = run + r0;
        tile_rows[nt] = min(gm, c - r0);
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

// out[row0 + r][n] = sum_k A_e[r][k] * W_e[n][k] for the tile's rows r and columns n0 .. n0 + 63.
// A_e's row r is a[e * a_group + (gather ? gather[row0 + r] / gather_div : row0 + r) * lda ..];
// out's row is out[e * out_group + (row0 + r) * ldo ..]. GATED: W_e has N gate rows followed by N up
// rows (or the packed layout, see `packed`), and out (bfloat16) is act(gate, up). With a tile list (tile_expert ...) the CTA reads its
// group and rows from it; without, blockIdx.z is the group and every group has `rows_all` rows.
// The CTA is WM x WN warps, a warp's tile (MI * 16) x (NP * 16): 128 x 64 for groups of many rows,
// 16 x 64 for a few rows per group, where a taller tile would be padding. GATED with in_scale: the
// products of row r are multiplied by in_scale[gather[row0 + r]] before the activation (a factor on
// the expert's input, in which both products are linear).
template <int WM, int WN, int MI, int NP, bool GATED, typename OT>
__global__ void __launch_bounds__(WM * WN * 32)
grouped_gemm_kernel(const __nv_bfloat16* __restrict__ a, int lda, long long a_group, const int32_t* __restrict__ gather,
                    int gather_div, const __nv_bfloat16* __restrict__ w, long long w_group, OT* __restrict__ out, int ldo,
                    long long out_group, int N, int K, const int32_t* __restrict__ tile_expert,
                    const int32_t* __restrict__ tile_row0, const int32_t* __restrict__ tile_rows,
                    const int32_t* __restrict__ num_tiles, int rows_all, int kind, float limit, int packed,
                    const float* __restrict__ in_scale) {
  constexpr int TM = WM * MI * 16, TN = WN * NP * 16, THREADS = WM * WN * 32;
  constexpr int BROWS = GATED ? 2 * TN : TN;
  constexpr int CH = GK / 8;                       // 16-byte chunks of a tile's row
  extern __shared__ __align__(16) unsigned char tiles[];       // STAGES x (A tile, B tile)
  auto a_tile = [&](int stage) { return tiles + (size_t)stage * (TM + BROWS) * GPITCH; };
  auto b_tile = [&](int stage) { return tiles + ((size_t)stage * (TM + BROWS) + TM) * GPITCH; };
  __shared__ int32_t src_row[TM];
  __shared__ float row_scale[GATED ? TM : 1];
  int e, row0, rows;
  if (tile_expert != nullptr) {
    const int tile = blockIdx.y;
    if (tile >= *num_tiles) return;
    e = tile_expert[tile], row0 = tile_row0[tile], rows = tile_rows[tile];
  } else {
    e = blockIdx.z, row0 = blockIdx.y * TM, rows = min(TM, rows_all - row0);
    if (rows <= 0) return;
  }
  const int n0 = blockIdx.x * TN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int r = tid; r < TM; r += THREADS)
    src_row[r] = r < rows ? (gather ? gather[row0 + r] / gather_div : row0 + r) : -1;
  if (GATED)
    for (int r = tid; r < TM; r += THREADS)
      row_scale[r] = (in_scale != nullptr && gather != nullptr && r < rows) ? in_scale[gather[row0 + r]] : 1.0f;
  __syncthreads();
  const __nv_bfloat16* ae = a + (size_t)e * a_group;
  const __nv_bfloat16* we = w + (size_t)e * w_group;
  auto load = [&](int k0, int stage) {
    unsigned char* as = a_tile(stage);
    unsigned char* bs = b_tile(stage);
    for (int idx = tid; idx < TM * CH; idx += THREADS) {
      const int r = idx / CH, c = idx % CH;
      const int k = k0 + c * 8;
      const bool valid = src_row[r] >= 0 && k < K;
      cp16(as + r * GPITCH + c * 16, ae + (valid ? (size_t)src_row[r] * lda + k : 0), valid);
    }
    for (int idx = tid; idx < BROWS * CH; idx += THREADS) {
      const int r = idx / CH, c = idx % CH;
      const int k = k0 + c * 8;
      const int n = n0 + (r % TN);
      const bool valid = n < N && k < K;
      // gate row n and up row n of the group: N gate rows then N up rows, or (packed) gate and up rows
      // interleaved in groups of 64, which is the layout of the tcgen05 product's gated epilogue
      const size_t wrow = packed ? (size_t)((n >> 6) * 128 + (n & 63) + (r < TN ? 0 : 64)) : (size_t)(r < TN ? n : N + n);
      cp16(bs + r * GPITCH + c * 16, we + (valid ? wrow * K + k : 0), valid);
    }
  };
  const int wm = warp / WN, wn = warp % WN;
  float acc[MI][2 * NP][4], acc_u[GATED ? MI : 1][2 * NP][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < 2 * NP; ++j)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        acc[i][j][x] = 0.f;
        if (GATED) acc_u[GATED ? i : 0][j][x] = 0.f;
      }
  const int k_tiles = (K + GK - 1) / GK;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < k_tiles) load(st * GK, st);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    // tile kt has landed for every thread; the stage that tile kt - 1 was read from is free again
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    if (kt + STAGES - 1 < k_tiles) load((kt + STAGES - 1) * GK, (kt + STAGES - 1) % STAGES);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const unsigned char* as = a_tile(kt % STAGES);
    const unsigned char* bs = b_tile(kt % STAGES);
#pragma unroll
    for (int kk = 0; kk < GK; kk += 16) {
      uint32_t af[MI][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        ldmatrix_x4(af[mi], as + ((wm * MI + mi) * 16 + (lane & 15)) * GPITCH + (kk + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int np = 0; np < NP; ++np) {
        uint32_t b[4];
        const int brow = (wn * NP + np) * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldmatrix_x4(b, bs + brow * GPITCH + (kk + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
        for (int mi = 0; mi < MI; ++mi) {
          mma_16816(acc[mi][2 * np], af[mi], b[0], b[1]);
          mma_16816(acc[mi][2 * np + 1], af[mi], b[2], b[3]);
        }
        if (GATED) {
          ldmatrix_x4(b, bs + (TN + brow) * GPITCH + (kk + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
          for (int mi = 0; mi < MI; ++mi) {
            mma_16816(acc_u[GATED ? mi : 0][2 * np], af[mi], b[0], b[1]);
            mma_16816(acc_u[GATED ? mi : 0][2 * np + 1], af[mi], b[2], b[3]);
          }
        }
      }
    }
  }
  const int g = lane >> 2, tig = lane & 3;
  OT* oe = out + (size_t)e * out_group;
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int nt = 0; nt < 2 * NP; ++nt)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int r = (wm * MI + mi) * 16 + g + (x >> 1) * 8;
        const int n = n0 + wn * NP * 16 + nt * 8 + 2 * tig + (x & 1);
        if (r >= rows || n >= N) continue;
        float v = acc[mi][nt][x];
        if (GATED) v = gate_act(kind, limit, v * row_scale[GATED ? r : 0], acc_u[GATED ? mi : 0][nt][x] * row_scale[GATED ? r : 0]);
        oe[(size_t)(row0 + r) * ldo + n] = gb::from_float<OT>(v);
      }
}

// x[t][n] += alpha * sum_j weights[t][j] * y[pair_row[t * top + j]][n], j in the router's order; weights null: all one
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ pair_row, const float* __restrict__ weights,
                   float* __restrict__ x, int top, int N, float alpha) {
  const int t = blockIdx.x;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
      const int row = pair_row[(size_t)t * top + j];
      if (row >= 0) total = fmaf(weights ? weights[(size_t)t * top + j] : 1.0f, y[(size_t)row * N + n], total);
    }
    x[(size_t)t * N + n] = fmaf(alpha, total, x[(size_t)t * N + n]);
  }
}


template <int WM, int WN, int MI, int NP, bool GATED, typename OT, typename... Args>
int launch_grouped(dim3 grid, cudaStream_t stream, const char* what, Args... args) {
  constexpr int TM = WM * MI * 16, TN = WN * NP * 16;
  constexpr size_t smem = (size_t)STAGES * (TM + (GATED ? 2 * TN : TN)) * GPITCH;
  static gb::OncePerDevice attribute;
  auto kernel = grouped_gemm_kernel<WM, WN, MI, NP, GATED, OT>;
  if (smem > 48 * 1024 && attribute.needed()) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
    attribute.done();
  }
  kernel<<<grid, WM * WN * 32, smem, stream>>>(args...);
  return gb::check_launch(what);
}

}  // namespace

// Words of int32 work space for R = T * top pairs over E experts.
GB_EXPORT long long gb_moe_grouped_index_words(long long R, int E) {
  const long long tiles = (R + SHORT - 1) / SHORT + E;
  return 2 * R + 3 * tiles + 4;
}

// h [T, K], w_gate_up [E, 2F, K] (packed: [E, 128 * ceil(F / 64), K], gate and up rows in groups of 64),
// w_down [E, N, F] bfloat16; ids [T, top], weights [T, top]; x [T, N] 32-bit.
// index: gb_moe_grouped_index_words int32; act: [T * top, F] bfloat16; y: [T * top, N] 32-bit.
GB_EXPORT int gb_moe_grouped(const void* h, const void* w_gate_up, const void* w_down, const int32_t* ids,
                             const float* weights, float* x, int T, int top, int E, int F, int K, int N, int kind,
                             float limit, float alpha, int packed, int scale_input, int32_t* index, void* act, float* y,
                             cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (K % 8 || F % 8) return gb::fail(GB_UNSUPPORTED, "moe_grouped: widths %d and %d must be multiples of 8", K, F);
  if (E < 1 || (size_t)E * 2 * sizeof(int32_t) > 40 * 1024) return gb::fail(GB_UNSUPPORTED, "moe_grouped: %d experts", E);
  const long long R = (long long)T * top;
  const bool tall = R >= 48LL * E;             // on average 48 rows an expert or more
  const int gm = tall ? TALL : SHORT;
  const int max_tiles = (int)((R + gm - 1) / gm + E);
  const long long cap = (R + SHORT - 1) / SHORT + E;
  int32_t* row_pair = index;
  int32_t* pair_row = index + R;
  int32_t* tile_expert = index + 2 * R;
  int32_t* tile_row0 = tile_expert + cap;
  int32_t* tile_rows = tile_row0 + cap;
  int32_t* num_tiles = tile_rows + cap;
  moe_sort_kernel<<<1, SORT_THREADS, (size_t)E * 2 * sizeof(int32_t), stream>>>(ids, (int)R, E, gm, row_pair, pair_row,
                                                                               tile_expert, tile_row0, tile_rows, num_tiles);
  int rc = gb::check_launch("moe_sort");
  if (rc != GB_OK) return rc;
  const __nv_bfloat16* hh = (const __nv_bfloat16*)h;
  const __nv_bfloat16* wgu = (const __nv_bfloat16*)w_gate_up;
  const __nv_bfloat16* wd = (const __nv_bfloat16*)w_down;
  __nv_bfloat16* a = (__nv_bfloat16*)act;
  const dim3 grid_f((F + GN - 1) / GN, max_tiles), grid_n((N + GN - 1) / GN, max_tiles);
  const int32_t* none = nullptr;
  const int32_t *te = tile_expert, *t0 = tile_row0, *tr = tile_rows, *nt = num_tiles, *rp = row_pair;
  const float* in_scale = scale_input ? weights : nullptr;       // the weights scale what goes into an expert ...
  const float* out_weights = scale_input ? nullptr : weights;    // ... or what comes out of it
  const float* no_scale = nullptr;
  const long long zero = 0, gu_group = (long long)(packed ? 128 * ((F + 63) / 64) : 2 * F) * K, d_group = (long long)N * F;
  if (tall)
    rc = launch_grouped<4, 2, 2, 2, true, __nv_bfloat16>(grid_f, stream, "moe_gate_up_grouped", hh, K, zero, rp, top, wgu,
                                                        gu_group, a, F, zero, F, K, te, t0, tr, nt, 0, kind, limit, packed, in_scale);
  else
    rc = launch_grouped<1, 4, 1, 1, true, __nv_bfloat16>(grid_f, stream, "moe_gate_up_grouped", hh, K, zero, rp, top, wgu,
                                                        gu_group, a, F, zero, F, K, te, t0, tr, nt, 0, kind, limit, packed, in_scale);
  if (rc != GB_OK) return rc;
  const __nv_bfloat16* ac = a;
  if (tall)
    rc = launch_grouped<4, 2, 2, 2, false, float>(grid_n, stream, "moe_down_grouped", ac, F, zero, none, 1, wd, d_group, y, N,
                                                 zero, N, F, te, t0, tr, nt, 0, 0, 0.f, 0, no_scale);
  else
    rc = launch_grouped<1, 4, 1, 1, false, float>(grid_n, stream, "moe_down_grouped", ac, F, zero, none, 1, wd, d_group, y, N,
                                                 zero, N, F, te, t0, tr, nt, 0, 0, 0.f, 0, no_scale);
  if (rc != GB_OK) return rc;
  moe_combine_kernel<<<T, 256, 0, stream>>>(y, pair_row, out_weights, x, top, N, alpha);
  return gb::check_launch("moe_combine");
}

namespace {

constexpr int BLOCK_ROWS = 128;       // rows of a block of the tcgen05 grouped product: every block of one expert

// One block. Pair p = t * top + j goes to expert ids[p]; an expert's rows start at a multiple of
// BLOCK_ROWS. Out: pair_row[R] (pair -> row of the padded order) and, per block of rows, the first
// weight row of its expert in the stacked gate/up and down weights (blocks beyond the used ones: 0).
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_padded_kernel(const int32_t* __restrict__ ids, int R, int E, int gu_rows, int dn_rows, int blocks,
                       int32_t* __restrict__ pair_row, int32_t* __restrict__ block_w_gu, int32_t* __restrict__ block_w_dn) {
  extern __shared__ int32_t sm[];
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
    int blk = 0;
    for (int e = 0; e < E; ++e) {
      cursor[e] = blk * BLOCK_ROWS;
      for (int c = counts[e]; c > 0 && blk < blocks; c -= BLOCK_ROWS, ++blk) {
        block_w_gu[blk] = e * gu_rows;
        block_w_dn[blk] = e * dn_rows;
      }
    }
    for (; blk < blocks; ++blk) block_w_gu[blk] = block_w_dn[blk] = 0;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < R; p += blockDim.x) {
    const int e = ids[p];
    pair_row[p] = (e >= 0 && e < E) ? atomicAdd(&cursor[e], 1) : -1;
  }
}

// a[pair_row[p]] = h[p / top] (rows of K bfloat16, K a multiple of 8), one block per pair; with
// in_scale the row is multiplied by in_scale[p] (32-bit, rounded once)
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ h, const int32_t* __restrict__ pair_row, int top, int K,
                       __nv_bfloat16* __restrict__ a, const float* __restrict__ in_scale) {
  const int p = blockIdx.x, row = pair_row[p];
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(p / top) * K);
  uint4* dst = reinterpret_cast<uint4*>(a + (size_t)row * K);
  if (in_scale == nullptr) {
    for (int c = threadIdx.x; c < K / 8; c += blockDim.x) dst[c] = src[c];
    return;
  }
  const float s = in_scale[p];
  for (int c = threadIdx.x; c < K / 8; c += blockDim.x) {
    uint4 v = src[c];
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(pairs[i]);
      pairs[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
    }
    dst[c] = v;
  }
}

}  // namespace

// Rows of the padded order for R pairs over E experts (a multiple of 128), and its blocks.
GB_EXPORT long long gb_moe_padded_rows(long long R, int E) { return ((R + BLOCK_ROWS - 1) / BLOCK_ROWS + E) * BLOCK_ROWS; }

// For the tcgen05 grouped products: pairs sorted by expert into blocks of 128 rows, the tokens' rows
// gathered (padding rows zero). index: pair_row [R], then block_w_gu and block_w_dn [rows / 128 each].
GB_EXPORT int gb_moe_padded_prepare(const void* h, const int32_t* ids, int T, int top, int E, int K, int gu_rows,
                                    int dn_rows, int32_t* index, void* a_sorted, const float* in_scale,
                                    cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (K % 8 || E < 1 || (size_t)E * 2 * sizeof(int32_t) > 40 * 1024)
    return gb::fail(GB_UNSUPPORTED, "moe_padded_prepare: width %d, %d experts", K, E);
  const long long R = (long long)T * top, rows = gb_moe_padded_rows(R, E);
  const int blocks = (int)(rows / BLOCK_ROWS);
  int32_t* pair_row = index;
  int32_t* block_w_gu = index + R;
  int32_t* block_w_dn = block_w_gu + blocks;
  cudaError_t e = cudaMemsetAsync(a_sorted, 0, (size_t)rows * K * sizeof(__nv_bfloat16), stream);
  if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "moe_padded_prepare: %s", cudaGetErrorString(e));
  moe_sort_padded_kernel<<<1, SORT_THREADS, (size_t)E * 2 * sizeof(int32_t), stream>>>(ids, (int)R, E, gu_rows, dn_rows, blocks,
                                                                                      pair_row, block_w_gu, block_w_dn);
  int rc = gb::check_launch("moe_sort_padded");
  if (rc != GB_OK) return rc;
  moe_gather_rows_kernel<<<(unsigned)R, 128, 0, stream>>>((const __nv_bfloat16*)h, pair_row, top, K, (__nv_bfloat16*)a_sorted, in_scale);
  return gb::check_launch("moe_gather_rows");
}

// x[t] += alpha * sum_j weights[t][j] * y[pair_row[t * top + j]], j in the router's order
GB_EXPORT int gb_moe_combine(const float* y, const int32_t* pair_row, const float* weights, float* x, int T, int top,
                             int N, float alpha, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  moe_combine_kernel<<<T, 256, 0, stream>>>(y, pair_row, weights, x, top, N, alpha);
  return gb::check_launch("moe_combine");
}

// One product per group (a head) with the same number of rows in every group:
// out[g][r][n] = sum_k a[g][r][k] * w[g][n][k]; group strides in elements. bfloat16 operands.
GB_EXPORT int gb_grouped_gemm(const void* a, int lda, long long a_group, const void* w, long long w_group, void* out,
                              int ldo, long long out_group, int groups, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || groups <= 0) return GB_OK;
  if (K % 8 || lda % 8 || a_group % 8 || w_group % 8 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15))
    return gb::fail(GB_UNSUPPORTED, "grouped_gemm: operands must be 16-byte aligned row by row (K = %d)", K);
  if (groups > 65535) return gb::fail(GB_UNSUPPORTED, "grouped_gemm: %d groups", groups);
  const __nv_bfloat16* aa = (const __nv_bfloat16*)a;
  const __nv_bfloat16* ww = (const __nv_bfloat16*)w;
  __nv_bfloat16* oo = (__nv_bfloat16*)out;
  const int32_t* none = nullptr;
  if (M >= 48)
    return launch_grouped<4, 2, 2, 2, false, __nv_bfloat16>(dim3((N + GN - 1) / GN, (M + TALL - 1) / TALL, groups), stream,
                                                           "grouped_gemm", aa, lda, a_group, none, 1, ww, w_group, oo, ldo,
                                                           out_group, N, K, none, none, none, none, M, 0, 0.f, 0, (const float*)nullptr);
  return launch_grouped<1, 4, 1, 1, false, __nv_bfloat16>(dim3((N + GN - 1) / GN, (M + SHORT - 1) / SHORT, groups), stream,
                                                         "grouped_gemm", aa, lda, a_group, none, 1, ww, w_group, oo, ldo,
                                                         out_group, N, K, none, none, none, none, M, 0, 0.f, 0, (const float*)nullptr);
}
