// The experts' products for steps of many tokens, bfloat16: rows sorted by expert (xrt_moe_group in moe.cu), ONE
// launch for all experts.  C[r] = A[r] . W_e^T for the rows r of expert e, with A [rows, K] and W [experts, N, K] both
// K-contiguous.  A block owns 64 rows of one expert and 64 output columns; its four warps take 16 rows each; tiles of
// 32 along K come by cp.async, two in flight; mma.sync m16n8k16 with 32-bit accumulators.  Which expert a block
// serves follows from the experts' row offsets: expert e has ceil(rows_e / 64) row tiles, numbered one expert after
// the other.
//   first product   N = 2 ff (an expert's gate rows, then its up rows): the block computes the gate columns and the
//                   matching up columns and writes act = g * sigmoid(alpha g) * (u + 1), g = min(gate, limit),
//                   u = clamp(up, -limit, limit), in bfloat16
//   second product  N = width: 32-bit results
//   first product of experts without a gate (MODE 2): N = ff, act = gelu(W_up h) with the exact (erf) gelu, bfloat16
// A row's result does not depend on which other rows share its tile.
#include "attention_mma.cuh"

namespace xrt {

constexpr int GG_ROWS = 64, GG_COLS = 64, GG_K = 32;
constexpr int GG_STRIDE = GG_K * 2 + 16;  // bytes of a shared row: 32 bfloat16 and padding against bank conflicts

struct GroupedArgs {
  const __nv_bfloat16* a;      // [rows, K]
  const __nv_bfloat16* w;      // [experts, N, K]
  const int* offsets;          // [experts + 1]
  void* out;                   // act bfloat16 [rows, ff] (first) or float [rows, N] (second)
  int n_experts, n, k, ff;
  float limit, alpha, up_shift;
};

// MODE 0: second product; 1: first product of gated experts; 2: first product of experts without a gate.
template <int MODE>
__global__ void __launch_bounds__(128) moe_grouped_product_kernel(const GroupedArgs g) {
  constexpr bool FIRST = MODE == 1;
  constexpr int W_TILES = FIRST ? 2 : 1;  // weight tiles a step: gate and up, or one
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_trigger();
  pdl_wait();
  // which expert, which of its row tiles
  int e = 0, tile = blockIdx.x, row0 = 0, row1 = 0;
  for (; e < g.n_experts; ++e) {
    row0 = g.offsets[e];
    row1 = g.offsets[e + 1];
    const int tiles = (row1 - row0 + GG_ROWS - 1) / GG_ROWS;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (e == g.n_experts) return;
  row0 += tile * GG_ROWS;
  const int col0 = blockIdx.y * GG_COLS;
  const int cols = FIRST ? g.ff : g.n;  // output columns of the block's kind
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
  const int j = lane >> 3, r = lane & 7;
  const __nv_bfloat16* w_e = g.w + (size_t)e * g.n * g.k;
  const int stage_bytes = (GG_ROWS + W_TILES * GG_COLS) * GG_STRIDE;

  auto issue = [&](int k0, int stage) {
    unsigned char* base = smem + stage * stage_bytes;
    // 64 rows x 4 pieces of 16 bytes for A, the same for every weight tile: 128 threads take two pieces of each
    for (int p = threadIdx.x; p < GG_ROWS * 4; p += blockDim.x) {
      const int row = p >> 2, piece = p & 3, kk = k0 + piece * 8;
      const bool live = row0 + row < row1 && kk < g.k;
      cp_async_16(smem_addr(base + row * GG_STRIDE + piece * 16), live ? g.a + (size_t)(row0 + row) * g.k + kk : g.a,
                  live ? 16 : 0);
#pragma unroll
      for (int wt = 0; wt < W_TILES; ++wt) {
        const int n = col0 + row + wt * g.ff;
        const bool there = col0 + row < cols && kk < g.k;
        cp_async_16(smem_addr(base + (GG_ROWS + wt * GG_COLS + row) * GG_STRIDE + piece * 16),
                    there ? w_e + (size_t)n * g.k + kk : w_e, there ? 16 : 0);
      }
    }
    cp_async_commit();
  };

  float acc[W_TILES][8][4];
#pragma unroll
  for (int wt = 0; wt < W_TILES; ++wt)
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[wt][nt][i] = 0.f;

  const int steps = (g.k + GG_K - 1) / GG_K;
  issue(0, 0);
  for (int s = 0; s < steps; ++s) {
    if (s + 1 < steps) { issue((s + 1) * GG_K, (s + 1) & 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const unsigned char* base = smem + (s & 1) * stage_bytes;
#pragma unroll
    for (int ks = 0; ks < GG_K / 16; ++ks) {
      uint32_t af[4];
      // matrix j of the x4 load: rows (j % 2) * 8 .., k (j / 2) * 8 ..
      ldmatrix_x4(af, smem_addr(base + (warp * 16 + (j & 1) * 8 + r) * GG_STRIDE + ks * 32 + (j >> 1) * 16));
#pragma unroll
      for (int wt = 0; wt < W_TILES; ++wt)
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bf[4];
          // matrix j: weight rows np * 16 + (j / 2) * 8 .., k (j % 2) * 8 ..
          ldmatrix_x4(bf, smem_addr(base + (GG_ROWS + wt * GG_COLS + np * 16 + (j >> 1) * 8 + r) * GG_STRIDE + ks * 32 +
                                    (j & 1) * 16));
          mma_16816(acc[wt][2 * np], af, bf[0], bf[1]);
          mma_16816(acc[wt][2 * np + 1], af, bf[2], bf[3]);
        }
    }
    __syncthreads();
  }
  // accumulator (nt, i): row warp * 16 + gq + 8 * (i / 2), column nt * 8 + 2 t + (i % 2)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = row0 + warp * 16 + gq + 8 * half;
    if (row >= row1) continue;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int col = col0 + nt * 8 + 2 * t + i;
        if (col >= cols) continue;
        if (FIRST) {
          const float gate = fminf(acc[0][nt][2 * half + i], g.limit);
          const float up = fminf(fmaxf(acc[W_TILES - 1][nt][2 * half + i], -g.limit), g.limit);
          ((__nv_bfloat16*)g.out)[(size_t)row * g.ff + col] =
              __float2bfloat16_rn(gate / (1.0f + expf(-g.alpha * gate)) * (up + g.up_shift));
        } else if (MODE == 2) {
          const float u = acc[0][nt][2 * half + i];
          ((__nv_bfloat16*)g.out)[(size_t)row * g.n + col] =
              __float2bfloat16_rn(0.5f * u * (1.0f + erff(u * 0.70710678118654752f)));
        } else {
          ((float*)g.out)[(size_t)row * g.n + col] = acc[0][nt][2 * half + i];
        }
      }
    }
  }
}

}  // namespace xrt

// first == 2: act [rows, n] bfloat16 = gelu(a . w^T) from w [experts, n, k] (experts without a gate).
// first == 3: as first == 1 with act = silu(gate) * up.
// first == 1: act [rows, ff] bfloat16 from a [rows, k] and w [experts, 2 ff, k]; else out [rows, n] float32 from
// a [rows, k] and w [experts, n, k].  offsets [experts + 1] int32 on the device; `rows` is their last entry's bound
// (the number of (token, choice) pairs).  k must be a multiple of 8 and the bases 16-byte aligned.
XRT_EXPORT int xrt_moe_grouped_product(void* out, const void* a, const void* w, const int* offsets, int rows, int n_experts,
                                       int n, int k, int ff, float limit, float alpha, int first, cudaStream_t stream) {
  float up_shift = 1.0f;
  if (first == 3) {  // gated silu experts: the gated form without limits and without the one added to the up rows
    first = 1;
    limit = INFINITY;
    alpha = 1.0f;
    up_shift = 0.0f;
  }
  if (rows < 0 || n_experts <= 0 || n <= 0 || k <= 0 || (first == 1 && (ff <= 0 || n != 2 * ff))) return XRT_ERR_ARGUMENT;
  if (k % 8 || (((uintptr_t)a | (uintptr_t)w) & 15)) return XRT_ERR_UNSUPPORTED;
  if (rows == 0) return XRT_OK;
  xrt::GroupedArgs g;
  g.a = (const __nv_bfloat16*)a; g.w = (const __nv_bfloat16*)w; g.offsets = offsets; g.out = out;
  g.n_experts = n_experts; g.n = n; g.k = k; g.ff = ff; g.limit = limit; g.alpha = alpha; g.up_shift = up_shift;
  const int row_tiles = (rows + xrt::GG_ROWS - 1) / xrt::GG_ROWS + n_experts;  // every expert may leave one tile partly empty
  const int cols = first == 1 ? ff : n;
  const int col_tiles = (cols + xrt::GG_COLS - 1) / xrt::GG_COLS;
  if (col_tiles > 65535) return XRT_ERR_UNSUPPORTED;
  const dim3 grid(row_tiles, col_tiles);
  if (first == 1) {
    const size_t smem = 2 * (size_t)(xrt::GG_ROWS + 2 * xrt::GG_COLS) * xrt::GG_STRIDE;
    xrt::launch_kernel(xrt::moe_grouped_product_kernel<1>, grid, dim3(128), smem, stream, g);
  } else {
    const size_t smem = 2 * (size_t)(xrt::GG_ROWS + xrt::GG_COLS) * xrt::GG_STRIDE;
    if (first == 2) xrt::launch_kernel(xrt::moe_grouped_product_kernel<2>, grid, dim3(128), smem, stream, g);
    else xrt::launch_kernel(xrt::moe_grouped_product_kernel<0>, grid, dim3(128), smem, stream, g);
  }
  return xrt::launch_status();
}
