// Latent attention: keys and values of all heads are read out of ONE small vector c a token (the latent), and one
// rotated key part is shared by all heads.  The cache keeps a token's row [c | rotated part] once, not a key and a
// value a head, and attention runs in the latent space:
//
//   score(t, j, head) = ( (W_uk,head^T q_plain) . c_j  +  q_rot . k_rot,j ) * scale
//   out(t, head)      = W_uv,head ( sum_j p_j c_j )
//
// since q_plain . (W_uk c) = (W_uk^T q_plain) . c and sum_j p_j (W_uv c_j) = W_uv sum_j p_j c_j.  So every head's
// query becomes [W_uk^T q_plain | q_rot], all heads attend to the same cached rows (one kv head, keys and values in
// the same pool), and W_uv is applied to the attended latent afterwards.  Two kernels serve this:
//
//   xrt_latent_prepare   from the 32-bit result of the [q | down] product: the latent's RMSNorm (32-bit), the rotation
//                        of the shared key part and of every head's rotated query part (32-bit angles), the cache row,
//                        and the rotated query parts at their place in the attention kernel's query rows
//   xrt_head_product     out[t, head, n] = sum_k x[t, head, k] W[head, n, k]: one small matrix a head, for both
//                        W_uk^T (before attention) and W_uv (after it); operands at any offset inside wider rows.
//                        bfloat16 matrices and results run on the tensor cores (m16n8k16, 32-bit sums), in a form for
//                        prompts and one for steps of up to 16 tokens; everything else by 32-bit multiply-adds
#include "attention_mma.cuh"

namespace xrt {

// One block a token.  Warp 0 writes the cache row; all warps walk the heads' rotated query parts.
// qd row: [heads x (dim | rot)] then, at down_offset, [rank | rot].  q_rows row: heads x [rank | rot | padding]
// of head_size.  cos_sin [T, rot / 2, 2]; pairs are (2i, 2i + 1) with `interleaved`, else (i, i + rot / 2).
template <typename TN, typename TQ, typename TC>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(TQ* __restrict__ q_rows, TC* __restrict__ pool, const float* __restrict__ qd, int row_stride,
                      int down_offset, const TN* __restrict__ norm_w, float eps, const float2* __restrict__ cos_sin,
                      const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                      const int* __restrict__ block_table, int max_blocks, int n_heads, int dim, int rot, int rank,
                      int head_size, int write_cache, int interleaved) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = tok_slot[t];
  TQ* q_row = q_rows + (size_t)t * n_heads * head_size;
  if (slot < 0) {  // a padding row: its queries are zero, the cache is not touched
    for (int e = threadIdx.x; e < n_heads * head_size; e += blockDim.x) q_row[e] = from_float<TQ>(0.f);
    return;
  }
  const int pos = tok_pos[t];
  const float* row = qd + (size_t)t * row_stride;
  const float2* cs = cos_sin + (size_t)t * (rot / 2);
  const int half = rot / 2;
  auto rotated = [&](const float* part, int d) {  // entry d of the rotated `part` (rot floats)
    if (interleaved) {
      const float2 a = cs[d >> 1];
      return (d & 1) ? part[d] * a.x + part[d - 1] * a.y : part[d] * a.x - part[d + 1] * a.y;
    }
    const float2 a = cs[d < half ? d : d - half];
    return d < half ? part[d] * a.x - part[d + half] * a.y : part[d] * a.x + part[d - half] * a.y;
  };
  if (warp == 0 && write_cache) {
    const int block = block_table[(size_t)slot * max_blocks + pos / XRT_BLOCK_TOKENS];
    if (block >= 0) {  // the host reserves blocks before the step
      TC* dst = pool + ((size_t)block * XRT_BLOCK_TOKENS + pos % XRT_BLOCK_TOKENS) * head_size;
      const float* down = row + down_offset;
      float sq = 0.f;
      for (int d = lane; d < rank; d += 32) sq = fmaf(down[d], down[d], sq);
      const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)rank + eps);
      for (int d = lane; d < rank; d += 32) dst[d] = from_float<TC>((down[d] * inv) * to_float(norm_w[d]));
      for (int d = lane; d < rot; d += 32) dst[rank + d] = from_float<TC>(rotated(down + rank, d));
      for (int d = rank + rot + lane; d < head_size; d += 32) dst[d] = from_float<TC>(0.f);
    }
  }
  // every head's rotated query part, and zeros in the padding columns; [0, rank) is the head product's to write
  const int tail = head_size - rank;
  for (int e = threadIdx.x; e < n_heads * tail; e += blockDim.x) {
    const int head = e / tail, d = e - head * tail;
    const float v = d < rot ? rotated(row + (size_t)head * (dim + rot) + dim, d) : 0.f;
    q_row[(size_t)head * head_size + rank + d] = from_float<TQ>(v);
  }
}

// out[t, head * out_head + out_off + n] = sum_k x[t, head * x_head + x_off + k] * w[head][n][k], 32-bit sums in one
// fixed order of k whatever the step holds.  Tiles of 64 tokens x 64 outputs, 16 along k; 256 threads, 4 x 4 each.
// ROUND_X: x is rounded to bfloat16 first (a 32-bit input of a bfloat16 product).
constexpr int HP_T = 64, HP_N = 64, HP_K = 16;
template <typename TX, typename TW, typename TO, bool ROUND_X>
__global__ void __launch_bounds__(256)
head_product_kernel(TO* __restrict__ out, int out_stride, int out_head, int out_off, const TX* __restrict__ x,
                    int x_stride, int x_head, int x_off, const TW* __restrict__ w, int n_tokens, int n, int k) {
  __shared__ float xs[HP_K][HP_T + 4];
  __shared__ float ws[HP_K][HP_N + 4];
  pdl_trigger();
  pdl_wait();
  const int t0 = blockIdx.x * HP_T, head = blockIdx.y, n0 = blockIdx.z * HP_N;
  const TX* xh = x + (size_t)head * x_head + x_off;
  const TW* wh = w + (size_t)head * n * k;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // outputs n0 + 4 tx .., tokens t0 + 4 ty ..
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < k; k0 += HP_K) {
    for (int e = threadIdx.x; e < HP_T * HP_K; e += 256) {
      const int r = e / HP_K, kk = e - r * HP_K;
      float v = 0.f;
      if (t0 + r < n_tokens && k0 + kk < k) {
        v = to_float(xh[(size_t)(t0 + r) * x_stride + k0 + kk]);
        if (ROUND_X) v = __bfloat162float(__float2bfloat16_rn(v));
      }
      xs[kk][r] = v;
    }
    for (int e = threadIdx.x; e < HP_N * HP_K; e += 256) {
      const int r = e / HP_K, kk = e - r * HP_K;
      ws[kk][r] = (n0 + r < n && k0 + kk < k) ? to_float(wh[(size_t)(n0 + r) * k + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HP_K; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[kk][4 * ty]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[kk][4 * tx]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + 4 * ty + i;
    if (t >= n_tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + 4 * tx + j;
      if (c < n) out[(size_t)t * out_stride + (size_t)head * out_head + out_off + c] = from_float<TO>(acc[i][j]);
    }
  }
}

// The same product on the tensor cores for bfloat16 matrices and results (x 32-bit, rounded first, or bfloat16):
// m16n8k16 steps over k in rising order with 32-bit sums, so a token's result does not depend on the tile it is in.
// 4 warps.  WM = 4: a block is 64 tokens x 64 outputs, a warp 16 tokens x 64; WM = 1 (a step of few tokens): 16 tokens
// x 32 outputs, a warp 8 outputs, and all of k (up to BK) is in flight at once.  VEC: every piece starts on a 16-byte
// (x: 4 elements) boundary and k is a multiple of 8; otherwise element by element.
template <typename TX, int WM, int NT, int BK, bool VEC>
__global__ void __launch_bounds__(128)
head_product_mma_kernel(__nv_bfloat16* __restrict__ out, int out_stride, int out_head, int out_off,
                        const TX* __restrict__ x, int x_stride, int x_head, int x_off,
                        const __nv_bfloat16* __restrict__ w, int n_tokens, int n, int k) {
  constexpr int BM = 16 * WM, BN = (4 / WM) * NT * 8, LD = BK + 8;
  __shared__ __align__(16) __nv_bfloat16 xs[BM][LD];
  __shared__ __align__(16) __nv_bfloat16 ws[BN][LD];
  pdl_trigger();
  pdl_wait();
  const int t0 = blockIdx.x * BM, head = blockIdx.y, n0 = blockIdx.z * BN;
  const TX* xh = x + (size_t)head * x_head + x_off;
  const __nv_bfloat16* wh = w + (size_t)head * n * k;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int row0 = (warp % WM) * 16, col0 = (warp / WM) * NT * 8;
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
  // VEC: a thread's pieces of the next stretch of k wait in registers while the tensor cores work on this one
  constexpr int XV = BM * (BK / 4) / 128, WV = BN * (BK / 8) / 128;
  static_assert(BM * (BK / 4) % 128 == 0 && BN * (BK / 8) % 128 == 0, "whole rounds of the block's threads");
  uint2 xr[XV];
  uint4 wr4[WV];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < XV; ++i) {
      const int e = threadIdx.x + i * 128, r = e / (BK / 4), c = (e - r * (BK / 4)) * 4;
      xr[i] = make_uint2(0u, 0u);
      if (t0 + r < n_tokens && k0 + c < k) {
        const TX* src = xh + (size_t)(t0 + r) * x_stride + k0 + c;
        if constexpr (sizeof(TX) == 4) {
          const float4 f = *reinterpret_cast<const float4*>(src);
          xr[i] = make_uint2(pack_bf16(f.x, f.y), pack_bf16(f.z, f.w));
        } else {
          xr[i] = *reinterpret_cast<const uint2*>(src);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < WV; ++i) {
      const int e = threadIdx.x + i * 128, r = e / (BK / 8), c = (e - r * (BK / 8)) * 8;
      wr4[i] = make_uint4(0u, 0u, 0u, 0u);
      if (n0 + r < n && k0 + c < k) wr4[i] = *reinterpret_cast<const uint4*>(wh + (size_t)(n0 + r) * k + k0 + c);
    }
  };
  if (VEC) fetch(0);
  for (int k0 = 0; k0 < k; k0 += BK) {
    if (VEC) {
#pragma unroll
      for (int i = 0; i < XV; ++i) {
        const int e = threadIdx.x + i * 128, r = e / (BK / 4), c = (e - r * (BK / 4)) * 4;
        *reinterpret_cast<uint2*>(&xs[r][c]) = xr[i];
      }
#pragma unroll
      for (int i = 0; i < WV; ++i) {
        const int e = threadIdx.x + i * 128, r = e / (BK / 8), c = (e - r * (BK / 8)) * 8;
        *reinterpret_cast<uint4*>(&ws[r][c]) = wr4[i];
      }
    } else {
      for (int e = threadIdx.x; e < BM * BK; e += 128) {
        const int r = e / BK, c = e - r * BK;
        float v = 0.f;
        if (t0 + r < n_tokens && k0 + c < k) v = to_float(xh[(size_t)(t0 + r) * x_stride + k0 + c]);
        xs[r][c] = __float2bfloat16_rn(v);
      }
      for (int e = threadIdx.x; e < BN * BK; e += 128) {
        const int r = e / BK, c = e - r * BK;
        ws[r][c] = (n0 + r < n && k0 + c < k) ? wh[(size_t)(n0 + r) * k + k0 + c] : __float2bfloat16_rn(0.f);
      }
    }
    __syncthreads();
    if (VEC && k0 + BK < k) fetch(k0 + BK);
#pragma unroll 4
    for (int kk = 0; kk < BK; kk += 16) {
      if (k0 + kk >= k) break;
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(&xs[row0 + g][kk + 2 * tq]);
      a[1] = *reinterpret_cast<const uint32_t*>(&xs[row0 + g + 8][kk + 2 * tq]);
      a[2] = *reinterpret_cast<const uint32_t*>(&xs[row0 + g][kk + 8 + 2 * tq]);
      a[3] = *reinterpret_cast<const uint32_t*>(&xs[row0 + g + 8][kk + 8 + 2 * tq]);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const __nv_bfloat16* wr = &ws[col0 + j * 8 + g][kk + 2 * tq];
        mma_16816(acc[j], a, *reinterpret_cast<const uint32_t*>(wr), *reinterpret_cast<const uint32_t*>(wr + 8));
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = t0 + row0 + g + (i >> 1) * 8, c = n0 + col0 + j * 8 + 2 * tq + (i & 1);
      if (t < n_tokens && c < n)
        out[(size_t)t * out_stride + (size_t)head * out_head + out_off + c] = __float2bfloat16_rn(acc[j][i]);
    }
}

template <typename TX, int WM, int NT, int BK>
static void launch_head_product_mma(bool vec, void* out, int out_stride, int out_head, int out_off, const void* x,
                                    int x_stride, int x_head, int x_off, const void* w, int n_tokens, int n_heads, int n,
                                    int k, cudaStream_t stream) {
  constexpr int BM = 16 * WM, BN = (4 / WM) * NT * 8;
  const dim3 grid((n_tokens + BM - 1) / BM, n_heads, (n + BN - 1) / BN);
  if (vec)
    launch_kernel(head_product_mma_kernel<TX, WM, NT, BK, true>, grid, dim3(128), 0, stream, (__nv_bfloat16*)out,
                  out_stride, out_head, out_off, (const TX*)x, x_stride, x_head, x_off, (const __nv_bfloat16*)w, n_tokens, n, k);
  else
    launch_kernel(head_product_mma_kernel<TX, WM, NT, BK, false>, grid, dim3(128), 0, stream, (__nv_bfloat16*)out,
                  out_stride, out_head, out_off, (const TX*)x, x_stride, x_head, x_off, (const __nv_bfloat16*)w, n_tokens, n, k);
}

template <typename TX>
static void head_product_mma(void* out, int out_stride, int out_head, int out_off, const void* x, int x_stride,
                             int x_head, int x_off, const void* w, int n_tokens, int n_heads, int n, int k,
                             cudaStream_t stream) {
  const bool vec = k % 8 == 0 && x_stride % 4 == 0 && x_head % 4 == 0 && x_off % 4 == 0 &&
                   (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0;
  if (n_tokens <= 16)
    launch_head_product_mma<TX, 1, 1, 256>(vec, out, out_stride, out_head, out_off, x, x_stride, x_head, x_off, w,
                                           n_tokens, n_heads, n, k, stream);
  else
    launch_head_product_mma<TX, 4, 8, 32>(vec, out, out_stride, out_head, out_off, x, x_stride, x_head, x_off, w,
                                          n_tokens, n_heads, n, k, stream);
}

}  // namespace xrt

// q_rows [T, heads * head_size] in q_dtype; pool [blocks, 1, 64, head_size] in cache_dtype (null with write_cache 0);
// qd float32 rows of row_stride floats; norm_w [rank]; cos_sin float32 [T, rot / 2, 2].
XRT_EXPORT int xrt_latent_prepare(void* q_rows, void* pool, const float* qd, int row_stride, int down_offset,
                                  const void* norm_w, float eps, const float* cos_sin, const int* tok_slot,
                                  const int* tok_pos, const int* block_table, int max_blocks, int n_tokens, int n_heads,
                                  int dim, int rot, int rank, int head_size, int write_cache, int interleaved,
                                  int norm_dtype, int q_dtype, int cache_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || dim <= 0 || rot < 0 || rot % 2 || rank <= 0 || head_size < rank + rot)
    return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  XRT_DISPATCH_DTYPE(norm_dtype, TN, {
    XRT_DISPATCH_DTYPE(q_dtype, TQ, {
      XRT_DISPATCH_DTYPE(cache_dtype, TC, {
        xrt::launch_kernel(xrt::latent_prepare_kernel<TN, TQ, TC>, dim3(n_tokens), dim3(128), 0, stream, (TQ*)q_rows,
                           (TC*)pool, qd, row_stride, down_offset, (const TN*)norm_w, eps, (const float2*)cos_sin,
                           tok_slot, tok_pos, block_table, max_blocks, n_heads, dim, rot, rank, head_size, write_cache,
                           interleaved);
      });
    });
  });
  return xrt::launch_status();
}

// Strides and offsets in elements.  w [heads, n, k] contiguous.
XRT_EXPORT int xrt_head_product(void* out, int out_stride, int out_head, int out_off, const void* x, int x_stride,
                                int x_head, int x_off, const void* w, int n_tokens, int n_heads, int n, int k,
                                int x_dtype, int w_dtype, int out_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || n <= 0 || k <= 0) return XRT_ERR_ARGUMENT;
  if (n_heads > 65535 || (n + xrt::HP_N - 1) / xrt::HP_N > 65535) return XRT_ERR_UNSUPPORTED;
  if (n_tokens == 0) return XRT_OK;
  if (w_dtype == XRT_BF16 && out_dtype == XRT_BF16 && (x_dtype == XRT_F32 || x_dtype == XRT_BF16)) {
    if (x_dtype == XRT_F32)
      xrt::head_product_mma<float>(out, out_stride, out_head, out_off, x, x_stride, x_head, x_off, w, n_tokens, n_heads,
                                   n, k, stream);
    else
      xrt::head_product_mma<__nv_bfloat16>(out, out_stride, out_head, out_off, x, x_stride, x_head, x_off, w, n_tokens,
                                           n_heads, n, k, stream);
    return xrt::launch_status();
  }
  const dim3 grid((n_tokens + xrt::HP_T - 1) / xrt::HP_T, n_heads, (n + xrt::HP_N - 1) / xrt::HP_N);
  XRT_DISPATCH_DTYPE(x_dtype, TX, {
    XRT_DISPATCH_DTYPE(w_dtype, TW, {
      XRT_DISPATCH_DTYPE(out_dtype, TO, {
        if (x_dtype == XRT_F32 && w_dtype == XRT_BF16)
          xrt::launch_kernel(xrt::head_product_kernel<TX, TW, TO, true>, grid, dim3(256), 0, stream, (TO*)out, out_stride,
                             out_head, out_off, (const TX*)x, x_stride, x_head, x_off, (const TW*)w, n_tokens, n, k);
        else
          xrt::launch_kernel(xrt::head_product_kernel<TX, TW, TO, false>, grid, dim3(256), 0, stream, (TO*)out, out_stride,
                             out_head, out_off, (const TX*)x, x_stride, x_head, x_off, (const TW*)w, n_tokens, n, k);
      });
    });
  });
  return xrt::launch_status();
}
