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
//                        W_uk^T (before attention) and W_uv (after it); operands at any offset inside wider rows
#include "common.cuh"

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
