// Token shift: what a mixer reads is blended, channel by channel, with what it read for the token before,
//
//   n_t = RMSNorm(x_t) * w          (32-bit)
//   h_t = n_t + (n_(t-1) - n_t) * shift[c]
//
// with n_(t-1) = 0 for a sequence's first token.  The norm and the blend are one kernel: a block has one token,
// norms its own row and, where the token before it lies in the same step, that row too (recomputed: the row is
// short and in the L2); the step's first token of a sequence reads n_(t-1) from the sequence's state
// [slot][width] (zero when the slot opens), and the step's last token leaves its n_t there.
//
// A step whose sequences bring one token each does all of that in one launch (the thread that reads a state
// entry is the one that writes it).  With longer portions the block of a sequence's first token reads the state
// that the block of its last token would write, so the state is written by a second launch of one block a
// sequence, after the first has read it.
//
// Beside it: x[t] += row, the vector that a pass over a stretch of layers begins with.
#include "common.cuh"

namespace xrt {

// mode 0: h for every token, the state is only read; mode 1: also the state (steps of single tokens)
template <typename TW, typename TO, int PER>
__global__ void rmsnorm_shift_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                                     const float* __restrict__ shift, float* __restrict__ state,
                                     const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, int n_tokens,
                                     int width, float eps, int mode) {
  __shared__ float scratch[33];
  pdl_trigger();
  const int t = blockIdx.x;
  float wv[PER], sv[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < width ? to_float(w[c]) : 0.f;
    sv[i] = c < width ? shift[c] : 0.f;
  }
  const int slot = tok_slot[t];  // the step's arrays were written before the step began
  const int pos = tok_pos[t];
  const bool inside = t > 0 && tok_slot[t - 1] == slot;  // the token before is a row of this step
  const bool last = t + 1 >= n_tokens || tok_slot[t + 1] != slot;
  pdl_wait();
  TO* dst = out + (size_t)t * width;
  if (slot < 0) {  // a padding row
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = from_float<TO>(0.f);
    return;
  }
  const float* row = x + (size_t)t * width;
  float cur[PER], prev[PER];
  float sum = 0.f, sum_prev = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    cur[i] = c < width ? row[c] : 0.f;
    prev[i] = 0.f;
    if (c < width && pos > 0) prev[i] = inside ? row[c - width] : state[(size_t)slot * width + c];
    sum = fmaf(cur[i], cur[i], sum);
    sum_prev = fmaf(prev[i], prev[i], sum_prev);
  }
  const float inv = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps);
  float inv_prev = 1.0f;
  if (inside) {  // uniform over the block
    __syncthreads();
    inv_prev = 1.0f / sqrtf(block_sum(sum_prev, scratch) / (float)width + eps);
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c >= width) continue;
    const float n = (cur[i] * inv) * wv[i];
    const float before = inside ? (prev[i] * inv_prev) * wv[i] : prev[i];
    dst[c] = from_float<TO>(n + (before - n) * sv[i]);
    if (mode == 1 && last) state[(size_t)slot * width + c] = n;
  }
}

// The state after a step of longer portions: the norm of every sequence's last row.  One block a sequence.
template <typename TW, int PER>
__global__ void rmsnorm_shift_state_kernel(float* __restrict__ state, const float* __restrict__ x,
                                           const TW* __restrict__ w, const int* __restrict__ cu_seqlens,
                                           const int* __restrict__ seq_slot, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x;
  const int slot = seq_slot[s];
  const int begin = cu_seqlens[s], end = cu_seqlens[s + 1];
  if (slot < 0 || end <= begin) return;
  const float* row = x + (size_t)(end - 1) * width;
  float cur[PER];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    cur[i] = c < width ? row[c] : 0.f;
    sum = fmaf(cur[i], cur[i], sum);
  }
  const float inv = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < width) state[(size_t)slot * width + c] = (cur[i] * inv) * to_float(w[c]);
  }
}

template <typename TW>
__global__ void add_row_kernel(float* __restrict__ x, const TW* __restrict__ row, size_t total, int width) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    x[i] += to_float(row[i % width]);
}

}  // namespace xrt

// out [T, width] in out_dtype; x float32 [T, width]; weight [width] in weight_dtype; shift float32 [width];
// state float32 [slots, width]; single_tokens: every sequence of the step brings one token.
XRT_EXPORT int xrt_rmsnorm_shift(void* out, const float* x, const void* weight, const float* shift, float* state,
                                 const int* tok_slot, const int* tok_pos, const int* cu_seqlens, const int* seq_slot,
                                 int n_seqs, int n_tokens, int width, float eps, int single_tokens, int weight_dtype,
                                 int out_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n_seqs < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const int threads = width >= 4096 ? 512 : (width >= 1024 ? 256 : (width >= 256 ? 128 : 64));
  const int per = (width + threads - 1) / threads;
  if (per > 32) return XRT_ERR_UNSUPPORTED;
#define XRT_SHIFT(PER)                                                                                                  \
  do {                                                                                                                  \
    xrt::launch_kernel(xrt::rmsnorm_shift_kernel<TW, TO, PER>, dim3(n_tokens), dim3(threads), 0, stream, (TO*)out, x,   \
                       (const TW*)weight, shift, state, tok_slot, tok_pos, n_tokens, width, eps,                        \
                       single_tokens ? 1 : 0);                                                                          \
    if (!single_tokens && n_seqs > 0)                                                                                   \
      xrt::launch_kernel(xrt::rmsnorm_shift_state_kernel<TW, PER>, dim3(n_seqs), dim3(threads), 0, stream, state, x,    \
                         (const TW*)weight, cu_seqlens, seq_slot, width, eps);                                          \
  } while (0)
  XRT_DISPATCH_DTYPE(weight_dtype, TW, {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      if (per <= 4) XRT_SHIFT(4);
      else if (per <= 8) XRT_SHIFT(8);
      else if (per <= 16) XRT_SHIFT(16);
      else XRT_SHIFT(32);
    });
  });
#undef XRT_SHIFT
  return xrt::launch_status();
}

// x[t, c] += row[c] in place; x float32 [T, width].
XRT_EXPORT int xrt_add_row(float* x, const void* row, int n_tokens, int width, int row_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t total = (size_t)n_tokens * width;
  const size_t blocks = (total + 255) / 256;
  XRT_DISPATCH_DTYPE(row_dtype, TW, {
    xrt::launch_kernel(xrt::add_row_kernel<TW>, dim3((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16)), dim3(256), 0,
                       stream, x, (const TW*)row, total, width);
  });
  return xrt::launch_status();
}
