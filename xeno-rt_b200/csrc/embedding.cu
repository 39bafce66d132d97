// Embedding gather: rows of the table to the 32-bit residual stream.
// Restates crates/xrt-cuda/src/lib.rs:815-882 (embedding_kernel) of the reference, which writes
// zeros for an id outside the table while its host wrapper refuses such ids (1217-1225); here the
// kernel writes zeros and raises an error flag that the host reads.
#include "common.cuh"

namespace xrt {

template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab,
                                 int* __restrict__ error_flag, float scale) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
  const TW* row = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = ok ? to_float(row[c]) * scale : 0.f;
}

// 16 bytes of the table a thread and step (hidden a multiple of 8 for bfloat16, of 4 for float32)
template <typename TW>
__global__ void embedding_vec_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                     const int* __restrict__ ids, int hidden, int vocab,
                                     int* __restrict__ error_flag, float scale) {
  constexpr int PER = 16 / (int)sizeof(TW);
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
  const TW* row = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)t * hidden;
#pragma unroll 4
  for (int c = threadIdx.x * PER; c < hidden; c += blockDim.x * PER) {
    const uint4 raw = ok ? *reinterpret_cast<const uint4*>(row + c) : make_uint4(0u, 0u, 0u, 0u);
    const TW* vals = reinterpret_cast<const TW*>(&raw);
    float f[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) f[j] = ok ? to_float(vals[j]) * scale : 0.f;
#pragma unroll
    for (int j = 0; j < PER; j += 4) *reinterpret_cast<float4*>(dst + c + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
  }
}

// Token embedding plus a hashed embedding of the (previous, current) token pair:
//   out[t] = table[id] + pairs[(previous * mul_prev + id * mul_cur) mod buckets],   pairs[buckets] at a sequence's start.
// The previous token of a step's first token is the sequence's state `last_token[slot]`; the second kernel leaves the
// step's last token of every sequence there.  Rows of no sequence (slot < 0) are zeros.
template <typename TW>
__global__ void embedding_pair_kernel(float* __restrict__ out, const TW* __restrict__ table, const TW* __restrict__ pairs,
                                      const int* __restrict__ ids, const int* __restrict__ tok_slot,
                                      const int* __restrict__ tok_pos, const int* __restrict__ last_token, int hidden,
                                      int vocab, int buckets, int mul_prev, int mul_cur, int* __restrict__ error_flag) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t], slot = tok_slot[t];
  float* dst = out + (size_t)t * hidden;
  const bool ok = id >= 0 && id < vocab;
  if (slot < 0 || !ok) {
    if (slot >= 0 && threadIdx.x == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = 0.f;
    return;
  }
  long long row = buckets;
  if (tok_pos[t] > 0) {
    const int previous = (t > 0 && tok_slot[t - 1] == slot) ? ids[t - 1] : last_token[slot];
    row = ((long long)previous * mul_prev + (long long)id * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  const TW* a = table + (size_t)id * hidden;
  const TW* b = pairs + (size_t)row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_float(a[c]) + to_float(b[c]);
}

__global__ void embedding_pair_state_kernel(int* __restrict__ last_token, const int* __restrict__ ids,
                                            const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                                            int n_seqs) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_seqs) return;
  const int slot = seq_slot[s], end = cu_seqlens[s + 1];
  if (slot >= 0 && end > cu_seqlens[s]) last_token[slot] = ids[end - 1];
}

}  // namespace xrt

XRT_EXPORT int xrt_embedding_pair(float* out, const void* table, const void* pairs, const int* ids, const int* tok_slot,
                                  const int* tok_pos, int* last_token, const int* cu_seqlens, const int* seq_slot,
                                  int n_tokens, int n_seqs, int hidden, int vocab, int buckets, int mul_prev, int mul_cur,
                                  int table_dtype, int* error_flag, cudaStream_t stream) {
  if (n_tokens < 0 || n_seqs < 0 || hidden <= 0 || vocab <= 0 || buckets <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  XRT_DISPATCH_DTYPE(table_dtype, TW, {
    xrt::launch_kernel(xrt::embedding_pair_kernel<TW>, dim3(n_tokens), dim3(128), 0, stream, out, (const TW*)table,
                       (const TW*)pairs, ids, tok_slot, tok_pos, (const int*)last_token, hidden, vocab, buckets, mul_prev,
                       mul_cur, error_flag);
  });
  if (n_seqs > 0)
    xrt::launch_kernel(xrt::embedding_pair_state_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, last_token, ids,
                       cu_seqlens, seq_slot, n_seqs);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_embedding(float* out, const void* table, const int* ids, int n_tokens, int hidden,
                             int vocab, int table_dtype, int* error_flag, float scale, cudaStream_t stream) {
  if (n_tokens < 0 || hidden <= 0 || vocab <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const bool vec = hidden % 8 == 0 && (((uintptr_t)out | (uintptr_t)table) & 15) == 0;
  XRT_DISPATCH_DTYPE(table_dtype, TW, {
    if (vec)
      xrt::launch_kernel(xrt::embedding_vec_kernel<TW>, dim3(n_tokens), dim3(128), 0, stream, out, (const TW*)table, ids, hidden, vocab, error_flag, scale);
    else
      xrt::launch_kernel(xrt::embedding_kernel<TW>, dim3(n_tokens), dim3(256), 0, stream, out, (const TW*)table, ids, hidden, vocab, error_flag, scale);
  });
  return xrt::launch_status();
}
