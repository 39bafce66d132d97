// Attention of single new tokens for layers with score options (ScoreOptions in common.cuh: a window that keeps a
// sequence's first keys, a tanh cap, a distance slope, a sink term in the denominator), bfloat16 cache, 32-bit
// scores and sums.
//
// The keys a token sees are its kept first keys [0, kept) and its window [first, pos]: `total` keys, numbered
// 0 .. total - 1 in that order.  Grid (tokens, kv heads, splits): a block takes `chunk` of those numbers, its four
// warps 32 at a time, lane = key.  A lane reads its key's row once (16 bytes a load) and scores it against all
// query heads of the kv head's group (the queries wait in shared memory), so keys and values are fetched once a
// group, not once a head.  Every warp keeps a running maximum, sum and output per head; the warps of a block, then
// the splits of a token (second kernel), are merged in index order.  With one split the block writes the result.
#include "common.cuh"

namespace xrt {

constexpr int DS_WARPS = 4;

struct DecodeScoredArgs {
  __nv_bfloat16* out;            // [tokens, heads * head_dim]
  float* partial;                // [tokens, heads, splits, head_dim + 2] (o, then m, l), or null with one split
  const __nv_bfloat16 *q, *k_pool, *v_pool;
  const int *tok_slot, *tok_pos, *block_table;
  int max_blocks, n_heads, n_kv_heads, head_dim, window, chunk, n_splits;
  float scale;
  ScoreOptions opt;
};

// G: query heads a pass (a group of more heads takes several passes); PAIRS: value dims a lane holds, in pairs
// (dims 2 lane + 64 j, + 1): 64 PAIRS >= head_dim.
template <int G, int PAIRS>
__global__ void __launch_bounds__(DS_WARPS * 32) attention_decode_scored_kernel(const DecodeScoredArgs a) {
  extern __shared__ __align__(16) float shared[];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, kv = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hd = a.head_dim, group = a.n_heads / a.n_kv_heads;
  const int slot = a.tok_slot[t];
  if (slot < 0) {  // a padding row
    if (split == 0)
      for (int e = threadIdx.x; e < group * hd; e += blockDim.x)
        a.out[((size_t)t * a.n_heads + kv * group) * hd + e] = __float2bfloat16_rn(0.f);
    return;
  }
  const int pos = a.tok_pos[t];
  const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int kept = min(a.opt.keep_first, first);
  const int total = kept + pos - first + 1;
  const int v_begin = split * a.chunk, v_end = min(total, v_begin + a.chunk);
  const int* blocks = a.block_table + (size_t)slot * a.max_blocks;
  float* qs = shared;                                   // [G][hd]
  float* merge = shared + G * hd;                       // [warps][G][hd + 2]

  for (int h0 = 0; h0 < group; h0 += G) {
    const int n_g = min(G, group - h0);
    __syncthreads();
    for (int e = threadIdx.x; e < G * hd; e += blockDim.x) {
      const int g = e / hd, d = e - g * hd;
      qs[e] = g < n_g ? __bfloat162float(a.q[((size_t)t * a.n_heads + kv * group + h0 + g) * hd + d]) : 0.f;
    }
    __syncthreads();
    float slope[G], m[G], l[G], acc[G][2 * PAIRS];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int head = kv * group + h0 + g;
      slope[g] = a.opt.distance_rate > 0.f ? exp2f(-a.opt.distance_rate * (float)(head + 1) / (float)a.n_heads) : 0.f;
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int j = 0; j < 2 * PAIRS; ++j) acc[g][j] = 0.f;
    }
    for (int v0 = v_begin + warp * 32; v0 < v_end; v0 += DS_WARPS * 32) {
      const int v = v0 + lane;
      const bool live = v < v_end;
      const int key = live ? (v < kept ? v : first + v - kept) : pos;
      const size_t row = (((size_t)blocks[key / XRT_BLOCK_TOKENS] * a.n_kv_heads + kv) * XRT_BLOCK_TOKENS +
                          key % XRT_BLOCK_TOKENS) * hd;
      float s[G];
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = 0.f;
      if (live) {
        const __nv_bfloat16* kr = a.k_pool + row;
#pragma unroll 4
        for (int d = 0; d < hd; d += 8) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
          const __nv_bfloat162* kk = reinterpret_cast<const __nv_bfloat162*>(&raw);
          float kf[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(kk[j]);
            kf[2 * j] = f.x;
            kf[2 * j + 1] = f.y;
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 q0 = *reinterpret_cast<const float4*>(qs + g * hd + d);
            const float4 q1 = *reinterpret_cast<const float4*>(qs + g * hd + d + 4);
            s[g] = fmaf(kf[0], q0.x, s[g]); s[g] = fmaf(kf[1], q0.y, s[g]);
            s[g] = fmaf(kf[2], q0.z, s[g]); s[g] = fmaf(kf[3], q0.w, s[g]);
            s[g] = fmaf(kf[4], q1.x, s[g]); s[g] = fmaf(kf[5], q1.y, s[g]);
            s[g] = fmaf(kf[6], q1.z, s[g]); s[g] = fmaf(kf[7], q1.w, s[g]);
          }
        }
      }
      float p[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sc = s[g] * a.scale;
        if (a.opt.softcap > 0.f) sc = a.opt.softcap * tanhf(sc / a.opt.softcap);
        sc = live ? sc - slope[g] * (float)(pos - key) : -INFINITY;
        const float m_new = fmaxf(m[g], warp_max(sc));  // the warp's first key of the range is always live
        const float corr = expf(m[g] - m_new);
        p[g] = live ? expf(sc - m_new) : 0.f;
        l[g] = l[g] * corr + warp_sum(p[g]);
        m[g] = m_new;
#pragma unroll
        for (int j = 0; j < 2 * PAIRS; ++j) acc[g][j] *= corr;
      }
      // all 32 keys of the tile, several keys' loads in flight: a lane beyond the range holds weight 0 and the row
      // of the token's own key, which is there to be read
#pragma unroll 8
      for (int kk = 0; kk < 32; ++kk) {
        const size_t vrow = __shfl_sync(0xffffffffu, (unsigned long long)row, kk);
        float pk[G];
#pragma unroll
        for (int g = 0; g < G; ++g) pk[g] = __shfl_sync(0xffffffffu, p[g], kk);
        const __nv_bfloat16* vr = a.v_pool + vrow;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
          const int d = 2 * lane + 64 * j;
          if (d < hd) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vr + d));
#pragma unroll
            for (int g = 0; g < G; ++g) {
              acc[g][2 * j] = fmaf(pk[g], f.x, acc[g][2 * j]);
              acc[g][2 * j + 1] = fmaf(pk[g], f.y, acc[g][2 * j + 1]);
            }
          }
        }
      }
    }
    // the block's warps, in index order
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* mine = merge + ((size_t)warp * G + g) * (hd + 2);
#pragma unroll
      for (int j = 0; j < PAIRS; ++j) {
        const int d = 2 * lane + 64 * j;
        if (d < hd) { mine[d] = acc[g][2 * j]; mine[d + 1] = acc[g][2 * j + 1]; }
      }
      if (lane == 0) { mine[hd] = m[g]; mine[hd + 1] = l[g]; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_g * hd; e += blockDim.x) {
      const int g = e / hd, d = e - g * hd;
      float top = -INFINITY;
      for (int w = 0; w < DS_WARPS; ++w) top = fmaxf(top, merge[((size_t)w * G + g) * (hd + 2) + hd]);
      float sum = 0.f, o = 0.f;
      for (int w = 0; w < DS_WARPS; ++w) {
        const float* from = merge + ((size_t)w * G + g) * (hd + 2);
        const float f = from[hd] == -INFINITY ? 0.f : expf(from[hd] - top);
        sum = fmaf(from[hd + 1], f, sum);
        o = fmaf(from[d], f, o);
      }
      const int head = kv * group + h0 + g;
      if (a.partial == nullptr) {
        if (a.opt.sink) sum += expf(a.opt.sink_score - top);
        a.out[((size_t)t * a.n_heads + head) * hd + d] = __float2bfloat16_rn(o / sum);
      } else {
        float* dst = a.partial + (((size_t)t * a.n_heads + head) * a.n_splits + split) * (hd + 2);
        dst[d] = o;
        if (d == 0) { dst[hd] = top; dst[hd + 1] = sum; }
      }
    }
  }
}

// The splits of a (token, head), in index order.
__global__ void attention_decode_scored_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ partial,
                                                     const int* __restrict__ tok_slot, int n_heads, int head_dim,
                                                     int n_splits, int sink, float sink_score) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  if (tok_slot[t] < 0) return;  // the first kernel wrote the padding row's zeros
  const float* from = partial + ((size_t)t * n_heads + head) * n_splits * (head_dim + 2);
  float top = -INFINITY;
  for (int s = 0; s < n_splits; ++s) top = fmaxf(top, from[(size_t)s * (head_dim + 2) + head_dim]);
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float sum = 0.f, o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float* p = from + (size_t)s * (head_dim + 2);
      const float f = p[head_dim] == -INFINITY ? 0.f : expf(p[head_dim] - top);
      sum = fmaf(p[head_dim + 1], f, sum);
      o = fmaf(p[d], f, o);
    }
    if (sink) sum += expf(sink_score - top);
    out[((size_t)t * n_heads + head) * head_dim + d] = __float2bfloat16_rn(o / sum);
  }
}

template <int G, int PAIRS>
int launch_decode_scored(const DecodeScoredArgs& a, int n_tokens, cudaStream_t stream) {
  const size_t smem = ((size_t)G * a.head_dim + (size_t)DS_WARPS * G * (a.head_dim + 2)) * sizeof(float);
  auto kernel = attention_decode_scored_kernel<G, PAIRS>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(kernel, dim3(n_tokens, a.n_kv_heads, a.n_splits), dim3(DS_WARPS * 32), smem, stream, a);
  return launch_status();
}

}  // namespace xrt

// q, out: bfloat16 [tokens, heads * head_dim], one new token a row at tok_pos (rows with tok_slot < 0 give zeros);
// pools bfloat16 [blocks, kv heads, 64, head_dim].  A token's visible keys are cut into n_splits stretches of `chunk`
// (a multiple of 32; n_splits * chunk must cover window + keep_first, or the longest context without a window);
// partial: float32 scratch [tokens, heads, n_splits, head_dim + 2], unused with one split.
XRT_EXPORT int xrt_attention_decode_scored(void* out, float* partial, const void* q, const void* k_pool, const void* v_pool,
                                           const int* tok_slot, const int* tok_pos, const int* block_table, int max_blocks,
                                           int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                           int keep_first, float softcap, float distance_rate, int sink, float sink_score,
                                           int chunk, int n_splits, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || head_dim <= 0 || chunk <= 0 || n_splits <= 0)
    return XRT_ERR_ARGUMENT;
  if (head_dim % 8 || head_dim > 256 || chunk % 32 || n_tokens > 65535 * 32 || n_kv_heads > 65535 || n_splits > 65535 ||
      (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15))
    return XRT_ERR_UNSUPPORTED;
  if (n_splits > 1 && partial == nullptr) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  xrt::DecodeScoredArgs a;
  a.out = (__nv_bfloat16*)out;
  a.partial = n_splits > 1 ? partial : nullptr;
  a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
  a.tok_slot = tok_slot; a.tok_pos = tok_pos; a.block_table = block_table;
  a.max_blocks = max_blocks; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim;
  a.window = window; a.chunk = chunk; a.n_splits = n_splits; a.scale = scale;
  a.opt.keep_first = window > 0 && keep_first > 0 ? keep_first : 0;
  a.opt.softcap = softcap;
  a.opt.distance_rate = distance_rate;
  a.opt.sink = sink;
  a.opt.sink_score = sink_score;
  const int group = n_heads / n_kv_heads;
  const int pairs = head_dim <= 64 ? 1 : (head_dim <= 128 ? 2 : 4);
  int status;
#define XRT_DS(G)                                                                      \
  status = pairs == 1 ? xrt::launch_decode_scored<G, 1>(a, n_tokens, stream)           \
         : pairs == 2 ? xrt::launch_decode_scored<G, 2>(a, n_tokens, stream)           \
                      : xrt::launch_decode_scored<G, 4>(a, n_tokens, stream)
  if (group == 1) XRT_DS(1);
  else if (group == 2) XRT_DS(2);
  else if (group <= 4) XRT_DS(4);
  else XRT_DS(8);
#undef XRT_DS
  if (status != XRT_OK || n_splits == 1) return status;
  xrt::launch_kernel(xrt::attention_decode_scored_merge_kernel, dim3(n_tokens, n_heads), dim3(head_dim >= 128 ? 128 : 64), 0,
                     stream, (__nv_bfloat16*)out, (const float*)partial, tok_slot, n_heads, head_dim, n_splits, sink, sink_score);
  return xrt::launch_status();
}
