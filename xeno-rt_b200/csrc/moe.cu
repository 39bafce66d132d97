// A feed-forward made of many small gated experts of which every token uses a few.
//
//   routing   from the router's 32-bit logits z (bias added here): the `top` largest (the lower index wins a tie),
//             weights = softmax over those alone
//   expert    g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g * sigmoid(alpha g) * (u + 1),
//             result W_down y, times the token's weight for that expert
//
// The experts' matrices lie one after another: w_in [experts][gate rows | up rows][width], w_out [experts][width][ff].
// xrt_moe_experts computes every (token, choice) pair by itself (two kernels: the gated hidden units, then the
// output rows; blocks of 32 units or rows each stream their part of the expert's matrices) and writes
// out[choice][token][width];
// whoever follows adds a token's choices in index order, so the sum has one order whatever else is in the step.
// For steps of many tokens the rows are sorted by expert instead (xrt_moe_group, xrt_moe_gather), every expert's rows
// go through the library's matrix products with xrt_moe_activation between them, and xrt_moe_combine writes the same
// out[choice][token][width].
// A second kind of expert and of routing, chosen by a number (`act` 1, xrt_moe_route_scores):
//   expert    W_down gelu(W_up h) with the exact (erf) gelu; w_in then holds one block of ff rows an expert
//   routing   scores = softmax of the logits over ALL experts; the experts form `groups` equal groups of neighbours, a
//             group counts by its largest score and only experts of the `keep` best groups can be chosen; the `top`
//             largest scores among those win, and a chosen expert's weight is its score as it is (no renormalizing)
//   options of that routing (RouteOptions): scores = sigmoid of each logit instead of the softmax; a `correction` a
//             expert that is added to the score for every choice (of groups and of experts) but not for the weight; a
//             group that counts by the sum of its `group_best` largest choice scores instead of the largest; weights
//             divided by their sum (+ `sum_eps`) and multiplied by `scale`
#include "common.cuh"

namespace xrt {

constexpr int MOE_ACT_GATED = 0, MOE_ACT_GELU = 1, MOE_ACT_SILU = 2;

// A third kind of expert (`act` 2): W_down (silu(W_gate h) * (W_up h)), the gated form without limits and without the
// one added to the up rows: the gated kernels run it with limit = infinity, alpha = 1 and `up_shift` = 0.
struct GateForm { float limit, alpha, up_shift; };
inline GateForm gate_form(int act_kind, float limit, float alpha) {
  if (act_kind == MOE_ACT_SILU) return {INFINITY, 1.0f, 0.0f};
  return {limit, alpha, 1.0f};
}

__device__ __forceinline__ float gelu_erf(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f)); }

struct RouteOptions {
  int sigmoid = 0;                    // scores = 1 / (1 + exp(-z)) each, not the softmax over all
  const float* correction = nullptr;  // [experts]: choice score = score + correction
  int group_best = 1;                 // a group counts by the sum of so many of its largest choice scores
  int normalize = 0;                  // weights / (their sum + sum_eps) ...
  float sum_eps = 0.f;
  float scale = 1.f;                  // ... times scale
};

// One warp a token.  Lane l holds logits l, l + 32, ...; group_best [warps][groups] in shared memory.
template <int PER_LANE>
__global__ void moe_route_scores_kernel(int* __restrict__ ids, float* __restrict__ weights,
                                        const float* __restrict__ logits, int n_tokens, int n_experts, int top,
                                        int groups, int keep, const RouteOptions opt) {
  extern __shared__ float group_best[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tokens) return;
  float z[PER_LANE];
  float top_z = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = lane + 32 * i;
    z[i] = e < n_experts ? logits[(size_t)t * n_experts + e] : -INFINITY;
    top_z = fmaxf(top_z, z[i]);
  }
  top_z = warp_max(top_z);
  float score[PER_LANE];  // what a chosen expert's weight is made of; z becomes what the choice goes by
  if (opt.sigmoid) {
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < n_experts ? 1.0f / (1.0f + expf(-z[i])) : 0.f;
      z[i] = e < n_experts ? score[i] : -INFINITY;
    }
  } else {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      z[i] = lane + 32 * i < n_experts ? expf(z[i] - top_z) : -INFINITY;  // from here on z holds the scores' numerators
      if (lane + 32 * i < n_experts) sum += z[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      if (lane + 32 * i < n_experts) z[i] /= sum;
      score[i] = z[i];
    }
  }
  if (opt.correction != nullptr) {
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts) z[i] += opt.correction[e];
    }
  }
  if (keep < groups) {
    float* best_of = group_best + (size_t)warp * groups;
    const int size = n_experts / groups;
    for (int g = 0; g < groups; ++g) {
      // the sum of the group's `group_best` largest choice scores (one: the largest), taken one at a time
      float worth = 0.f;
      unsigned taken = 0u;  // bit i: this lane's i-th entry went into the sum already
      for (int r = 0; r < opt.group_best && r < size; ++r) {
        float b = -INFINITY;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
          const int e = lane + 32 * i;
          if (e < n_experts && e / size == g && !(taken >> i & 1u) && (z[i] > b || be == 0x7fffffff)) { b = z[i]; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float other = __shfl_xor_sync(0xffffffffu, b, o);
          const int other_e = __shfl_xor_sync(0xffffffffu, be, o);
          if (other_e != 0x7fffffff && (be == 0x7fffffff || other > b || (other == b && other_e < be))) { b = other; be = other_e; }
        }
        if (be == 0x7fffffff) break;
        if ((be & 31) == lane) taken |= 1u << (be >> 5);
        worth = r == 0 ? b : worth + b;
      }
      if (lane == 0) best_of[g] = worth;
    }
    __syncwarp();
    // the keep best groups, one at a time (the lower number wins a tie); a taken group's entry becomes +inf
    for (int r = 0; r < keep; ++r) {
      float b = -INFINITY;
      int bg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = best_of[g];
        if (v != INFINITY && (v > b || (v == b && g < bg) || bg == 0x7fffffff)) { b = v; bg = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, b, o);
        const int other_g = __shfl_xor_sync(0xffffffffu, bg, o);
        if (other_g != 0x7fffffff && (bg == 0x7fffffff || other > b || (other == b && other_g < bg))) { b = other; bg = other_g; }
      }
      __syncwarp();
      if (lane == 0 && bg != 0x7fffffff) best_of[bg] = INFINITY;
      __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < n_experts && best_of[e / size] != INFINITY) z[i] = -INFINITY;  // not of a kept group
    }
  }
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (z[i] > best || (z[i] == best && e < best_e && z[i] > -INFINITY)) { best = z[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    float weight = 0.f;  // the chosen expert's score without the correction
    if (best_e >= n_experts) {  // a row of logits that are no numbers (a padding row's): any expert, no weight
      best_e = c;
    } else {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (i == (best_e >> 5)) weight = __shfl_sync(0xffffffffu, score[i], best_e & 31);
    }
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i)
      if (lane + 32 * i == best_e) z[i] = -INFINITY;  // taken
    if (lane == 0) {
      ids[(size_t)t * top + c] = best_e;
      weights[(size_t)t * top + c] = weight;
    }
  }
  if (opt.normalize) {  // lane 0 wrote the weights; it adds them up in the order of the choices
    __syncwarp();
    if (lane == 0) {
      float sum = 0.f;
      for (int c = 0; c < top; ++c) sum += weights[(size_t)t * top + c];
      const float f = opt.scale / (sum + opt.sum_eps);
      for (int c = 0; c < top; ++c) weights[(size_t)t * top + c] *= f;
    }
  } else if (opt.scale != 1.f) {
    __syncwarp();
    if (lane == 0)
      for (int c = 0; c < top; ++c) weights[(size_t)t * top + c] *= opt.scale;
  }
}

// One warp a token.  Lane l holds logits l, l + 32, ...
template <int PER_LANE>
__global__ void moe_route_kernel(int* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits,
                                 const float* __restrict__ bias, int n_tokens, int n_experts, int top) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  float z[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = lane + 32 * i;
    z[i] = e < n_experts ? logits[(size_t)t * n_experts + e] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
  }
  float first = 0.f, sum = 0.f;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (z[i] > best || (z[i] == best && e < best_e && z[i] > -INFINITY)) { best = z[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (best_e >= n_experts) {  // a row of logits that are no numbers (a padding row's): any expert, weight as it comes
      best_e = c;
      best = first;
    }
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i)
      if (lane + 32 * i == best_e) z[i] = -INFINITY;  // taken
    if (c == 0) first = best;
    const float p = expf(best - first);  // the first choice is the largest logit
    sum += p;
    if (lane == 0) {
      ids[(size_t)t * top + c] = best_e;
      weights[(size_t)t * top + c] = p;
    }
  }
  __syncwarp();
  for (int c = lane; c < top; c += 32) weights[(size_t)t * top + c] /= sum;
}

// R dot products of weight rows with one vector in shared memory at once (rows[i] null: none), 16 bytes of a row a
// lane and step where VEC (the row's length a multiple of 16 bytes' worth and the rows 16-byte aligned), else one
// element a lane and step; a row's sum runs over k in rising order a lane, then over the lanes, whatever R is.  A
// warp has R rows' loads of DEPTH steps in flight and reads the vector once for all of them.
template <typename TW, bool VEC, int R, int DEPTH>
__device__ __forceinline__ void rows_dot(float (&out)[R], const TW* const (&rows)[R], const float* __restrict__ x, int n,
                                         int lane) {
  constexpr int PER = 16 / (int)sizeof(TW);
  float acc[R];
#pragma unroll
  for (int i = 0; i < R; ++i) acc[i] = 0.f;
  if (VEC) {
#pragma unroll DEPTH
    for (int k = lane * PER; k < n; k += 32 * PER) {
      uint4 raw[R];
#pragma unroll
      for (int i = 0; i < R; ++i)
        raw[i] = rows[i] != nullptr ? *reinterpret_cast<const uint4*>(rows[i] + k) : make_uint4(0u, 0u, 0u, 0u);
      float xv[PER];
#pragma unroll
      for (int j = 0; j < PER; ++j) xv[j] = x[k + j];
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const TW* v = reinterpret_cast<const TW*>(&raw[i]);
#pragma unroll
        for (int j = 0; j < PER; ++j) acc[i] = fmaf(to_float(v[j]), xv[j], acc[i]);
      }
    }
  } else {
    for (int k = lane; k < n; k += 32) {
      const float xv = x[k];
#pragma unroll
      for (int i = 0; i < R; ++i)
        if (rows[i] != nullptr) acc[i] = fmaf(to_float(rows[i][k]), xv, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) out[i] = warp_sum(acc[i]);
}

// First half of a (token, choice) pair: act[pair][j] for the hidden units j of this block (UNITS a block, one warp a
// unit at a time).  grid (tokens, top, ceil(ff / UNITS)).
// UNITS = 32: a warp takes four units (or the gate and up rows of two) at a time; UNITS = 8 (few pairs: more,
// smaller blocks so that every multiprocessor streams): one unit a warp, its row's loads further ahead instead.
constexpr int MOE_UNITS = 32, MOE_UNITS_FEW = 8, MOE_WARPS = 8;
template <typename TX, typename TW, bool VEC, int UNITS>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_experts_in_kernel(float* __restrict__ act, const TX* __restrict__ h, const TW* __restrict__ w_in,
                      const int* __restrict__ ids, int width, int ff, int top, float limit, float alpha, float up_shift,
                      int act_kind) {
  extern __shared__ float hs[];  // [width]
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y;
  constexpr int n_warps = MOE_WARPS, R = UNITS / MOE_WARPS, DEPTH = R >= 4 ? 4 : 8, G = R >= 2 ? R / 2 : 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = ids[(size_t)t * top + c];
  for (int k = threadIdx.x; k < width; k += blockDim.x) hs[k] = to_float(h[(size_t)t * width + k]);
  __syncthreads();
  const int j1 = min(ff, (int)(blockIdx.z + 1) * UNITS);
  if (act_kind == MOE_ACT_GELU) {  // one block of ff rows an expert, no gate
    const TW* only = w_in + (size_t)e * ff * width;
    for (int j = blockIdx.z * UNITS + warp; j < j1; j += R * n_warps) {  // R of the warp's units at a time
      const TW* rows[R];
      float u[R];
#pragma unroll
      for (int i = 0; i < R; ++i) rows[i] = j + i * n_warps < j1 ? only + (size_t)(j + i * n_warps) * width : nullptr;
      rows_dot<TW, VEC, R, DEPTH>(u, rows, hs, width, lane);
#pragma unroll
      for (int i = 0; i < R; ++i)
        if (lane == 0 && rows[i] != nullptr) act[((size_t)t * top + c) * ff + j + i * n_warps] = gelu_erf(u[i]);
    }
    return;
  }
  const TW* gate = w_in + (size_t)e * 2 * ff * width;
  const TW* up = gate + (size_t)ff * width;
  for (int j = blockIdx.z * UNITS + warp; j < j1; j += G * n_warps) {  // gate and up rows of G units at a time
    const TW* rows[2 * G];
    float gu[2 * G];
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const bool live = j + i * n_warps < j1;
      rows[2 * i] = live ? gate + (size_t)(j + i * n_warps) * width : nullptr;
      rows[2 * i + 1] = live ? up + (size_t)(j + i * n_warps) * width : nullptr;
    }
    rows_dot<TW, VEC, 2 * G, DEPTH>(gu, rows, hs, width, lane);
#pragma unroll
    for (int i = 0; i < G; ++i)
      if (lane == 0 && rows[2 * i] != nullptr) {
        const float g = fminf(gu[2 * i], limit);
        const float u = fminf(fmaxf(gu[2 * i + 1], -limit), limit);
        act[((size_t)t * top + c) * ff + j + i * n_warps] = g / (1.0f + expf(-alpha * g)) * (u + up_shift);
      }
  }
}

// Second half: out[c][t][r] = weight * (W_down[e] act)[r] for the rows r of this block.  grid (tokens, top, ceil(width / UNITS)).
template <typename TW, bool VEC, int UNITS>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_experts_out_kernel(float* __restrict__ out, const float* __restrict__ act, const TW* __restrict__ w_out,
                       const int* __restrict__ ids, const float* __restrict__ weights, int n_tokens, int width, int ff,
                       int top) {
  extern __shared__ float ys[];  // [ff]
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y;
  constexpr int n_warps = MOE_WARPS, R = UNITS / MOE_WARPS, DEPTH = R >= 4 ? 4 : 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = ids[(size_t)t * top + c];
  const float weight = weights[(size_t)t * top + c];
  for (int k = threadIdx.x; k < ff; k += blockDim.x) ys[k] = act[((size_t)t * top + c) * ff + k];
  __syncthreads();
  const TW* down = w_out + (size_t)e * width * ff;
  float* dst = out + ((size_t)c * n_tokens + t) * width;
  const int r1 = min(width, (int)(blockIdx.z + 1) * UNITS);
  for (int r = blockIdx.z * UNITS + warp; r < r1; r += R * n_warps) {  // R of the warp's rows at a time
    const TW* rows[R];
    float acc[R];
#pragma unroll
    for (int i = 0; i < R; ++i) rows[i] = r + i * n_warps < r1 ? down + (size_t)(r + i * n_warps) * ff : nullptr;
    rows_dot<TW, VEC, R, DEPTH>(acc, rows, ys, ff, lane);
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (lane == 0 && rows[i] != nullptr) dst[r + i * n_warps] = weight * acc[i];
  }
}

// ---- the same for many tokens: rows sorted by expert, one product an expert -----------------------------------
// One block.  offsets[e] .. offsets[e + 1] are the rows of expert e in the sorted order; pos[pair] is the row of
// (token, choice) pair `pair`, row_token[row] the token of a row.  The order of an expert's rows among themselves
// is whatever the atomics give: no row's result depends on its neighbours.
__global__ void __launch_bounds__(1024)
moe_group_kernel(int* __restrict__ offsets, int* __restrict__ pos, int* __restrict__ row_token,
                 const int* __restrict__ ids, int n_pairs, int n_experts, int top) {
  extern __shared__ int counts[];  // [experts] counts, then [experts] cursors
  int* cursor = counts + n_experts;
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&counts[ids[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      at += counts[e];
    }
    offsets[n_experts] = at;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int row = atomicAdd(&cursor[ids[p]], 1);
    pos[p] = row;
    row_token[row] = p / top;
  }
}

template <typename TX>
__global__ void moe_gather_kernel(TX* __restrict__ out, const TX* __restrict__ h, const int* __restrict__ row_token,
                                  int width) {
  pdl_trigger();
  pdl_wait();
  const TX* src = h + (size_t)row_token[blockIdx.x] * width;
  TX* dst = out + (size_t)blockIdx.x * width;
  for (int k = threadIdx.x; k < width; k += blockDim.x) dst[k] = src[k];
}

// act[r, j] = g * sigmoid(alpha g) * (u + 1) with g = min(gu[r, j], limit), u = clamp(gu[r, ff + j], -limit, limit)
template <typename TO>
__global__ void moe_activation_kernel(TO* __restrict__ act, const float* __restrict__ gate_up, size_t total, int ff,
                                      float limit, float alpha, float up_shift, int act_kind) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    if (act_kind == MOE_ACT_GELU) {  // gate_up holds [rows, ff]
      act[i] = from_float<TO>(gelu_erf(gate_up[i]));
      continue;
    }
    const size_t r = i / ff, j = i - r * ff;
    const float g = fminf(gate_up[r * 2 * ff + j], limit);
    const float u = fminf(fmaxf(gate_up[r * 2 * ff + ff + j], -limit), limit);
    act[i] = from_float<TO>(g / (1.0f + expf(-alpha * g)) * (u + up_shift));
  }
}

// out[c][t] = weights[t][c] * y[pos[t * top + c]]
__global__ void moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y, const int* __restrict__ pos,
                                   const float* __restrict__ weights, int n_tokens, int width, int top) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y;
  const float w = weights[(size_t)t * top + c];
  const float* src = y + (size_t)pos[(size_t)t * top + c] * width;
  float* dst = out + ((size_t)c * n_tokens + t) * width;
  for (int k = threadIdx.x; k < width; k += blockDim.x) dst[k] = w * src[k];
}

}  // namespace xrt

XRT_EXPORT int xrt_moe_group(int* offsets, int* pos, int* row_token, const int* ids, int n_tokens, int n_experts, int top,
                             cudaStream_t stream) {
  if (n_tokens < 0 || n_experts <= 0 || top <= 0) return XRT_ERR_ARGUMENT;
  if (n_experts > 4096) return XRT_ERR_UNSUPPORTED;
  xrt::launch_kernel(xrt::moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * n_experts * sizeof(int), stream, offsets, pos,
                     row_token, ids, n_tokens * top, n_experts, top);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_moe_gather(void* out, const void* h, const int* row_token, int n_rows, int width, int dtype,
                              cudaStream_t stream) {
  if (n_rows < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_rows == 0) return XRT_OK;
  XRT_DISPATCH_DTYPE(dtype, TX, {
    xrt::launch_kernel(xrt::moe_gather_kernel<TX>, dim3(n_rows), dim3(128), 0, stream, (TX*)out, (const TX*)h, row_token,
                       width);
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_moe_activation(void* act, const float* gate_up, int n_rows, int ff, float limit, float alpha,
                                  int act_kind, int out_dtype, cudaStream_t stream) {
  if (n_rows < 0 || ff <= 0) return XRT_ERR_ARGUMENT;
  if (n_rows == 0) return XRT_OK;
  const size_t total = (size_t)n_rows * ff;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  const xrt::GateForm form = xrt::gate_form(act_kind, limit, alpha);
  XRT_DISPATCH_DTYPE(out_dtype, TO, {
    xrt::launch_kernel(xrt::moe_activation_kernel<TO>, dim3(blocks), dim3(256), 0, stream, (TO*)act, gate_up, total, ff,
                       form.limit, form.alpha, form.up_shift, act_kind);
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_moe_combine(float* out, const float* y, const int* pos, const float* weights, int n_tokens, int width,
                               int top, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0 || top <= 0 || top > 65535) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  xrt::launch_kernel(xrt::moe_combine_kernel, dim3(n_tokens, top), dim3(128), 0, stream, out, y, pos, weights, n_tokens,
                     width, top);
  return xrt::launch_status();
}

// logits [T, experts] float32 (without the bias); ids [T, top] int32 and weights [T, top] float32 are written.
XRT_EXPORT int xrt_moe_route(int* ids, float* weights, const float* logits, const float* bias, int n_tokens,
                             int n_experts, int top, cudaStream_t stream) {
  if (n_tokens < 0 || n_experts <= 0 || top <= 0 || top > n_experts) return XRT_ERR_ARGUMENT;
  if (n_experts > 512) return XRT_ERR_UNSUPPORTED;
  if (n_tokens == 0) return XRT_OK;
  const dim3 grid((n_tokens + 3) / 4), block(128);
  if (n_experts <= 32) xrt::launch_kernel(xrt::moe_route_kernel<1>, grid, block, 0, stream, ids, weights, logits, bias, n_tokens, n_experts, top);
  else if (n_experts <= 64) xrt::launch_kernel(xrt::moe_route_kernel<2>, grid, block, 0, stream, ids, weights, logits, bias, n_tokens, n_experts, top);
  else if (n_experts <= 128) xrt::launch_kernel(xrt::moe_route_kernel<4>, grid, block, 0, stream, ids, weights, logits, bias, n_tokens, n_experts, top);
  else if (n_experts <= 256) xrt::launch_kernel(xrt::moe_route_kernel<8>, grid, block, 0, stream, ids, weights, logits, bias, n_tokens, n_experts, top);
  else xrt::launch_kernel(xrt::moe_route_kernel<16>, grid, block, 0, stream, ids, weights, logits, bias, n_tokens, n_experts, top);
  return xrt::launch_status();
}

// The second kind of routing (see the top of the file).  logits [T, experts] float32.
XRT_EXPORT int xrt_moe_route_scores(int* ids, float* weights, const float* logits, int n_tokens, int n_experts, int top,
                                    int groups, int keep, int sigmoid, const float* correction, int group_best,
                                    int normalize, float sum_eps, float scale, cudaStream_t stream) {
  if (group_best < 1) return XRT_ERR_ARGUMENT;
  xrt::RouteOptions opt;
  opt.sigmoid = sigmoid;
  opt.correction = correction;
  opt.group_best = group_best;
  opt.normalize = normalize;
  opt.sum_eps = sum_eps;
  opt.scale = scale;
  if (n_tokens < 0 || n_experts <= 0 || top <= 0 || groups <= 0 || keep <= 0 || keep > groups || n_experts % groups)
    return XRT_ERR_ARGUMENT;
  if (top > n_experts / groups * keep) return XRT_ERR_ARGUMENT;
  if (n_experts > 512) return XRT_ERR_UNSUPPORTED;
  if (n_tokens == 0) return XRT_OK;
  const dim3 grid((n_tokens + 3) / 4), block(128);
  const size_t smem = (size_t)4 * groups * sizeof(float);
#define XRT_ROUTE(PER) xrt::launch_kernel(xrt::moe_route_scores_kernel<PER>, grid, block, smem, stream, ids, weights, logits, n_tokens, n_experts, top, groups, keep, opt)
  if (n_experts <= 32) XRT_ROUTE(1);
  else if (n_experts <= 64) XRT_ROUTE(2);
  else if (n_experts <= 128) XRT_ROUTE(4);
  else if (n_experts <= 256) XRT_ROUTE(8);
  else XRT_ROUTE(16);
#undef XRT_ROUTE
  return xrt::launch_status();
}

// out [top, T, width] float32; h [T, width]; w_in [experts * 2 * ff, width] (act 1: [experts * ff, width]); w_out [experts * width, ff];
// act [T * top, ff] float32 scratch between the two halves.
XRT_EXPORT int xrt_moe_experts(float* out, float* act, const void* h, const void* w_in, const void* w_out, const int* ids,
                               const float* weights, int n_tokens, int width, int ff, int top, float limit, float alpha,
                               int act_kind, int h_dtype, int w_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0 || ff <= 0 || top <= 0) return XRT_ERR_ARGUMENT;
  if (top > 65535 || (ff + xrt::MOE_UNITS - 1) / xrt::MOE_UNITS > 65535 || (width + xrt::MOE_UNITS - 1) / xrt::MOE_UNITS > 65535)
    return XRT_ERR_UNSUPPORTED;
  if (n_tokens == 0) return XRT_OK;
  if ((size_t)(width > ff ? width : ff) * sizeof(float) > 48 * 1024) return XRT_ERR_UNSUPPORTED;
  const int per = w_dtype == XRT_BF16 ? 8 : 4;
  const bool vec = width % per == 0 && ff % per == 0 && (((uintptr_t)w_in | (uintptr_t)w_out) & 15) == 0;
  // few pairs: blocks of 8 units, so that there are about two blocks a multiprocessor or more
  const bool few = (long long)n_tokens * top * ((ff + xrt::MOE_UNITS - 1) / xrt::MOE_UNITS) < 2 * 148;
  const int units = few ? xrt::MOE_UNITS_FEW : xrt::MOE_UNITS;
  const dim3 grid_in(n_tokens, top, (ff + units - 1) / units);
  const dim3 grid_out(n_tokens, top, (width + units - 1) / units);
  const dim3 block(xrt::MOE_WARPS * 32);
  const xrt::GateForm form = xrt::gate_form(act_kind, limit, alpha);
#define XRT_EXPERTS(VEC, UNITS)                                                                                           \
  do {                                                                                                                    \
    xrt::launch_kernel(xrt::moe_experts_in_kernel<TX, TW, VEC, UNITS>, grid_in, block, (size_t)width * sizeof(float),     \
                       stream, act, (const TX*)h, (const TW*)w_in, ids, width, ff, top, form.limit, form.alpha,          \
                       form.up_shift, act_kind);                                                                          \
    xrt::launch_kernel(xrt::moe_experts_out_kernel<TW, VEC, UNITS>, grid_out, block, (size_t)ff * sizeof(float), stream,  \
                       out, (const float*)act, (const TW*)w_out, ids, weights, n_tokens, width, ff, top);                 \
  } while (0)
  XRT_DISPATCH_DTYPE(h_dtype, TX, {
    XRT_DISPATCH_DTYPE(w_dtype, TW, {
      if (vec && few) XRT_EXPERTS(true, xrt::MOE_UNITS_FEW);
      else if (vec) XRT_EXPERTS(true, xrt::MOE_UNITS);
      else if (few) XRT_EXPERTS(false, xrt::MOE_UNITS_FEW);
      else XRT_EXPERTS(false, xrt::MOE_UNITS);
    });
  });
#undef XRT_EXPERTS
  return xrt::launch_status();
}
