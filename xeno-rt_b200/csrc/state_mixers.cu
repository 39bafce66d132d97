// Mixers that keep a matrix state per head instead of keys: the scan over a step's tokens, and the
// small steps around it.  Everything here is 32-bit: the state, decays, gates of the recurrence,
// unit norms and head norms.
//
//   state scan        S_t = diag(a_t) S_(t-1) + k_t u_t^T,   o_t = S_t^T q_t
//                     plain:       u_t = v_t                                   (gated linear attention)
//                     delta rule:  u_t = b_t (v_t - (diag(a_t) S_(t-1))^T k_t) (the read-out sees the write)
//                     removal:     S_t = diag(a_t) S_(t-1) - e_t (n_t^T S_(t-1)) + k_t v_t^T, with two more vectors a
//                                  token and head, n_t (a unit key) and e_t (a removal rate times n_t); the decay and
//                                  the removal both read the state as the token found it
//   removal gates     from raw products: a = exp(-rate * sigmoid(z + bias)), n = k / sqrt(sum(k^2) + eps) per head,
//                     e = sigmoid(y + bias) * n
//   short convolution y_t = act(bias[c] + sum_j w[c, j] x_(t - (taps - 1) + j)) per channel (the bias is optional), zeros before a sequence's
//                     start; the last taps - 1 inputs of a sequence are its state; with `in_bias` every input inside
//                     the sequence is x + in_bias[c] (a product's bias, added here), and the state holds them so
//   decays            a = sigmoid(z + bias)^(1 / tau)   or   a = exp(-exp(A) softplus(z + bias))
//   unit heads        x / sqrt(sum(x^2) + eps) * scale per head
//   head norm + gate  o / sqrt(mean(o^2) + eps) * w * act(g) per head
//
// A sequence is a row of the step's cu_seqlens / seq_slot arrays; a row with slot -1 or no tokens is
// skipped, so padding rows of a captured step leave every state alone.
#include "common.cuh"

namespace xrt {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float activate(float z, int act) {  // 0 none, 1 silu, 2 sigmoid, 3 tanh
  return act == 1 ? z * sigmoidf_(z) : (act == 2 ? sigmoidf_(z) : (act == 3 ? tanhf(z) : z));
}

// ------------------------------------------------------------------------------------------ the scan
// One block: one sequence, one head, COLS value columns.  A column's state S[:, j] (dim rows) is held
// in registers by PARTS neighbouring lanes, R rows each; sums over rows are finished by a butterfly
// among those lanes, so every lane of a column holds the same total.  The state is kept column by
// column, [slot][head][vdim][dim], so that a warp reads and writes it in whole lines.
// Tiles of TT tokens' q, k, a (padded to PARTS * R rows: k = q = 0 there) and the columns' v and b are
// staged in shared memory by cp.async, two tiles in flight: the next tile lands while this one is
// worked on.  A lane's rows are every PARTS-th group of four (lane p holds rows 4 (i PARTS + p) .. + 3), so
// that the lanes of a column read neighbouring 16 bytes at a time: whole lines of the state in global
// memory, different banks of shared memory.  Sums over a lane's rows run as two chains.
template <int BYTES>
__device__ __forceinline__ void cp_async(float* smem, const float* global) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  if (BYTES == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(global) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct ScanArgs {
  float* out;
  const float *q, *k, *v, *decay, *beta;
  const float *unit, *removal;  // MODE 2: n_t and e_t, rows of heads * dim
  int unit_stride, removal_stride;
  int q_stride, k_stride, v_stride, decay_stride, beta_stride;
  float* state;
  const int *cu_seqlens, *seq_slot;
  int n_heads, heads_per_qk, dim, vdim;
  float q_scale;
  int parts, cols, tile_tokens, stage_floats;
};

// VEC: 16-byte copies (dim, vdim, cols and every row stride are multiples of 4 floats, every base 16-byte aligned).
// C2: value columns a lane holds (C2 * R state registers): what a lane reads of q, k and a serves C2 columns, and
// the kernel is bound by what its warps ask of shared memory.
// MODE 0: plain, 1: delta rule, 2: removal along a unit key (two more vectors in a stage).
template <int R, int C2, int MODE, bool VEC>
__global__ void __launch_bounds__(128) state_scan_kernel(const ScanArgs a) {
  constexpr bool DELTA = MODE == 1;
  constexpr int NVEC = MODE == 2 ? 5 : 3;  // vectors of `padded` floats a token in a stage
  extern __shared__ float4 tile4[];
  float* tile = reinterpret_cast<float*>(tile4);
  pdl_trigger();
  const int parts = a.parts, cols = a.cols, TT = a.tile_tokens, dim = a.dim, vdim = a.vdim;
  const int padded = parts * R;
  // a stage: q | k | a (| n | e), each [TT][padded]; then v [TT][cols]; then b [TT] (regions of whole 16 bytes)
  const int vec_floats = TT * padded, v_floats = (TT * cols + 3) & ~3;
  if (padded != dim || vdim % cols != 0)  // rows and columns beyond the head's stay zero
    for (int e = threadIdx.x; e < 2 * a.stage_floats; e += blockDim.x) tile[e] = 0.f;
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y;
  const int slot = a.seq_slot[s];
  const int begin = a.cu_seqlens[s], end = a.cu_seqlens[s + 1];
  if (slot < 0 || end <= begin) return;
  const int part = threadIdx.x % parts, jl = (threadIdx.x / parts) * C2;  // the lane's first column in the block
  const int col0 = blockIdx.z * cols;
  const int j = col0 + jl;
  const int qh = h / a.heads_per_qk;
  constexpr int B = VEC ? 16 : 4, E = VEC ? 4 : 1;  // bytes and floats a copy
  auto row_of = [&](int i) { return 4 * ((i / 4) * parts + part) + (i & 3); };  // the lane's i-th row

  auto issue = [&](int t0, int stage) {
    float* sq = tile + stage * a.stage_floats;
    float* sk = sq + vec_floats;
    float* sa = sk + vec_floats;
    float* sv = sq + NVEC * vec_floats;
    float* sb = sv + v_floats;
    const int nt = min(TT, end - t0);
    const int per = dim / E;
    for (int e = threadIdx.x; e < nt * per; e += blockDim.x) {
      const int tt = e / per, d = (e - tt * per) * E;
      const int at = tt * padded + d;
      const size_t t = (size_t)(t0 + tt);
      cp_async<B>(sq + at, a.q + t * a.q_stride + qh * dim + d);
      cp_async<B>(sk + at, a.k + t * a.k_stride + qh * dim + d);
      cp_async<B>(sa + at, a.decay + t * a.decay_stride + h * dim + d);
      if (MODE == 2) {
        cp_async<B>(sa + vec_floats + at, a.unit + t * a.unit_stride + h * dim + d);
        cp_async<B>(sa + 2 * vec_floats + at, a.removal + t * a.removal_stride + h * dim + d);
      }
    }
    const int vper = cols / E;
    for (int e = threadIdx.x; e < nt * vper; e += blockDim.x) {
      const int tt = e / vper, c = (e - tt * vper) * E;
      if (col0 + c < vdim) cp_async<B>(sv + tt * cols + c, a.v + (size_t)(t0 + tt) * a.v_stride + h * vdim + col0 + c);
    }
    if (DELTA)
      for (int tt = threadIdx.x; tt < nt; tt += blockDim.x)
        cp_async<4>(sb + tt, a.beta + (size_t)(t0 + tt) * a.beta_stride + h);
    cp_async_commit();
  };

  // the state as pairs: the multiply-adds below are the packed 2 x fp32 instructions of sm_100 (each half a true
  // 32-bit fused multiply-add, rounded to nearest), half as many instructions for the same arithmetic
  float2 S[C2][R / 2];
  float* sp = a.state + (((size_t)slot * a.n_heads + h) * vdim + j) * dim;  // column j + c is c * dim further
#pragma unroll
  for (int c = 0; c < C2; ++c) {
    const bool live = j + c < vdim;
    if (VEC) {
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live && row_of(i) < dim) t = *reinterpret_cast<const float4*>(sp + (size_t)c * dim + row_of(i));
        S[c][i / 2] = make_float2(t.x, t.y);
        S[c][i / 2 + 1] = make_float2(t.z, t.w);
      }
    } else {
#pragma unroll
      for (int i = 0; i < R; i += 2)
        S[c][i / 2] = make_float2((live && row_of(i) < dim) ? sp[(size_t)c * dim + row_of(i)] : 0.f,
                                  (live && row_of(i + 1) < dim) ? sp[(size_t)c * dim + row_of(i + 1)] : 0.f);
    }
  }
  __syncthreads();  // the zero fill is done before the first copies land
  issue(begin, 0);
  int stage = 0;
  for (int t0 = begin; t0 < end; t0 += TT, stage ^= 1) {
    const int nt = min(TT, end - t0);
    if (t0 + TT < end) {
      issue(t0 + TT, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    const float* sq = tile + stage * a.stage_floats;
    const float* sk = sq + vec_floats;
    const float* sa = sk + vec_floats;
    const float* sv = sq + NVEC * vec_floats;
    float* sb = tile + stage * a.stage_floats + NVEC * vec_floats + v_floats;
    if (DELTA)  // b = sigmoid(raw), once a tile, by the thread whose own copy brought the raw value
      for (int tt = threadIdx.x; tt < nt; tt += blockDim.x) sb[tt] = sigmoidf_(sb[tt]);
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      // the lane's i-th group of four rows is 16-byte element i * parts of these
      const float4* pq = reinterpret_cast<const float4*>(sq + tt * padded) + part;
      const float4* pk = reinterpret_cast<const float4*>(sk + tt * padded) + part;
      const float4* pa = reinterpret_cast<const float4*>(sa + tt * padded) + part;
      float u[C2];
#pragma unroll
      for (int c = 0; c < C2; ++c) u[c] = sv[tt * cols + jl + c];
      float2 kr[R / 2];
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        const float4 t = pk[(i / 4) * parts];
        kr[i / 2] = make_float2(t.x, t.y);
        kr[i / 2 + 1] = make_float2(t.z, t.w);
      }
      if (DELTA) {
        const float b = sb[tt];
        float2 seen[C2][2];
#pragma unroll
        for (int c = 0; c < C2; ++c) seen[c][0] = seen[c][1] = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 d = pa[(i / 4) * parts];
#pragma unroll
          for (int c = 0; c < C2; ++c) {
            S[c][i / 2] = __fmul2_rn(S[c][i / 2], make_float2(d.x, d.y));
            S[c][i / 2 + 1] = __fmul2_rn(S[c][i / 2 + 1], make_float2(d.z, d.w));
            seen[c][0] = __ffma2_rn(S[c][i / 2], kr[i / 2], seen[c][0]);
            seen[c][1] = __ffma2_rn(S[c][i / 2 + 1], kr[i / 2 + 1], seen[c][1]);
          }
        }
#pragma unroll
        for (int c = 0; c < C2; ++c) {
          float total = (seen[c][0].x + seen[c][0].y) + (seen[c][1].x + seen[c][1].y);
          for (int o = 1; o < parts; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
          u[c] = b * (u[c] - total);
        }
#pragma unroll
        for (int c = 0; c < C2; ++c)
#pragma unroll
          for (int i = 0; i < R / 2; ++i) S[c][i] = __ffma2_rn(kr[i], make_float2(u[c], u[c]), S[c][i]);
      } else if (MODE == 2) {
        // what the state answers along the unit key, from the state as the token found it
        const float4* pn = reinterpret_cast<const float4*>(sa + vec_floats + tt * padded) + part;
        const float4* pe = reinterpret_cast<const float4*>(sa + 2 * vec_floats + tt * padded) + part;
        float2 seen[C2][2];
#pragma unroll
        for (int c = 0; c < C2; ++c) seen[c][0] = seen[c][1] = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 n = pn[(i / 4) * parts];
#pragma unroll
          for (int c = 0; c < C2; ++c) {
            seen[c][0] = __ffma2_rn(S[c][i / 2], make_float2(n.x, n.y), seen[c][0]);
            seen[c][1] = __ffma2_rn(S[c][i / 2 + 1], make_float2(n.z, n.w), seen[c][1]);
          }
        }
        float gone[C2];
#pragma unroll
        for (int c = 0; c < C2; ++c) {
          float total = (seen[c][0].x + seen[c][0].y) + (seen[c][1].x + seen[c][1].y);
          for (int o = 1; o < parts; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
          gone[c] = -total;
        }
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 d = pa[(i / 4) * parts];
          const float4 e = pe[(i / 4) * parts];
#pragma unroll
          for (int c = 0; c < C2; ++c) {
            const float2 uu = make_float2(u[c], u[c]), gg = make_float2(gone[c], gone[c]);
            // diag(a) S - e (n^T S) + k v^T, the two corrections first
            const float2 lo = __ffma2_rn(make_float2(e.x, e.y), gg, __fmul2_rn(kr[i / 2], uu));
            const float2 hi = __ffma2_rn(make_float2(e.z, e.w), gg, __fmul2_rn(kr[i / 2 + 1], uu));
            S[c][i / 2] = __ffma2_rn(S[c][i / 2], make_float2(d.x, d.y), lo);
            S[c][i / 2 + 1] = __ffma2_rn(S[c][i / 2 + 1], make_float2(d.z, d.w), hi);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 d = pa[(i / 4) * parts];
#pragma unroll
          for (int c = 0; c < C2; ++c) {
            const float2 uu = make_float2(u[c], u[c]);
            S[c][i / 2] = __ffma2_rn(S[c][i / 2], make_float2(d.x, d.y), __fmul2_rn(kr[i / 2], uu));
            S[c][i / 2 + 1] = __ffma2_rn(S[c][i / 2 + 1], make_float2(d.z, d.w), __fmul2_rn(kr[i / 2 + 1], uu));
          }
        }
      }
      float2 read[C2][2];
#pragma unroll
      for (int c = 0; c < C2; ++c) read[c][0] = read[c][1] = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        const float4 qq = pq[(i / 4) * parts];
#pragma unroll
        for (int c = 0; c < C2; ++c) {
          read[c][0] = __ffma2_rn(S[c][i / 2], make_float2(qq.x, qq.y), read[c][0]);
          read[c][1] = __ffma2_rn(S[c][i / 2 + 1], make_float2(qq.z, qq.w), read[c][1]);
        }
      }
#pragma unroll
      for (int c = 0; c < C2; ++c) {
        float total = (read[c][0].x + read[c][0].y) + (read[c][1].x + read[c][1].y);
        for (int o = 1; o < parts; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (part == 0 && j + c < vdim) a.out[(size_t)(t0 + tt) * a.n_heads * vdim + h * vdim + j + c] = total * a.q_scale;
      }
    }
    __syncthreads();  // the stage is read out before the copies of the tile after next overwrite it
  }
#pragma unroll
  for (int c = 0; c < C2; ++c) {
    if (j + c >= vdim) continue;
    if (VEC) {
#pragma unroll
      for (int i = 0; i < R; i += 4)
        if (row_of(i) < dim)
          *reinterpret_cast<float4*>(sp + (size_t)c * dim + row_of(i)) =
              make_float4(S[c][i / 2].x, S[c][i / 2].y, S[c][i / 2 + 1].x, S[c][i / 2 + 1].y);
    } else {
#pragma unroll
      for (int i = 0; i < R; i += 2) {
        if (row_of(i) < dim) sp[(size_t)c * dim + row_of(i)] = S[c][i / 2].x;
        if (row_of(i + 1) < dim) sp[(size_t)c * dim + row_of(i + 1)] = S[c][i / 2].y;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ convolution
// grid (sequences, token tiles, channel blocks); a thread has one channel of a tile's tokens.  Inputs before the step's first token
// come from the sequence's state [slot][taps - 1][channels] (the newest last).
__global__ void short_conv_kernel(float* __restrict__ out, const float* __restrict__ x, int x_stride,
                                  const float* __restrict__ w, const float* __restrict__ bias,
                                  const float* __restrict__ in_bias, const float* __restrict__ state,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, int channels,
                                  int taps, int tile_tokens, int act) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x;
  const int slot = seq_slot[s];
  const int begin = cu_seqlens[s], len = cu_seqlens[s + 1] - begin;
  const int l0 = blockIdx.y * tile_tokens;
  if (slot < 0 || l0 >= len) return;
  const int l1 = min(len, l0 + tile_tokens);
  const float* st = state + (size_t)slot * (taps - 1) * channels;
  for (int c = blockIdx.z * blockDim.x + threadIdx.x; c < channels; c += gridDim.z * blockDim.x) {
    const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
    for (int l = l0; l < l1; ++l) {
      float acc = bias != nullptr ? bias[c] : 0.f;
      for (int jj = 0; jj < taps; ++jj) {
        const int src = l - (taps - 1) + jj;  // local index of the input under tap jj
        const float xv = src >= 0 ? x[(size_t)(begin + src) * x_stride + c] + ib : st[(size_t)(taps - 1 + src) * channels + c];
        acc = fmaf(w[c * taps + jj], xv, acc);
      }
      out[(size_t)(begin + l) * channels + c] = activate(acc, act);
    }
  }
}

// The state after the step: the last taps - 1 inputs of the sequence (older ones shift out).
template <int MAX_KEEP>
__global__ void short_conv_state_kernel(float* __restrict__ state, const float* __restrict__ x, int x_stride,
                                        const float* __restrict__ in_bias,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                                        int channels, int taps) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x;
  const int slot = seq_slot[s];
  const int begin = cu_seqlens[s], len = cu_seqlens[s + 1] - begin;
  if (slot < 0 || len <= 0) return;
  const int keep = taps - 1;
  float* st = state + (size_t)slot * keep * channels;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float next[MAX_KEEP];
#pragma unroll
    for (int i = 0; i < MAX_KEEP; ++i) {
      if (i < keep) {
        const int src = len - keep + i;
        next[i] = src >= 0 ? x[(size_t)(begin + src) * x_stride + c] + (in_bias != nullptr ? in_bias[c] : 0.f)
                           : st[(size_t)(keep + src) * channels + c];
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_KEEP; ++i)
      if (i < keep) st[(size_t)i * channels + c] = next[i];
  }
}

// A step whose sequences bring one token each: output and new state in one launch.  A thread has one channel of one
// sequence, so what it reads of the state it writes itself; the taps are walked in the order of the kernel above
// (the state's entries, then the new input), which gives the same bits.
template <int MAX_KEEP>
__global__ void short_conv_single_kernel(float* __restrict__ out, const float* __restrict__ x, int x_stride,
                                         const float* __restrict__ w, const float* __restrict__ bias,
                                         const float* __restrict__ in_bias, float* __restrict__ state,
                                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                                         int channels, int taps, int act) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x;
  const int slot = seq_slot[s];
  const int begin = cu_seqlens[s], len = cu_seqlens[s + 1] - begin;
  if (slot < 0 || len <= 0) return;
  const int keep = taps - 1;
  float* st = state + (size_t)slot * keep * channels;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float xv = x[(size_t)begin * x_stride + c] + (in_bias != nullptr ? in_bias[c] : 0.f);
    float acc = bias != nullptr ? bias[c] : 0.f;
    float old[MAX_KEEP];
#pragma unroll
    for (int i = 0; i < MAX_KEEP; ++i)
      if (i < keep) {
        old[i] = st[(size_t)i * channels + c];
        acc = fmaf(w[c * taps + i], old[i], acc);
      }
    acc = fmaf(w[c * taps + keep], xv, acc);
    out[(size_t)begin * channels + c] = activate(acc, act);
#pragma unroll
    for (int i = 0; i < MAX_KEEP; ++i)
      if (i < keep) st[(size_t)i * channels + c] = i + 1 < keep ? old[i + 1] : xv;
  }
}

// ------------------------------------------------------------------------------------------ small steps
// mode 0: a = sigmoid(z + bias)^(1 / tau) = exp(-softplus(-(z + bias)) / tau)
// mode 1: a = exp(-exp(a_log[head]) * softplus(z + bias))
__global__ void decay_kernel(float* __restrict__ a, const float* __restrict__ bias, const float* __restrict__ a_log,
                             size_t total, int width, int dim, int mode, float tau) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % width);
    const float z = a[i] + (bias != nullptr ? bias[c] : 0.f);
    a[i] = mode == 0 ? expf(-softplusf_(-z) / tau) : expf(-expf(a_log[c / dim]) * softplusf_(z));
  }
}

// One warp a (token, head): x <- x / sqrt(sum(x^2) + eps) * scale, in place; heads [first, first + n).
__global__ void unit_heads_kernel(float* __restrict__ x, int stride, int n_tokens, int n_heads, int dim, float eps,
                                  int scaled_heads, float scale) {
  pdl_trigger();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_tokens * n_heads) return;
  const int t = warp / n_heads, head = warp - t * n_heads;
  float* p = x + (size_t)t * stride + head * dim;
  float sum = 0.f;
  for (int d = lane; d < dim; d += 32) sum = fmaf(p[d], p[d], sum);
  sum = warp_sum(sum);
  const float f = (head < scaled_heads ? scale : 1.0f) / sqrtf(sum + eps);
  for (int d = lane; d < dim; d += 32) p[d] *= f;
}

// One warp a (token, head): the three vectors that the removal form of the scan reads beside q, k and v.
//   decay[c]   <- exp(-rate * sigmoid(decay[c] + decay_bias[c]))            (in place over the raw product)
//   unit[c]     = k[c] / sqrt(sum over the head of k^2 + unit_eps)
//   removal[c] <- sigmoid(removal[c] + removal_bias[c]) * unit[c]            (in place over the raw product)
__global__ void removal_gates_kernel(float* __restrict__ decay, int decay_stride, const float* __restrict__ decay_bias,
                                     float* __restrict__ removal, int removal_stride,
                                     const float* __restrict__ removal_bias, float* __restrict__ unit, int unit_stride,
                                     const float* __restrict__ k, int k_stride, int n_tokens, int n_heads, int dim,
                                     float rate, float unit_eps) {
  pdl_trigger();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_tokens * n_heads) return;
  const int t = warp / n_heads, head = warp - t * n_heads;
  const float* kp = k + (size_t)t * k_stride + head * dim;
  float sum = 0.f;
  for (int d = lane; d < dim; d += 32) sum = fmaf(kp[d], kp[d], sum);
  const float inv = 1.0f / sqrtf(warp_sum(sum) + unit_eps);
  float* dp = decay + (size_t)t * decay_stride + head * dim;
  float* rp = removal + (size_t)t * removal_stride + head * dim;
  float* up = unit + (size_t)t * unit_stride + head * dim;
  for (int d = lane; d < dim; d += 32) {
    const int c = head * dim + d;
    const float n = kp[d] * inv;
    dp[d] = expf(-rate * sigmoidf_(dp[d] + decay_bias[c]));
    rp[d] = sigmoidf_(rp[d] + removal_bias[c]) * n;
    up[d] = n;
  }
}

// One warp a (token, head): y = o / sqrt(mean(o^2) + eps) * w * act(gate).
template <typename TO>
__global__ void head_norm_gate_kernel(TO* __restrict__ y, const float* __restrict__ o, const float* __restrict__ w,
                                      const float* __restrict__ gate, int gate_stride, int n_tokens, int n_heads,
                                      int vdim, float eps, int act, int w_per_head) {
  pdl_trigger();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= n_tokens * n_heads) return;
  const int t = warp / n_heads, head = warp - t * n_heads;
  const float* p = o + ((size_t)t * n_heads + head) * vdim;
  const float* g = gate + (size_t)t * gate_stride + head * vdim;
  float sum = 0.f;
  for (int d = lane; d < vdim; d += 32) sum = fmaf(p[d], p[d], sum);
  sum = warp_sum(sum);
  const float inv = 1.0f / sqrtf(sum / (float)vdim + eps);
  TO* dst = y + ((size_t)t * n_heads + head) * vdim;
  const float* wh = w + (w_per_head ? head * vdim : 0);  // one weight a column of all heads, or one shared by the heads
  for (int d = lane; d < vdim; d += 32) dst[d] = from_float<TO>((p[d] * inv) * wh[d] * activate(g[d], act));
}

// x[t, c] *= act(gate[t, c]) in place.
template <typename TX>
__global__ void gate_mul_kernel(TX* __restrict__ x, const float* __restrict__ gate, int gate_stride, int n_tokens,
                                int width, int act, int group) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n_tokens * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width, c = i - t * width;
    x[i] = from_float<TX>(to_float(x[i]) * activate(gate[t * gate_stride + c / group], act));  // one gate a group of columns
  }
}

// residual[t] += factor * y[t] / sqrt(mean(y[t]^2) + eps) * w; one block a row.  The row, the weight and the
// residual are all asked for before the sum (a few rows a step: the time is load latency).
template <int PER>
__global__ void rms_scale_add_kernel(float* __restrict__ residual, const float* __restrict__ y,
                                     const float* __restrict__ w, int width, float eps, float factor) {
  __shared__ float scratch[33];
  pdl_trigger();
  float wv[PER], yv[PER], rv[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < width ? w[c] : 0.f;
  }
  pdl_wait();
  const float* p = y + (size_t)blockIdx.x * width;
  float* r = residual + (size_t)blockIdx.x * width;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    yv[i] = c < width ? p[c] : 0.f;
    rv[i] = c < width ? r[c] : 0.f;
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) sum = fmaf(yv[i], yv[i], sum);
  for (int c = threadIdx.x + PER * blockDim.x; c < width; c += blockDim.x) sum = fmaf(p[c], p[c], sum);
  const float total = block_sum(sum, scratch);
  const float f = factor / sqrtf(total / (float)width + eps);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < width) r[c] = rv[i] + (yv[i] * f) * wv[i];
  }
  for (int c = threadIdx.x + PER * blockDim.x; c < width; c += blockDim.x) r[c] += (p[c] * f) * w[c];
}

// out[t] = [a[t] | b[t]] in the compute dtype.
template <typename TO>
__global__ void concat_cast_kernel(TO* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                   int n_tokens, int width) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n_tokens * 2 * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / (2 * width), c = i - t * 2 * width;
    out[i] = from_float<TO>(c < (size_t)width ? a[t * width + c] : b[t * width + c - width]);
  }
}

// out[t, c] = act(x[t, c]) in the compute dtype; x rows may be slices of wider rows.
template <typename TO>
__global__ void act_cast_kernel(TO* __restrict__ out, const float* __restrict__ x, int x_stride, int n_tokens, int width,
                                int act) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)n_tokens * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width, c = i - t * width;
    out[i] = from_float<TO>(activate(x[t * x_stride + c], act));
  }
}

// residual[t, c] += sum_p scales[p] * parts[p][t, c], the parts in index order.
__global__ void add_scaled_parts_kernel(float* __restrict__ residual, const float* __restrict__ parts,
                                        const float* __restrict__ scales, size_t total, int n_parts) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float sum = 0.f;
    for (int p = 0; p < n_parts; ++p) sum = fmaf(parts[(size_t)p * total + i], scales[p], sum);
    residual[i] += sum;
  }
}

// x <- cap * tanh(x * scale / cap), or x * scale without a cap.
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t total, float scale, float cap) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = x[i] * scale;
    x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

inline int grid_for(size_t total, int threads) {
  const size_t blocks = (total + threads - 1) / threads;
  return (int)(blocks < 148 * 16 ? (blocks ? blocks : 1) : 148 * 16);
}

}  // namespace xrt

// Rows of a column's state that one lane holds, for a key size.  Few lanes a column (4 up to a key size of 64,
// 2 at 128) keep the butterflies short; measured at 32 heads of 128 x 128 (16 / 32 / 64 rows a lane): one prompt
// of 2,048 tokens 1.11 / 1.11 / 1.17 ms, four such prompts 2.1 / 2.05 / 1.64 ms, 64 single tokens 130 / 109 / 95 us.
static int scan_rows_per_lane(int dim) { return dim <= 32 ? 8 : (dim <= 64 ? 16 : (dim <= 128 ? 64 : 32)); }

XRT_EXPORT int xrt_state_scan(float* out, const float* q, int q_stride, const float* k, int k_stride, const float* v,
                              int v_stride, const float* decay, int decay_stride, const float* beta, int beta_stride,
                              const float* unit, int unit_stride, const float* removal, int removal_stride,
                              float* state, const int* cu_seqlens, const int* seq_slot, int n_seqs, int n_heads,
                              int n_qk_heads, int dim, int vdim, float q_scale, int mode, int max_new,
                              cudaStream_t stream) {
  const bool delta = mode == 1;
  if (mode < 0 || mode > 2 || (mode == 2 && (unit == nullptr || removal == nullptr))) return XRT_ERR_ARGUMENT;
  if (max_new < 1) max_new = 1 << 30;
  if (n_seqs < 0 || n_heads <= 0 || n_qk_heads <= 0 || n_heads % n_qk_heads || dim <= 0 || vdim <= 0)
    return XRT_ERR_ARGUMENT;
  if (dim > 1024 || n_heads > 65535) return XRT_ERR_UNSUPPORTED;
  if (delta && beta == nullptr) return XRT_ERR_ARGUMENT;
  if (n_seqs == 0) return XRT_OK;
  const int R = scan_rows_per_lane(dim);
  int parts = 1;
  while (parts * R < dim) parts <<= 1;
  // columns a lane holds: one.  (Several, so that what a lane reads of q, k and a serves more columns, was
  // measured slower: 1.77 against 0.96 ms for 2,048 tokens of 32 heads of 128 x 128; a token's time is the
  // chain of dependent instructions of ONE warp, and more columns a lane make that chain longer.)
  const int per_lane = 1;
  // 128 threads a block at most, whole warps at least
  int groups = 128 / parts;
  if (groups < 1) groups = 1;
  while (groups > 1 && (groups / 2) * per_lane >= vdim && (groups / 2) * parts >= 32) groups >>= 1;
  if (groups * parts < 32) groups = 32 / parts;
  const int cols = groups * per_lane;
  const int padded = parts * R;
  const int n_vec = mode == 2 ? 5 : 3;
  auto stage_floats = [&](int tt) { return n_vec * tt * padded + ((tt * cols + 3) & ~3) + ((tt + 3) & ~3); };
  int tile_tokens = 16;
  while (tile_tokens > 1 && 2 * (size_t)stage_floats(tile_tokens) * sizeof(float) > 44 * 1024) tile_tokens >>= 1;
  // no more than the step's longest sequence brings: a decode step's blocks are small and many fit a multiprocessor
  while (tile_tokens > 1 && tile_tokens / 2 >= max_new) tile_tokens >>= 1;
  const size_t smem = 2 * (size_t)stage_floats(tile_tokens) * sizeof(float);
  if (smem > 48 * 1024) return XRT_ERR_UNSUPPORTED;
  const bool vec = dim % 4 == 0 && vdim % 4 == 0 && cols % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 &&
                   v_stride % 4 == 0 && decay_stride % 4 == 0 && unit_stride % 4 == 0 && removal_stride % 4 == 0 &&
                   (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)decay | (uintptr_t)state |
                     (uintptr_t)unit | (uintptr_t)removal) & 15) == 0;
  xrt::ScanArgs a = {out, q, k, v, decay, beta, unit, removal, unit_stride, removal_stride,
                     q_stride, k_stride, v_stride, decay_stride, beta_stride, state,
                     cu_seqlens, seq_slot, n_heads, n_heads / n_qk_heads, dim, vdim, q_scale, parts, cols, tile_tokens,
                     stage_floats(tile_tokens)};
  const dim3 grid(n_seqs, n_heads, (vdim + cols - 1) / cols), block(parts * groups);
#define XRT_SCAN(RR, CC, DD, VV) xrt::launch_kernel(xrt::state_scan_kernel<RR, CC, DD, VV>, grid, block, smem, stream, a)
#define XRT_SCAN_R(RR, CC)                                     \
  do {                                                         \
    if (mode == 2 && vec) XRT_SCAN(RR, CC, 2, true);           \
    else if (mode == 2) XRT_SCAN(RR, CC, 2, false);            \
    else if (delta && vec) XRT_SCAN(RR, CC, 1, true);          \
    else if (delta) XRT_SCAN(RR, CC, 1, false);                \
    else if (vec) XRT_SCAN(RR, CC, 0, true);                   \
    else XRT_SCAN(RR, CC, 0, false);                           \
  } while (0)
  if (R == 8) XRT_SCAN_R(8, 1);
  else if (R == 16) XRT_SCAN_R(16, 1);
  else if (R == 64) XRT_SCAN_R(64, 1);
  else XRT_SCAN_R(32, 1);
#undef XRT_SCAN_R
#undef XRT_SCAN
  return xrt::launch_status();
}

XRT_EXPORT int xrt_short_conv(float* out, const float* x, int x_stride, const float* w, const float* bias,
                              const float* in_bias, float* state, const int* cu_seqlens, const int* seq_slot, int n_seqs, int max_new, int channels,
                              int taps, int act, cudaStream_t stream) {
  if (n_seqs < 0 || channels <= 0 || taps < 1 || max_new < 0) return XRT_ERR_ARGUMENT;
  if (taps > 9 || n_seqs > 65535) return XRT_ERR_UNSUPPORTED;
  if (n_seqs == 0 || max_new == 0) return XRT_OK;
  const int tile_tokens = 8;
  const int threads = channels >= 128 ? 128 : 64;
  const int channel_blocks = (channels + threads - 1) / threads;
  if (max_new == 1 && taps > 1) {  // single tokens: one launch
    xrt::launch_kernel(xrt::short_conv_single_kernel<8>, dim3(n_seqs, channel_blocks < 65535 ? channel_blocks : 65535),
                       dim3(threads), 0, stream, out, x, x_stride, w, bias, in_bias, state, cu_seqlens, seq_slot, channels,
                       taps, act);
    return xrt::launch_status();
  }
  xrt::launch_kernel(xrt::short_conv_kernel,
                     dim3(n_seqs, (max_new + tile_tokens - 1) / tile_tokens, channel_blocks < 65535 ? channel_blocks : 65535),
                     dim3(threads), 0, stream, out, x, x_stride, w, bias, in_bias, (const float*)state, cu_seqlens, seq_slot, channels, taps, tile_tokens,
                     act);
  if (taps > 1)
    xrt::launch_kernel(xrt::short_conv_state_kernel<8>, dim3(n_seqs, (channels + 255) / 256), dim3(256), 0, stream, state,
                       x, x_stride, in_bias, cu_seqlens, seq_slot, channels, taps);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_decay(float* a, const float* bias, const float* a_log, int n_tokens, int n_heads, int dim, int mode,
                         float tau, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || dim <= 0 || (mode != 0 && mode != 1)) return XRT_ERR_ARGUMENT;
  if ((mode == 0 && !(tau > 0.f)) || (mode == 1 && a_log == nullptr)) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t total = (size_t)n_tokens * n_heads * dim;
  xrt::launch_kernel(xrt::decay_kernel, dim3(xrt::grid_for(total, 256)), dim3(256), 0, stream, a, bias, a_log, total,
                     n_heads * dim, dim, mode, tau);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_unit_heads(float* x, int stride, int n_tokens, int n_heads, int dim, float eps, int scaled_heads,
                              float scale, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || dim <= 0 || stride < n_heads * dim) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t warps = (size_t)n_tokens * n_heads;
  xrt::launch_kernel(xrt::unit_heads_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, stream, x, stride, n_tokens,
                     n_heads, dim, eps, scaled_heads, scale);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_removal_gates(float* decay, int decay_stride, const float* decay_bias, float* removal,
                                 int removal_stride, const float* removal_bias, float* unit, int unit_stride,
                                 const float* k, int k_stride, int n_tokens, int n_heads, int dim, float rate,
                                 float unit_eps, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || dim <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t warps = (size_t)n_tokens * n_heads;
  xrt::launch_kernel(xrt::removal_gates_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, stream, decay,
                     decay_stride, decay_bias, removal, removal_stride, removal_bias, unit, unit_stride, k, k_stride,
                     n_tokens, n_heads, dim, rate, unit_eps);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_head_norm_gate(void* y, const float* o, const float* w, const float* gate, int gate_stride,
                                  int n_tokens, int n_heads, int vdim, float eps, int act, int out_dtype,
                                  int w_per_head, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || vdim <= 0 || gate_stride < n_heads * vdim) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t warps = (size_t)n_tokens * n_heads;
  XRT_DISPATCH_DTYPE(out_dtype, TO, {
    xrt::launch_kernel(xrt::head_norm_gate_kernel<TO>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, stream, (TO*)y, o,
                       w, gate, gate_stride, n_tokens, n_heads, vdim, eps, act, w_per_head);
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_gate_mul(void* x, const float* gate, int gate_stride, int n_tokens, int width, int act, int dtype,
                            int group, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0 || group <= 0 || width % group || gate_stride < width / group) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  XRT_DISPATCH_DTYPE(dtype, TX, {
    xrt::launch_kernel(xrt::gate_mul_kernel<TX>, dim3(xrt::grid_for((size_t)n_tokens * width, 256)), dim3(256), 0, stream,
                       (TX*)x, gate, gate_stride, n_tokens, width, act, group);
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_rms_scale_add(float* residual, const float* y, const float* w, int n_tokens, int width, float eps,
                                 float factor, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  if (width <= 4 * threads)
    xrt::launch_kernel(xrt::rms_scale_add_kernel<4>, dim3(n_tokens), dim3(threads), 0, stream, residual, y, w, width, eps,
                       factor);
  else
    xrt::launch_kernel(xrt::rms_scale_add_kernel<16>, dim3(n_tokens), dim3(threads), 0, stream, residual, y, w, width,
                       eps, factor);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_concat_cast(void* out, const float* a, const float* b, int n_tokens, int width, int out_dtype,
                               cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  XRT_DISPATCH_DTYPE(out_dtype, TO, {
    xrt::launch_kernel(xrt::concat_cast_kernel<TO>, dim3(xrt::grid_for((size_t)n_tokens * 2 * width, 256)), dim3(256), 0,
                       stream, (TO*)out, a, b, n_tokens, width);
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_act_cast(void* out, const float* x, int x_stride, int n_tokens, int width, int act, int out_dtype,
                            cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0 || x_stride < width) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  XRT_DISPATCH_DTYPE(out_dtype, TO, {
    xrt::launch_kernel(xrt::act_cast_kernel<TO>, dim3(xrt::grid_for((size_t)n_tokens * width, 256)), dim3(256), 0, stream,
                       (TO*)out, x, x_stride, n_tokens, width, act);
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_add_scaled_parts(float* residual, const float* parts, const float* scales, long long total, int n_parts,
                                    cudaStream_t stream) {
  if (total < 0 || n_parts <= 0) return XRT_ERR_ARGUMENT;
  if (total == 0) return XRT_OK;
  xrt::launch_kernel(xrt::add_scaled_parts_kernel, dim3(xrt::grid_for((size_t)total, 256)), dim3(256), 0, stream, residual,
                     parts, scales, (size_t)total, n_parts);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_scale_softcap(float* x, int n_rows, int width, float scale, float cap, cudaStream_t stream) {
  if (n_rows < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_rows == 0) return XRT_OK;
  const size_t total = (size_t)n_rows * width;
  xrt::launch_kernel(xrt::scale_softcap_kernel, dim3(xrt::grid_for(total, 256)), dim3(256), 0, stream, x, total, scale,
                     cap);
  return xrt::launch_status();
}
