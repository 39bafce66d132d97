// A norm on what a sublayer GIVES: residual[t] += RMSNorm(y[t]) * w, for layers that read the residual stream
// itself and norm only the sublayer's result.
//
//   y may come in `n_parts` parts [parts][T][width] (the chosen experts' weighted results): they are added in index
//   order first, so the sum has one order whatever else is in the step.  Each part may have a factor of its own
//   (`part_scales`, mixers side by side that are added with a weight each) and a row `bias` may be added to the sum
//   (a product's bias that was left for here).  What is added into the stream may be scaled (`factor`), and the new
//   row can be normed once more with a second weight into `then_out` (the norm that the next sublayer begins with).
//   Statistics, the division and the sum into the stream are 32-bit.  The new residual row can also be written once
//   more in the compute dtype (`copy`), which is what the next sublayer's products read: the pass that adds is the
//   pass that rounds, and no kernel of its own runs for that.
// One block a row; the row, the weight and the residual are asked for before the sum.
#include "common.cuh"

namespace xrt {

struct PostNormExtras {
  const float* part_scales = nullptr;  // [n_parts]
  const float* bias = nullptr;         // [width], added to the sum of the parts
  float factor = 1.0f;                 // residual += factor * norm
  const void* then_w = nullptr;        // [width] in the first weight's dtype: a second norm over the new row ...
  void* then_out = nullptr;            // ... written here in the copy's dtype
  float then_eps = 0.f;
};

template <typename TW, typename TC, int PER>
__global__ void rmsnorm_add_kernel(float* __restrict__ residual, const float* __restrict__ y, size_t part_stride,
                                   int n_parts, const TW* __restrict__ w, TC* __restrict__ copy, int width, float eps,
                                   const PostNormExtras ex) {
  __shared__ float scratch[33];
  pdl_trigger();
  float wv[PER], yv[PER], rv[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < width ? to_float(w[c]) : 0.f;
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
  if (ex.part_scales != nullptr) {
    const float s0 = ex.part_scales[0];
#pragma unroll
    for (int i = 0; i < PER; ++i) yv[i] *= s0;
  }
  for (int part = 1; part < n_parts; ++part) {
    const float sp = ex.part_scales != nullptr ? ex.part_scales[part] : 1.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < width) yv[i] = fmaf(p[(size_t)part * part_stride + c], sp, yv[i]);
    }
  }
  if (ex.bias != nullptr) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < width) yv[i] += ex.bias[c];
    }
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) sum = fmaf(yv[i], yv[i], sum);
  const float total = block_sum(sum, scratch);
  const float f = 1.0f / sqrtf(total / (float)width + eps);
  float again = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < width) {
      const float v = rv[i] + ex.factor * ((yv[i] * f) * wv[i]);
      r[c] = v;
      if (copy != nullptr) copy[(size_t)blockIdx.x * width + c] = from_float<TC>(v);
      rv[i] = v;
      again = fmaf(v, v, again);
    }
  }
  if (ex.then_out != nullptr) {  // uniform over the grid
    const float f2 = 1.0f / sqrtf(block_sum(again, scratch) / (float)width + ex.then_eps);
    const TW* w2 = static_cast<const TW*>(ex.then_w);
    TC* out2 = static_cast<TC*>(ex.then_out) + (size_t)blockIdx.x * width;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < width) out2[c] = from_float<TC>((rv[i] * f2) * to_float(w2[c]));
    }
  }
}

template <typename TC>
__global__ void cast_rows_kernel(TC* __restrict__ out, const float* __restrict__ x, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<TC>(x[i]);
}

}  // namespace xrt

// residual [T, width] float32; y [parts, T, width] float32 with `part_stride` floats between parts; weight [width];
// copy (may be null) [T, width] in copy_dtype.
XRT_EXPORT int xrt_rmsnorm_add(float* residual, const float* y, long long part_stride, int n_parts, const void* weight,
                               void* copy, int n_tokens, int width, float eps, int weight_dtype, int copy_dtype,
                               const float* part_scales, const float* bias, float factor, const void* then_weight,
                               void* then_out, float then_eps, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0 || n_parts <= 0) return XRT_ERR_ARGUMENT;
  if ((then_weight == nullptr) != (then_out == nullptr)) return XRT_ERR_ARGUMENT;
  xrt::PostNormExtras ex;
  ex.part_scales = part_scales;
  ex.bias = bias;
  ex.factor = factor;
  ex.then_w = then_weight;
  ex.then_out = then_out;
  ex.then_eps = then_eps;
  if (n_tokens == 0) return XRT_OK;
  const int threads = width >= 4096 ? 512 : (width >= 1024 ? 256 : (width >= 256 ? 128 : 64));
  const int per = (width + threads - 1) / threads;
  if (per > 32) return XRT_ERR_UNSUPPORTED;
#define XRT_POST(PER)                                                                                                   \
  xrt::launch_kernel(xrt::rmsnorm_add_kernel<TW, TC, PER>, dim3(n_tokens), dim3(threads), 0, stream, residual, y,       \
                     (size_t)part_stride, n_parts, (const TW*)weight, (TC*)copy, width, eps, ex)
  XRT_DISPATCH_DTYPE(weight_dtype, TW, {
    XRT_DISPATCH_DTYPE(copy_dtype, TC, {
      if (per <= 4) XRT_POST(4);
      else if (per <= 8) XRT_POST(8);
      else if (per <= 16) XRT_POST(16);
      else XRT_POST(32);
    });
  });
#undef XRT_POST
  return xrt::launch_status();
}

// out = x in out_dtype, elementwise; x float32.
XRT_EXPORT int xrt_cast_rows(void* out, const float* x, long long total, int out_dtype, cudaStream_t stream) {
  if (total < 0) return XRT_ERR_ARGUMENT;
  if (total == 0) return XRT_OK;
  const long long blocks = (total + 255) / 256;
  XRT_DISPATCH_DTYPE(out_dtype, TC, {
    xrt::launch_kernel(xrt::cast_rows_kernel<TC>, dim3((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16)), dim3(256), 0,
                       stream, (TC*)out, x, (size_t)total);
  });
  return xrt::launch_status();
}
