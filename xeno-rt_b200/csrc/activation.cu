// SwiGLU on the fused gate/up product: out[t, f] = silu(gu[t, f]) * gu[t, F + f],
// silu(g) = g / (1 + exp(-g)).  Restates crates/xrt-kernels/src/cpu/silu.rs:1-3, 22-24; the
// reference's PTX silu_kernel (crates/xrt-cuda/src/lib.rs:596-635) has no gate product.
#include "common.cuh"

namespace xrt {

// `act` 1: the gate passes the tanh form of gelu instead, 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))).
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return g / (1.0f + expf(-g));
}

template <typename TI, typename TO>
__global__ void swiglu_kernel(TO* __restrict__ out, const TI* __restrict__ gate_up, int n_tokens, int width, int act) {
  const size_t total = (size_t)n_tokens * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width, f = i - t * width;
    const float g = to_float(gate_up[t * 2 * width + f]);
    const float u = to_float(gate_up[t * 2 * width + width + f]);
    out[i] = from_float<TO>(gate_act(g, act) * u);
  }
}

// Squared relu: out[i] = max(x[i], 0)^2 (the activation of a feed-forward without a gate).
template <typename TO>
__global__ void relu_squared_kernel(TO* __restrict__ out, const float* __restrict__ x, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(x[i], 0.f);
    out[i] = from_float<TO>(v * v);
  }
}

}  // namespace xrt

XRT_EXPORT int xrt_relu_squared(void* out, const float* x, int n_tokens, int width, int out_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t total = (size_t)n_tokens * width;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  XRT_DISPATCH_DTYPE(out_dtype, TO, {
    xrt::launch_kernel(xrt::relu_squared_kernel<TO>, dim3(blocks), dim3(256), 0, stream, (TO*)out, x, total);
  });
  return xrt::launch_status();
}

XRT_EXPORT int xrt_swiglu(void* out, const void* gate_up, int n_tokens, int width, int in_dtype,
                          int out_dtype, int act, cudaStream_t stream) {
  if (act != 0 && act != 1) return XRT_ERR_ARGUMENT;
  if (n_tokens < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t total = (size_t)n_tokens * width;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  XRT_DISPATCH_DTYPE(in_dtype, TI, {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      xrt::swiglu_kernel<TI, TO><<<blocks, 256, 0, stream>>>((TO*)out, (const TI*)gate_up, n_tokens, width, act);
    });
  });
  return xrt::launch_status();
}
