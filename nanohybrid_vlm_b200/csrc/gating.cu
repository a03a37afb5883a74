// Small elementwise steps around gated sub-blocks, all computed in fp32 and rounded once:
//
//   sigmoid_mul     out[t, c] = x[t, c] * sigmoid(g[t, c])          (an output gate before the output projection)
//   add_row_bias    x[t, c] += bias[c], in place                     (the bias of a projection whose product has none)
//   clamped_glu     out[t, c] = g' * sigmoid(alpha * g') * (u' + 1), g' = min(gate, limit), u' = clamp(up, -limit, limit)
//                   for gate_up [T, 2 I] with the gate in the first half of each row
#include <math.h>

#include "nhv_common.cuh"

template <typename T>
__global__ void sigmoid_mul_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ x, int x_stride,
                                   const T* __restrict__ g, int g_stride, int width, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width;
    const int c = (int)(i - t * width);
    const float gv = to_f32<T>(g[t * g_stride + c]);
    out[t * out_stride + c] = from_f32<T>(to_f32<T>(x[t * x_stride + c]) / (1.0f + expf(-gv)));
  }
}

NHV_API int nhv_sigmoid_mul(int dtype, void* out, int out_stride, const void* x, int x_stride, const void* g, int g_stride,
                            int n_rows, int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0, "sigmoid_mul: bad sizes");
  const size_t total = (size_t)n_rows * width;
  const int blocks = (int)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
#define GO(T) \
  nhv_launch(sigmoid_mul_kernel<T>, blocks, 256, 0, stream, (T*)out, out_stride, (const T*)x, x_stride, (const T*)g, g_stride, width, total)
  if (dtype == NHV_F32) GO(float);
  else if (dtype == NHV_BF16) GO(__nv_bfloat16);
  else NHV_REQUIRE(false, "sigmoid_mul: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("sigmoid_mul");
  return 0;
}

template <typename T>
__global__ void add_row_bias_kernel(T* __restrict__ x, const T* __restrict__ bias, int width, size_t total) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    x[i] = from_f32<T>(to_f32<T>(x[i]) + to_f32<T>(bias[i % width]));
}

NHV_API int nhv_add_row_bias(int dtype, void* x, const void* bias, int n_rows, int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0, "add_row_bias: bad sizes");
  const size_t total = (size_t)n_rows * width;
  const int blocks = (int)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
  if (dtype == NHV_F32) nhv_launch(add_row_bias_kernel<float>, blocks, 256, 0, stream, (float*)x, (const float*)bias, width, total);
  else if (dtype == NHV_BF16)
    nhv_launch(add_row_bias_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)x, (const __nv_bfloat16*)bias, width, total);
  else NHV_REQUIRE(false, "add_row_bias: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("add_row_bias");
  return 0;
}

__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, size_t total, float limit,
                                   float alpha) {
  pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / inter;
    const int c = (int)(i - t * inter);
    const T* row = gate_up + t * 2 * inter;
    out[i] = from_f32<T>(clamped_glu(to_f32<T>(row[c]), to_f32<T>(row[inter + c]), limit, alpha));
  }
}

NHV_API int nhv_clamped_glu(int dtype, void* out, const void* gate_up, int n_rows, int inter, float limit, float alpha,
                            cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && inter > 0, "clamped_glu: bad sizes");
  const size_t total = (size_t)n_rows * inter;
  const int blocks = (int)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
  if (dtype == NHV_F32)
    nhv_launch(clamped_glu_kernel<float>, blocks, 256, 0, stream, (float*)out, (const float*)gate_up, inter, total, limit, alpha);
  else if (dtype == NHV_BF16)
    nhv_launch(clamped_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter,
               total, limit, alpha);
  else NHV_REQUIRE(false, "clamped_glu: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("clamped_glu");
  return 0;
}
