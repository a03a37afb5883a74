// out[M, N] (fp32) = x[M, K] @ w[N, K]^T for bfloat16 operands and few outputs: the small projections whose results
// enter a recurrence or a gate in 32-bit (a handful of rows of w, a step of a few tokens).  One warp per output:
// the lanes walk K in 16-byte pieces, sum in fp32 in a fixed order and meet in a shuffle tree, so an output does
// not depend on what else is in the batch.  Large M goes to the library product instead (the caller decides).
#include "nhv_common.cuh"

constexpr int GR_WARPS = 4;

__global__ void __launch_bounds__(GR_WARPS * 32) gemm_rows_f32_kernel(float* __restrict__ out, int out_stride,
                                                                       const __nv_bfloat16* __restrict__ x, int x_stride,
                                                                       const __nv_bfloat16* __restrict__ w, int w_stride,
                                                                       int M, int N, int K) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * GR_WARPS + warp;
  if (item >= (long)M * N) return;
  const int m = (int)(item / N), n = (int)(item - (long)m * N);
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)m * x_stride);
  const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)n * w_stride);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int c = lane; c < (K >> 3); c += 32) {
    const uint4 a = xr[c], b = wr[c];
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fa = __bfloat1622float2(ap[e]), fb = __bfloat1622float2(bp[e]);
      acc[e] = fmaf(fa.x, fb.x, acc[e]);
      acc[e] = fmaf(fa.y, fb.y, acc[e]);
    }
  }
  const float sum = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
  if (lane == 0) out[(size_t)m * out_stride + n] = sum;
}

NHV_API int nhv_gemm_rows_f32(float* out, int out_stride, const void* x, int x_stride, const void* w, int w_stride, int M,
                              int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  NHV_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0 && x_stride % 8 == 0 && w_stride % 8 == 0 &&
                  ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0,
              "gemm_rows_f32: K and the row strides must be multiples of 8 elements, the operands 16-byte aligned");
  const long items = (long)M * N;
  nhv_launch(gemm_rows_f32_kernel, (int)((items + GR_WARPS - 1) / GR_WARPS), GR_WARPS * 32, 0, stream, out, out_stride,
             (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)w, w_stride, M, N, K);
  NHV_CHECK_LAUNCH("gemm_rows_f32");
  return 0;
}
