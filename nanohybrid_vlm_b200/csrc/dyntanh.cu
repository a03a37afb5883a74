// Dynamic Tanh: a norm that takes no statistics, y = tanh(alpha * x) * w + b, with a learned scalar alpha and
// learned vectors w and b.  Being elementwise it fuses with whatever stands around it; three forms:
//
//   dyntanh          out = f(x) for rows of any of the two types in and out
//   embed_dyntanh    out (fp32) = f(table[ids]): the start of a residual stream kept in 32-bit
//   dyntanh_stream   the norm over a float32 residual stream between two sub-blocks of a layer whose sub-block
//                    outputs pass a norm of their own before they are added:
//                      s = stream[src] + (a ? f_post(a[src]) : 0)     (32-bit; written back unless rows are gathered;
//                                                                      without f_post the addend is added as it is)
//                      out[r] = f_pre(s)                              (rounded once to the storage type)
//                    with src = rows[r] or r.  One kernel does the add of the last sub-block and the norm of the next;
//                    elementwise over rows x width, so a decode step of a few rows spreads over many blocks.
//
// All arithmetic is fp32 (tanhf); alpha, w and b are stored in the model's type.
#include <math.h>

#include "nhv_common.cuh"

template <typename T>
struct DytParams {
  const T* alpha;   // one element
  const T* w;       // [width]
  const T* b;       // [width]
};

template <typename T>
__device__ __forceinline__ float dyt_apply(float x, float alpha, const DytParams<T>& p, int c) {
  return fmaf(tanhf(alpha * x), to_f32<T>(p.w[c]), to_f32<T>(p.b[c]));
}

template <typename TI, typename TO, typename TP>
__global__ void dyntanh_kernel(TO* __restrict__ out, const TI* __restrict__ x, DytParams<TP> p, size_t total, int width) {
  pdl_prologue();
  const float alpha = to_f32<TP>(p.alpha[0]);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f32<TO>(dyt_apply<TP>(to_f32<TI>(x[i]), alpha, p, (int)(i % width)));
}

NHV_API int nhv_dyntanh(int param_dtype, int in_f32, int out_f32, void* out, const void* x, const void* alpha,
                        const void* w, const void* b, int n_rows, int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0, "dyntanh: bad sizes");
  const size_t total = (size_t)n_rows * width;
  const int blocks = (int)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
#define GO(TI, TO, TP)                                                                                         \
  nhv_launch(dyntanh_kernel<TI, TO, TP>, blocks, 256, 0, stream, (TO*)out, (const TI*)x,                       \
             DytParams<TP>{(const TP*)alpha, (const TP*)w, (const TP*)b}, total, width)
#define PICK(TP)                                     \
  do {                                               \
    if (in_f32 && out_f32) GO(float, float, TP);     \
    else if (in_f32) GO(float, TP, TP);              \
    else if (out_f32) GO(TP, float, TP);             \
    else GO(TP, TP, TP);                             \
  } while (0)
  if (param_dtype == NHV_F32) PICK(float);
  else if (param_dtype == NHV_BF16) PICK(__nv_bfloat16);
  else NHV_REQUIRE(false, "dyntanh: unknown dtype %d", param_dtype);
#undef PICK
#undef GO
  NHV_CHECK_LAUNCH("dyntanh");
  return 0;
}

template <typename T>
__global__ void embed_dyntanh_kernel(float* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                     DytParams<T> p, int width, int vocab) {
  pdl_prologue();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const float alpha = to_f32<T>(p.alpha[0]);
  const T* row = table + (size_t)id * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)t * width + c] = dyt_apply<T>(to_f32<T>(row[c]), alpha, p, c);
}

NHV_API int nhv_embed_dyntanh(int dtype, float* out, const void* table, const int* ids, const void* alpha, const void* w,
                              const void* b, int n_tokens, int width, int vocab, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_tokens > 0 && width > 0 && vocab > 0, "embed_dyntanh: bad sizes");
  const int threads = width >= 256 ? 256 : 128;
#define GO(T)                                                                                              \
  nhv_launch(embed_dyntanh_kernel<T>, n_tokens, threads, 0, stream, out, (const T*)table, ids,             \
             DytParams<T>{(const T*)alpha, (const T*)w, (const T*)b}, width, vocab)
  if (dtype == NHV_F32) GO(float);
  else if (dtype == NHV_BF16) GO(__nv_bfloat16);
  else NHV_REQUIRE(false, "embed_dyntanh: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("embed_dyntanh");
  return 0;
}

// Four neighbouring columns of a row per thread (width in steps of 4), or one; the elements do not depend on one
// another, so a step of few rows still fills the device.
template <typename T> __device__ __forceinline__ void dyt_load4(float (&o)[4], const T* p);
template <> __device__ __forceinline__ void dyt_load4<float>(float (&o)[4], const float* p) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void dyt_load4<__nv_bfloat16>(float (&o)[4], const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
__device__ __forceinline__ void dyt_store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void dyt_store4(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
  h[0] = __floats2bfloat162_rn(v[0], v[1]);
  h[1] = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) dyntanh_stream_kernel(T* __restrict__ out, float* __restrict__ stream,
                                                             const T* __restrict__ a, DytParams<T> post, DytParams<T> pre,
                                                             const int* __restrict__ rows, int width, int write_stream,
                                                             size_t total) {
  pdl_prologue();
  const float a_pre = to_f32<T>(pre.alpha[0]);
  const bool has_post = a && post.alpha;                        // an addend without a norm of its own is added as it is
  const float a_post = has_post ? to_f32<T>(post.alpha[0]) : 0.f;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < total; i += (size_t)gridDim.x * blockDim.x * VEC) {
    const size_t r = i / width;
    const int c = (int)(i - r * width);
    const size_t src = (rows ? (size_t)rows[r] : r) * width + c;
    float s[VEC], y[VEC];
    if constexpr (VEC == 4) {
      float s4[4];
      dyt_load4<float>(s4, stream + src);
#pragma unroll
      for (int e = 0; e < VEC; ++e) s[e] = s4[e];
      if (a) {
        float a4[4];
        dyt_load4<T>(a4, a + src);
#pragma unroll
        for (int e = 0; e < VEC; ++e) s[e] += has_post ? dyt_apply<T>(a4[e], a_post, post, c + e) : a4[e];
        if (write_stream) {
          dyt_store4(stream + src, s);
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) y[e] = dyt_apply<T>(s[e], a_pre, pre, c + e);
      dyt_store4(out + i, y);
    } else {
      s[0] = stream[src];
      if (a) {
        const float av = to_f32<T>(a[src]);
        s[0] += has_post ? dyt_apply<T>(av, a_post, post, c) : av;
        if (write_stream) stream[src] = s[0];
      }
      out[i] = from_f32<T>(dyt_apply<T>(s[0], a_pre, pre, c));
    }
  }
}

NHV_API int nhv_dyntanh_stream(int dtype, void* out, float* stream, const void* a, const void* post_alpha,
                               const void* post_w, const void* post_b, const void* pre_alpha, const void* pre_w,
                               const void* pre_b, const int* rows, int n_rows, int width, int write_stream,
                               cudaStream_t stream_) {
  if (n_rows == 0) return 0;
  NHV_REQUIRE(n_rows > 0 && width > 0, "dyntanh_stream: bad sizes");
  NHV_REQUIRE(!post_alpha || (post_w && post_b), "dyntanh_stream: a norm is alpha, weight and bias together");
  const size_t total = (size_t)n_rows * width;
  const bool vec = width % 4 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)stream % 16) == 0 && ((uintptr_t)a % 16) == 0;
  const size_t per_block = 256 * (vec ? 4 : 1);
  const int blocks = (int)((total + per_block - 1) / per_block < 65535 * 8 ? (total + per_block - 1) / per_block : 65535 * 8);
#define GO(T, V)                                                                                                  \
  nhv_launch(dyntanh_stream_kernel<T, V>, blocks, 256, 0, stream_, (T*)out, stream, (const T*)a,                  \
             DytParams<T>{(const T*)post_alpha, (const T*)post_w, (const T*)post_b},                              \
             DytParams<T>{(const T*)pre_alpha, (const T*)pre_w, (const T*)pre_b}, rows, width,                    \
             (write_stream && !rows) ? 1 : 0, total)
  if (dtype == NHV_F32) { if (vec) GO(float, 4); else GO(float, 1); }
  else if (dtype == NHV_BF16) { if (vec) GO(__nv_bfloat16, 4); else GO(__nv_bfloat16, 1); }
  else NHV_REQUIRE(false, "dyntanh_stream: unknown dtype %d", dtype);
#undef GO
  NHV_CHECK_LAUNCH("dyntanh_stream");
  return 0;
}
