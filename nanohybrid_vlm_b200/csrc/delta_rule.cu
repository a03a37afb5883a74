// The gated delta rule as a recurrence over a packed step of several requests.
//
// Per head, with the state S [d, dv] (fp32, carried per request):
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// where q_t and k_t are unit vectors (x / sqrt(sum x^2 + 1e-6)), q_t also times d^-1/2,
//   beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log) * softplus(a_t + dt_bias)).
// Each o_t is then divided by its root mean square over dv, multiplied by a weight [dv] and by silu(gate_t).
//
// delta_prepare: one warp per (token, q/k head): the unit vectors in fp32; one thread per (token, head): beta, g.
// delta_scan:    one block per (request, head, tile of 64 columns of S).  Thread (column j, part p of P = 4) keeps
//                rows p, p + 4, ... of column j in registers; sums over rows end with two shuffles.  Tokens go
//                through shared memory in chunks of 16.  It writes o_t in fp32; the norm and the gate follow in
//                nhv_gated_rmsnorm (state_space.cu).
// The state of a slot is stored transposed, [head][dv][d].  A request with q_start == 0 starts from zeros; one
// without a slot (slot < 0) is skipped and its outputs are cleared.
#include <math.h>

#include "nhv_common.cuh"

constexpr int DR_PARTS = 4;
constexpr int DR_CHUNK = 16;
constexpr int DR_COLS = 64;         // columns of S per block

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void delta_prepare_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ beta,
                                     float* __restrict__ decay, const T* __restrict__ qkv, int qkv_stride,
                                     const float* __restrict__ ba, const float* __restrict__ a_log,
                                     const float* __restrict__ dt_bias, int n_tokens, int G, int H, int d) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + warp;
  const long n_vec = (long)n_tokens * 2 * G;
  if (item < n_vec) {
    const int t = (int)(item / (2 * G)), hh = (int)(item % (2 * G));       // hh < G: a q head, else a k head
    const T* src = qkv + (size_t)t * qkv_stride + (size_t)hh * d;
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float x = to_f32<T>(src[c]);
      ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    float r = 1.0f / sqrtf(ss + 1e-6f);
    float* dst;
    if (hh < G) {
      r *= 1.0f / sqrtf((float)d);
      dst = qn + ((size_t)t * G + hh) * d;
    } else {
      dst = kn + ((size_t)t * G + (hh - G)) * d;
    }
    for (int c = lane; c < d; c += 32) dst[c] = to_f32<T>(src[c]) * r;
  }
  const long gi = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gi < (long)n_tokens * H) {
    const int t = (int)(gi / H), h = (int)(gi % H);
    const float b = ba[(size_t)t * 2 * H + h], a = ba[(size_t)t * 2 * H + H + h];
    beta[gi] = 1.0f / (1.0f + expf(-b));
    decay[gi] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
  }
}

template <typename T, int R>
__global__ void __launch_bounds__(DR_COLS * DR_PARTS) delta_scan_kernel(
    float* __restrict__ o_out, const float* __restrict__ qn, const float* __restrict__ kn, const T* __restrict__ v,
    int v_stride, const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
    long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ slots,
    int G, int H, int d, int dv) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DR_COLS;
  const int g = h / (H / G);
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(DR_COLS, dv - col0);
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += blockDim.x)
      o_out[((size_t)(first + i / ncol) * H + h) * dv + col0 + i % ncol] = 0.f;
    return;
  }
  float* qs = smem;                         // [CHUNK][d]
  float* ks = qs + DR_CHUNK * d;            // [CHUNK][d]
  float* vs = ks + DR_CHUNK * d;            // [CHUNK][DR_COLS]
  float* gb = vs + DR_CHUNK * DR_COLS;      // [CHUNK][2]: decay, beta
  const int cl = tid / DR_PARTS, part = tid % DR_PARTS;
  const bool live = cl < ncol;
  const int col = col0 + (live ? cl : 0);
  float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + col) * d;
  float S[R];
  const bool fresh = q_start[s] == 0;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = part + r * DR_PARTS;
    S[r] = (live && !fresh && i < d) ? st[i] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += DR_CHUNK) {
    const int cn = min(DR_CHUNK, n - c0);
    __syncthreads();
    for (int i = tid; i < cn * d; i += blockDim.x) {
      const int tt = i / d, c = i - tt * d;
      const size_t row = ((size_t)(first + c0 + tt) * G + g) * d + c;
      qs[i] = qn[row];
      ks[i] = kn[row];
    }
    for (int i = tid; i < cn * ncol; i += blockDim.x) {
      const int tt = i / ncol, c = i - tt * ncol;
      vs[tt * DR_COLS + c] = to_f32<T>(v[(size_t)(first + c0 + tt) * v_stride + h * dv + col0 + c]);
    }
    for (int i = tid; i < cn; i += blockDim.x) {
      gb[2 * i] = decay[(size_t)(first + c0 + i) * H + h];
      gb[2 * i + 1] = beta[(size_t)(first + c0 + i) * H + h];
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float gt = gb[2 * tt], bt = gb[2 * tt + 1];
      const float* kt = ks + tt * d;
      const float* qt = qs + tt * d;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = part + r * DR_PARTS;
        if (i < d) {
          S[r] *= gt;
          acc = fmaf(S[r], kt[i], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      const float u = bt * ((live ? vs[tt * DR_COLS + cl] : 0.f) - acc);
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = part + r * DR_PARTS;
        if (i < d) {
          S[r] = fmaf(kt[i], u, S[r]);
          o = fmaf(S[r], qt[i], o);
        }
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (live && part == 0) o_out[((size_t)(first + c0 + tt) * H + h) * dv + col] = o;
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = part + r * DR_PARTS;
      if (i < d) st[i] = S[r];
    }
  }
}

// o_out [T, H, dv] fp32.  Scratch given by the caller: qn, kn [T, G, d] and beta, decay [T, H], all fp32.
NHV_API int nhv_delta_rule(int dtype, float* o_out, const void* qkv, int qkv_stride, const float* ba,
                           const float* a_log, const float* dt_bias, float* state, long state_stride, float* qn,
                           float* kn, float* beta, float* decay, const int* cu_q, const int* q_start,
                           const int* slots, int n_seqs, int n_tokens, int G, int H, int d, int dv,
                           cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(G > 0 && H > 0 && H % G == 0, "delta_rule: %d heads do not divide into %d q/k heads", H, G);
  NHV_REQUIRE(d > 0 && d <= 256 && dv > 0, "delta_rule: a q/k head of %d is beyond the supported 256", d);
  NHV_REQUIRE(state_stride >= (long)H * d * dv, "delta_rule: the state holds fewer than heads * d * dv floats");
  const int rows = (d + DR_PARTS - 1) / DR_PARTS;
  const int threads = DR_COLS * DR_PARTS;
  const size_t smem = ((size_t)DR_CHUNK * (2 * d + DR_COLS) + 2 * DR_CHUNK) * sizeof(float);
  const long vec = (long)n_tokens * 2 * G, gates = ((long)n_tokens * H + 31) / 32;
  const int prep_blocks = (int)(((vec > gates ? vec : gates) + 3) / 4);
  dim3 grid(n_seqs, H, (dv + DR_COLS - 1) / DR_COLS);
  const int v_off = 2 * G * d;
#define SCAN(T, R)                                                                                                  \
  nhv_launch(delta_scan_kernel<T, R>, grid, threads, smem, stream, o_out, (const float*)qn, (const float*)kn,       \
             (const T*)qkv + v_off, qkv_stride, (const float*)beta, (const float*)decay, state, state_stride, cu_q, \
             q_start, slots, G, H, d, dv)
#define LAUNCH(T)                                                                                                   \
  do {                                                                                                              \
    nhv_launch(delta_prepare_kernel<T>, prep_blocks, 128, 0, stream, qn, kn, beta, decay, (const T*)qkv, qkv_stride, \
               ba, a_log, dt_bias, n_tokens, G, H, d);                                                              \
    if (rows <= 8) SCAN(T, 8);                                                                                      \
    else if (rows <= 16) SCAN(T, 16);                                                                               \
    else if (rows <= 32) SCAN(T, 32);                                                                               \
    else SCAN(T, 64);                                                                                               \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "delta_rule: unknown dtype %d", dtype);
#undef LAUNCH
#undef SCAN
  NHV_CHECK_LAUNCH("delta_rule");
  return 0;
}
