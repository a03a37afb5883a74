// The state-space recurrence of Mamba-2 (scalar decay per head) over a packed step of several requests, and the
// gated RMS norm that follows it (also used behind the delta rule).
//
// Per head, with the state S [N, P] (fp32, carried per request), group gr of the head:
//   dt = softplus(dt_raw + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B_t x_t^T;  y_t = S^T C_t + D x_t
//
// ssd_scan: one block per (request, head, tile of 64 columns of S).  Thread (column j, part p of 4) keeps rows
// p, p + 4, ... of column j in registers; the sum over rows ends with two shuffles.  Tokens go through shared memory
// in chunks of 16.  The state of a slot is stored transposed, [head][P][N].  A request with q_start == 0 starts from
// zeros; one without a slot (slot < 0) is skipped and its outputs are cleared.
//
// gated_rmsnorm: rows of fp32 values y [T, n_groups * size], a gate z in the storage type, a weight w:
//   gate_first:  out = unit_rms(y * silu(z)) * w          (each group of `size` by its own root mean square)
//   else:        out = unit_rms(y) * w * silu(z)
// with w indexed by (column mod w_period).
#include <math.h>

#include "nhv_common.cuh"

constexpr int SS_PARTS = 4;
constexpr int SS_CHUNK = 16;
constexpr int SS_COLS = 64;

__device__ __forceinline__ float ss_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T, int R>
__global__ void __launch_bounds__(SS_COLS * SS_PARTS) ssd_scan_kernel(
    float* __restrict__ y, const T* __restrict__ xbc, int xbc_stride, const float* __restrict__ dt_raw, int dt_stride,
    const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int H, int P, int N, int G) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * SS_COLS;
  const int gr = h / (H / G);
  const int inner = H * P;
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(SS_COLS, P - col0);
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += blockDim.x) y[(size_t)(first + i / ncol) * inner + h * P + col0 + i % ncol] = 0.f;
    return;
  }
  float* Bs = smem;                          // [CHUNK][N]
  float* Cs = Bs + SS_CHUNK * N;             // [CHUNK][N]
  float* xs = Cs + SS_CHUNK * N;             // [CHUNK][SS_COLS]
  float* ds = xs + SS_CHUNK * SS_COLS;       // [CHUNK][2]: decay, dt
  const int cl = tid / SS_PARTS, part = tid % SS_PARTS;
  const bool live = cl < ncol;
  const int col = col0 + (live ? cl : 0);
  float* st = state + (size_t)slot * state_stride + ((size_t)h * P + col) * N;
  const float rate = expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];
  float S[R];
  const bool fresh = q_start[s] == 0;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = part + r * SS_PARTS;
    S[r] = (live && !fresh && i < N) ? st[i] : 0.f;
  }
  for (int c0 = 0; c0 < n; c0 += SS_CHUNK) {
    const int cn = min(SS_CHUNK, n - c0);
    __syncthreads();
    for (int i = tid; i < cn * N; i += blockDim.x) {
      const int tt = i / N, c = i - tt * N;
      const T* row = xbc + (size_t)(first + c0 + tt) * xbc_stride + inner + gr * N + c;
      Bs[i] = to_f32<T>(row[0]);
      Cs[i] = to_f32<T>(row[(size_t)G * N]);
    }
    for (int i = tid; i < cn * ncol; i += blockDim.x) {
      const int tt = i / ncol, c = i - tt * ncol;
      xs[tt * SS_COLS + c] = to_f32<T>(xbc[(size_t)(first + c0 + tt) * xbc_stride + h * P + col0 + c]);
    }
    for (int i = tid; i < cn; i += blockDim.x) {
      const float dt = ss_softplus(dt_raw[(size_t)(first + c0 + i) * dt_stride + h] + bias);
      ds[2 * i] = expf(-rate * dt);
      ds[2 * i + 1] = dt;
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float a = ds[2 * tt], dt = ds[2 * tt + 1];
      const float xv = live ? xs[tt * SS_COLS + cl] : 0.f;
      const float dx = dt * xv;
      const float* Bt = Bs + tt * N;
      const float* Ct = Cs + tt * N;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = part + r * SS_PARTS;
        if (i < N) {
          S[r] = fmaf(a, S[r], dx * Bt[i]);
          acc = fmaf(S[r], Ct[i], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (live && part == 0) y[(size_t)(first + c0 + tt) * inner + h * P + col] = acc + skip * xv;
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int i = part + r * SS_PARTS;
      if (i < N) st[i] = S[r];
    }
  }
}

// xbc [T, H*P + 2*G*N] (x, then B, then C), dt_raw [T, >= H] fp32, y [T, H*P] fp32
NHV_API int nhv_ssd_scan(int dtype, float* y, const void* xbc, int xbc_stride, const float* dt_raw, int dt_stride,
                         const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                         long state_stride, const int* cu_q, const int* q_start, const int* slots, int n_seqs,
                         int n_tokens, int H, int P, int N, int G, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(G > 0 && H > 0 && H % G == 0, "ssd_scan: %d heads do not divide into %d groups", H, G);
  NHV_REQUIRE(N > 0 && N <= 256 && P > 0, "ssd_scan: a state of %d rows is beyond the supported 256", N);
  NHV_REQUIRE(state_stride >= (long)H * P * N, "ssd_scan: the state holds fewer than heads * P * N floats");
  const int rows = (N + SS_PARTS - 1) / SS_PARTS;
  const size_t smem = ((size_t)SS_CHUNK * (2 * N + SS_COLS) + 2 * SS_CHUNK) * sizeof(float);
  dim3 grid(n_seqs, H, (P + SS_COLS - 1) / SS_COLS);
#define SCAN(T, R)                                                                                               \
  nhv_launch(ssd_scan_kernel<T, R>, grid, SS_COLS * SS_PARTS, smem, stream, y, (const T*)xbc, xbc_stride, dt_raw, \
             dt_stride, dt_bias, a_log, d_skip, state, state_stride, cu_q, q_start, slots, H, P, N, G)
#define LAUNCH(T)                          \
  do {                                     \
    if (rows <= 8) SCAN(T, 8);             \
    else if (rows <= 16) SCAN(T, 16);      \
    else if (rows <= 32) SCAN(T, 32);      \
    else SCAN(T, 64);                      \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "ssd_scan: unknown dtype %d", dtype);
#undef LAUNCH
#undef SCAN
  NHV_CHECK_LAUNCH("ssd_scan");
  return 0;
}

// One block per (token, group).
template <typename T>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, int out_stride, const float* __restrict__ y,
                                     const T* __restrict__ z, int z_stride, const T* __restrict__ w, int w_period,
                                     int n_groups, int size, float eps, int gate_first) {
  __shared__ float red[33];
  pdl_prologue();
  const int t = blockIdx.x / n_groups, gidx = blockIdx.x % n_groups;
  const float* yr = y + ((size_t)t * n_groups + gidx) * size;
  const T* zr = z + (size_t)t * z_stride + (size_t)gidx * size;
  T* dst = out + (size_t)t * out_stride + (size_t)gidx * size;
  float ss = 0.f;
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    float v = yr[c];
    if (gate_first) {
      const float g = to_f32<T>(zr[c]);
      v *= g / (1.0f + expf(-g));
    }
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)size + eps);
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    const float g = to_f32<T>(zr[c]);
    const float sg = g / (1.0f + expf(-g));
    const float wv = to_f32<T>(w[(gidx * size + c) % w_period]);
    dst[c] = from_f32<T>(yr[c] * sg * rstd * wv);
  }
}

NHV_API int nhv_gated_rmsnorm(int dtype, void* out, int out_stride, const float* y, const void* z, int z_stride,
                              const void* w, int w_period, int n_tokens, int n_groups, int size, float eps,
                              int gate_first, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_groups > 0 && size > 0 && w_period > 0, "gated_rmsnorm: bad sizes");
  int threads = 32;
  while (threads < 256 && threads * 2 <= size) threads <<= 1;
  const long blocks = (long)n_tokens * n_groups;
  NHV_REQUIRE(blocks < (1L << 31), "gated_rmsnorm: too many rows");
  if (dtype == NHV_F32)
    nhv_launch(gated_rmsnorm_kernel<float>, (int)blocks, threads, 0, stream, (float*)out, out_stride, y, (const float*)z,
               z_stride, (const float*)w, w_period, n_groups, size, eps, gate_first);
  else if (dtype == NHV_BF16)
    nhv_launch(gated_rmsnorm_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (__nv_bfloat16*)out, out_stride, y,
               (const __nv_bfloat16*)z, z_stride, (const __nv_bfloat16*)w, w_period, n_groups, size, eps, gate_first);
  else
    NHV_REQUIRE(false, "gated_rmsnorm: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("gated_rmsnorm");
  return 0;
}
