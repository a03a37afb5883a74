// The matrix-memory recurrence of xLSTM (mLSTM) over a packed step of several requests.
//
// Per head, with the memory S [d, dv], the normaliser n [d] and the running maximum m (all fp32, carried per
// request; S and n start at zero and m at 0):
//   i_t = cap tanh((i_raw + b_i) / cap)                         log input gate
//   f_t = logsigmoid(cap tanh((f_raw + b_f) / cap))             log forget gate
//   m_t = max(f_t + m_(t-1), i_t)
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),     q_t already times d^-1/2
//
// The columns of S are independent of one another (column j: S_j <- a S_j + b v_j k, o_j = S_j . q / den), so a
// block takes (request, head, ML_COLS columns) and a column lives in the registers of ML_PARTS lanes, each with
// d / ML_PARTS rows; every column block carries the rows of n as well (its own copy, so that no block reads what
// another writes).  The gates of ML_CHUNK tokens are prepared together: their tanh and logsigmoid in parallel, the
// chain of maxima by one thread, the exponentials in parallel again.
//
// State of a slot: S transposed, [head][dv][d], then per (head, column block) the d rows of n and m.
// A request with q_start == 0 starts fresh; one without a slot (slot < 0) is skipped and its outputs are cleared.
#include <math.h>

#include "nhv_common.cuh"

constexpr int ML_COLS = 16;
constexpr int ML_PARTS = 8;
constexpr int ML_CHUNK = 16;

__device__ __forceinline__ float ml_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T, int R>
__global__ void __launch_bounds__(ML_COLS * ML_PARTS) mlstm_scan_kernel(
    float* __restrict__ y, const T* __restrict__ proj, int proj_stride, const float* __restrict__ gates, int gate_stride,
    const float* __restrict__ gate_bias, float cap, float* __restrict__ state, long state_stride,
    const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ slots, int H, int d, int dv) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int s = blockIdx.x, h = blockIdx.y, cb = blockIdx.z, col0 = cb * ML_COLS;
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(ML_COLS, dv - col0);
  const int inner = H * dv;
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += blockDim.x) y[(size_t)(first + i / ncol) * inner + h * dv + col0 + i % ncol] = 0.f;
    return;
  }
  float* ks = smem;                          // [CHUNK][d]
  float* qs = ks + ML_CHUNK * d;             // [CHUNK][d], times d^-1/2
  float* vs = qs + ML_CHUNK * d;             // [CHUNK][COLS]
  float* ga = vs + ML_CHUNK * ML_COLS;       // [CHUNK] decay of the old state; before that the log forget gate
  float* gb = ga + ML_CHUNK;                 // [CHUNK] weight of the new pair; before that the log input gate
  float* gm = gb + ML_CHUNK;                 // [CHUNK + 1] m before each token and after the last; then exp(-m_t)
  const int cl = tid / ML_PARTS, part = tid % ML_PARTS;
  const bool live = cl < ncol;
  const int col = col0 + (live ? cl : 0);
  float* base = state + (size_t)slot * state_stride;
  float* st = base + ((size_t)h * dv + col) * d;
  float* nm = base + (size_t)H * dv * d + ((size_t)h * gridDim.z + cb) * (d + 1);
  const bool fresh = q_start[s] == 0;
  float S[R], Nn[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = part + r * ML_PARTS;
    S[r] = (live && !fresh && i < d) ? st[i] : 0.f;
    Nn[r] = (!fresh && i < d) ? nm[i] : 0.f;
  }
  float m_carry = fresh ? 0.f : nm[d];        // every thread keeps it; only thread 0's copy is written back
  const float qscale = 1.0f / sqrtf((float)d);
  const float bi = gate_bias[h], bf = gate_bias[H + h];
  const int q_off = h * d, k_off = H * d + h * d, v_off = 2 * H * d + h * dv + col0;
  for (int c0 = 0; c0 < n; c0 += ML_CHUNK) {
    const int cn = min(ML_CHUNK, n - c0);
    __syncthreads();
    for (int i = tid; i < cn * d; i += blockDim.x) {
      const int tt = i / d, c = i - tt * d;
      const T* row = proj + (size_t)(first + c0 + tt) * proj_stride;
      qs[i] = to_f32<T>(row[q_off + c]) * qscale;
      ks[i] = to_f32<T>(row[k_off + c]);
    }
    for (int i = tid; i < cn * ncol; i += blockDim.x) {
      const int tt = i / ncol, c = i - tt * ncol;
      vs[tt * ML_COLS + c] = to_f32<T>(proj[(size_t)(first + c0 + tt) * proj_stride + v_off + c]);
    }
    if (tid < cn) {
      const float* g = gates + (size_t)(first + c0 + tid) * gate_stride;
      gb[tid] = cap * tanhf((g[h] + bi) / cap);
      ga[tid] = ml_logsigmoid(cap * tanhf((g[H + h] + bf) / cap));
    }
    __syncthreads();
    if (tid == 0) {
      float m = m_carry;
      for (int tt = 0; tt < cn; ++tt) {
        gm[tt] = m;
        m = fmaxf(ga[tt] + m, gb[tt]);
      }
      gm[cn] = m;
    }
    __syncthreads();
    float m_prev = 0.f, m_new = 0.f, fg = 0.f, ig = 0.f;
    if (tid < cn) {
      m_prev = gm[tid];
      m_new = gm[tid + 1];
      fg = ga[tid];
      ig = gb[tid];
    }
    m_carry = gm[cn];
    __syncthreads();
    if (tid < cn) {
      ga[tid] = expf(fg + m_prev - m_new);
      gb[tid] = expf(ig - m_new);
      gm[tid] = expf(-m_new);
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float a = ga[tt], b = gb[tt];
      const float bv = live ? b * vs[tt * ML_COLS + cl] : 0.f;
      const float* kt = ks + tt * d;
      const float* qt = qs + tt * d;
      float acc = 0.f, accn = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int i = part + r * ML_PARTS;
        if (i < d) {
          const float kk = kt[i], qq = qt[i];
          S[r] = fmaf(a, S[r], bv * kk);
          Nn[r] = fmaf(a, Nn[r], b * kk);
          acc = fmaf(S[r], qq, acc);
          accn = fmaf(Nn[r], qq, accn);
        }
      }
#pragma unroll
      for (int o = 1; o < ML_PARTS; o <<= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
        accn += __shfl_xor_sync(0xffffffffu, accn, o);
      }
      if (live && part == 0)
        y[(size_t)(first + c0 + tt) * inner + h * dv + col] = acc / (fmaxf(fabsf(accn), gm[tt]) + 1e-6f);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = part + r * ML_PARTS;
    if (i < d) {
      if (live) st[i] = S[r];
      if (cl == 0) nm[i] = Nn[r];
    }
  }
  if (tid == 0) nm[d] = m_carry;
}

// Floats of state that one request needs (the host sizes its slots with this).
NHV_API int nhv_mlstm_state_floats(int H, int d, int dv) {
  const int nb = (dv + ML_COLS - 1) / ML_COLS;
  return H * dv * d + H * nb * (d + 1);
}

// proj [T, >= 2*H*d + H*dv] (q, then k, then v, per head), gates [T, >= 2*H] fp32 (input gates, then forget gates,
// before bias and cap), gate_bias [2*H] fp32, y [T, H*dv] fp32.
NHV_API int nhv_mlstm_scan(int dtype, float* y, const void* proj, int proj_stride, const float* gates, int gate_stride,
                           const float* gate_bias, float cap, float* state, long state_stride, const int* cu_q,
                           const int* q_start, const int* slots, int n_seqs, int n_tokens, int H, int d, int dv,
                           cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(H > 0 && d > 0 && dv > 0 && cap > 0.f, "mlstm_scan: bad sizes");
  NHV_REQUIRE(d <= 64 * ML_PARTS, "mlstm_scan: a key head of %d elements is beyond the supported %d", d, 64 * ML_PARTS);
  NHV_REQUIRE(state_stride >= (long)nhv_mlstm_state_floats(H, d, dv), "mlstm_scan: the state holds fewer floats than S, n and m need");
  const int rows = (d + ML_PARTS - 1) / ML_PARTS;
  const size_t smem = ((size_t)ML_CHUNK * (2 * d + ML_COLS) + 3 * ML_CHUNK + 1) * sizeof(float);
  dim3 grid(n_seqs, H, (dv + ML_COLS - 1) / ML_COLS);
#define SCAN(T, R)                                                                                                  \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      NHV_CUDA(cudaFuncSetAttribute(mlstm_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), \
               "mlstm_scan");                                                                                       \
    nhv_launch(mlstm_scan_kernel<T, R>, grid, ML_COLS * ML_PARTS, smem, stream, y, (const T*)proj, proj_stride, gates, \
               gate_stride, gate_bias, cap, state, state_stride, cu_q, q_start, slots, H, d, dv);                   \
  } while (0)
#define LAUNCH(T)                          \
  do {                                     \
    if (rows <= 4) SCAN(T, 4);             \
    else if (rows <= 8) SCAN(T, 8);        \
    else if (rows <= 16) SCAN(T, 16);      \
    else if (rows <= 32) SCAN(T, 32);      \
    else SCAN(T, 64);                      \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "mlstm_scan: unknown dtype %d", dtype);
#undef LAUNCH
#undef SCAN
  NHV_CHECK_LAUNCH("mlstm_scan");
  return 0;
}
