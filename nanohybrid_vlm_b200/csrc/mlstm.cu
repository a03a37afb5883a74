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
// block takes (request, head, ML_COLS columns) and a column lives in the registers of 8 or 16 lanes, each with
// d / 8 or d / 16 rows; every column block carries the rows of n as well (its own copy, so that no block reads what
// another writes).  The gates of a stage of tokens (64, or 32 for the largest heads) are prepared together: their tanh and logsigmoid in parallel, the
// chain of maxima by one thread, the exponentials in parallel again.
//
// State of a slot: S transposed, [head][dv][d], then per (head, column block) the d rows of n and m.
// A request with q_start == 0 starts fresh; one without a slot (slot < 0) is skipped and its outputs are cleared.
#include <math.h>

#include "nhv_common.cuh"
#include "nhv_vec8.cuh"

constexpr int ML_COLS = 16;

__device__ __forceinline__ float ml_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// Which row of its column a lane's r-th register holds (a column lives in PARTS lanes).  VEC (d in steps of 4 * PARTS):
// groups of four consecutive rows, so that one 16-byte read of k and one of q from shared memory serve four rows, and
// two neighbouring rows share a packed fp32x2 instruction; else rows PARTS apart.
template <bool VEC, int PARTS> __device__ __forceinline__ int ml_row(int part, int r) {
  return VEC ? ((r >> 2) * (4 * PARTS) + part * 4 + (r & 3)) : (part + r * PARTS);
}

// VEC also reads the tokens' rows of proj eight elements at a time (the host checks sizes and alignment).
template <typename T, int R, bool VEC, int ML_PARTS>
__global__ void __launch_bounds__(ML_COLS * ML_PARTS) mlstm_scan_kernel(
    float* __restrict__ y, const T* __restrict__ proj, int proj_stride, const float* __restrict__ gates, int gate_stride,
    const float* __restrict__ gate_bias, float cap, float* __restrict__ state, long state_stride,
    const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ slots, int H, int d, int dv) {
  constexpr int stage_tokens = (R * ML_PARTS > 256) ? 32 : 64;   // tokens per stage: what fits a block's shared memory
  extern __shared__ __align__(16) float smem[];
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
  float* qs = ks + stage_tokens * d;             // [CHUNK][d], times d^-1/2
  float* vs = qs + stage_tokens * d;             // [CHUNK][COLS]
  float* ga = vs + stage_tokens * ML_COLS;       // [CHUNK] decay of the old state; before that the log forget gate
  float* gb = ga + stage_tokens;                 // [CHUNK] weight of the new pair; before that the log input gate
  float* gm = gb + stage_tokens;                 // [CHUNK + 1] m before each token and after the last; then exp(-m_t)
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
    const int i = ml_row<VEC, ML_PARTS>(part, r);
    S[r] = (live && !fresh && i < d) ? st[i] : 0.f;
    Nn[r] = (!fresh && i < d) ? nm[i] : 0.f;
  }
  float m_carry = fresh ? 0.f : nm[d];        // every thread keeps it; only thread 0's copy is written back
  const float qscale = 1.0f / sqrtf((float)d);
  const float bi = gate_bias[h], bf = gate_bias[H + h];
  const int q_off = h * d, k_off = H * d + h * d, v_off = 2 * H * d + h * dv + col0;
  for (int c0 = 0; c0 < n; c0 += stage_tokens) {
    const int cn = min(stage_tokens, n - c0);
    __syncthreads();
    if (VEC) {
      const int d8 = d >> 3;
      for (int i = tid; i < cn * d8; i += blockDim.x) {
        const int tt = i / d8, c = (i - tt * d8) * 8;
        const T* row = proj + (size_t)(first + c0 + tt) * proj_stride;
        float q8[8], k8[8];
        nhv_load8(q8, row + q_off + c);
        nhv_load8(k8, row + k_off + c);
        float* qd = qs + tt * d + c;
        float* kd = ks + tt * d + c;
        *reinterpret_cast<float4*>(qd) = make_float4(q8[0] * qscale, q8[1] * qscale, q8[2] * qscale, q8[3] * qscale);
        *reinterpret_cast<float4*>(qd + 4) = make_float4(q8[4] * qscale, q8[5] * qscale, q8[6] * qscale, q8[7] * qscale);
        *reinterpret_cast<float4*>(kd) = make_float4(k8[0], k8[1], k8[2], k8[3]);
        *reinterpret_cast<float4*>(kd + 4) = make_float4(k8[4], k8[5], k8[6], k8[7]);
      }
    } else {
      for (int i = tid; i < cn * d; i += blockDim.x) {
        const int tt = i / d, c = i - tt * d;
        const T* row = proj + (size_t)(first + c0 + tt) * proj_stride;
        qs[i] = to_f32<T>(row[q_off + c]) * qscale;
        ks[i] = to_f32<T>(row[k_off + c]);
      }
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
    // Only S and n are carried from token to token (one multiply-add each); the sums over rows, their shuffles and the
    // division of one token overlap with the next tokens' updates once the loop is unrolled.
#pragma unroll 4
    for (int tt = 0; tt < cn; ++tt) {
      const float a = ga[tt], b = gb[tt];
      const float bv = live ? b * vs[tt * ML_COLS + cl] : 0.f;
      const float* kt = ks + tt * d;
      const float* qt = qs + tt * d;
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, accn[4] = {0.f, 0.f, 0.f, 0.f};
      if (VEC) {
        // two neighbouring rows per packed instruction (each half rounded as the scalar operation would be)
        const f32x2 a2 = f2_pack(a, a), bv2 = f2_pack(bv, bv), b2 = f2_pack(b, b);
        f32x2 so2[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)}, sn2[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          const int i0 = j * (4 * ML_PARTS) + part * 4;
          if (i0 < d) {
            const float4 k4 = *reinterpret_cast<const float4*>(kt + i0), q4 = *reinterpret_cast<const float4*>(qt + i0);
            const f32x2 kk[2] = {f2_pack(k4.x, k4.y), f2_pack(k4.z, k4.w)}, qq[2] = {f2_pack(q4.x, q4.y), f2_pack(q4.z, q4.w)};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              f32x2 s2 = f2_pack(S[4 * j + 2 * e], S[4 * j + 2 * e + 1]), n2 = f2_pack(Nn[4 * j + 2 * e], Nn[4 * j + 2 * e + 1]);
              s2 = f2_fma(a2, s2, f2_mul(bv2, kk[e]));
              n2 = f2_fma(a2, n2, f2_mul(b2, kk[e]));
              so2[e] = f2_fma(s2, qq[e], so2[e]);
              sn2[e] = f2_fma(n2, qq[e], sn2[e]);
              f2_unpack(s2, S[4 * j + 2 * e], S[4 * j + 2 * e + 1]);
              f2_unpack(n2, Nn[4 * j + 2 * e], Nn[4 * j + 2 * e + 1]);
            }
          }
        }
        f2_unpack(so2[0], acc[0], acc[1]);
        f2_unpack(so2[1], acc[2], acc[3]);
        f2_unpack(sn2[0], accn[0], accn[1]);
        f2_unpack(sn2[1], accn[2], accn[3]);
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int i = part + r * ML_PARTS;
          if (i < d) {
            const float kk = kt[i], qq = qt[i];
            S[r] = fmaf(a, S[r], bv * kk);
            Nn[r] = fmaf(a, Nn[r], b * kk);
            acc[r & 3] = fmaf(S[r], qq, acc[r & 3]);
            accn[r & 3] = fmaf(Nn[r], qq, accn[r & 3]);
          }
        }
      }
      float so = (acc[0] + acc[1]) + (acc[2] + acc[3]), sn = (accn[0] + accn[1]) + (accn[2] + accn[3]);
#pragma unroll
      for (int o = 1; o < ML_PARTS; o <<= 1) {
        so += __shfl_xor_sync(0xffffffffu, so, o);
        sn += __shfl_xor_sync(0xffffffffu, sn, o);
      }
      if (live && part == 0)
        y[(size_t)(first + c0 + tt) * inner + h * dv + col] = so / (fmaxf(fabsf(sn), gm[tt]) + 1e-6f);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = ml_row<VEC, ML_PARTS>(part, r);
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
                           const int* q_start, const int* slots, int n_seqs, int n_tokens, int H, int d, int dv, int lanes,
                           cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(H > 0 && d > 0 && dv > 0 && cap > 0.f, "mlstm_scan: bad sizes");
  NHV_REQUIRE(d <= 512, "mlstm_scan: a key head of %d elements is beyond the supported 512", d);
  NHV_REQUIRE(state_stride >= (long)nhv_mlstm_state_floats(H, d, dv), "mlstm_scan: the state holds fewer floats than S, n and m need");
  // lanes per column of the memory: 8, or 16 (twice the warps for the same columns, half the rows in each lane) where
  // heads are large enough to fill them; `lanes` 8 or 16 asks for one of them
  const int parts = (lanes == 8 || lanes == 16) ? lanes : (d >= 64 ? 16 : 8);
  const int rows = (d + parts - 1) / parts;
  const int r_lanes = rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : rows <= 32 ? 32 : 64;      // the kernel's R
  const int chunk = r_lanes * parts > 256 ? 32 : 64;           // the kernel's tokens per stage
  const size_t smem = ((size_t)chunk * (2 * d + ML_COLS) + 3 * chunk + 1) * sizeof(float);
  dim3 grid(n_seqs, H, (dv + ML_COLS - 1) / ML_COLS);
  // rows in groups of four and tokens read eight elements at a time, where sizes and alignment allow it
  const size_t item = dtype == NHV_F32 ? 4 : 2;
  const bool vec = d % (4 * parts) == 0 && dv % 8 == 0 && proj_stride % 8 == 0 && ((uintptr_t)proj % 16) == 0 &&
                   ((size_t)H * d * item) % 16 == 0;
#define SCAN(T, R, V, P)                                                                                            \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      NHV_CUDA(cudaFuncSetAttribute(mlstm_scan_kernel<T, R, V, P>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                    (int)smem), "mlstm_scan");                                                      \
    nhv_launch(mlstm_scan_kernel<T, R, V, P>, grid, ML_COLS * P, smem, stream, y, (const T*)proj, proj_stride,      \
               gates, gate_stride, gate_bias, cap, state, state_stride, cu_q, q_start, slots, H, d, dv);            \
  } while (0)
#define SCAN_V(T, R, P)                                     \
  do {                                                      \
    if (vec) SCAN(T, R, true, P); else SCAN(T, R, false, P); \
  } while (0)
#define SCAN_R(T, P)                         \
  do {                                       \
    if (rows <= 4) SCAN_V(T, 4, P);          \
    else if (rows <= 8) SCAN_V(T, 8, P);     \
    else if (rows <= 16) SCAN_V(T, 16, P);   \
    else if (rows <= 32) SCAN_V(T, 32, P);   \
    else SCAN_V(T, 64, P);                   \
  } while (0)
#define LAUNCH(T)                            \
  do {                                       \
    if (parts == 16) SCAN_R(T, 16);          \
    else SCAN_R(T, 8);                       \
  } while (0)
  if (dtype == NHV_F32) LAUNCH(float);
  else if (dtype == NHV_BF16) LAUNCH(__nv_bfloat16);
  else NHV_REQUIRE(false, "mlstm_scan: unknown dtype %d", dtype);
#undef LAUNCH
#undef SCAN_R
#undef SCAN_V
#undef SCAN
  NHV_CHECK_LAUNCH("mlstm_scan");
  return 0;
}
