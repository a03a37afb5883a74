// The gated delta rule as a recurrence over a packed step of several requests.
//
// Per head, with the state S [d, dv] (fp32, carried per request):
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// where q_t and k_t are unit vectors (x / sqrt(sum x^2 + 1e-6)), q_t also times d^-1/2,
//   beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log) * softplus(a_t + dt_bias)).
// Each o_t is then divided by its root mean square over dv, multiplied by a weight [dv] and by silu(gate_t).
//
// delta_prepare: one warp per (token, q/k head pair): the unit vectors in fp32 and their product k_t . q_t; one
//                thread per (token, head): beta, g; the values v_t widened to fp32.
// delta_scan:    the columns of S are independent of one another (column j: u_j = beta (v_j - S_j . k),
//                S_j += u_j k, o_j = S_j . q), so a block takes (request, head, 16 columns) and a column lives in
//                the registers of 8 lanes, each with d / 8 rows in groups of 4 (one 16-byte read of k and of q
//                from shared memory serves 4 rows).  Per token the two sums S_j . k and S_j . q are taken from
//                the state BEFORE the write, side by side (four partial sums each, then three shuffles), and
//                  o_j = g S_j . q + u_j (k . q),   S_j <- g S_j + u_j k
//                which is the read-out after the write, since (g S + k u^T)^T q = g S^T q + u (k . q).  Tokens
//                reach shared memory by cp.async, 16 at a time, the next 16 while these are worked on.
// delta_scan_any: the same recurrence for sizes that are no multiple of 4 (no 16-byte copies): 64 columns a
//                block, 4 lanes a column, plain loads.
// Both write o_t in fp32; the norm and the gate follow in nhv_gated_rmsnorm (state_space.cu).
// The state of a slot is stored transposed, [head][dv][d].  A request with q_start == 0 starts from zeros; one
// without a slot (slot < 0) is skipped and its outputs are cleared.
#include <math.h>

#include "nhv_common.cuh"

constexpr int DR_PARTS = 4;
constexpr int DR_CHUNK = 16;
constexpr int DR_COLS = 64;         // columns of S per block

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void delta_prepare_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ kq,
                                     float* __restrict__ v32, float* __restrict__ beta, float* __restrict__ decay,
                                     const T* __restrict__ qkv, int qkv_stride, const float* __restrict__ ba,
                                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                     int n_tokens, int G, int H, int d, int dv) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long n_warps = (long)gridDim.x * (blockDim.x >> 5);
  for (long item = (long)blockIdx.x * (blockDim.x >> 5) + warp; item < (long)n_tokens * G; item += n_warps) {
    const int t = (int)(item / G), g = (int)(item % G);
    const T* qs = qkv + (size_t)t * qkv_stride + (size_t)g * d;
    const T* ks = qs + (size_t)G * d;
    float sq = 0.f, sk = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float a = to_f32<T>(qs[c]), b = to_f32<T>(ks[c]);
      sq = fmaf(a, a, sq);
      sk = fmaf(b, b, sk);
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float rq = 1.0f / sqrtf(sq + 1e-6f) * (1.0f / sqrtf((float)d)), rk = 1.0f / sqrtf(sk + 1e-6f);
    float dot = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float a = to_f32<T>(qs[c]) * rq, b = to_f32<T>(ks[c]) * rk;
      qn[(size_t)item * d + c] = a;
      kn[(size_t)item * d + c] = b;
      dot = fmaf(a, b, dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) kq[item] = dot;
  }
  const long n_threads = (long)gridDim.x * blockDim.x, me = (long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long i = me; i < (long)n_tokens * H; i += n_threads) {
    const int t = (int)(i / H), h = (int)(i % H);
    const float b = ba[(size_t)t * 2 * H + h], a = ba[(size_t)t * 2 * H + H + h];
    beta[i] = 1.0f / (1.0f + expf(-b));
    decay[i] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
  }
  if (v32) {
    const int hv = H * dv;
    const T* vs = qkv + (size_t)2 * G * d;
    for (long i = me; i < (long)n_tokens * hv; i += n_threads) {
      const long t = i / hv;
      v32[i] = to_f32<T>(vs[(size_t)t * qkv_stride + (i - t * hv)]);
    }
  }
}

// ---------------------------------------------------------------- the scan for sizes in steps of 4
constexpr int DF_CHUNK = 16;        // tokens per stage
constexpr int DF_THREADS = 128;     // LANES lanes per column of S (8, 16 or 32), 128 / LANES columns per block

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// R: rows of a column per lane (a multiple of 4, R * 8 >= d).  qn, kn [T, G, d]; kq [T, G]; v32: rows of v_stride
// floats whose first H * dv are the token's values; all fp32.
template <int R, int LANES>
__global__ void __launch_bounds__(DF_THREADS) delta_scan_fast_kernel(
    float* __restrict__ o_out, const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ kq,
    const float* __restrict__ v32, int v_stride, const float* __restrict__ beta, const float* __restrict__ decay,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int G, int H, int d, int dv) {
  constexpr int COLS = DF_THREADS / LANES;             // columns of S per block
  extern __shared__ __align__(16) float smem[];
  // a long kernel of few blocks: the kernel behind it is let in only at the end, so that its blocks do not sit on
  // the SMs beside these for the whole scan
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
  const int g = h / (H / G);
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(COLS, dv - col0);            // a multiple of 4
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += DF_THREADS)
      o_out[((size_t)(first + i / ncol) * H + h) * dv + col0 + i % ncol] = 0.f;
    return;
  }
  constexpr int DP = R * LANES;                      // a row of q or k in shared memory: d floats, then zeros
  constexpr int stage_floats = DF_CHUNK * (2 * DP + COLS + 4);
  if (d < DP)                                          // (cp.async never writes the padding)
    for (int i = tid; i < 2 * 2 * DF_CHUNK * (DP - d); i += DF_THREADS) {
      const int row = i / (DP - d), c = i - row * (DP - d);          // row: stage, q or k, token
      smem[(row / (2 * DF_CHUNK)) * stage_floats + (row % (2 * DF_CHUNK)) * DP + d + c] = 0.f;
    }
  const int cl = tid / LANES, part = tid % LANES;
  const bool live = cl < ncol;
  const int col = col0 + (live ? cl : 0);
  float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + col) * d;
  f32x2 S[R / 2];                                      // rows 4c, 4c+1 | 4c+2, 4c+3 of the lane's groups of four
  const bool fresh = q_start[s] == 0;
  const bool st_vec = ((uintptr_t)st % 16) == 0;       // d is a multiple of 4: then every group of 4 rows is 16-byte aligned
#pragma unroll
  for (int j = 0; j < R / 4; ++j) {
    const int i = 4 * (part + LANES * j);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && !fresh && i < d) {
      if (st_vec) v = *reinterpret_cast<const float4*>(st + i);
      else v = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
    }
    S[2 * j] = f2_pack(v.x, v.y);
    S[2 * j + 1] = f2_pack(v.z, v.w);
  }

  auto fetch = [&](int c0, int stage) {
    float* qs = smem + stage * stage_floats;           // [CHUNK][DP]
    float* ks = qs + DF_CHUNK * DP;                    // [CHUNK][DP]
    float* vs = ks + DF_CHUNK * DP;                    // [CHUNK][COLS]
    float* sc = vs + DF_CHUNK * COLS;               // [CHUNK][4]: decay, beta, k . q
    const int cn = min(DF_CHUNK, n - c0);
    const int d4 = d >> 2, c4 = ncol >> 2;
    for (int i = tid; i < cn * d4; i += DF_THREADS) {
      const int tt = i / d4, c = i - tt * d4;
      const size_t row = ((size_t)(first + c0 + tt) * G + g) * d + 4 * c;
      cp_async16(qs + tt * DP + 4 * c, qn + row);
      cp_async16(ks + tt * DP + 4 * c, kn + row);
    }
    for (int i = tid; i < cn * c4; i += DF_THREADS) {
      const int tt = i / c4, c = i - tt * c4;
      cp_async16(vs + tt * COLS + 4 * c, v32 + (size_t)(first + c0 + tt) * v_stride + h * dv + col0 + 4 * c);
    }
    for (int i = tid; i < cn * 3; i += DF_THREADS) {
      const int tt = i / 3, w = i - tt * 3;
      const size_t tok = first + c0 + tt;
      cp_async4(sc + tt * 4 + w, w == 0 ? decay + tok * H + h : (w == 1 ? beta + tok * H + h : kq + tok * G + g));
    }
  };

  const int n_chunks = (n + DF_CHUNK - 1) / DF_CHUNK;
  if (n_chunks > 0) fetch(0, 0);
  cp_async_commit();
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int c0 = ci * DF_CHUNK, stage = ci & 1;
    if (ci + 1 < n_chunks) fetch(c0 + DF_CHUNK, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* qs = smem + stage * stage_floats + 4 * part;
    const float* ks = qs + DF_CHUNK * DP;
    const float* vs = smem + stage * stage_floats + 2 * DF_CHUNK * DP;
    const float* sc = vs + DF_CHUNK * COLS;
    const int cn = min(DF_CHUNK, n - c0);
    // a token's k, q, v and scalars are read from shared memory one token ahead, so that the reads are under
    // way while the token before goes through its shuffles
    ulonglong2 kk[R / 4], qq[R / 4], kk_n[R / 4], qq_n[R / 4];      // four floats as two pairs
    float4 sc_n = *reinterpret_cast<const float4*>(sc);
    float v_n = live ? vs[cl] : 0.f;
#pragma unroll
    for (int j = 0; j < R / 4; ++j) {
      kk_n[j] = *reinterpret_cast<const ulonglong2*>(ks + 4 * LANES * j);
      qq_n[j] = *reinterpret_cast<const ulonglong2*>(qs + 4 * LANES * j);
    }
    for (int tt = 0; tt < cn; ++tt) {
      const float gt = sc_n.x, bt = sc_n.y, kqt = sc_n.z, vt = v_n;
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        kk[j] = kk_n[j];
        qq[j] = qq_n[j];
      }
      {
        const int tn = min(tt + 1, DF_CHUNK - 1);      // (the row behind the last token of a short chunk holds old data: read, not used)
        sc_n = *reinterpret_cast<const float4*>(sc + tn * 4);
        v_n = live ? vs[tn * COLS + cl] : 0.f;
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          kk_n[j] = *reinterpret_cast<const ulonglong2*>(ks + tn * DP + 4 * LANES * j);
          qq_n[j] = *reinterpret_cast<const ulonglong2*>(qs + tn * DP + 4 * LANES * j);
        }
      }
      f32x2 ak[2] = {0ull, 0ull}, aq[2] = {0ull, 0ull};
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        ak[0] = f2_fma(S[2 * j], kk[j].x, ak[0]);     aq[0] = f2_fma(S[2 * j], qq[j].x, aq[0]);
        ak[1] = f2_fma(S[2 * j + 1], kk[j].y, ak[1]); aq[1] = f2_fma(S[2 * j + 1], qq[j].y, aq[1]);
      }
      float sk = f2_sum(ak[0], ak[1]), sq = f2_sum(aq[0], aq[1]);
      {
        // two sums over the column's lanes for the price of one: neighbours swap, so that even lanes go on with
        // S . k and odd lanes with S . q; at the end they swap back
        const bool odd = part & 1;
        float mine = odd ? sq : sk;
        mine += __shfl_xor_sync(0xffffffffu, odd ? sk : sq, 1);
#pragma unroll
        for (int off = 2; off < LANES; off <<= 1) mine += __shfl_xor_sync(0xffffffffu, mine, off);
        const float theirs = __shfl_xor_sync(0xffffffffu, mine, 1);
        sk = odd ? theirs : mine;
        sq = odd ? mine : theirs;
      }
      const float u = bt * (vt - gt * sk);
      const f32x2 uu = f2_pack(u, u), gg = f2_pack(gt, gt);
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        S[2 * j] = f2_fma(kk[j].x, uu, f2_mul(S[2 * j], gg));
        S[2 * j + 1] = f2_fma(kk[j].y, uu, f2_mul(S[2 * j + 1], gg));
      }
      if (live && part == 0) o_out[((size_t)(first + c0 + tt) * H + h) * dv + col] = fmaf(u, kqt, gt * sq);
    }
    __syncthreads();                                   // the stage is free for the fetch after next
  }
  cp_async_wait<0>();
  pdl_launch_dependents();
  if (live) {
#pragma unroll
    for (int j = 0; j < R / 4; ++j) {
      const int i = 4 * (part + LANES * j);
      if (i < d) {
        float4 v;
        f2_unpack(S[2 * j], v.x, v.y);
        f2_unpack(S[2 * j + 1], v.z, v.w);
        if (st_vec) {
          *reinterpret_cast<float4*>(st + i) = v;
        } else {
          st[i] = v.x; st[i + 1] = v.y; st[i + 2] = v.z; st[i + 3] = v.w;
        }
      }
    }
  }
}


// ---------------------------------------------------------------- four tokens per step of the chain
// For one long request the scan above is a chain of tokens: every token waits for the sums over the state, their
// shuffles and the write of the token before.  Four tokens can share one such round.  With s0 the column before the
// four, gam_i = g_1 .. g_i and D(m, i) = g_(m+1) .. g_i:
//   u_i = beta_i (v_i - gam_i (s0 . k_i) - sum_{m < i} D(m, i) (k_m . k_i) u_m)
//   o_i = gam_i (s0 . q_i) + sum_{m <= i} D(m, i) (k_m . q_i) u_m
//   s4  = gam_4 s0 + sum_m D(m, 4) u_m k_m
// which is the same recurrence written out (g_i s_(i-1) = gam_i s0 + sum_{m < i} D(m, i) u_m k_m).  The eight sums
// over s0 are independent and go through the shuffles together; the products between tokens (k_m . k_i, k_m . q_i
// for neighbours up to three apart) come from delta_pairs_kernel; what is left of the chain are a few scalar
// operations per token.  The sums are taken in another order than token by token, so results agree with the
// plain scan to rounding, not to the bit; groups of four start at the first token of the step's portion.

// pairs [T, G, 8]: k_t . k_(t-1), k_t . k_(t-2), k_t . k_(t-3), k_t . q_t, k_(t-1) . q_t, k_(t-2) . q_t, k_(t-3) . q_t, 0
// (over the packed tokens; a neighbour before the array's start counts as zero, one of another request is never used)
__global__ void delta_pairs_kernel(float* __restrict__ pairs, const float* __restrict__ qn, const float* __restrict__ kn,
                                   int n_tokens, int G, int d) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long)n_tokens * G) return;
  const int t = (int)(item / G), g = (int)(item % G);
  const float* kt = kn + (size_t)item * d;
  const float* qt = qn + (size_t)item * d;
  float acc[7] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int c = lane; c < d; c += 32) {
    const float k0 = kt[c], q0 = qt[c];
    acc[3] = fmaf(k0, q0, acc[3]);
#pragma unroll
    for (int j = 1; j <= 3; ++j)
      if (t - j >= 0) {
        const float kj = kn[((size_t)(t - j) * G + g) * d + c];
        acc[j - 1] = fmaf(k0, kj, acc[j - 1]);
        acc[3 + j] = fmaf(kj, q0, acc[3 + j]);
      }
  }
#pragma unroll
  for (int j = 0; j < 7; ++j) acc[j] = warp_sum(acc[j]);
  if (lane < 8) {
    float v = 0.f;
#pragma unroll
    for (int j = 0; j < 7; ++j) v = lane == j ? acc[j] : v;
    pairs[(size_t)item * 8 + lane] = v;
  }
}

constexpr int DB_LANES = 8;
constexpr int DB_COLS = DF_THREADS / DB_LANES;

template <int R>
__global__ void __launch_bounds__(DF_THREADS) delta_scan_block4_kernel(
    float* __restrict__ o_out, const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ pairs,
    const float* __restrict__ v32, int v_stride, const float* __restrict__ beta, const float* __restrict__ decay,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int G, int H, int d, int dv) {
  constexpr int LANES = DB_LANES, COLS = DB_COLS;
  extern __shared__ __align__(16) float smem[];
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
  const int g = h / (H / G);
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(COLS, dv - col0);               // a multiple of 4
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += DF_THREADS)
      o_out[((size_t)(first + i / ncol) * H + h) * dv + col0 + i % ncol] = 0.f;
    return;
  }
  constexpr int DP = R * LANES;                        // a row of q or k in shared memory: d floats, then zeros
  constexpr int stage_floats = DF_CHUNK * (2 * DP + COLS + 4 + 8);
  if (d < DP)                                          // (cp.async never writes the padding)
    for (int i = tid; i < 2 * 2 * DF_CHUNK * (DP - d); i += DF_THREADS) {
      const int row = i / (DP - d), c = i - row * (DP - d);          // row: stage, q or k, token
      smem[(row / (2 * DF_CHUNK)) * stage_floats + (row % (2 * DF_CHUNK)) * DP + d + c] = 0.f;
    }
  const int cl = tid / LANES, part = tid % LANES;
  const bool live = cl < ncol;
  const int col = col0 + (live ? cl : 0);
  float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + col) * d;
  f32x2 S[R / 2];
  const bool fresh = q_start[s] == 0;
  const bool st_vec = ((uintptr_t)st % 16) == 0;
#pragma unroll
  for (int j = 0; j < R / 4; ++j) {
    const int i = 4 * (part + LANES * j);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && !fresh && i < d) {
      if (st_vec) v = *reinterpret_cast<const float4*>(st + i);
      else v = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
    }
    S[2 * j] = f2_pack(v.x, v.y);
    S[2 * j + 1] = f2_pack(v.z, v.w);
  }

  auto fetch = [&](int c0, int stage) {
    float* qs = smem + stage * stage_floats;           // [CHUNK][DP]
    float* ks = qs + DF_CHUNK * DP;                    // [CHUNK][DP]
    float* vs = ks + DF_CHUNK * DP;                    // [CHUNK][COLS]
    float* sc = vs + DF_CHUNK * COLS;                  // [CHUNK][4]: decay, beta
    float* pr = sc + DF_CHUNK * 4;                     // [CHUNK][8]: products between neighbouring tokens
    const int cn = min(DF_CHUNK, n - c0);
    const int d4 = d >> 2, c4 = ncol >> 2;
    for (int i = tid; i < cn * d4; i += DF_THREADS) {
      const int tt = i / d4, c = i - tt * d4;
      const size_t row = ((size_t)(first + c0 + tt) * G + g) * d + 4 * c;
      cp_async16(qs + tt * DP + 4 * c, qn + row);
      cp_async16(ks + tt * DP + 4 * c, kn + row);
    }
    for (int i = tid; i < cn * c4; i += DF_THREADS) {
      const int tt = i / c4, c = i - tt * c4;
      cp_async16(vs + tt * COLS + 4 * c, v32 + (size_t)(first + c0 + tt) * v_stride + h * dv + col0 + 4 * c);
    }
    for (int i = tid; i < cn * 2; i += DF_THREADS) {
      const int tt = i >> 1, w = i & 1;
      const size_t tok = first + c0 + tt;
      cp_async4(sc + tt * 4 + w, w == 0 ? decay + tok * H + h : beta + tok * H + h);
      cp_async16(pr + tt * 8 + 4 * w, pairs + (tok * G + g) * 8 + 4 * w);
    }
    // the tokens that fill the last group of four: no decay, no write, nothing read
    const int pad_end = min(DF_CHUNK, (cn + 3) & ~3);
    for (int i = tid; i < (pad_end - cn) * DP; i += DF_THREADS) {
      const int tt = cn + i / DP, c = i % DP;
      qs[tt * DP + c] = 0.f;
      ks[tt * DP + c] = 0.f;
    }
    for (int i = tid; i < (pad_end - cn) * 16; i += DF_THREADS) {
      const int tt = cn + i / 16, c = i % 16;
      if (c < 8) pr[tt * 8 + c] = 0.f;
      else if (c < 12) sc[tt * 4 + (c - 8)] = c == 8 ? 1.f : 0.f;
    }
    for (int i = tid; i < (pad_end - cn) * COLS; i += DF_THREADS) vs[cn * COLS + i] = 0.f;
  };

  const int n_chunks = (n + DF_CHUNK - 1) / DF_CHUNK;
  if (n_chunks > 0) fetch(0, 0);
  cp_async_commit();
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int c0 = ci * DF_CHUNK, stage = ci & 1;
    if (ci + 1 < n_chunks) fetch(c0 + DF_CHUNK, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* qs = smem + stage * stage_floats + 4 * part;
    const float* ks = qs + DF_CHUNK * DP;
    const float* vs = smem + stage * stage_floats + 2 * DF_CHUNK * DP;
    const float* sc = vs + DF_CHUNK * COLS;
    const float* pr = sc + DF_CHUNK * 4;
    const int cn = min(DF_CHUNK, n - c0);
    for (int t0 = 0; t0 < cn; t0 += 4) {
      // the eight sums over the column as it stands before these four tokens
      float r[4], p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f32x2 a0 = 0ull, a1 = 0ull, b0 = 0ull, b1 = 0ull;
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          const ulonglong2 kk = *reinterpret_cast<const ulonglong2*>(ks + (t0 + i) * DP + 4 * LANES * j);
          const ulonglong2 qq = *reinterpret_cast<const ulonglong2*>(qs + (t0 + i) * DP + 4 * LANES * j);
          a0 = f2_fma(S[2 * j], kk.x, a0);     b0 = f2_fma(S[2 * j], qq.x, b0);
          a1 = f2_fma(S[2 * j + 1], kk.y, a1); b1 = f2_fma(S[2 * j + 1], qq.y, b1);
        }
        r[i] = f2_sum(a0, a1);
        p[i] = f2_sum(b0, b1);
      }
#pragma unroll
      for (int off = 1; off < LANES; off <<= 1)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          r[i] += __shfl_xor_sync(0xffffffffu, r[i], off);
          p[i] += __shfl_xor_sync(0xffffffffu, p[i], off);
        }
      // scalars of the four tokens (off the chain: they do not depend on the state)
      float gd[4], be[4], vv[4], K[4][3], Q[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 c4v = *reinterpret_cast<const float4*>(sc + (t0 + i) * 4);
        const float4 pa = *reinterpret_cast<const float4*>(pr + (t0 + i) * 8);
        const float4 pb = *reinterpret_cast<const float4*>(pr + (t0 + i) * 8 + 4);
        gd[i] = c4v.x; be[i] = c4v.y;
        vv[i] = live ? vs[(t0 + i) * COLS + cl] : 0.f;
        K[i][0] = pa.x; K[i][1] = pa.y; K[i][2] = pa.z;          // k_i . k_(i-1), k_(i-2), k_(i-3)
        Q[i][0] = pa.w; Q[i][1] = pb.x; Q[i][2] = pb.y; Q[i][3] = pb.z;   // k_i, k_(i-1), k_(i-2), k_(i-3) . q_i
      }
      const float gam0 = gd[0], gam1 = gam0 * gd[1], gam2 = gam1 * gd[2], gam3 = gam2 * gd[3];
      const float D01 = gd[1], D02 = gd[1] * gd[2], D03 = D02 * gd[3], D12 = gd[2], D13 = gd[2] * gd[3], D23 = gd[3];
      const float u0 = be[0] * (vv[0] - gam0 * r[0]);
      const float u1 = be[1] * (vv[1] - gam1 * r[1] - D01 * K[1][0] * u0);
      const float u2 = be[2] * (vv[2] - gam2 * r[2] - D02 * K[2][1] * u0 - D12 * K[2][0] * u1);
      const float u3 = be[3] * (vv[3] - gam3 * r[3] - D03 * K[3][2] * u0 - D13 * K[3][1] * u1 - D23 * K[3][0] * u2);
      const float o0 = gam0 * p[0] + Q[0][0] * u0;
      const float o1 = gam1 * p[1] + D01 * Q[1][1] * u0 + Q[1][0] * u1;
      const float o2 = gam2 * p[2] + D02 * Q[2][2] * u0 + D12 * Q[2][1] * u1 + Q[2][0] * u2;
      const float o3 = gam3 * p[3] + D03 * Q[3][3] * u0 + D13 * Q[3][2] * u1 + D23 * Q[3][1] * u2 + Q[3][0] * u3;
      if (live && part < 4 && t0 + part < cn) {
        const float o = part == 0 ? o0 : (part == 1 ? o1 : (part == 2 ? o2 : o3));
        o_out[((size_t)(first + c0 + t0 + part) * H + h) * dv + col] = o;
      }
      // the column after the four: gam3 s0 + sum_m D(m, 3) u_m k_m
      const f32x2 gg = f2_pack(gam3, gam3);
      const f32x2 e0 = f2_pack(D03 * u0, D03 * u0), e1 = f2_pack(D13 * u1, D13 * u1), e2 = f2_pack(D23 * u2, D23 * u2),
                  e3 = f2_pack(u3, u3);
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const ulonglong2 k0 = *reinterpret_cast<const ulonglong2*>(ks + (t0 + 0) * DP + 4 * LANES * j);
        const ulonglong2 k1 = *reinterpret_cast<const ulonglong2*>(ks + (t0 + 1) * DP + 4 * LANES * j);
        const ulonglong2 k2 = *reinterpret_cast<const ulonglong2*>(ks + (t0 + 2) * DP + 4 * LANES * j);
        const ulonglong2 k3 = *reinterpret_cast<const ulonglong2*>(ks + (t0 + 3) * DP + 4 * LANES * j);
        S[2 * j] = f2_fma(k3.x, e3, f2_fma(k2.x, e2, f2_fma(k1.x, e1, f2_fma(k0.x, e0, f2_mul(S[2 * j], gg)))));
        S[2 * j + 1] = f2_fma(k3.y, e3, f2_fma(k2.y, e2, f2_fma(k1.y, e1, f2_fma(k0.y, e0, f2_mul(S[2 * j + 1], gg)))));
      }
    }
    __syncthreads();                                   // the stage is free for the fetch after next
  }
  cp_async_wait<0>();
  pdl_launch_dependents();
  if (live) {
#pragma unroll
    for (int j = 0; j < R / 4; ++j) {
      const int i = 4 * (part + LANES * j);
      if (i < d) {
        float4 v;
        f2_unpack(S[2 * j], v.x, v.y);
        f2_unpack(S[2 * j + 1], v.z, v.w);
        if (st_vec) {
          *reinterpret_cast<float4*>(st + i) = v;
        } else {
          st[i] = v.x; st[i + 1] = v.y; st[i + 2] = v.z; st[i + 3] = v.w;
        }
      }
    }
  }
}


// ---------------------------------------------------------------- several columns per lane
// The same scan, token by token in the same order per column (the same bits), with CPT columns of the state in
// each lane: a lane's rows of k and q, read once from shared memory, serve all its columns, and the columns' chains
// run side by side in one warp.  A block holds 16 * CPT columns (column c of a lane is 16 * c to the right).
template <int R, int CPT>
__global__ void __launch_bounds__(DF_THREADS) delta_scan_wide_kernel(
    float* __restrict__ o_out, const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ kq,
    const float* __restrict__ v32, int v_stride, const float* __restrict__ beta, const float* __restrict__ decay,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int G, int H, int d, int dv) {
  constexpr int LANES = 8, NTC = DF_THREADS / LANES, COLS = NTC * CPT;
  extern __shared__ __align__(16) float smem[];
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
  const int g = h / (H / G);
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(COLS, dv - col0);               // a multiple of 4
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += DF_THREADS)
      o_out[((size_t)(first + i / ncol) * H + h) * dv + col0 + i % ncol] = 0.f;
    return;
  }
  constexpr int DP = R * LANES;
  constexpr int stage_floats = DF_CHUNK * (2 * DP + COLS + 4);
  if (d < DP)
    for (int i = tid; i < 2 * 2 * DF_CHUNK * (DP - d); i += DF_THREADS) {
      const int row = i / (DP - d), c = i - row * (DP - d);
      smem[(row / (2 * DF_CHUNK)) * stage_floats + (row % (2 * DF_CHUNK)) * DP + d + c] = 0.f;
    }
  const int cl = tid / LANES, part = tid % LANES;
  bool live[CPT];
  float* st[CPT];
  f32x2 S[CPT][R / 2];
  const bool fresh = q_start[s] == 0;
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    live[c] = cl + NTC * c < ncol;
    st[c] = state + (size_t)slot * state_stride + ((size_t)h * dv + col0 + (live[c] ? cl + NTC * c : 0)) * d;
#pragma unroll
    for (int j = 0; j < R / 4; ++j) {
      const int i = 4 * (part + LANES * j);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live[c] && !fresh && i < d) v = make_float4(st[c][i], st[c][i + 1], st[c][i + 2], st[c][i + 3]);
      S[c][2 * j] = f2_pack(v.x, v.y);
      S[c][2 * j + 1] = f2_pack(v.z, v.w);
    }
  }

  auto fetch = [&](int c0, int stage) {
    float* qs = smem + stage * stage_floats;           // [CHUNK][DP]
    float* ks = qs + DF_CHUNK * DP;                    // [CHUNK][DP]
    float* vs = ks + DF_CHUNK * DP;                    // [CHUNK][COLS]
    float* sc = vs + DF_CHUNK * COLS;                  // [CHUNK][4]: decay, beta, k . q
    const int cn = min(DF_CHUNK, n - c0);
    const int d4 = d >> 2, c4 = ncol >> 2;
    for (int i = tid; i < cn * d4; i += DF_THREADS) {
      const int tt = i / d4, c = i - tt * d4;
      const size_t row = ((size_t)(first + c0 + tt) * G + g) * d + 4 * c;
      cp_async16(qs + tt * DP + 4 * c, qn + row);
      cp_async16(ks + tt * DP + 4 * c, kn + row);
    }
    for (int i = tid; i < cn * c4; i += DF_THREADS) {
      const int tt = i / c4, c = i - tt * c4;
      cp_async16(vs + tt * COLS + 4 * c, v32 + (size_t)(first + c0 + tt) * v_stride + h * dv + col0 + 4 * c);
    }
    for (int i = tid; i < cn * 3; i += DF_THREADS) {
      const int tt = i / 3, w = i - tt * 3;
      const size_t tok = first + c0 + tt;
      cp_async4(sc + tt * 4 + w, w == 0 ? decay + tok * H + h : (w == 1 ? beta + tok * H + h : kq + tok * G + g));
    }
  };

  const int n_chunks = (n + DF_CHUNK - 1) / DF_CHUNK;
  if (n_chunks > 0) fetch(0, 0);
  cp_async_commit();
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int c0 = ci * DF_CHUNK, stage = ci & 1;
    if (ci + 1 < n_chunks) fetch(c0 + DF_CHUNK, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* qs = smem + stage * stage_floats + 4 * part;
    const float* ks = qs + DF_CHUNK * DP;
    const float* vs = smem + stage * stage_floats + 2 * DF_CHUNK * DP;
    const float* sc = vs + DF_CHUNK * COLS;
    const int cn = min(DF_CHUNK, n - c0);
    for (int tt = 0; tt < cn; ++tt) {
      const float4 scv = *reinterpret_cast<const float4*>(sc + tt * 4);
      const float gt = scv.x, bt = scv.y, kqt = scv.z;
      ulonglong2 kk[R / 4], qq[R / 4];
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        kk[j] = *reinterpret_cast<const ulonglong2*>(ks + tt * DP + 4 * LANES * j);
        qq[j] = *reinterpret_cast<const ulonglong2*>(qs + tt * DP + 4 * LANES * j);
      }
      float sk[CPT], sq[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        f32x2 ak[2] = {0ull, 0ull}, aq[2] = {0ull, 0ull};
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          ak[0] = f2_fma(S[c][2 * j], kk[j].x, ak[0]);     aq[0] = f2_fma(S[c][2 * j], qq[j].x, aq[0]);
          ak[1] = f2_fma(S[c][2 * j + 1], kk[j].y, ak[1]); aq[1] = f2_fma(S[c][2 * j + 1], qq[j].y, aq[1]);
        }
        sk[c] = f2_sum(ak[0], ak[1]);
        sq[c] = f2_sum(aq[0], aq[1]);
      }
      const bool odd = part & 1;
      float mine[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) mine[c] = (odd ? sq[c] : sk[c]) + __shfl_xor_sync(0xffffffffu, odd ? sk[c] : sq[c], 1);
#pragma unroll
      for (int off = 2; off < LANES; off <<= 1)
#pragma unroll
        for (int c = 0; c < CPT; ++c) mine[c] += __shfl_xor_sync(0xffffffffu, mine[c], off);
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const float theirs = __shfl_xor_sync(0xffffffffu, mine[c], 1);
        const float skc = odd ? theirs : mine[c], sqc = odd ? mine[c] : theirs;
        const float u = bt * ((live[c] ? vs[tt * COLS + cl + NTC * c] : 0.f) - gt * skc);
        const f32x2 uu = f2_pack(u, u), gg = f2_pack(gt, gt);
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          S[c][2 * j] = f2_fma(kk[j].x, uu, f2_mul(S[c][2 * j], gg));
          S[c][2 * j + 1] = f2_fma(kk[j].y, uu, f2_mul(S[c][2 * j + 1], gg));
        }
        if (live[c] && part == 0)
          o_out[((size_t)(first + c0 + tt) * H + h) * dv + col0 + cl + NTC * c] = fmaf(u, kqt, gt * sqc);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  pdl_launch_dependents();
#pragma unroll
  for (int c = 0; c < CPT; ++c)
    if (live[c]) {
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const int i = 4 * (part + LANES * j);
        if (i < d) {
          float4 v;
          f2_unpack(S[c][2 * j], v.x, v.y);
          f2_unpack(S[c][2 * j + 1], v.z, v.w);
          st[c][i] = v.x; st[c][i + 1] = v.y; st[c][i + 2] = v.z; st[c][i + 3] = v.w;
        }
      }
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

// o_out [T, H, dv] fp32.  lanes: 4, 8, 16 or 32 lanes per column of the state, or 0 for the kernel's own choice.
// group4: 1 takes four tokens per round of the chain (needs pairs [T, G, 8] as scratch), 0 one, -1 chooses by the
// size of the step.  cpt: 2 or 4 columns of the state per lane (8 lanes a column, d up to 128), 1 one, 0 the
// kernel's choice.
// Scratch given by the caller, all fp32: qn, kn [T, G, d]; kq [T, G]; v32 [T, H, dv]; beta,
// decay [T, H].
NHV_API int nhv_delta_rule(int dtype, float* o_out, const void* qkv, int qkv_stride, const float* ba,
                           const float* a_log, const float* dt_bias, float* state, long state_stride, float* qn,
                           float* kn, float* kq, float* v32, float* beta, float* decay, const int* cu_q,
                           const int* q_start, const int* slots, int n_seqs, int n_tokens, int G, int H, int d, int dv,
                           int lanes, int group4, float* pairs, int cpt, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(G > 0 && H > 0 && H % G == 0, "delta_rule: %d heads do not divide into %d q/k heads", H, G);
  NHV_REQUIRE(d > 0 && d <= 256 && dv > 0, "delta_rule: a q/k head of %d is beyond the supported 256", d);
  NHV_REQUIRE(state_stride >= (long)H * d * dv, "delta_rule: the state holds fewer than heads * d * dv floats");
  const bool fast = d % 4 == 0 && dv % 4 == 0;
  // values that are fp32 already are read where they lie (16-byte pieces: the rows' stride and start in steps of 4)
  const bool v_in_place = fast && dtype == NHV_F32 && qkv_stride % 4 == 0 && ((uintptr_t)qkv % 16) == 0;
  const float* v_src = v_in_place ? (const float*)qkv + 2 * G * d : v32;
  const int v_stride = v_in_place ? qkv_stride : H * dv;
  const long work = (long)n_tokens * (H * dv > 32 * G ? H * dv : 32 * G);
  const int prep_blocks = (int)(work / 256 + 1 < 148 * 8 ? work / 256 + 1 : 148 * 8);
  const int v_off = 2 * G * d;
#define PREP(T)                                                                                                      \
  nhv_launch(delta_prepare_kernel<T>, prep_blocks, 256, 0, stream, qn, kn, kq, fast && !v_in_place ? v32 : (float*)nullptr, beta, \
             decay, (const T*)qkv, qkv_stride, ba, a_log, dt_bias, n_tokens, G, H, d, dv)
  if (dtype == NHV_F32) PREP(float);
  else if (dtype == NHV_BF16) PREP(__nv_bfloat16);
  else NHV_REQUIRE(false, "delta_rule: unknown dtype %d", dtype);
#undef PREP
  // four tokens per round of the chain: 225 against 252 ns a token for one 4,096-token request (16 heads, d = dv =
  // 128), the same at 4 or more requests.  Too little to give up sums in one fixed order for: off unless asked for.
  if (group4 < 0) group4 = 0;
  // columns per lane: one while the blocks of 16 columns leave SMs idle (one or two long requests: 259 ns a token
  // against 265 and 347 with 2 and 4 columns), more when the SMs are full and reads of k and q from shared memory
  // are what costs (8 requests of 512 tokens: 878, 673, 604 ns per token-step; 64 single tokens: 36, 32, 31 µs)
  if (cpt <= 0) {
    const long blocks16 = (long)n_seqs * H * ((dv + 15) / 16);
    if (n_tokens >= 8 * (long)n_seqs) cpt = blocks16 <= 2 * 148 ? 1 : (blocks16 <= 6 * 148 ? 2 : 4);
    else cpt = blocks16 >= 16 * 148 ? 4 : (blocks16 >= 8 * 148 ? 2 : 1);     // single tokens: the states stream in and out, and many small blocks keep more reads in flight
  }
  if (fast && group4 && pairs) {
    const long items = (long)n_tokens * G;
    nhv_launch(delta_pairs_kernel, (int)((items + 7) / 8), 256, 0, stream, pairs, (const float*)qn, (const float*)kn,
               n_tokens, G, d);
    dim3 grid(n_seqs, H, (dv + DB_COLS - 1) / DB_COLS);
    const int need = (d + DB_LANES - 1) / DB_LANES;
#define BLOCK4(R)                                                                                                    \
  do {                                                                                                               \
    static bool attr = false;                                                                                        \
    if (!attr) {                                                                                                     \
      NHV_CUDA(cudaFuncSetAttribute(delta_scan_block4_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                    232448), "delta_rule");                                                          \
      attr = true;                                                                                                   \
    }                                                                                                                \
    nhv_launch(delta_scan_block4_kernel<R>, grid, DF_THREADS,                                                        \
               nhv_spread_smem((size_t)2 * DF_CHUNK * (2 * R * DB_LANES + DB_COLS + 12) * sizeof(float),             \
                               (long)grid.x * grid.y * grid.z), stream,                                             \
               o_out, (const float*)qn, (const float*)kn, (const float*)pairs, v_src, v_stride, (const float*)beta, \
               (const float*)decay, state, state_stride, cu_q, q_start, slots, G, H, d, dv);                        \
  } while (0)
    if (need <= 4) BLOCK4(4);
    else if (need <= 8) BLOCK4(8);
    else if (need <= 16) BLOCK4(16);
    else BLOCK4(32);
#undef BLOCK4
  } else if (fast && cpt > 1 && d <= 128 && (lanes == 0 || lanes == 8)) {
    if (cpt != 2) cpt = 4;
    const int cols = 16 * cpt;
    dim3 grid(n_seqs, H, (dv + cols - 1) / cols);
    const int need = (d + 7) / 8;
#define WIDE(R, C)                                                                                                   \
  do {                                                                                                               \
    static bool attr = false;                                                                                        \
    if (!attr) {                                                                                                     \
      NHV_CUDA(cudaFuncSetAttribute(delta_scan_wide_kernel<R, C>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                    232448), "delta_rule");                                                          \
      attr = true;                                                                                                   \
    }                                                                                                                \
    nhv_launch(delta_scan_wide_kernel<R, C>, grid, DF_THREADS,                                                       \
               nhv_spread_smem((size_t)2 * DF_CHUNK * (2 * R * 8 + 16 * C + 4) * sizeof(float),                      \
                               (long)grid.x * grid.y * grid.z), stream,                                             \
               o_out, (const float*)qn, (const float*)kn, (const float*)kq, v_src, v_stride, (const float*)beta,    \
               (const float*)decay, state, state_stride, cu_q, q_start, slots, G, H, d, dv);                        \
  } while (0)
#define WIDE_C(C)                          \
  do {                                     \
    if (need <= 4) WIDE(4, C);             \
    else if (need <= 8) WIDE(8, C);        \
    else WIDE(16, C);                      \
  } while (0)
    if (cpt == 2) WIDE_C(2);
    else WIDE_C(4);
#undef WIDE_C
#undef WIDE
  } else if (fast) {
    // lanes per column: 8 measured fastest for one long request (244 ns a token against 254 with 16 lanes and 299
    // with 32: the shuffle rounds of the sum over lanes are the longest stretch of a token's chain) and for full
    // batches (fewest instructions in all); 16 and 32 stay for the tests
    if (lanes != 4 && lanes != 8 && lanes != 16 && lanes != 32) lanes = 8;
    if (lanes == 4 && d > 128) lanes = 8;                                    // 4 lanes hold at most 32 rows each
    const int cols = DF_THREADS / lanes;
    dim3 grid(n_seqs, H, (dv + cols - 1) / cols);
    const int need = (d + lanes - 1) / lanes;                                // rows per lane, then rounded up to 4, 8, 16, 32
#define FAST(R, L)                                                                                                   \
  do {                                                                                                               \
    static bool attr = false;                                                                                        \
    if (!attr) {                                                                                                     \
      NHV_CUDA(cudaFuncSetAttribute(delta_scan_fast_kernel<R, L>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                    232448), "delta_rule");                                                          \
      attr = true;                                                                                                   \
    }                                                                                                                \
    nhv_launch(delta_scan_fast_kernel<R, L>, grid, DF_THREADS,                                                       \
               nhv_spread_smem((size_t)2 * DF_CHUNK * (2 * R * L + DF_THREADS / L + 4) * sizeof(float),              \
                               (long)grid.x * grid.y * grid.z), stream,                                             \
               o_out, (const float*)qn, (const float*)kn, (const float*)kq, v_src, v_stride, (const float*)beta,    \
               (const float*)decay, state, state_stride, cu_q, q_start, slots, G, H, d, dv);                        \
  } while (0)
#define FAST_L(L)                          \
  do {                                     \
    if (need <= 4) FAST(4, L);             \
    else if (need <= 8) FAST(8, L);        \
    else if (need <= 16) FAST(16, L);      \
    else FAST(32, L);                      \
  } while (0)
    if (lanes == 4) FAST_L(4);
    else if (lanes == 8) FAST_L(8);
    else if (lanes == 16) {
      if (need <= 4) FAST(4, 16);
      else if (need <= 8) FAST(8, 16);
      else FAST(16, 16);
    } else {
      if (need <= 4) FAST(4, 32);
      else FAST(8, 32);
    }
#undef FAST_L
#undef FAST
  } else {
    const int rows = (d + DR_PARTS - 1) / DR_PARTS;
    const size_t smem = ((size_t)DR_CHUNK * (2 * d + DR_COLS) + 2 * DR_CHUNK) * sizeof(float);
    dim3 grid(n_seqs, H, (dv + DR_COLS - 1) / DR_COLS);
#define SCAN(T, R)                                                                                                  \
  nhv_launch(delta_scan_kernel<T, R>, grid, DR_COLS * DR_PARTS, smem, stream, o_out, (const float*)qn, (const float*)kn, \
             (const T*)qkv + v_off, qkv_stride, (const float*)beta, (const float*)decay, state, state_stride, cu_q, \
             q_start, slots, G, H, d, dv)
#define LAUNCH(T)                          \
  do {                                     \
    if (rows <= 8) SCAN(T, 8);             \
    else if (rows <= 16) SCAN(T, 16);      \
    else if (rows <= 32) SCAN(T, 32);      \
    else SCAN(T, 64);                      \
  } while (0)
    if (dtype == NHV_F32) LAUNCH(float);
    else LAUNCH(__nv_bfloat16);
#undef LAUNCH
#undef SCAN
  }
  NHV_CHECK_LAUNCH("delta_rule");
  return 0;
}
