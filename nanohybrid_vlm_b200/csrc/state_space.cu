// The state-space recurrence of Mamba-2 (scalar decay per head) over a packed step of several requests, and the
// gated RMS norm that follows it (also used behind the delta rule).
//
// Per head, with the state S [N, P] (fp32, carried per request), group gr of the head:
//   dt = softplus(dt_raw + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B_t x_t^T;  y_t = S^T C_t + D x_t
//
// ssd_scan_fast (fp32 inputs, sizes in steps of 4): the columns of S are independent of one another (column j:
// S_j <- a S_j + dt x_j B, y_j = S_j . C + D x_j), so a block takes (request, head, 16 columns) and a column lives
// in the registers of 8 lanes, each with N / 8 rows in groups of 4 (one 16-byte read of B and of C from shared
// memory serves 4 rows); the sum over rows ends with three shuffles.  Tokens reach shared memory by cp.async, 16 at
// a time, the next 16 while these are worked on; dt and the decay of the next 16 are computed meanwhile.
// ssd_scan (any size and type): 64 columns a block, 4 lanes a column, plain loads.
// The state of a slot is stored transposed, [head][P][N].  A request with q_start == 0 starts from
// zeros; one without a slot (slot < 0) is skipped and its outputs are cleared.
//
// gated_rmsnorm: rows of fp32 values y [T, n_groups * size], a gate z in the storage type, a weight w:
//   gate_first:  out = unit_rms(y * silu(z)) * w          (each group of `size` by its own root mean square)
//   else:        out = unit_rms(y) * w * silu(z)
// with w indexed by (column mod w_period).  gate_kind 1 puts sigmoid(z) in the place of silu(z).
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


// ---------------------------------------------------------------- the scan for fp32 inputs and sizes in steps of 4
constexpr int SF_CHUNK = 16;        // tokens per stage
constexpr int SF_THREADS = 128;     // LANES lanes per column of S (8, 16 or 32), 128 / LANES columns per block

__device__ __forceinline__ void ss_cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void ss_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N_> __device__ __forceinline__ void ss_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N_)); }

template <int R, int LANES>
__global__ void __launch_bounds__(SF_THREADS) ssd_scan_fast_kernel(
    float* __restrict__ y, const float* __restrict__ xbc, int xbc_stride, const float* __restrict__ dt_raw, int dt_stride,
    const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int H, int P, int N, int G) {
  constexpr int COLS = SF_THREADS / LANES;             // columns of S per block
  extern __shared__ __align__(16) float smem[];
  // a long kernel of few blocks: the kernel behind it is let in only at the end, so that its blocks do not sit on
  // the SMs beside these for the whole scan
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
  const int gr = h / (H / G);
  const int inner = H * P;
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(COLS, P - col0);             // a multiple of 4
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += SF_THREADS) y[(size_t)(first + i / ncol) * inner + h * P + col0 + i % ncol] = 0.f;
    return;
  }
  constexpr int NP = R * LANES;                      // a row of B or C in shared memory: N floats, then zeros
  constexpr int stage_floats = SF_CHUNK * (2 * NP + COLS + 2);
  if (N < NP)                                          // (cp.async never writes the padding)
    for (int i = tid; i < 2 * 2 * SF_CHUNK * (NP - N); i += SF_THREADS) {
      const int row = i / (NP - N), c = i - row * (NP - N);          // row: stage, B or C, token
      smem[(row / (2 * SF_CHUNK)) * stage_floats + (row % (2 * SF_CHUNK)) * NP + N + c] = 0.f;
    }
  const int cl = tid / LANES, part = tid % LANES;
  const bool live = cl < ncol;
  const int col = col0 + (live ? cl : 0);
  float* st = state + (size_t)slot * state_stride + ((size_t)h * P + col) * N;
  const float rate = expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];
  f32x2 S[R / 2];                                      // rows 4c, 4c+1 | 4c+2, 4c+3 of the lane's groups of four
  const bool fresh = q_start[s] == 0;
  const bool st_vec = ((uintptr_t)st % 16) == 0;       // N is a multiple of 4: then every group of 4 rows is 16-byte aligned
#pragma unroll
  for (int j = 0; j < R / 4; ++j) {
    const int i = 4 * (part + LANES * j);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && !fresh && i < N) {
      if (st_vec) v = *reinterpret_cast<const float4*>(st + i);
      else v = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
    }
    S[2 * j] = f2_pack(v.x, v.y);
    S[2 * j + 1] = f2_pack(v.z, v.w);
  }

  auto fetch = [&](int c0, int stage) {
    float* Bs = smem + stage * stage_floats;           // [CHUNK][NP]
    float* Cs = Bs + SF_CHUNK * NP;                    // [CHUNK][NP]
    float* xs = Cs + SF_CHUNK * NP;                    // [CHUNK][COLS]
    const int cn = min(SF_CHUNK, n - c0);
    const int n4 = N >> 2, c4 = ncol >> 2;
    for (int i = tid; i < cn * n4; i += SF_THREADS) {
      const int tt = i / n4, c = i - tt * n4;
      const float* row = xbc + (size_t)(first + c0 + tt) * xbc_stride + inner + gr * N + 4 * c;
      ss_cp_async16(Bs + tt * NP + 4 * c, row);
      ss_cp_async16(Cs + tt * NP + 4 * c, row + (size_t)G * N);
    }
    for (int i = tid; i < cn * c4; i += SF_THREADS) {
      const int tt = i / c4, c = i - tt * c4;
      ss_cp_async16(xs + tt * COLS + 4 * c, xbc + (size_t)(first + c0 + tt) * xbc_stride + h * P + col0 + 4 * c);
    }
  };

  const int n_chunks = (n + SF_CHUNK - 1) / SF_CHUNK;
  float dt_next = 0.f;                                 // thread tt < CHUNK: the raw dt of token tt of the chunk to come
  if (n_chunks > 0) {
    fetch(0, 0);
    if (tid < min(SF_CHUNK, n)) dt_next = dt_raw[(size_t)(first + tid) * dt_stride + h];
  }
  ss_cp_async_commit();
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int c0 = ci * SF_CHUNK, stage = ci & 1;
    const int cn = min(SF_CHUNK, n - c0);
    if (ci + 1 < n_chunks) fetch(c0 + SF_CHUNK, stage ^ 1);
    ss_cp_async_commit();
    float* ds = smem + stage * stage_floats + SF_CHUNK * (2 * NP + COLS);    // [CHUNK][2]: decay, dt
    if (tid < cn) {
      const float dt = ss_softplus(dt_next + bias);
      ds[2 * tid] = expf(-rate * dt);
      ds[2 * tid + 1] = dt;
    }
    ss_cp_async_wait<1>();
    __syncthreads();
    if (ci + 1 < n_chunks && tid < min(SF_CHUNK, n - c0 - SF_CHUNK))
      dt_next = dt_raw[(size_t)(first + c0 + SF_CHUNK + tid) * dt_stride + h];
    const float* Bs = smem + stage * stage_floats + 4 * part;
    const float* Cs = Bs + SF_CHUNK * NP;
    const float* xs = smem + stage * stage_floats + 2 * SF_CHUNK * NP;
#pragma unroll 2
    for (int tt = 0; tt < cn; ++tt) {
      const float a = ds[2 * tt], dt = ds[2 * tt + 1];
      const float xv = live ? xs[tt * COLS + cl] : 0.f;
      const float dx = dt * xv;
      const f32x2 aa = f2_pack(a, a), dd = f2_pack(dx, dx);
      f32x2 acc[2] = {0ull, 0ull};
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const ulonglong2 bb = *reinterpret_cast<const ulonglong2*>(Bs + tt * NP + 4 * LANES * j);   // four floats, two pairs
        const ulonglong2 cc = *reinterpret_cast<const ulonglong2*>(Cs + tt * NP + 4 * LANES * j);
        S[2 * j] = f2_fma(aa, S[2 * j], f2_mul(dd, bb.x));         acc[0] = f2_fma(S[2 * j], cc.x, acc[0]);
        S[2 * j + 1] = f2_fma(aa, S[2 * j + 1], f2_mul(dd, bb.y)); acc[1] = f2_fma(S[2 * j + 1], cc.y, acc[1]);
      }
      float sum = f2_sum(acc[0], acc[1]);
#pragma unroll
      for (int off = 1; off < LANES; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (live && part == 0) y[(size_t)(first + c0 + tt) * inner + h * P + col] = fmaf(skip, xv, sum);
    }
    __syncthreads();                                   // the stage is free for the fetch after next
  }
  ss_cp_async_wait<0>();
  pdl_launch_dependents();
  if (live) {
#pragma unroll
    for (int j = 0; j < R / 4; ++j) {
      const int i = 4 * (part + LANES * j);
      if (i < N) {
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

// The same scan with CPT columns of the state in each lane (8 lanes a column): a lane's rows of B and C, read once
// from shared memory, serve all its columns.  A block holds 16 * CPT columns (column c of a lane is 16 * c to the
// right).  Every column sees its tokens in the same order as above: the same bits.
template <int R, int CPT>
__global__ void __launch_bounds__(SF_THREADS) ssd_scan_wide_kernel(
    float* __restrict__ y, const float* __restrict__ xbc, int xbc_stride, const float* __restrict__ dt_raw, int dt_stride,
    const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
    float* __restrict__ state, long state_stride, const int* __restrict__ cu_q, const int* __restrict__ q_start,
    const int* __restrict__ slots, int H, int P, int N, int G) {
  constexpr int LANES = 8, NTC = SF_THREADS / LANES, COLS = NTC * CPT;
  extern __shared__ __align__(16) float smem[];
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * COLS;
  const int gr = h / (H / G);
  const int inner = H * P;
  const int first = cu_q[s], n = cu_q[s + 1] - first;
  const int slot = slots[s];
  const int tid = threadIdx.x;
  const int ncol = min(COLS, P - col0);                // a multiple of 4
  if (slot < 0) {
    for (int i = tid; i < n * ncol; i += SF_THREADS) y[(size_t)(first + i / ncol) * inner + h * P + col0 + i % ncol] = 0.f;
    return;
  }
  constexpr int NP = R * LANES;
  constexpr int stage_floats = SF_CHUNK * (2 * NP + COLS + 2);
  if (N < NP)
    for (int i = tid; i < 2 * 2 * SF_CHUNK * (NP - N); i += SF_THREADS) {
      const int row = i / (NP - N), c = i - row * (NP - N);
      smem[(row / (2 * SF_CHUNK)) * stage_floats + (row % (2 * SF_CHUNK)) * NP + N + c] = 0.f;
    }
  const int cl = tid / LANES, part = tid % LANES;
  const float rate = expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];
  bool live[CPT];
  float* st[CPT];
  f32x2 S[CPT][R / 2];
  const bool fresh = q_start[s] == 0;
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    live[c] = cl + NTC * c < ncol;
    st[c] = state + (size_t)slot * state_stride + ((size_t)h * P + col0 + (live[c] ? cl + NTC * c : 0)) * N;
#pragma unroll
    for (int j = 0; j < R / 4; ++j) {
      const int i = 4 * (part + LANES * j);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live[c] && !fresh && i < N) v = make_float4(st[c][i], st[c][i + 1], st[c][i + 2], st[c][i + 3]);
      S[c][2 * j] = f2_pack(v.x, v.y);
      S[c][2 * j + 1] = f2_pack(v.z, v.w);
    }
  }

  auto fetch = [&](int c0, int stage) {
    float* Bs = smem + stage * stage_floats;           // [CHUNK][NP]
    float* Cs = Bs + SF_CHUNK * NP;                    // [CHUNK][NP]
    float* xs = Cs + SF_CHUNK * NP;                    // [CHUNK][COLS]
    const int cn = min(SF_CHUNK, n - c0);
    const int n4 = N >> 2, c4 = ncol >> 2;
    for (int i = tid; i < cn * n4; i += SF_THREADS) {
      const int tt = i / n4, c = i - tt * n4;
      const float* row = xbc + (size_t)(first + c0 + tt) * xbc_stride + inner + gr * N + 4 * c;
      ss_cp_async16(Bs + tt * NP + 4 * c, row);
      ss_cp_async16(Cs + tt * NP + 4 * c, row + (size_t)G * N);
    }
    for (int i = tid; i < cn * c4; i += SF_THREADS) {
      const int tt = i / c4, c = i - tt * c4;
      ss_cp_async16(xs + tt * COLS + 4 * c, xbc + (size_t)(first + c0 + tt) * xbc_stride + h * P + col0 + 4 * c);
    }
  };

  const int n_chunks = (n + SF_CHUNK - 1) / SF_CHUNK;
  float dt_next = 0.f;
  if (n_chunks > 0) {
    fetch(0, 0);
    if (tid < min(SF_CHUNK, n)) dt_next = dt_raw[(size_t)(first + tid) * dt_stride + h];
  }
  ss_cp_async_commit();
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int c0 = ci * SF_CHUNK, stage = ci & 1;
    const int cn = min(SF_CHUNK, n - c0);
    if (ci + 1 < n_chunks) fetch(c0 + SF_CHUNK, stage ^ 1);
    ss_cp_async_commit();
    float* ds = smem + stage * stage_floats + SF_CHUNK * (2 * NP + COLS);      // [CHUNK][2]: decay, dt
    if (tid < cn) {
      const float dt = ss_softplus(dt_next + bias);
      ds[2 * tid] = expf(-rate * dt);
      ds[2 * tid + 1] = dt;
    }
    ss_cp_async_wait<1>();
    __syncthreads();
    if (ci + 1 < n_chunks && tid < min(SF_CHUNK, n - c0 - SF_CHUNK))
      dt_next = dt_raw[(size_t)(first + c0 + SF_CHUNK + tid) * dt_stride + h];
    const float* Bs = smem + stage * stage_floats + 4 * part;
    const float* Cs = Bs + SF_CHUNK * NP;
    const float* xs = smem + stage * stage_floats + 2 * SF_CHUNK * NP;
    for (int tt = 0; tt < cn; ++tt) {
      const float a = ds[2 * tt], dt = ds[2 * tt + 1];
      const f32x2 aa = f2_pack(a, a);
      ulonglong2 bb[R / 4], cc[R / 4];
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        bb[j] = *reinterpret_cast<const ulonglong2*>(Bs + tt * NP + 4 * LANES * j);
        cc[j] = *reinterpret_cast<const ulonglong2*>(Cs + tt * NP + 4 * LANES * j);
      }
      float sum[CPT], xv[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        xv[c] = live[c] ? xs[tt * COLS + cl + NTC * c] : 0.f;
        const float dx = dt * xv[c];
        const f32x2 dd = f2_pack(dx, dx);
        f32x2 acc[2] = {0ull, 0ull};
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          S[c][2 * j] = f2_fma(aa, S[c][2 * j], f2_mul(dd, bb[j].x));         acc[0] = f2_fma(S[c][2 * j], cc[j].x, acc[0]);
          S[c][2 * j + 1] = f2_fma(aa, S[c][2 * j + 1], f2_mul(dd, bb[j].y)); acc[1] = f2_fma(S[c][2 * j + 1], cc[j].y, acc[1]);
        }
        sum[c] = f2_sum(acc[0], acc[1]);
      }
#pragma unroll
      for (int off = 1; off < LANES; off <<= 1)
#pragma unroll
        for (int c = 0; c < CPT; ++c) sum[c] += __shfl_xor_sync(0xffffffffu, sum[c], off);
#pragma unroll
      for (int c = 0; c < CPT; ++c)
        if (live[c] && part == 0)
          y[(size_t)(first + c0 + tt) * inner + h * P + col0 + cl + NTC * c] = fmaf(skip, xv[c], sum[c]);
    }
    __syncthreads();
  }
  ss_cp_async_wait<0>();
  pdl_launch_dependents();
#pragma unroll
  for (int c = 0; c < CPT; ++c)
    if (live[c]) {
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const int i = 4 * (part + LANES * j);
        if (i < N) {
          float4 v;
          f2_unpack(S[c][2 * j], v.x, v.y);
          f2_unpack(S[c][2 * j + 1], v.z, v.w);
          st[c][i] = v.x; st[c][i + 1] = v.y; st[c][i + 2] = v.z; st[c][i + 3] = v.w;
        }
      }
    }
}


// xbc [T, H*P + 2*G*N] (x, then B, then C), dt_raw [T, >= H] fp32, y [T, H*P] fp32.  lanes: 8, 16 or 32 lanes per
// column of the state in the fast form, or 0 to choose by the size of the step.
NHV_API int nhv_ssd_scan(int dtype, float* y, const void* xbc, int xbc_stride, const float* dt_raw, int dt_stride,
                         const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                         long state_stride, const int* cu_q, const int* q_start, const int* slots, int n_seqs,
                         int n_tokens, int H, int P, int N, int G, int lanes, int cpt, cudaStream_t stream) {
  if (n_tokens == 0 || n_seqs == 0) return 0;
  NHV_REQUIRE(G > 0 && H > 0 && H % G == 0, "ssd_scan: %d heads do not divide into %d groups", H, G);
  NHV_REQUIRE(N > 0 && N <= 256 && P > 0, "ssd_scan: a state of %d rows is beyond the supported 256", N);
  NHV_REQUIRE(state_stride >= (long)H * P * N, "ssd_scan: the state holds fewer than heads * P * N floats");
  const bool fast = dtype == NHV_F32 && N % 4 == 0 && P % 4 == 0 && xbc_stride % 4 == 0 && ((uintptr_t)xbc % 16) == 0;
  // columns per lane (cpt: 1, 2, 4, or 0 to choose): one while the blocks of 16 columns leave SMs idle, more when
  // the SMs are full and the reads of B and C from shared memory are what costs
  if (cpt <= 0) {
    const long blocks16 = (long)n_seqs * H * ((P + 15) / 16);
    if (n_tokens >= 8 * (long)n_seqs) cpt = blocks16 <= 2 * 148 ? 1 : (blocks16 <= 6 * 148 ? 2 : 4);
    else cpt = blocks16 >= 16 * 148 ? 4 : (blocks16 >= 8 * 148 ? 2 : 1);     // single tokens: the states stream in and out, and many small blocks keep more reads in flight
  }
  if (fast && cpt > 1 && N <= 128 && lanes != 4 && lanes != 16 && lanes != 32) {
    if (cpt != 2) cpt = 4;
    const int cols = 16 * cpt;
    dim3 wgrid(n_seqs, H, (P + cols - 1) / cols);
    const int need = (N + 7) / 8;
#define WIDE(R, C)                                                                                                   \
  do {                                                                                                               \
    static bool attr = false;                                                                                        \
    if (!attr) {                                                                                                     \
      NHV_CUDA(cudaFuncSetAttribute(ssd_scan_wide_kernel<R, C>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                    232448), "ssd_scan");                                                            \
      attr = true;                                                                                                   \
    }                                                                                                                \
    nhv_launch(ssd_scan_wide_kernel<R, C>, wgrid, SF_THREADS,                                                        \
               nhv_spread_smem((size_t)2 * SF_CHUNK * (2 * R * 8 + 16 * C + 2) * sizeof(float),                      \
                               (long)wgrid.x * wgrid.y * wgrid.z), stream,                                          \
               y, (const float*)xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, d_skip, state, state_stride,    \
               cu_q, q_start, slots, H, P, N, G);                                                                    \
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
    NHV_CHECK_LAUNCH("ssd_scan");
    return 0;
  }
  if (fast) {
    // lanes per column: 8 measured fastest for one long request (244 ns a token against 254 with 16 lanes and 299
    // with 32: the shuffle rounds of the sum over lanes are the longest stretch of a token's chain) and for full
    // batches (fewest instructions in all); 16 and 32 stay for the tests
    if (lanes != 8 && lanes != 16 && lanes != 32) lanes = 8;
    const int cols = SF_THREADS / lanes;
    dim3 fgrid(n_seqs, H, (P + cols - 1) / cols);
    const int need = (N + lanes - 1) / lanes;
#define FAST(R, L)                                                                                                   \
  do {                                                                                                               \
    static bool attr = false;                                                                                        \
    if (!attr) {                                                                                                     \
      NHV_CUDA(cudaFuncSetAttribute(ssd_scan_fast_kernel<R, L>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                    232448), "ssd_scan");                                                            \
      attr = true;                                                                                                   \
    }                                                                                                                \
    nhv_launch(ssd_scan_fast_kernel<R, L>, fgrid, SF_THREADS,                                                        \
               nhv_spread_smem((size_t)2 * SF_CHUNK * (2 * R * L + SF_THREADS / L + 2) * sizeof(float),              \
                               (long)fgrid.x * fgrid.y * fgrid.z), stream,                                          \
               y, (const float*)xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, d_skip, state, state_stride,    \
               cu_q, q_start, slots, H, P, N, G);                                                                    \
  } while (0)
    if (lanes == 8) {
      if (need <= 4) FAST(4, 8);
      else if (need <= 8) FAST(8, 8);
      else if (need <= 16) FAST(16, 8);
      else FAST(32, 8);
    } else if (lanes == 16) {
      if (need <= 4) FAST(4, 16);
      else if (need <= 8) FAST(8, 16);
      else FAST(16, 16);
    } else {
      if (need <= 4) FAST(4, 32);
      else FAST(8, 32);
    }
#undef FAST
    NHV_CHECK_LAUNCH("ssd_scan");
    return 0;
  }
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

__device__ __forceinline__ float gn_gate(float g, int kind) {
  const float sg = 1.0f / (1.0f + expf(-g));
  return kind == 1 ? sg : g * sg;
}

// One block per (token, group).
template <typename T>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, int out_stride, const float* __restrict__ y,
                                     const T* __restrict__ z, int z_stride, const T* __restrict__ w, int w_period,
                                     int n_groups, int size, float eps, int gate_first, int gate_kind) {
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
      v *= gn_gate(to_f32<T>(zr[c]), gate_kind);
    }
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(total / (float)size + eps);
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    const float sg = gn_gate(to_f32<T>(zr[c]), gate_kind);
    const float wv = to_f32<T>(w[(gidx * size + c) % w_period]);
    dst[c] = from_f32<T>(yr[c] * sg * rstd * wv);
  }
}

// One warp per (token, group), for groups of up to 256 elements (a head of the delta rule): no barrier, the group's values stay in registers
// between the sum of squares and the output.
constexpr int GN_WARPS = 8;
constexpr int GN_MAX = 256;

template <typename T>
__global__ void __launch_bounds__(GN_WARPS * 32) gated_rmsnorm_warp_kernel(
    T* __restrict__ out, int out_stride, const float* __restrict__ y, const T* __restrict__ z, int z_stride,
    const T* __restrict__ w, int w_period, long n_items, int n_groups, int size, float eps, int gate_first,
    int gate_kind) {
  pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * GN_WARPS + warp;
  if (item >= n_items) return;
  const long t = item / n_groups;
  const int gidx = (int)(item - t * n_groups);
  const float* yr = y + (size_t)item * size;
  const T* zr = z + (size_t)t * z_stride + (size_t)gidx * size;
  T* dst = out + (size_t)t * out_stride + (size_t)gidx * size;
  float vals[GN_MAX / 32], gates[GN_MAX / 32];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < GN_MAX / 32; ++k) {
    const int c = lane + k * 32;
    if (c < size) {
      const float sg = gn_gate(to_f32<T>(zr[c]), gate_kind);
      const float v = gate_first ? yr[c] * sg : yr[c];
      vals[k] = v;
      gates[k] = gate_first ? 1.0f : sg;
      ss = fmaf(v, v, ss);
    }
  }
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)size + eps);
#pragma unroll
  for (int k = 0; k < GN_MAX / 32; ++k) {
    const int c = lane + k * 32;
    if (c < size) dst[c] = from_f32<T>(vals[k] * gates[k] * rstd * to_f32<T>(w[(gidx * size + c) % w_period]));
  }
}

NHV_API int nhv_gated_rmsnorm(int dtype, void* out, int out_stride, const float* y, const void* z, int z_stride,
                              const void* w, int w_period, int n_tokens, int n_groups, int size, float eps,
                              int gate_first, int gate_kind, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  NHV_REQUIRE(n_groups > 0 && size > 0 && w_period > 0, "gated_rmsnorm: bad sizes");
  if (size <= GN_MAX) {           // larger groups: a block per (token, group) below
    const long items = (long)n_tokens * n_groups;
    const long wblocks = (items + GN_WARPS - 1) / GN_WARPS;
    NHV_REQUIRE(wblocks < (1L << 31), "gated_rmsnorm: too many rows");
    if (dtype == NHV_F32)
      nhv_launch(gated_rmsnorm_warp_kernel<float>, (int)wblocks, GN_WARPS * 32, 0, stream, (float*)out, out_stride, y,
                 (const float*)z, z_stride, (const float*)w, w_period, items, n_groups, size, eps, gate_first, gate_kind);
    else if (dtype == NHV_BF16)
      nhv_launch(gated_rmsnorm_warp_kernel<__nv_bfloat16>, (int)wblocks, GN_WARPS * 32, 0, stream, (__nv_bfloat16*)out,
                 out_stride, y, (const __nv_bfloat16*)z, z_stride, (const __nv_bfloat16*)w, w_period, items, n_groups, size,
                 eps, gate_first, gate_kind);
    else
      NHV_REQUIRE(false, "gated_rmsnorm: unknown dtype %d", dtype);
    NHV_CHECK_LAUNCH("gated_rmsnorm");
    return 0;
  }
  int threads = 32;
  while (threads < 256 && threads * 2 <= size) threads <<= 1;
  const long blocks = (long)n_tokens * n_groups;
  NHV_REQUIRE(blocks < (1L << 31), "gated_rmsnorm: too many rows");
  if (dtype == NHV_F32)
    nhv_launch(gated_rmsnorm_kernel<float>, (int)blocks, threads, 0, stream, (float*)out, out_stride, y, (const float*)z,
               z_stride, (const float*)w, w_period, n_groups, size, eps, gate_first, gate_kind);
  else if (dtype == NHV_BF16)
    nhv_launch(gated_rmsnorm_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (__nv_bfloat16*)out, out_stride, y,
               (const __nv_bfloat16*)z, z_stride, (const __nv_bfloat16*)w, w_period, n_groups, size, eps, gate_first, gate_kind);
  else
    NHV_REQUIRE(false, "gated_rmsnorm: unknown dtype %d", dtype);
  NHV_CHECK_LAUNCH("gated_rmsnorm");
  return 0;
}
