// Gated linear attention: a matrix memory S [key channels, value columns] per head with a decay per key channel,
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t,
//   alpha_t = sigmoid(z_t)^(1/tau),              z_t = A2 (A1 h_t) + b        (a low-rank product, laid out heads x channels)
//
// The memory is float32 and is kept by value column ([slot][head][column][channel]), so that what one thread owns
// is contiguous.  rows: float32 [T, ...] of the mixer's stacked projection, holding q, k, v and A1 h at the given
// columns.  A step's rows of one sequence are a run; the memory is read at a run's start and written at its end.
//
// gla_decay_kernel   alpha for every row and channel: exp(-softplus(-z) / tau), all float32
// gla_scan_kernel    a block per (run, head, tile of value columns).  A column lies on P lanes, each holding R = 16
//                    channels of it in registers; a chunk of rows' q, k and alpha is staged in shared memory for all
//                    the block's columns; per row a lane does R decays, R updates and R products, and log2 P
//                    exchanges finish a column's output.
#include "rb_common.cuh"

namespace {

constexpr int GLA_R = 16;        // channels a lane holds

__device__ __forceinline__ float softplus_(float v) { return v > 20.f ? v : log1pf(expf(v)); }

__global__ void gla_decay_kernel(float* __restrict__ alpha, const float* __restrict__ rows, int64_t ld, int a_off,
                                 const float* __restrict__ A2, const float* __restrict__ bias, int T, int C, int rank,
                                 float inv_tau) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t = blockIdx.x;
  extern __shared__ float s_low[];                 // A1 h of this row
  for (int r = threadIdx.x; r < rank; r += blockDim.x) s_low[r] = rows[(int64_t)t * ld + a_off + r];
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float z = bias != nullptr ? bias[c] : 0.f;
    const float* w = A2 + (int64_t)c * rank;
    for (int r = 0; r < rank; ++r) z = fmaf(w[r], s_low[r], z);
    alpha[(int64_t)t * C + c] = expf(-softplus_(-z) * inv_tau);
  }
}

template <int P>
__global__ void __launch_bounds__(128) gla_scan_kernel(float* __restrict__ o, const float* __restrict__ rows, int64_t ld,
                                                       int q_off, int k_off, int v_off, const float* __restrict__ alpha,
                                                       float q_scale, float* __restrict__ state,
                                                       const int* __restrict__ seq_first, const int* __restrict__ seq_count,
                                                       const int* __restrict__ tok_slot, int H, int D, int Dv) {
  rb_pdl_launch_dependents();
  constexpr int COLS = 128 / P;                    // value columns of a block
  constexpr int DP = P * GLA_R;                    // channels with padding
  constexpr int GLA_CHUNK = P <= 8 ? 16 : (P == 16 ? 8 : 4);   // rows staged at once: 24 KB of q, k and alpha at most
  __shared__ __align__(16) float s_q[GLA_CHUNK][DP], s_k[GLA_CHUNK][DP], s_a[GLA_CHUNK][DP];
  __shared__ float s_v[GLA_CHUNK][COLS];
  const int run = blockIdx.x, head = blockIdx.y;
  const int col = threadIdx.x / P, p = threadIdx.x % P;
  const int j = blockIdx.z * COLS + col;           // this thread's value column
  rb_pdl_wait();
  const int first = seq_first != nullptr ? seq_first[run] : run;
  const int n = seq_count != nullptr ? seq_count[run] : 1;
  const int slot = tok_slot[first];
  float S[GLA_R];
  float* mine = state + (((int64_t)slot * H + head) * Dv + j) * D + p * GLA_R;
#pragma unroll
  for (int r = 0; r < GLA_R; ++r) S[r] = (j < Dv && p * GLA_R + r < D) ? mine[r] : 0.f;
  for (int t0 = 0; t0 < n; t0 += GLA_CHUNK) {
    const int nt = min(GLA_CHUNK, n - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < nt * DP; e += blockDim.x) {
      const int i = e / DP, d = e % DP;
      const int64_t row = (int64_t)(first + t0 + i) * ld;
      const bool in = d < D;
      s_q[i][d] = in ? rows[row + q_off + head * D + d] * q_scale : 0.f;
      s_k[i][d] = in ? rows[row + k_off + head * D + d] : 0.f;
      s_a[i][d] = in ? alpha[(int64_t)(first + t0 + i) * H * D + head * D + d] : 0.f;
    }
    for (int e = threadIdx.x; e < nt * COLS; e += blockDim.x) {
      const int i = e / COLS, c = e % COLS;
      const int jj = blockIdx.z * COLS + c;
      s_v[i][c] = jj < Dv ? rows[(int64_t)(first + t0 + i) * ld + v_off + head * Dv + jj] : 0.f;
    }
    __syncthreads();
    for (int i = 0; i < nt; ++i) {
      const float v = s_v[i][col];
      float acc = 0.f;
#pragma unroll
      for (int r4 = 0; r4 < GLA_R; r4 += 4) {
        const float4 a = *reinterpret_cast<const float4*>(&s_a[i][p * GLA_R + r4]);
        const float4 k = *reinterpret_cast<const float4*>(&s_k[i][p * GLA_R + r4]);
        const float4 q = *reinterpret_cast<const float4*>(&s_q[i][p * GLA_R + r4]);
        S[r4 + 0] = fmaf(a.x, S[r4 + 0], k.x * v); acc = fmaf(S[r4 + 0], q.x, acc);
        S[r4 + 1] = fmaf(a.y, S[r4 + 1], k.y * v); acc = fmaf(S[r4 + 1], q.y, acc);
        S[r4 + 2] = fmaf(a.z, S[r4 + 2], k.z * v); acc = fmaf(S[r4 + 2], q.z, acc);
        S[r4 + 3] = fmaf(a.w, S[r4 + 3], k.w * v); acc = fmaf(S[r4 + 3], q.w, acc);
      }
#pragma unroll
      for (int off = P / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (p == 0 && j < Dv) o[((int64_t)(first + t0 + i) * H + head) * Dv + j] = acc;
    }
  }
#pragma unroll
  for (int r = 0; r < GLA_R; ++r)
    if (j < Dv && p * GLA_R + r < D) mine[r] = S[r];
}

template <int P>
int launch_scan(float* o, const float* rows, int64_t ld, int q_off, int k_off, int v_off, const float* alpha, float q_scale,
                float* state, const int* seq_first, const int* seq_count, const int* tok_slot, int n_runs, int H, int D,
                int Dv, cudaStream_t stream) {
  constexpr int COLS = 128 / P;
  const dim3 grid(n_runs, H, (Dv + COLS - 1) / COLS);
  RB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "rb_gla_scan: %d heads of %d value columns are too many for one launch", H, Dv);
  RB_LAUNCH("gla_scan_kernel", (gla_scan_kernel<P>), grid, 128, 0, stream, o, rows, ld, q_off, k_off, v_off, alpha, q_scale,
            state, seq_first, seq_count, tok_slot, H, D, Dv);
  RB_CHECK_LAUNCH("rb_gla_scan");
  return 0;
}

}  // namespace

// alpha [T, C] from rows[t, a_off .. a_off + rank): C = heads x channels outputs of A2 [C, rank] plus bias [C].
RB_EXPORT int rb_gla_decay(float* alpha, const float* rows, int64_t ld, int a_off, const float* A2, const float* bias, int T,
                           int C, int rank, float tau, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(C > 0 && rank > 0 && tau > 0.f, "rb_gla_decay: bad sizes C=%d rank=%d tau=%g", C, rank, (double)tau);
  RB_REQUIRE((size_t)rank * sizeof(float) <= 48 * 1024, "rb_gla_decay: a rank of %d is more than a block's shared memory holds", rank);
  int by = (C + 127) / 128;
  if (by > 32) by = 32;
  RB_LAUNCH("gla_decay_kernel", (gla_decay_kernel), dim3(T, by), 128, (size_t)rank * sizeof(float), stream, alpha, rows, ld,
            a_off, A2, bias, T, C, rank, 1.0f / tau);
  RB_CHECK_LAUNCH("rb_gla_decay");
  return 0;
}

RB_EXPORT int rb_gla_max_dim() { return 32 * GLA_R; }

// o [T, H, Dv] float32.  n_runs runs (seq_first, seq_count; null: every one of the n_runs rows is its own run).
// state: [n_slots, H, Dv, D] float32.
RB_EXPORT int rb_gla_scan(float* o, const float* rows, int64_t ld, int q_off, int k_off, int v_off, const float* alpha,
                          float q_scale, float* state, const int* seq_first, const int* seq_count, const int* tok_slot,
                          int n_runs, int H, int D, int Dv, cudaStream_t stream) {
  if (n_runs == 0) return 0;
  RB_REQUIRE(H > 0 && D > 0 && Dv > 0 && D <= 32 * GLA_R, "rb_gla_scan: bad sizes H=%d D=%d Dv=%d (at most %d key channels)", H,
             D, Dv, 32 * GLA_R);
  int P = 1;
  while (P * GLA_R < D) P *= 2;
#define GO(PP) return launch_scan<PP>(o, rows, ld, q_off, k_off, v_off, alpha, q_scale, state, seq_first, seq_count, tok_slot, n_runs, H, D, Dv, stream)
  switch (P) {
    case 1: GO(1);
    case 2: GO(2);
    case 4: GO(4);
    case 8: GO(8);
    case 16: GO(16);
    default: GO(32);
  }
#undef GO
}
