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
//                    exchanges finish a column's output.  Token by token: the plain form.
// gla_chunk_*        runs of several tokens in chunks of 32, the chain in time only from chunk to chunk (below).
// gla_step_kernel    a decode step in one launch: decays, the memory's step, the norm per head and the gate.
#include "rb_common.cuh"

namespace {

constexpr int GLA_R = 16;        // channels a lane holds

__device__ __forceinline__ float softplus_(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// A block takes GLA_DT rows and 128 channels at a time: a channel's row of A2 is read once for all of them.
constexpr int GLA_DT = 8;
__global__ void __launch_bounds__(128) gla_decay_kernel(float* __restrict__ alpha, const float* __restrict__ rows, int64_t ld,
                                                        int a_off, const float* __restrict__ A2,
                                                        const float* __restrict__ bias, int T, int C, int rank,
                                                        float inv_tau, int as_log) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t0 = blockIdx.x * GLA_DT, nt = min(GLA_DT, T - t0);
  extern __shared__ float s_low[];                 // A1 h of these rows: [GLA_DT][rank], zeros for rows beyond the last
  for (int e = threadIdx.x; e < GLA_DT * rank; e += blockDim.x) {
    const int i = e / rank, r = e - i * rank;
    s_low[e] = i < nt ? rows[(int64_t)(t0 + i) * ld + a_off + r] : 0.f;
  }
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float z[GLA_DT];
    const float b = bias != nullptr ? bias[c] : 0.f;
#pragma unroll
    for (int i = 0; i < GLA_DT; ++i) z[i] = b;
    const float* w = A2 + (int64_t)c * rank;
    for (int r = 0; r < rank; ++r) {
      const float wr = w[r];
#pragma unroll
      for (int i = 0; i < GLA_DT; ++i) z[i] = fmaf(wr, s_low[i * rank + r], z[i]);
    }
#pragma unroll
    for (int i = 0; i < GLA_DT; ++i) {
      if (i < nt) {
        const float lg = -softplus_(-z[i]) * inv_tau;            // log alpha
        alpha[(int64_t)(t0 + i) * C + c] = as_log ? lg : expf(lg);
      }
    }
  }
}

template <int P>
__global__ void __launch_bounds__(128) gla_scan_kernel(float* __restrict__ o, const float* __restrict__ rows, int64_t ld,
                                                       int q_off, int k_off, int v_off, const float* __restrict__ alpha,
                                                       float q_scale, float* __restrict__ state,
                                                       const int* __restrict__ seq_first, const int* __restrict__ seq_count,
                                                       const int* __restrict__ tok_slot, int H, int D, int Dv,
                                                       int64_t a_ld) {
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
      s_a[i][d] = in ? alpha[(int64_t)(first + t0 + i) * a_ld + head * D + d] : 0.f;
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
                int Dv, int64_t a_ld, cudaStream_t stream) {
  constexpr int COLS = 128 / P;
  const dim3 grid(n_runs, H, (Dv + COLS - 1) / COLS);
  RB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "rb_gla_scan: %d heads of %d value columns are too many for one launch", H, Dv);
  RB_LAUNCH("gla_scan_kernel", (gla_scan_kernel<P>), grid, 128, 0, stream, o, rows, ld, q_off, k_off, v_off, alpha, q_scale,
            state, seq_first, seq_count, tok_slot, H, D, Dv, a_ld);
  RB_CHECK_LAUNCH("rb_gla_scan");
  return 0;
}

// ---------------------------------------------------------------- long runs: chunks of 32 tokens
// Within a chunk that starts from the memory S0, with B_i[d] the sum of the logarithms of channel d's decays over the
// chunk's tokens up to and including i (so that exp(B_i - B_j) is the decay from token j to token i, never above one):
//   o_i   = (q_i * e^{B_i})^T S0 + sum_{j <= i} M_ij v_j,      M_ij = sum_d q_i[d] k_j[d] e^{B_i[d] - B_j[d]}
//   S_end = diag(e^{B_end}) S0 + sum_j (k_j * e^{B_end - B_j}) v_j^T
// Every exponent is taken of a difference that is zero or negative, channel by channel, so nothing overflows however
// fast a channel forgets.  The first kernel makes Qt = q e^{B}, Kt = k e^{B_end - B}, M and e^{B_end} for every
// (chunk, head) at once; the second walks a run's chunks with the memory: two small products per chunk.  A chunk's
// missing tokens (the run's end) count as decay 1 and k = q = v = 0.
constexpr int GCH = 32;          // tokens of a chunk
constexpr int GCT = 16;          // value columns of a block of the second kernel
constexpr int GSCAN_NT = 256;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_or_zeros(void* dst, const void* src, bool real) {
  const int bytes = real ? 16 : 0;            // fewer source bytes than 16: the rest is filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__host__ __device__ constexpr int gla_item_floats(int D) { return 2 * GCH * D + GCH * GCH + D; }   // Qt, Kt, M, e^{B_end}

// grid (chunks, H), 128 threads.  log_alpha: [T, H * D].  Scratch per (chunk, head): Qt [32][D], Kt [32][D], M [32][32],
// e^{B_end} [D].
__global__ void __launch_bounds__(128) gla_chunk_prepare_kernel(float* __restrict__ scratch, const float* __restrict__ rows,
                                                                int64_t ld, int q_off, int k_off,
                                                                const float* __restrict__ log_alpha, float q_scale,
                                                                const int* __restrict__ chunk_row,
                                                                const int* __restrict__ chunk_len, int H, int D,
                                                                int64_t a_ld) {
  rb_pdl_launch_dependents();
  extern __shared__ __align__(16) float s_gprep[];
  const int KS = D + 4;                          // row stride: the lanes' 16-byte loads of their own rows spread over the banks
  float* Bs = s_gprep;                           // [32][D + 4]
  float* Qs = Bs + GCH * KS;
  float* Ks = Qs + GCH * KS;
  const int chunk = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D4 = D >> 2;
  rb_pdl_wait();
  const int row0 = chunk_row[chunk], m = chunk_len[chunk];
  for (int i = tid; i < GCH * D4; i += 128) {
    const int j = i / D4, d = (i - j * D4) << 2;
    float4 bb = make_float4(0.f, 0.f, 0.f, 0.f), qq = bb, kk = bb;
    if (j < m) {
      const float* row = rows + (int64_t)(row0 + j) * ld;
      bb = *reinterpret_cast<const float4*>(log_alpha + (int64_t)(row0 + j) * a_ld + h * D + d);
      qq = *reinterpret_cast<const float4*>(row + q_off + h * D + d);
      kk = *reinterpret_cast<const float4*>(row + k_off + h * D + d);
      qq.x *= q_scale; qq.y *= q_scale; qq.z *= q_scale; qq.w *= q_scale;
    }
    *reinterpret_cast<float4*>(Bs + j * KS + d) = bb;
    *reinterpret_cast<float4*>(Qs + j * KS + d) = qq;
    *reinterpret_cast<float4*>(Ks + j * KS + d) = kk;
  }
  __syncthreads();
  for (int d = tid; d < D; d += 128) {           // the running sums, channel by channel
    float run = 0.f;
#pragma unroll 8
    for (int i = 0; i < GCH; ++i) {
      run += Bs[i * KS + d];
      Bs[i * KS + d] = run;
    }
  }
  __syncthreads();
  float* item = scratch + ((int64_t)chunk * H + h) * gla_item_floats(D);
  {
    // thread: column j = lane, rows i = warp + 4 r
    const int j = lane;
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
    for (int d = 0; d < D; d += 4) {
      const float4 kj = *reinterpret_cast<const float4*>(Ks + j * KS + d);
      const float4 bj = *reinterpret_cast<const float4*>(Bs + j * KS + d);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int i = warp + 4 * r;
        if (j <= i) {
          const float4 qi = *reinterpret_cast<const float4*>(Qs + i * KS + d);
          const float4 bi = *reinterpret_cast<const float4*>(Bs + i * KS + d);
          acc[r] = fmaf(qi.x * kj.x, expf(bi.x - bj.x), acc[r]);
          acc[r] = fmaf(qi.y * kj.y, expf(bi.y - bj.y), acc[r]);
          acc[r] = fmaf(qi.z * kj.z, expf(bi.z - bj.z), acc[r]);
          acc[r] = fmaf(qi.w * kj.w, expf(bi.w - bj.w), acc[r]);
        }
      }
    }
    float* Mo = item + 2 * GCH * D;
#pragma unroll
    for (int r = 0; r < 8; ++r) Mo[(warp + 4 * r) * GCH + j] = acc[r];
  }
  float* Qt = item;
  float* Kt = item + GCH * D;
  float* Eo = item + 2 * GCH * D + GCH * GCH;
  for (int i = tid; i < GCH * D; i += 128) {
    const int j = i / D, d = i - j * D;
    const float b = Bs[j * KS + d], be = Bs[(GCH - 1) * KS + d];
    Qt[i] = Qs[j * KS + d] * expf(b);
    Kt[i] = Ks[j * KS + d] * expf(be - b);
  }
  for (int d = tid; d < D; d += 128) Eo[d] = expf(Bs[(GCH - 1) * KS + d]);
}

// grid (runs, H, tiles of 16 value columns), 256 threads.  Shared memory: two buffers of a chunk's item (as the first
// kernel left it) and the tile's values [32][16], filled a chunk ahead with cp.async; the memory's tile S [16][D + 4]
// twice: a chunk reads one and writes the other, so that its read-out and its update need no barrier between them.
__global__ void __launch_bounds__(GSCAN_NT) gla_chunk_scan_kernel(
    float* __restrict__ o, const float* __restrict__ scratch, const float* __restrict__ rows, int64_t ld, int v_off,
    float* __restrict__ state, const int* __restrict__ seq_first, const int* __restrict__ seq_count,
    const int* __restrict__ run_chunk0, const int* __restrict__ tok_slot, int H, int D, int Dv) {
  rb_pdl_launch_dependents();
  extern __shared__ __align__(16) float s_gscan[];
  const int item_floats = gla_item_floats(D);
  const int per_buf = item_floats + GCH * GCT;
  const int SS = D + 4;
  float* Sa = s_gscan + 2 * per_buf;    // [16][D + 4]: the memory as this chunk finds it
  float* Sb = Sa + GCT * SS;            // the memory as this chunk leaves it (the two change places after every chunk)
  const int run = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GCT;
  const int tid = threadIdx.x;
  rb_pdl_wait();
  const int first = seq_first[run], n = seq_count[run], chunk0 = run_chunk0[run];
  const int slot = tok_slot[first];
  auto copy_chunk = [&](int ci, int buf) {
    const int row0 = first + ci * GCH, m = min(GCH, n - ci * GCH);
    const float* src = scratch + ((int64_t)(chunk0 + ci) * H + h) * item_floats;
    float* dst = s_gscan + (size_t)buf * per_buf;
    for (int i = tid; i < (item_floats >> 2); i += GSCAN_NT) cp_async16(dst + 4 * i, src + 4 * i);
    if (tid < GCH * GCT / 4) {
      const int j = tid >> 2, c4 = (tid & 3) << 2;
      const bool real = j < m && col0 + c4 < Dv;
      const float* v = real ? rows + (int64_t)(row0 + j) * ld + v_off + h * Dv + col0 + c4 : rows;
      cp_async16_or_zeros(dst + item_floats + j * GCT + c4, v, real);
    }
  };
  const int n_chunks = (n + GCH - 1) / GCH;
  copy_chunk(0, 0);
  cp_async_commit();
  float* mine = state + (((int64_t)slot * H + h) * Dv + col0) * D;      // [column][D]
  for (int i = tid; i < D * GCT; i += GSCAN_NT) {
    const int cc = i / D, d = i - cc * D;
    Sa[cc * SS + d] = col0 + cc < Dv ? mine[(int64_t)cc * D + d] : 0.f;
  }
  const int c = tid & 15, g = tid >> 4;              // read-out: column c, rows g and g + 16
  const int dq = (tid & 31) << 2, cp = (tid >> 5) << 1;   // update: channels dq .. dq + 3 of columns cp and cp + 1
  for (int ci = 0, buf = 0; ci < n_chunks; ++ci, buf ^= 1) {
    const int row0 = first + ci * GCH, m = min(GCH, n - ci * GCH);
    cp_async_wait<0>();
    __syncthreads();                  // this chunk's copies have landed, the memory the last chunk left is whole, and
                                      // nobody reads the other buffer any more: the one barrier of a chunk
    if (ci + 1 < n_chunks) {
      copy_chunk(ci + 1, buf ^ 1);    // lands while this chunk is multiplied
      cp_async_commit();
    }
    const float* Ss = (ci & 1) ? Sb : Sa;
    float* Sn = (ci & 1) ? Sa : Sb;
    const float* Qt = s_gscan + (size_t)buf * per_buf;
    const float* Kt = Qt + GCH * D;
    const float* Ms = Kt + GCH * D;
    const float* Es = Ms + GCH * GCH;
    const float* Vs = Qt + item_floats;
    {
      float acc0 = 0.f, acc1 = 0.f;
      const float* s = Ss + c * SS;
      const float* q0 = Qt + g * D;
      const float* q1 = Qt + (g + 16) * D;
      for (int d = 0; d < D; d += 4) {
        const float4 s4 = *reinterpret_cast<const float4*>(s + d);
        const float4 a4 = *reinterpret_cast<const float4*>(q0 + d);
        const float4 b4 = *reinterpret_cast<const float4*>(q1 + d);
        acc0 = fmaf(a4.x, s4.x, fmaf(a4.y, s4.y, fmaf(a4.z, s4.z, fmaf(a4.w, s4.w, acc0))));
        acc1 = fmaf(b4.x, s4.x, fmaf(b4.y, s4.y, fmaf(b4.z, s4.z, fmaf(b4.w, s4.w, acc1))));
      }
      // M is zero above its diagonal, so both rows take all 32 columns: a loop of fixed length whose loads run ahead
      const float4* m0 = reinterpret_cast<const float4*>(Ms + g * GCH);
      const float4* m1 = reinterpret_cast<const float4*>(Ms + (g + 16) * GCH);
#pragma unroll
      for (int j4 = 0; j4 < GCH / 4; ++j4) {
        const float4 a4 = m0[j4], b4 = m1[j4];
        const float v0 = Vs[(4 * j4 + 0) * GCT + c], v1 = Vs[(4 * j4 + 1) * GCT + c];
        const float v2 = Vs[(4 * j4 + 2) * GCT + c], v3 = Vs[(4 * j4 + 3) * GCT + c];
        acc0 = fmaf(a4.x, v0, fmaf(a4.y, v1, fmaf(a4.z, v2, fmaf(a4.w, v3, acc0))));
        acc1 = fmaf(b4.x, v0, fmaf(b4.y, v1, fmaf(b4.z, v2, fmaf(b4.w, v3, acc1))));
      }
      if (col0 + c < Dv) {
        if (g < m) o[((int64_t)(row0 + g) * H + h) * Dv + col0 + c] = acc0;
        if (g + 16 < m) o[((int64_t)(row0 + g + 16) * H + h) * Dv + col0 + c] = acc1;
      }
    }
    // the memory moves on into the other buffer, so that no thread waits here for the read-outs of the others
    if (dq < D) {
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
#pragma unroll 8
      for (int j = 0; j < GCH; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(Kt + j * D + dq);
        const float2 v2 = *reinterpret_cast<const float2*>(Vs + j * GCT + cp);
        a0.x = fmaf(k4.x, v2.x, a0.x); a0.y = fmaf(k4.y, v2.x, a0.y); a0.z = fmaf(k4.z, v2.x, a0.z); a0.w = fmaf(k4.w, v2.x, a0.w);
        a1.x = fmaf(k4.x, v2.y, a1.x); a1.y = fmaf(k4.y, v2.y, a1.y); a1.z = fmaf(k4.z, v2.y, a1.z); a1.w = fmaf(k4.w, v2.y, a1.w);
      }
      const float4 e4 = *reinterpret_cast<const float4*>(Es + dq);
      float4 x = *reinterpret_cast<const float4*>(Ss + cp * SS + dq);
      float4 y = *reinterpret_cast<const float4*>(Ss + (cp + 1) * SS + dq);
      float4* s0 = reinterpret_cast<float4*>(Sn + cp * SS + dq);
      float4* s1 = reinterpret_cast<float4*>(Sn + (cp + 1) * SS + dq);
      x.x = fmaf(e4.x, x.x, a0.x); x.y = fmaf(e4.y, x.y, a0.y); x.z = fmaf(e4.z, x.z, a0.z); x.w = fmaf(e4.w, x.w, a0.w);
      y.x = fmaf(e4.x, y.x, a1.x); y.y = fmaf(e4.y, y.y, a1.y); y.z = fmaf(e4.z, y.z, a1.z); y.w = fmaf(e4.w, y.w, a1.w);
      *s0 = x;
      *s1 = y;
    }
  }
  __syncthreads();
  const float* Se = (n_chunks & 1) ? Sb : Sa;
  for (int i = tid; i < D * GCT; i += GSCAN_NT) {
    const int cc = i / D, d = i - cc * D;
    if (col0 + cc < Dv) mine[(int64_t)cc * D + d] = Se[cc * SS + d];
  }
}

}  // namespace

// alpha [T, C] from rows[t, a_off .. a_off + rank): C = heads x channels outputs of A2 [C, rank] plus bias [C].
// as_log: its logarithm instead (what the chunked kernels add up).
RB_EXPORT int rb_gla_decay(float* alpha, const float* rows, int64_t ld, int a_off, const float* A2, const float* bias, int T,
                           int C, int rank, float tau, int as_log, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(C > 0 && rank > 0 && tau > 0.f, "rb_gla_decay: bad sizes C=%d rank=%d tau=%g", C, rank, (double)tau);
  RB_REQUIRE((size_t)GLA_DT * rank * sizeof(float) <= 48 * 1024, "rb_gla_decay: a rank of %d is more than a block's shared memory holds", rank);
  int by = (C + 127) / 128;
  if (by > 32) by = 32;
  RB_LAUNCH("gla_decay_kernel", (gla_decay_kernel), dim3((T + GLA_DT - 1) / GLA_DT, by), 128, (size_t)GLA_DT * rank * sizeof(float),
            stream, alpha, rows, ld, a_off, A2, bias, T, C, rank, 1.0f / tau, as_log);
  RB_CHECK_LAUNCH("rb_gla_decay");
  return 0;
}

RB_EXPORT int rb_gla_max_dim() { return 32 * GLA_R; }

// Decays that do not depend on the token (a fixed decay per head, say): after rb_gla_shared_decays() the calling
// thread's next rb_gla_scan or rb_gla_chunked reads ONE row [H * D] of decays (or of their logarithms) for every token.
static thread_local bool t_shared_decays = false;
static bool take_shared_decays() {
  const bool v = t_shared_decays;
  t_shared_decays = false;
  return v;
}
RB_EXPORT int rb_gla_shared_decays() {
  t_shared_decays = true;
  return 0;
}

// o [T, H, Dv] float32.  n_runs runs (seq_first, seq_count; null: every one of the n_runs rows is its own run).
// state: [n_slots, H, Dv, D] float32.
RB_EXPORT int rb_gla_scan(float* o, const float* rows, int64_t ld, int q_off, int k_off, int v_off, const float* alpha,
                          float q_scale, float* state, const int* seq_first, const int* seq_count, const int* tok_slot,
                          int n_runs, int H, int D, int Dv, cudaStream_t stream) {
  const int64_t a_ld = take_shared_decays() ? 0 : (int64_t)H * D;
  if (n_runs == 0) return 0;
  RB_REQUIRE(H > 0 && D > 0 && Dv > 0 && D <= 32 * GLA_R, "rb_gla_scan: bad sizes H=%d D=%d Dv=%d (at most %d key channels)", H,
             D, Dv, 32 * GLA_R);
  int P = 1;
  while (P * GLA_R < D) P *= 2;
#define GO(PP) return launch_scan<PP>(o, rows, ld, q_off, k_off, v_off, alpha, q_scale, state, seq_first, seq_count, tok_slot, n_runs, H, D, Dv, a_ld, stream)
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

// Whether runs of several tokens take the chunked kernels: key sizes that are multiples of 4, up to 128; value sizes
// and row strides that keep every 16-byte copy aligned.
RB_EXPORT int rb_gla_chunked_supports(int D, int Dv, long long ld, int q_off, int k_off, int v_off) {
  return D % 4 == 0 && D > 0 && D <= 128 && Dv > 0 && Dv % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0;
}

// Floats of scratch per (chunk, head).
RB_EXPORT long long rb_gla_chunk_floats(int D) { return gla_item_floats(D); }

// The same recurrence for runs of several tokens, in chunks of 32 (see above).  log_alpha [T, H * D]: rb_gla_decay's
// logarithms.  chunk_row, chunk_len: every chunk of every run, the runs' chunks in order; run_chunk0[r]: the first
// chunk of run r.  scratch: n_chunks * H * rb_gla_chunk_floats(D) floats.
RB_EXPORT int rb_gla_chunked(float* o, const float* rows, int64_t ld, int q_off, int k_off, int v_off, const float* log_alpha,
                             float q_scale, float* state, float* scratch, const int* seq_first, const int* seq_count,
                             const int* run_chunk0, const int* chunk_row, const int* chunk_len, const int* tok_slot,
                             int n_runs, int n_chunks, int H, int D, int Dv, cudaStream_t stream) {
  const int64_t a_ld = take_shared_decays() ? 0 : (int64_t)H * D;
  if (n_runs == 0 || n_chunks == 0) return 0;
  RB_REQUIRE(H > 0 && H <= 65535 && rb_gla_chunked_supports(D, Dv, ld, q_off, k_off, v_off) && (uintptr_t)rows % 16 == 0 &&
                 (uintptr_t)scratch % 16 == 0 && (uintptr_t)log_alpha % 16 == 0,
             "rb_gla_chunked: bad sizes H=%d D=%d Dv=%d", H, D, Dv);
  const size_t smem_a = (size_t)(3 * GCH * (D + 4)) * sizeof(float);
  const size_t smem_b = (size_t)(2 * (gla_item_floats(D) + GCH * GCT) + 2 * GCT * (D + 4)) * sizeof(float);
  static RbOncePerDevice configured;
  if (configured.first()) {
    RB_CUDA(cudaFuncSetAttribute(gla_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    RB_CUDA(cudaFuncSetAttribute(gla_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
  }
  RB_REQUIRE(smem_a <= 64 * 1024 && smem_b <= 128 * 1024, "rb_gla_chunked: key size %d needs too much shared memory", D);
  RB_LAUNCH("gla_chunk_prepare_kernel", (gla_chunk_prepare_kernel), dim3(n_chunks, H), 128, smem_a, stream, scratch, rows, ld,
            q_off, k_off, log_alpha, q_scale, chunk_row, chunk_len, H, D, a_ld);
  RB_CHECK_LAUNCH("rb_gla_chunked");
  const dim3 grid(n_runs, H, (Dv + GCT - 1) / GCT);
  RB_REQUIRE(grid.z <= 65535, "rb_gla_chunked: too many columns");
  RB_LAUNCH("gla_chunk_scan_kernel", (gla_chunk_scan_kernel), grid, GSCAN_NT, smem_b, stream, o, scratch, rows, ld, v_off, state,
            seq_first, seq_count, run_chunk0, tok_slot, H, D, Dv);
  RB_CHECK_LAUNCH("rb_gla_chunked");
  return 0;
}
