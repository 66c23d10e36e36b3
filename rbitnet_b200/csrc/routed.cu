// A feed-forward of routed experts: the router, the plan that sorts a step's (token, choice) pairs by expert,
// the gather of the pairs' input rows, the grouped float32 product, and the weighted sum.
//
//   z = Wr h (float32), s = softmax(z) over all n outputs; the choice score of output e is s_e + c_e
//   outputs form `groups` equal groups of neighbours; a group's score is its largest choice score, and
//   only outputs of the `keep` best groups can be chosen; the `top` largest choice scores are chosen;
//   a chosen output's weight is s_e (not renormalised)
//   outputs n_experts .. n-1 are identity experts: their result is the input row itself
//   result_t = sum over the chosen e of s_e * expert_e(h_t)
//
// Variants, each a parameter: `scoring` 1 takes s = sigmoid(z), output by output, instead of the softmax; the router's
// matrix may hold `n_extra` further rows after the n outputs, whose sums leave as they are (a gate that reads the same
// rows); the gather may multiply a pair's input row by the pair's weight (experts whose weight acts on the input).
//
// The pairs whose expert has weights are sorted by expert into rows of a padded buffer in which every
// expert's rows start on a tile border, so that a tile of rows multiplies by one expert's matrix
// (tile_group[tile]: the expert, or -1 for a tile without rows).  Where a pair lands inside its
// expert's rows depends on the order in which threads arrive; no result depends on it, because a row's
// products are sums over k in a fixed order whatever rows are beside it, and a token's weighted sum
// adds its choices in the order of the choice.
#include "rb_common.cuh"

namespace {

// ---------------------------------------------------------------- router
// A block of 8 warps takes TB tokens (up to 8).  Its warps share the router's outputs: a warp makes output e for all
// of the block's tokens at once, so that a row of Wr is read once per block (lanes stride over k four values at a
// time; a token's sum is the lanes' partial sums added in a fixed tree, whatever other tokens the block holds).  Then
// warp w makes the choice of token w.  Shared memory: per token 2 n + 2 groups floats.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// One warp: from the token's router sums z[0..n) (shared memory; choice, gscore: n and 2 groups floats of scratch) to
// its `top` outputs and their weights.
__device__ __forceinline__ void route_select(float* z, float* choice, float* gscore, const float* __restrict__ correction,
                                             int n, int top, int groups, int keep, int lane, int* __restrict__ ids,
                                             float* __restrict__ weights, int64_t t, int scoring = 0) {
  if (scoring == 1) {
    for (int e = lane; e < n; e += 32) {
      const float s = 1.0f / (1.0f + expf(-z[e]));
      z[e] = s;
      choice[e] = s + (correction != nullptr ? correction[e] : 0.f);
    }
    __syncwarp();
  } else {
  float m = -INFINITY;
  for (int e = lane; e < n; e += 32) m = fmaxf(m, z[e]);
  m = rb_warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < n; e += 32) sum += expf(z[e] - m);
  sum = rb_warp_sum(sum);
  const float inv = 1.0f / sum;
  __syncwarp();
  for (int e = lane; e < n; e += 32) {
    const float s = expf(z[e] - m) * inv;
    z[e] = s;
    choice[e] = s + (correction != nullptr ? correction[e] : 0.f);
  }
  __syncwarp();
  }
  // the largest value of v[0..count) that is not -inf, lowest index on ties; every lane gets the index
  auto arg_max = [&](const float* v, int count) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < count; e += 32)
      if (v[e] > best) { best = v[e]; at = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    return at;
  };
  if (groups > 1 && keep < groups) {
    const int per = n / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, choice[e]);
      gscore[g] = best;
    }
    __syncwarp();
    float* gkeep = gscore + groups;
    for (int g = lane; g < groups; g += 32) gkeep[g] = 0.f;
    __syncwarp();
    for (int j = 0; j < keep; ++j) {
      const int g = arg_max(gscore, groups);
      if (g >= groups) break;                          // nothing left to take
      __syncwarp();
      if (lane == 0) { gscore[g] = -INFINITY; gkeep[g] = 1.f; }
      __syncwarp();
    }
    for (int e = lane; e < n; e += 32)
      if (gkeep[e / per] == 0.f) choice[e] = -INFINITY;
    __syncwarp();
  }
  for (int j = 0; j < top; ++j) {
    const int e = arg_max(choice, n);
    __syncwarp();
    if (lane == 0) {
      const bool found = e < n;
      ids[(int64_t)t * top + j] = found ? e : 0;
      weights[(int64_t)t * top + j] = found ? z[e] : 0.f;
      if (found) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
}

constexpr int ROUTE_TB = 8;

template <typename TI>
__global__ void __launch_bounds__(256) route_kernel(int* __restrict__ ids, float* __restrict__ weights,
                                                    const TI* __restrict__ h, int64_t ldh,
                                                    const float* __restrict__ Wr, const float* __restrict__ correction,
                                                    int T, int K, int n_out, int top, int groups, int keep, int TB, int vec,
                                                    int scoring, int n_extra, float* __restrict__ extra) {
  rb_pdl_launch_dependents();
  extern __shared__ float s_route[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = n_out + n_extra;                       // rows of Wr: the outputs, then the extra rows
  const int per_token = 2 * n + 2 * groups;
  const int t0 = blockIdx.x * TB;
  const int nt = min(TB, T - t0);
  rb_pdl_wait();
  if (TB == 1 && vec) {
    // one token: a warp makes four of its outputs at once, so that four rows of Wr are asked for together
    const TI* row = h + (int64_t)t0 * ldh;
    for (int e0 = warp; e0 < n; e0 += 32) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int k = lane * 4; k < K; k += 128) {
        float hv[4];
        load4(row + k, hv);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const int e = e0 + 8 * a;
          if (e < n) {
            float wv[4];
            load4(Wr + (int64_t)e * K + k, wv);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[a] = fmaf(hv[i], wv[i], acc[a]);
          }
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float v = rb_warp_sum(acc[a]);
        if (lane == 0 && e0 + 8 * a < n) s_route[e0 + 8 * a] = v;
      }
    }
  } else
  for (int e = warp; e < n; e += 8) {
    const float* w = Wr + (int64_t)e * K;
    float acc[ROUTE_TB];
#pragma unroll
    for (int j = 0; j < ROUTE_TB; ++j) acc[j] = 0.f;
    if (vec) {
#pragma unroll 4
      for (int k = lane * 4; k < K; k += 128) {
        float wv[4];
        load4(w + k, wv);
#pragma unroll
        for (int j = 0; j < ROUTE_TB; ++j) {
          if (j < nt) {
            float hv[4];
            load4(h + (int64_t)(t0 + j) * ldh + k, hv);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j] = fmaf(hv[i], wv[i], acc[j]);
          }
        }
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float wk = w[k];
#pragma unroll
        for (int j = 0; j < ROUTE_TB; ++j)
          if (j < nt) acc[j] = fmaf(rb_to_float<TI>(h[(int64_t)(t0 + j) * ldh + k]), wk, acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < ROUTE_TB; ++j) {
      const float v = rb_warp_sum(acc[j]);
      if (lane == 0 && j < nt) s_route[(size_t)j * per_token + e] = v;
    }
  }
  __syncthreads();
  if (warp >= nt) return;
  float* z = s_route + (size_t)warp * per_token;     // scores, choice scores, group scores, kept groups
  for (int i = lane; i < n_extra; i += 32) extra[(int64_t)(t0 + warp) * n_extra + i] = z[n_out + i];
  route_select(z, z + n, z + 2 * n, correction, n_out, top, groups, keep, lane, ids, weights, t0 + warp, scoring);
}

// Many tokens: the router's sums as a tiled float32 product (16 tokens by 64 outputs a block, k in steps of 32 through
// shared memory, the next step's values asked for before this one is multiplied; every sum runs over k in ascending
// order), then a warp per token for the choice.
constexpr int RL_TM = 16, RL_TN = 64, RL_TK = 32;
template <typename TI>
__global__ void __launch_bounds__(256) route_logits_kernel(float* __restrict__ z, const TI* __restrict__ h, int64_t ldh,
                                                           const float* __restrict__ Wr, int T, int K, int n) {
  rb_pdl_launch_dependents();
  __shared__ float As[RL_TK][RL_TM + 1];
  __shared__ __align__(16) float Ws[RL_TK][RL_TN + 4];
  const int tid = threadIdx.x, tok = tid >> 4, oo = (tid & 15) * 4;
  const int t0 = blockIdx.x * RL_TM;
  rb_pdl_wait();
  // what a thread brings per step: two values of the tokens' rows, eight of the router's
  const int a_row = tid >> 4, a_k = (tid & 15) * 2;           // token, k
  const int w_row = tid >> 2, w_k = (tid & 3) * 8;            // output, k
  for (int n0 = 0; n0 < n; n0 += RL_TN) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float a_next[2], w_next[8];
    auto fetch = [&](int k0) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int k = k0 + a_k + i;
        a_next[i] = (t0 + a_row < T && k < K) ? rb_to_float<TI>(h[(int64_t)(t0 + a_row) * ldh + k]) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int k = k0 + w_k + i;
        w_next[i] = (n0 + w_row < n && k < K) ? Wr[(int64_t)(n0 + w_row) * K + k] : 0.f;
      }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += RL_TK) {
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 2; ++i) As[a_k + i][a_row] = a_next[i];
#pragma unroll
      for (int i = 0; i < 8; ++i) Ws[w_k + i][w_row] = w_next[i];
      __syncthreads();
      if (k0 + RL_TK < K) fetch(k0 + RL_TK);
#pragma unroll
      for (int kk = 0; kk < RL_TK; ++kk) {
        const float a = As[kk][tok];
        const float4 w = *reinterpret_cast<const float4*>(&Ws[kk][oo]);
        acc[0] = fmaf(a, w.x, acc[0]); acc[1] = fmaf(a, w.y, acc[1]);
        acc[2] = fmaf(a, w.z, acc[2]); acc[3] = fmaf(a, w.w, acc[3]);
      }
    }
    if (t0 + tok < T) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (n0 + oo + i < n) z[(int64_t)(t0 + tok) * n + n0 + oo + i] = acc[i];
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(128) route_select_kernel(int* __restrict__ ids, float* __restrict__ weights,
                                                           const float* __restrict__ zg, const float* __restrict__ correction,
                                                           int T, int n, int top, int groups, int keep, int scoring,
                                                           int n_extra, float* __restrict__ extra) {
  rb_pdl_launch_dependents();
  extern __shared__ float s_route[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  float* z = s_route + (size_t)warp * (2 * n + 2 * groups);
  rb_pdl_wait();
  if (t >= T) return;
  const int64_t ldz = n + n_extra;                     // zg holds the outputs' sums, then the extra rows'
  for (int e = lane; e < n; e += 32) z[e] = zg[(int64_t)t * ldz + e];
  for (int i = lane; i < n_extra; i += 32) extra[(int64_t)t * n_extra + i] = zg[(int64_t)t * ldz + n + i];
  __syncwarp();
  route_select(z, z + n, z + 2 * n, correction, n, top, groups, keep, lane, ids, weights, t, scoring);
}

// ---------------------------------------------------------------- plan
// One block.  ids: [pairs] chosen outputs.  Outputs:
//   pos [pairs]        the pair's row in the padded buffer (-1: an identity expert)
//   row_token [rows]   the token whose input row a buffer row holds (-1: padding)
//   tile_group [tiles] the expert of a tile of rows (-1: none)
__global__ void __launch_bounds__(1024) plan_kernel(int* __restrict__ pos, int* __restrict__ row_token,
                                                    int* __restrict__ tile_group, const int* __restrict__ ids,
                                                    int pairs, int top, int n_experts, int tile, int n_tiles) {
  rb_pdl_launch_dependents();
  extern __shared__ int s_plan[];       // counts [n_experts], first rows [n_experts]
  int* counts = s_plan;
  int* first = s_plan + n_experts;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
  rb_pdl_wait();
  for (int r = threadIdx.x; r < n_tiles * tile; r += blockDim.x) row_token[r] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    pos[i] = e < n_experts ? atomicAdd(&counts[e], 1) : -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < n_experts; ++e) {
      first[e] = at;
      at += (counts[e] + tile - 1) / tile * tile;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int t0 = first[e] / tile, t1 = t0 + (counts[e] + tile - 1) / tile;
    for (int i = t0; i < t1 && i < n_tiles; ++i) tile_group[i] = e;
  }
  const int last = n_experts > 0 ? (first[n_experts - 1] + (counts[n_experts - 1] + tile - 1) / tile * tile) / tile : 0;
  for (int i = last + threadIdx.x; i < n_tiles; i += blockDim.x) tile_group[i] = -1;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < n_experts) {
      const int r = first[e] + pos[i];
      pos[i] = r;
      row_token[r] = i / top;
    }
  }
}

// ---------------------------------------------------------------- gather
// xp[r, :] = h[row_token[r], :], zeros for padding rows.
template <typename T>
__global__ void gather_kernel(T* __restrict__ xp, const T* __restrict__ h, int64_t ldh, const int* __restrict__ row_token,
                              int K) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int r = blockIdx.x;
  const int t = row_token[r];
  T* dst = xp + (int64_t)r * K;
  constexpr int PER = 16 / (int)sizeof(T);          // values in 16 bytes
  const bool vec = K % PER == 0 && ldh % PER == 0 && (uintptr_t)xp % 16 == 0 && (uintptr_t)h % 16 == 0;
  if (vec) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    if (t < 0) {
      for (int k = threadIdx.x; k < K / PER; k += blockDim.x) d4[k] = make_uint4(0, 0, 0, 0);
      return;
    }
    const uint4* s4 = reinterpret_cast<const uint4*>(h + (int64_t)t * ldh);
    for (int k = threadIdx.x; k < K / PER; k += blockDim.x) d4[k] = s4[k];
    return;
  }
  if (t < 0) {
    for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = rb_from_float<T>(0.f);
    return;
  }
  const T* src = h + (int64_t)t * ldh;
  for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = src[k];
}

// xp[r, :] = w * h[row_token[r], :] with w the weight of the pair that owns row r (the token's choice j with
// pos[token, j] == r), rounded to the rows' type; zeros for padding rows.
template <typename T>
__global__ void gather_scaled_kernel(T* __restrict__ xp, const T* __restrict__ h, int64_t ldh, const int* __restrict__ row_token,
                                     const int* __restrict__ pos, const float* __restrict__ weights, int top, int K) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int r = blockIdx.x;
  const int t = row_token[r];
  T* dst = xp + (int64_t)r * K;
  if (t < 0) {
    for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = rb_from_float<T>(0.f);
    return;
  }
  float w = 0.f;
  for (int j = 0; j < top; ++j)
    if (pos[(int64_t)t * top + j] == r) w = weights[(int64_t)t * top + j];
  const T* src = h + (int64_t)t * ldh;
  for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = rb_from_float<T>(w * rb_to_float<T>(src[k]));
}

// ---------------------------------------------------------------- weighted sum
// x[t, :] (+)= sum_j w[t, j] * (pos[t, j] >= 0 ? y[pos[t, j], :] : h[t, :]), the choices in their order.
template <typename T>
__global__ void combine_kernel(float* __restrict__ x, int64_t ldx, const float* __restrict__ y, const T* __restrict__ h,
                               int64_t ldh, const int* __restrict__ pos, const float* __restrict__ weights, int top, int E,
                               int accumulate, int vec4) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t = blockIdx.x;
  if (vec4) {
    // four columns a thread: 16-byte loads of the experts' rows and of the residual stream
    for (int c = threadIdx.x * 4; c < E; c += blockDim.x * 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < top; ++j) {
        const int r = pos[(int64_t)t * top + j];
        const float w = weights != nullptr ? weights[(int64_t)t * top + j] : 1.0f;
        float v[4];
        if (r >= 0) load4(y + (int64_t)r * E + c, v);
        else load4(h + (int64_t)t * ldh + c, v);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(w, v[i], acc[i]);
      }
      float4* dst = reinterpret_cast<float4*>(x + (int64_t)t * ldx + c);
      float4 out = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (accumulate) {
        const float4 old = *dst;
        out = make_float4(old.x + acc[0], old.y + acc[1], old.z + acc[2], old.w + acc[3]);
      }
      *dst = out;
    }
    return;
  }
  for (int c = threadIdx.x; c < E; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int r = pos[(int64_t)t * top + j];
      const float w = weights != nullptr ? weights[(int64_t)t * top + j] : 1.0f;
      const float v = r >= 0 ? y[(int64_t)r * E + c] : rb_to_float<T>(h[(int64_t)t * ldh + c]);
      acc = fmaf(w, v, acc);
    }
    float* dst = x + (int64_t)t * ldx + c;
    *dst = accumulate ? *dst + acc : acc;
  }
}

// ---------------------------------------------------------------- grouped float32 product
// C[rows, N] = act(A[rows, K] * W_g[N, K]^T) with g = tile_group[row / 64]: the plain tiled product of
// gemm_simple.cu (one sequential float32 sum over k per output element) whose weight matrix changes from
// one tile of 64 rows to the next.  Tiles without a group store zeros.
constexpr int GM = 64, GN = 64, GK = 16;

template <typename TA, typename TC>
__global__ void __launch_bounds__(256) gemm_grouped_kernel(TC* __restrict__ C, int64_t ldc, const TA* __restrict__ A,
                                                          int64_t lda, const TA* __restrict__ W, int64_t ldw,
                                                          const int* __restrict__ tile_group, int N, int K,
                                                          int square_relu) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  __shared__ float As[GK][GM + 1];
  __shared__ float Ws[GK][GN + 1];
  const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
  const int g = tile_group[blockIdx.y];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  if (g >= 0) {
    const TA* Wg = W + (int64_t)g * N * ldw;
    for (int k0 = 0; k0 < K; k0 += GK) {
      for (int e = threadIdx.x; e < GM * GK; e += 256) {
        const int r = e / GK, c = e % GK;
        const int gn = n0 + r, gk = k0 + c;
        As[c][r] = gk < K ? rb_to_float<TA>(A[(int64_t)(m0 + r) * lda + gk]) : 0.f;
        Ws[c][r] = (gn < N && gk < K) ? rb_to_float<TA>(Wg[(int64_t)gn * ldw + gk]) : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < GK; ++kk) {
        float a[4], w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (square_relu) { v = fmaxf(v, 0.f); v *= v; }
      C[(int64_t)gm * ldc + gn] = rb_from_float<TC>(v);
    }
  }
}

// ---------------------------------------------------------------- max(v, 0)^2, element by element
template <typename T>
__global__ void square_relu_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t n) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float v = fmaxf(rb_to_float<T>(in[i]), 0.f);
    out[i] = rb_from_float<T>(v * v);
  }
}

}  // namespace

// ids, weights: [T, top].  h: the input rows (dtype h_dtype).  Wr: float32 [n, K]; correction: float32 [n] or null.
// groups <= 1 or keep >= groups: every output can be chosen.  z_scratch: T * n floats (from 64 tokens on, the router's
// sums are a product of their own that leaves them there), or null.
static int route_impl(int* ids, float* weights, const void* h, int64_t ldh, int h_dtype, const float* Wr,
                      const float* correction, int T, int K, int n, int top, int groups, int keep, float* z_scratch,
                      int scoring, int n_extra, float* extra, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(scoring == 0 || scoring == 1, "rb_route: scoring %d is not built (0: softmax, 1: sigmoid)", scoring);
  RB_REQUIRE(n_extra >= 0 && (n_extra == 0 || extra != nullptr), "rb_route: %d extra rows and nowhere to leave them", n_extra);
  const int n_all = n + n_extra;
  RB_REQUIRE(K > 0 && n > 0 && top > 0 && top <= n, "rb_route: bad sizes K=%d outputs=%d top=%d", K, n, top);
  RB_REQUIRE(groups <= 1 || n % groups == 0, "rb_route: %d outputs are not %d equal groups", n, groups);
  if (groups < 1) groups = 1;
  // few tokens: a block each, so that the rows of Wr are read by many SMs at once; many: eight tokens a block
  if (T >= 64 && z_scratch != nullptr) {
    const size_t smem_sel = (size_t)4 * (2 * n + 2 * groups) * sizeof(float);
    RB_REQUIRE(smem_sel <= 48 * 1024, "rb_route: %d router outputs are more than a block's shared memory holds", n);
    const int blocks_l = (T + RL_TM - 1) / RL_TM;
    if (h_dtype == RB_F32)
      RB_LAUNCH("route_logits_kernel", (route_logits_kernel<float>), blocks_l, 256, 0, stream, z_scratch, (const float*)h, ldh, Wr, T, K, n_all);
    else if (h_dtype == RB_BF16)
      RB_LAUNCH("route_logits_kernel", (route_logits_kernel<__nv_bfloat16>), blocks_l, 256, 0, stream, z_scratch, (const __nv_bfloat16*)h, ldh, Wr, T, K, n_all);
    else
      RB_FAIL("rb_route: unknown dtype %d", h_dtype);
    RB_CHECK_LAUNCH("rb_route");
    RB_LAUNCH("route_select_kernel", (route_select_kernel), (T + 3) / 4, 128, smem_sel, stream, ids, weights, z_scratch, correction, T, n, top,
              groups, keep, scoring, n_extra, extra);
    RB_CHECK_LAUNCH("rb_route");
    return 0;
  }
  const int TB = T >= 64 ? ROUTE_TB : 1;
  const size_t smem = (size_t)TB * (2 * n_all + 2 * groups) * sizeof(float);
  RB_REQUIRE(smem <= 48 * 1024, "rb_route: %d router outputs are more than a block's shared memory holds", n);
  const int blocks = (T + TB - 1) / TB;
  const int elem = h_dtype == RB_F32 ? 4 : 2;
  const int vec = K % 4 == 0 && ldh % 4 == 0 && (uintptr_t)h % (4 * elem) == 0 && (uintptr_t)Wr % 16 == 0;
  if (h_dtype == RB_F32)
    RB_LAUNCH("route_kernel", (route_kernel<float>), blocks, 256, smem, stream, ids, weights, (const float*)h, ldh, Wr, correction, T, K, n, top, groups, keep, TB, vec, scoring, n_extra, extra);
  else if (h_dtype == RB_BF16)
    RB_LAUNCH("route_kernel", (route_kernel<__nv_bfloat16>), blocks, 256, smem, stream, ids, weights, (const __nv_bfloat16*)h, ldh, Wr, correction, T, K, n, top, groups, keep, TB, vec, scoring, n_extra, extra);
  else
    RB_FAIL("rb_route: unknown dtype %d", h_dtype);
  RB_CHECK_LAUNCH("rb_route");
  return 0;
}

RB_EXPORT int rb_route(int* ids, float* weights, const void* h, int64_t ldh, int h_dtype, const float* Wr,
                       const float* correction, int T, int K, int n, int top, int groups, int keep, float* z_scratch,
                       cudaStream_t stream) {
  return route_impl(ids, weights, h, ldh, h_dtype, Wr, correction, T, K, n, top, groups, keep, z_scratch, 0, 0, nullptr, stream);
}

// The same with the variants: scoring (0: softmax over the outputs, 1: a sigmoid per output); Wr holds n + n_extra rows
// and the sums of the last n_extra leave in extra [T, n_extra]; z_scratch then holds T * (n + n_extra) floats.
RB_EXPORT int rb_route_scored(int* ids, float* weights, const void* h, int64_t ldh, int h_dtype, const float* Wr,
                              const float* correction, int T, int K, int n, int top, int groups, int keep, float* z_scratch,
                              int scoring, int n_extra, float* extra, cudaStream_t stream) {
  return route_impl(ids, weights, h, ldh, h_dtype, Wr, correction, T, K, n, top, groups, keep, z_scratch, scoring, n_extra, extra,
                    stream);
}

// The choice alone, from router sums z [T, n] that a product has left (float32).
RB_EXPORT int rb_route_select(int* ids, float* weights, const float* z, const float* correction, int T, int n, int top,
                              int groups, int keep, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(n > 0 && top > 0 && top <= n, "rb_route_select: bad sizes outputs=%d top=%d", n, top);
  RB_REQUIRE(groups <= 1 || n % groups == 0, "rb_route_select: %d outputs are not %d equal groups", n, groups);
  if (groups < 1) groups = 1;
  const size_t smem_sel = (size_t)4 * (2 * n + 2 * groups) * sizeof(float);
  RB_REQUIRE(smem_sel <= 48 * 1024, "rb_route_select: %d router outputs are more than a block's shared memory holds", n);
  RB_LAUNCH("route_select_kernel", (route_select_kernel), (T + 3) / 4, 128, smem_sel, stream, ids, weights, z, correction, T, n, top,
            groups, keep, 0, 0, (float*)nullptr);
  RB_CHECK_LAUNCH("rb_route_select");
  return 0;
}

// The choice with the variants of rb_route_scored, from sums z [T, n + n_extra] that a product has left.
RB_EXPORT int rb_route_select_scored(int* ids, float* weights, const float* z, const float* correction, int T, int n, int top,
                                     int groups, int keep, int scoring, int n_extra, float* extra, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(n > 0 && top > 0 && top <= n && n_extra >= 0 && (n_extra == 0 || extra != nullptr),
             "rb_route_select_scored: bad sizes outputs=%d top=%d extra=%d", n, top, n_extra);
  RB_REQUIRE(groups <= 1 || n % groups == 0, "rb_route_select_scored: %d outputs are not %d equal groups", n, groups);
  if (groups < 1) groups = 1;
  const size_t smem_sel = (size_t)4 * (2 * n + 2 * groups) * sizeof(float);
  RB_REQUIRE(smem_sel <= 48 * 1024, "rb_route_select_scored: %d router outputs are more than a block's shared memory holds", n);
  RB_LAUNCH("route_select_kernel", (route_select_kernel), (T + 3) / 4, 128, smem_sel, stream, ids, weights, z, correction, T, n, top,
            groups, keep, scoring, n_extra, extra);
  RB_CHECK_LAUNCH("rb_route_select_scored");
  return 0;
}

// Tiles of rows the padded buffer needs at most for `pairs` pairs over n_experts experts.
RB_EXPORT int rb_routed_tiles(int pairs, int n_experts, int tile) {
  if (pairs <= 0 || tile <= 0) return 0;
  const int used = pairs < n_experts ? pairs : n_experts;       // experts that can have rows
  return (pairs + tile - 1) / tile + used;
}

RB_EXPORT int rb_routed_plan(int* pos, int* row_token, int* tile_group, const int* ids, int pairs, int top, int n_experts,
                             int tile, int n_tiles, cudaStream_t stream) {
  if (pairs == 0) return 0;
  RB_REQUIRE(n_experts >= 0 && top > 0 && tile > 0 && n_tiles >= rb_routed_tiles(pairs, n_experts, tile),
             "rb_routed_plan: %d tiles of %d rows for %d pairs over %d experts", n_tiles, tile, pairs, n_experts);
  const size_t smem = (size_t)(2 * n_experts + 1) * sizeof(int);
  RB_REQUIRE(smem <= 48 * 1024, "rb_routed_plan: %d experts", n_experts);
  RB_LAUNCH("plan_kernel", (plan_kernel), 1, 1024, smem, stream, pos, row_token, tile_group, ids, pairs, top, n_experts, tile, n_tiles);
  RB_CHECK_LAUNCH("rb_routed_plan");
  return 0;
}

RB_EXPORT int rb_routed_gather(void* xp, const void* h, int64_t ldh, int dtype, const int* row_token, int rows, int K,
                               cudaStream_t stream) {
  if (rows == 0) return 0;
  const int threads = K >= 256 ? 256 : (K >= 128 ? 128 : 64);
  if (dtype == RB_F32)
    RB_LAUNCH("gather_kernel", (gather_kernel<float>), rows, threads, 0, stream, (float*)xp, (const float*)h, ldh, row_token, K);
  else if (dtype == RB_BF16)
    RB_LAUNCH("gather_kernel", (gather_kernel<__nv_bfloat16>), rows, threads, 0, stream, (__nv_bfloat16*)xp, (const __nv_bfloat16*)h, ldh, row_token, K);
  else
    RB_FAIL("rb_routed_gather: unknown dtype %d", dtype);
  RB_CHECK_LAUNCH("rb_routed_gather");
  return 0;
}

// The gather with every row multiplied by its pair's weight (pos, weights: [T, top] as the plan and the router left them).
RB_EXPORT int rb_routed_gather_scaled(void* xp, const void* h, int64_t ldh, int dtype, const int* row_token, const int* pos,
                                      const float* weights, int top, int rows, int K, cudaStream_t stream) {
  if (rows == 0) return 0;
  const int threads = K >= 256 ? 256 : (K >= 128 ? 128 : 64);
  if (dtype == RB_F32)
    RB_LAUNCH("gather_scaled_kernel", (gather_scaled_kernel<float>), rows, threads, 0, stream, (float*)xp, (const float*)h, ldh, row_token, pos, weights, top, K);
  else if (dtype == RB_BF16)
    RB_LAUNCH("gather_scaled_kernel", (gather_scaled_kernel<__nv_bfloat16>), rows, threads, 0, stream, (__nv_bfloat16*)xp, (const __nv_bfloat16*)h, ldh, row_token, pos, weights, top, K);
  else
    RB_FAIL("rb_routed_gather_scaled: unknown dtype %d", dtype);
  RB_CHECK_LAUNCH("rb_routed_gather_scaled");
  return 0;
}

RB_EXPORT int rb_routed_combine(float* x, int64_t ldx, const float* y, const void* h, int64_t ldh, int h_dtype,
                                const int* pos, const float* weights, int T, int top, int E, int accumulate,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  const int elem = h_dtype == RB_F32 ? 4 : 2;
  const int vec4 = E % 4 == 0 && ldx % 4 == 0 && ldh % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 &&
                   (uintptr_t)h % (4 * elem) == 0;
  const int threads = vec4 ? (E >= 1024 ? 256 : (E >= 512 ? 128 : 64)) : (E >= 256 ? 256 : (E >= 128 ? 128 : 64));
  if (h_dtype == RB_F32)
    RB_LAUNCH("combine_kernel", (combine_kernel<float>), T, threads, 0, stream, x, ldx, y, (const float*)h, ldh, pos, weights, top, E, accumulate, vec4);
  else if (h_dtype == RB_BF16)
    RB_LAUNCH("combine_kernel", (combine_kernel<__nv_bfloat16>), T, threads, 0, stream, x, ldx, y, (const __nv_bfloat16*)h, ldh, pos, weights, top, E, accumulate, vec4);
  else
    RB_FAIL("rb_routed_combine: unknown dtype %d", h_dtype);
  RB_CHECK_LAUNCH("rb_routed_combine");
  return 0;
}

// rows: a multiple of 64 (tile_group has rows / 64 entries).  W: [groups * N, K], one matrix per group.
RB_EXPORT int rb_gemm_grouped_simple(void* C, int64_t ldc, int c_dtype, const void* A, int64_t lda, const void* W,
                                     int64_t ldw, int a_dtype, const int* tile_group, int rows, int N, int K,
                                     int square_relu, cudaStream_t stream) {
  if (rows == 0 || N == 0) return 0;
  RB_REQUIRE(rows % GM == 0 && N > 0 && K > 0, "rb_gemm_grouped_simple: %d rows (tiles of %d), N=%d K=%d", rows, GM, N, K);
  const dim3 grid((N + GN - 1) / GN, rows / GM);
  RB_REQUIRE(grid.y <= 65535, "rb_gemm_grouped_simple: %d rows are too many for one launch", rows);
#define LAUNCH(TA, TC)                                                                                                 \
  RB_LAUNCH("gemm_grouped_kernel", (gemm_grouped_kernel<TA, TC>), grid, 256, 0, stream, (TC*)C, ldc, (const TA*)A, lda, \
            (const TA*)W, ldw, tile_group, N, K, square_relu)
  if (a_dtype == RB_F32 && c_dtype == RB_F32) LAUNCH(float, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_F32) LAUNCH(__nv_bfloat16, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else RB_FAIL("rb_gemm_grouped_simple: unsupported dtypes a=%d c=%d", a_dtype, c_dtype);
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_gemm_grouped_simple");
  return 0;
}

RB_EXPORT int rb_square_relu(void* out, const void* in, int dtype, long long n, cudaStream_t stream) {
  if (n == 0) return 0;
  const long long most = (long long)rb_sm_count() * 16;
  const int blocks = (int)((n + 255) / 256 < most ? (n + 255) / 256 : most);
  if (dtype == RB_F32)
    RB_LAUNCH("square_relu_kernel", (square_relu_kernel<float>), blocks, 256, 0, stream, (float*)out, (const float*)in, (int64_t)n);
  else if (dtype == RB_BF16)
    RB_LAUNCH("square_relu_kernel", (square_relu_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)in, (int64_t)n);
  else
    RB_FAIL("rb_square_relu: unknown dtype %d", dtype);
  RB_CHECK_LAUNCH("rb_square_relu");
  return 0;
}
