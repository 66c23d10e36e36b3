// What stands around a sublayer in a block with filtered inputs and gated results:
//
//   grouped RMS norm   a row cut into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps),
//                      the whole multiplied by w
//   input filter       h_t + sum_j taps[:, j] h_(t - K + 1 + j) over time on every channel (causal, zeros before a
//                      sequence's start); the last K - 1 inputs of a sequence live in a ring of K rows by position
//   gated residual     x += y * sigmoid(g + b), value by value
//   scaled rows        y += sigmoid(logit_t) * z, one number per row
//   soft cap           v <- cap * tanh(v / cap)
//
// All arithmetic is float32; rows enter and leave in the compute dtype where they feed a product.
#include "rb_common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_(float v) { return 1.0f / (1.0f + expf(-v)); }

// ---------------------------------------------------------------- grouped RMS norm
// A block per row; a warp takes the row's parts in turn (two passes over the part: the sum of squares, then the
// values; the second pass finds the part in the SM's cache).
__device__ __forceinline__ void store4(float* d, float a, float b, float c, float e) {
  *reinterpret_cast<float4*>(d) = make_float4(a, b, c, e);
}
__device__ __forceinline__ void store4(__nv_bfloat16* d, float a, float b, float c, float e) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(d) = u;
}

template <typename TO>
__global__ void __launch_bounds__(256) rmsnorm_grouped_kernel(TO* __restrict__ out, const float* __restrict__ x,
                                                              const float* __restrict__ w, int E, int groups, float eps,
                                                              int vec) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int per = E / groups;
  const float* row = x + (int64_t)blockIdx.x * E;
  TO* dst = out + (int64_t)blockIdx.x * E;
  for (int g = warp; g < groups; g += nw) {
    const float* p = row + (int64_t)g * per;
    float ss = 0.f;
    if (vec) {
      // 16 bytes a load; a part of up to 1,024 values stays in the lane's registers between the two passes
      float4 keep[8];
      const int n4 = per >> 2;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = lane + 32 * u;
        if (i < n4) {
          keep[u] = reinterpret_cast<const float4*>(p)[i];
          ss = fmaf(keep[u].x, keep[u].x, fmaf(keep[u].y, keep[u].y, fmaf(keep[u].z, keep[u].z, fmaf(keep[u].w, keep[u].w, ss))));
        }
      }
      for (int i = lane + 256; i < n4; i += 32) {
        const float4 v = reinterpret_cast<const float4*>(p)[i];
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
      }
      ss = rb_warp_sum(ss);
      const float r = 1.0f / sqrtf(ss / (float)per + eps);
      const float4* w4 = reinterpret_cast<const float4*>(w + (int64_t)g * per);
      TO* d = dst + (int64_t)g * per;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = lane + 32 * u;
        if (i < n4) {
          const float4 ww = w4[i];
          store4(d + 4 * i, keep[u].x * r * ww.x, keep[u].y * r * ww.y, keep[u].z * r * ww.z, keep[u].w * r * ww.w);
        }
      }
      for (int i = lane + 256; i < n4; i += 32) {
        const float4 v = reinterpret_cast<const float4*>(p)[i];
        const float4 ww = w4[i];
        store4(d + 4 * i, v.x * r * ww.x, v.y * r * ww.y, v.z * r * ww.z, v.w * r * ww.w);
      }
      continue;
    }
    for (int i = lane; i < per; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = rb_warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)per + eps);
    for (int i = lane; i < per; i += 32) dst[(int64_t)g * per + i] = rb_from_float<TO>(p[i] * r * w[g * per + i]);
  }
}

// ---------------------------------------------------------------- input filter
// out[t, c] = h[t, c] + sum_d taps[c, K-1-d] * h(d rows back), rows before the run taken from the ring (zeros before
// position 0).  With `update` (every row is its own run) the row also goes into the ring at its position: the rows it
// read lie at other positions of the ring.
template <typename T>
__global__ void input_filter_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ taps,
                                    float* __restrict__ ring, const int* __restrict__ tok_first,
                                    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, int n_tokens, int C,
                                    int K, int update, int per_block) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  for (int t = blockIdx.x * per_block; t < min(n_tokens, (int)(blockIdx.x + 1) * per_block); ++t) {
    const int first = tok_first != nullptr ? tok_first[t] : t;
    const int slot = tok_slot[t], pos = tok_pos[t];
    const int j = t - first;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
      const float own = rb_to_float<T>(h[(int64_t)t * C + c]);
      float acc = own;
      for (int d = 0; d < K; ++d) {
        float v;
        if (d == 0) v = own;
        else if (d <= j) v = rb_to_float<T>(h[(int64_t)(t - d) * C + c]);
        else if (pos - d < 0) v = 0.f;
        else v = ring[((int64_t)slot * K + (pos - d) % K) * C + c];
        acc = fmaf(taps[(int64_t)c * K + (K - 1 - d)], v, acc);
      }
      out[(int64_t)t * C + c] = rb_from_float<T>(acc);
      if (update && K > 1) ring[((int64_t)slot * K + pos % K) * C + c] = own;
    }
  }
}

// The same for widths and addresses that allow 16 bytes a load and at most KM taps: a thread owns V neighbouring
// channels, keeps their taps in registers, and takes the block's rows in turn (the rows behind a row were just read
// by the same block and come from the SM's cache).
template <typename T, int V> struct FilterVec;
template <> struct FilterVec<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct FilterVec<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(b[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 a;
    __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
    for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = a;
  }
};

template <typename T, int V, int KM>
__global__ void __launch_bounds__(256) input_filter_vec_kernel(T* __restrict__ out, const T* __restrict__ h,
                                                               const float* __restrict__ taps, float* __restrict__ ring,
                                                               const int* __restrict__ tok_first,
                                                               const int* __restrict__ tok_slot,
                                                               const int* __restrict__ tok_pos, int n_tokens, int C, int K,
                                                               int update, int per_block) {
  rb_pdl_launch_dependents();
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (c0 >= C) return;
  float w[KM][V];                                  // w[d][v]: the tap on the row d back
#pragma unroll
  for (int d = 0; d < KM; ++d)
#pragma unroll
    for (int v = 0; v < V; ++v) w[d][v] = d < K ? taps[(int64_t)(c0 + v) * K + (K - 1 - d)] : 0.f;
  rb_pdl_wait();
  for (int t = blockIdx.x * per_block; t < min(n_tokens, (int)(blockIdx.x + 1) * per_block); ++t) {
    const int first = tok_first != nullptr ? tok_first[t] : t;
    const int slot = tok_slot[t], pos = tok_pos[t];
    const int j = t - first;
    float own[V], acc[V];
    FilterVec<T, V>::load(h + (int64_t)t * C + c0, own);
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = fmaf(w[0][v], own[v], own[v]);
#pragma unroll
    for (int d = 1; d < KM; ++d) {
      if (d >= K || (d > j && pos - d < 0)) continue;
      float x[V];
      if (d <= j) {
        FilterVec<T, V>::load(h + (int64_t)(t - d) * C + c0, x);
      } else {
        const float* r = ring + ((int64_t)slot * K + (pos - d) % K) * C + c0;
#pragma unroll
        for (int v = 0; v < V; v += 4) FilterVec<float, 4>::load(r + v, x + v);
      }
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = fmaf(w[d][v], x[v], acc[v]);
    }
    FilterVec<T, V>::store(out + (int64_t)t * C + c0, acc);
    if (update && K > 1) {
      float* r = ring + ((int64_t)slot * K + pos % K) * C + c0;
#pragma unroll
      for (int v = 0; v < V; v += 4) FilterVec<float, 4>::store(r + v, own + v);
    }
  }
}

// ---------------------------------------------------------------- a decode step's rows between two sublayers
// For rows that are each their own run: the gated result of the sublayer before (x += y * sigmoid(g + b); y null: none),
// the norm in groups of the new x (h), and the filter on h from the ring (hf), whose row at the token's position
// becomes h.  A block of eight warps per row and part of the row.
template <typename TO>
__global__ void __launch_bounds__(256) norm_filter_rows_kernel(TO* __restrict__ h, TO* __restrict__ hf, float* __restrict__ x,
                                                               const float* __restrict__ y, const float* __restrict__ g,
                                                               int64_t ldg, const float* __restrict__ bias,
                                                               const float* __restrict__ w, int E, int groups, float eps,
                                                               const float* __restrict__ taps, float* __restrict__ ring,
                                                               const int* __restrict__ tok_slot,
                                                               const int* __restrict__ tok_pos, int K) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int t = blockIdx.x, per = E / groups;
  const int slot = tok_slot[t], pos = tok_pos[t];
  float* row = x + (int64_t)t * E;
  // blockIdx.y takes the row's parts in turn; all of the block's warps share a part
  __shared__ float s_parts[8];                     // the warps' sums of squares
  const int share = nw;
  const int per4 = per >> 2;                         // 16 bytes a load: a lane takes four neighbouring channels at a time
  for (int part = blockIdx.y; part < groups; part += gridDim.y) {
    const int sub = warp;
    const int c0 = part * per;
    float ss = 0.f;
    for (int i4 = sub * 32 + lane; i4 < per4; i4 += share * 32) {
      const int c = c0 + 4 * i4;
      float4 v = *reinterpret_cast<const float4*>(row + c);
      if (y != nullptr) {
        const float4 yy = *reinterpret_cast<const float4*>(y + (int64_t)t * E + c);
        float4 z = *reinterpret_cast<const float4*>(g + (int64_t)t * ldg + c);
        if (bias != nullptr) {
          const float4 bb = *reinterpret_cast<const float4*>(bias + c);
          z.x += bb.x; z.y += bb.y; z.z += bb.z; z.w += bb.w;
        }
        v.x = fmaf(yy.x, sigmoid_(z.x), v.x);
        v.y = fmaf(yy.y, sigmoid_(z.y), v.y);
        v.z = fmaf(yy.z, sigmoid_(z.z), v.z);
        v.w = fmaf(yy.w, sigmoid_(z.w), v.w);
        *reinterpret_cast<float4*>(row + c) = v;
      }
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = rb_warp_sum(ss);
    __syncthreads();                               // (the sums of the part before have been read)
    if (lane == 0) s_parts[warp] = ss;
    __syncthreads();
    ss = 0.f;
    for (int k = 0; k < share; ++k) ss += s_parts[k];
    const float r = 1.0f / sqrtf(ss / (float)per + eps);
    for (int i4 = sub * 32 + lane; i4 < per4; i4 += share * 32) {
      const int c = c0 + 4 * i4;
      const float4 v = *reinterpret_cast<const float4*>(row + c);          // (the lane reads what it wrote itself)
      const float4 ww = *reinterpret_cast<const float4*>(w + c);
      float own[4] = {v.x * r * ww.x, v.y * r * ww.y, v.z * r * ww.z, v.w * r * ww.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) own[q] = rb_to_float<TO>(rb_from_float<TO>(own[q]));    // as the rows leave
      store4(h + (int64_t)t * E + c, own[0], own[1], own[2], own[3]);
      float acc[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[q] = fmaf(taps[(int64_t)(c + q) * K + (K - 1)], own[q], own[q]);
      for (int d = 1; d < K; ++d) {
        if (pos - d < 0) break;
        const float4 rr = *reinterpret_cast<const float4*>(ring + ((int64_t)slot * K + (pos - d) % K) * E + c);
        acc[0] = fmaf(taps[(int64_t)(c + 0) * K + (K - 1 - d)], rr.x, acc[0]);
        acc[1] = fmaf(taps[(int64_t)(c + 1) * K + (K - 1 - d)], rr.y, acc[1]);
        acc[2] = fmaf(taps[(int64_t)(c + 2) * K + (K - 1 - d)], rr.z, acc[2]);
        acc[3] = fmaf(taps[(int64_t)(c + 3) * K + (K - 1 - d)], rr.w, acc[3]);
      }
      store4(hf + (int64_t)t * E + c, acc[0], acc[1], acc[2], acc[3]);
      if (K > 1) *reinterpret_cast<float4*>(ring + ((int64_t)slot * K + pos % K) * E + c) = make_float4(own[0], own[1], own[2], own[3]);
    }
  }
}

// ---------------------------------------------------------------- gated residual
template <typename TG>
__global__ void gated_add_kernel(float* __restrict__ x, const float* __restrict__ y, const TG* __restrict__ g, int64_t ldg,
                                 const float* __restrict__ bias, int64_t n, int E) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / E;
    const int c = (int)(i - t * E);
    const float z = rb_to_float<TG>(g[t * ldg + c]) + (bias != nullptr ? bias[c] : 0.f);
    x[i] = fmaf(y[i], sigmoid_(z), x[i]);
  }
}

__global__ void add_scaled_rows_kernel(float* __restrict__ y, const float* __restrict__ z, const float* __restrict__ logit,
                                       int64_t ldl, int64_t n, int E) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / E;
    y[i] = fmaf(z[i], sigmoid_(logit[t * ldl]), y[i]);
  }
}

__global__ void softcap_kernel(float* __restrict__ v, int64_t n, float cap) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const float inv = 1.0f / cap;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    v[i] = cap * tanhf(v[i] * inv);
}

inline int flat_blocks(int64_t n, int threads) {
  const int64_t most = (int64_t)rb_sm_count() * 16;
  const int64_t want = (n + threads - 1) / threads;
  return (int)(want < most ? want : most);
}

}  // namespace

RB_EXPORT int rb_rmsnorm_grouped(void* out, int out_dtype, const float* x, const float* w, int T, int E, int groups,
                                 float eps, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(groups >= 1 && E > 0 && E % groups == 0, "rb_rmsnorm_grouped: a row of %d values is not %d equal parts", E, groups);
  const int threads = groups >= 8 ? 256 : 32 * groups;
  const int vec = (E / groups) % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0;
  if (out_dtype == RB_F32)
    RB_LAUNCH("rmsnorm_grouped_kernel", (rmsnorm_grouped_kernel<float>), T, threads, 0, stream, (float*)out, x, w, E, groups, eps, vec);
  else if (out_dtype == RB_BF16)
    RB_LAUNCH("rmsnorm_grouped_kernel", (rmsnorm_grouped_kernel<__nv_bfloat16>), T, threads, 0, stream, (__nv_bfloat16*)out, x, w, E, groups, eps, vec);
  else
    RB_FAIL("rb_rmsnorm_grouped: unknown dtype %d", out_dtype);
  RB_CHECK_LAUNCH("rb_rmsnorm_grouped");
  return 0;
}

// h, out: [T, C] in `dtype`; taps: float32 [C, K]; ring: float32 [n_slots, K, C].  tok_first: per row the first row of
// its run, or null when every row is its own run (the ring is then moved on here; else rb_conv_tail_update does it).
RB_EXPORT int rb_input_filter(void* out, const void* h, int dtype, const float* taps, float* ring, const int* tok_first,
                              const int* tok_slot, const int* tok_pos, int T, int C, int K, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(C > 0 && K >= 1, "rb_input_filter: bad sizes C=%d K=%d", C, K);
  const int update = tok_first == nullptr ? 1 : 0;
  {
    constexpr int KM = 4;
    const int V = dtype == RB_F32 ? 4 : 8;
    const bool aligned = (uintptr_t)out % 16 == 0 && (uintptr_t)h % 16 == 0 && (ring == nullptr || (uintptr_t)ring % 16 == 0);
    if (K <= KM && C % V == 0 && aligned && (dtype == RB_F32 || dtype == RB_BF16)) {
      const int lanes = C / V;
      const int threads = lanes >= 256 ? 256 : ((lanes + 31) / 32) * 32;
      const int per_block = T >= 512 ? 4 : 1;
      const dim3 grid((T + per_block - 1) / per_block, (lanes + threads - 1) / threads);
      RB_REQUIRE(grid.y <= 65535, "rb_input_filter: %d channels are too many for one launch", C);
      if (dtype == RB_F32)
        RB_LAUNCH("input_filter_vec_kernel", (input_filter_vec_kernel<float, 4, KM>), grid, threads, 0, stream, (float*)out, (const float*)h, taps, ring, tok_first, tok_slot, tok_pos, T, C, K, update, per_block);
      else
        RB_LAUNCH("input_filter_vec_kernel", (input_filter_vec_kernel<__nv_bfloat16, 8, KM>), grid, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)h, taps, ring, tok_first, tok_slot, tok_pos, T, C, K, update, per_block);
      RB_CHECK_LAUNCH("rb_input_filter");
      return 0;
    }
  }
  const int threads = 128;
  int by = (C + threads - 1) / threads;
  if (by > 64) by = 64;
  const int per_block = T >= 512 ? 8 : 1;
  const dim3 grid((T + per_block - 1) / per_block, by);
  if (dtype == RB_F32)
    RB_LAUNCH("input_filter_kernel", (input_filter_kernel<float>), grid, threads, 0, stream, (float*)out, (const float*)h, taps, ring, tok_first, tok_slot, tok_pos, T, C, K, update, per_block);
  else if (dtype == RB_BF16)
    RB_LAUNCH("input_filter_kernel", (input_filter_kernel<__nv_bfloat16>), grid, threads, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)h, taps, ring, tok_first, tok_slot, tok_pos, T, C, K, update, per_block);
  else
    RB_FAIL("rb_input_filter: unknown dtype %d", dtype);
  RB_CHECK_LAUNCH("rb_input_filter");
  return 0;
}

// Whether these sizes take rb_norm_filter_rows: parts of the row and the gate's rows in multiples of four values.
RB_EXPORT int rb_norm_filter_rows_supports(int E, int groups, long long ldg) {
  return groups >= 1 && E > 0 && E % groups == 0 && (E / groups) % 4 == 0 && ldg % 4 == 0;
}

// Rows that are each their own run (a decode step): x += y * sigmoid(g + bias) (y null: nothing is added), then
// h = norm in groups of x, hf = h filtered from the ring [n_slots, K, E], which takes h at the row's position.
RB_EXPORT int rb_norm_filter_rows(void* h, void* hf, int dtype, float* x, const float* y, const float* g, int64_t ldg,
                                  const float* bias, const float* w, int T, int E, int groups, float eps, const float* taps,
                                  float* ring, const int* tok_slot, const int* tok_pos, int K, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(groups >= 1 && E > 0 && E % groups == 0 && K >= 1 && (K == 1 || ring != nullptr),
             "rb_norm_filter_rows: bad sizes E=%d groups=%d K=%d", E, groups, K);
  RB_REQUIRE(rb_norm_filter_rows_supports(E, groups, ldg) && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 &&
                 (uintptr_t)g % 16 == 0 && (uintptr_t)bias % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)ring % 16 == 0 &&
                 (uintptr_t)h % 16 == 0 && (uintptr_t)hf % 16 == 0,
             "rb_norm_filter_rows: parts of %d values or addresses do not allow 16 bytes a load", E / groups);
  const int threads = 256;
  const size_t smem = 0;
  const dim3 grid(T, groups < 64 ? groups : 64);
  if (dtype == RB_F32)
    RB_LAUNCH("norm_filter_rows_kernel", (norm_filter_rows_kernel<float>), grid, threads, smem, stream, (float*)h, (float*)hf, x, y, g, ldg, bias, w, E, groups, eps, taps, ring, tok_slot, tok_pos, K);
  else if (dtype == RB_BF16)
    RB_LAUNCH("norm_filter_rows_kernel", (norm_filter_rows_kernel<__nv_bfloat16>), grid, threads, smem, stream, (__nv_bfloat16*)h, (__nv_bfloat16*)hf, x, y, g, ldg, bias, w, E, groups, eps, taps, ring, tok_slot, tok_pos, K);
  else
    RB_FAIL("rb_norm_filter_rows: unknown dtype %d", dtype);
  RB_CHECK_LAUNCH("rb_norm_filter_rows");
  return 0;
}

// x [T, E] += y [T, E] * sigmoid(g[t, c] + bias[c]); g has rows of ldg values in g_dtype.
RB_EXPORT int rb_gated_add(float* x, const float* y, const void* g, int64_t ldg, int g_dtype, const float* bias, int T, int E,
                           cudaStream_t stream) {
  if (T == 0) return 0;
  const int64_t n = (int64_t)T * E;
  if (g_dtype == RB_F32)
    RB_LAUNCH("gated_add_kernel", (gated_add_kernel<float>), flat_blocks(n, 256), 256, 0, stream, x, y, (const float*)g, ldg, bias, n, E);
  else if (g_dtype == RB_BF16)
    RB_LAUNCH("gated_add_kernel", (gated_add_kernel<__nv_bfloat16>), flat_blocks(n, 256), 256, 0, stream, x, y, (const __nv_bfloat16*)g, ldg, bias, n, E);
  else
    RB_FAIL("rb_gated_add: unknown dtype %d", g_dtype);
  RB_CHECK_LAUNCH("rb_gated_add");
  return 0;
}

// y [T, E] += sigmoid(logit[t * ldl]) * z [T, E]
RB_EXPORT int rb_add_scaled_rows(float* y, const float* z, const float* logit, int64_t ldl, int T, int E, cudaStream_t stream) {
  if (T == 0) return 0;
  const int64_t n = (int64_t)T * E;
  RB_LAUNCH("add_scaled_rows_kernel", (add_scaled_rows_kernel), flat_blocks(n, 256), 256, 0, stream, y, z, logit, ldl, n, E);
  RB_CHECK_LAUNCH("rb_add_scaled_rows");
  return 0;
}

RB_EXPORT int rb_softcap(float* v, long long n, float cap, cudaStream_t stream) {
  if (n == 0) return 0;
  RB_REQUIRE(cap > 0.f, "rb_softcap: the cap must be positive");
  RB_LAUNCH("softcap_kernel", (softcap_kernel), flat_blocks(n, 256), 256, 0, stream, v, (int64_t)n, cap);
  RB_CHECK_LAUNCH("rb_softcap");
  return 0;
}
