// Kernels between the products of a layer whose sublayers read the residual stream itself and whose results are
// normed, and the kernels that prepare queries, keys and values from float32 projections.  All arithmetic is float32;
// T below is the compute dtype (of q, of the cache and of rows that enter a product).
//
//   round_rows_kernel          x (float32) -> compute dtype
//   norm_add_kernel            x += y / rms(y) * w  (y a sublayer's float32 result); optionally also x in the compute dtype
//   token_gate_kernel          gelu_tanh(a) * table[id]
//   embed_pairs_kernel         table[id] * scale + pairs[(previous * a + id * b) mod n] (a sequence's first token: row n);
//                              the sequence's last token is kept per slot
//   qk_prepare_kernel          per token, from rows [q | k | v | gates]: short causal convolution of q and k over time,
//                              RMS norm (over a whole projection, or per head with one shared weight), rotation of a
//                              prefix of every head, k and v (own, mixed with another layer's, or the keys before the
//                              norm) into the paged cache, the gates' logits passed on
//   latent_rotate_append_kernel  per token, from rows [q heads of D + R | latent C | shared key part R]: the latent
//                              under its RMS norm and the turned key part go into the cache row [c | k_r | 0], the
//                              queries leave with their last R values turned
//   rotate_rows_kernel         float32 rows in place: a prefix of every head turned by position
#include "rb_common.cuh"

namespace {

// position * frequency in float64, brought into (-pi, pi] before the float32 sine and cosine
__device__ __forceinline__ void angle_sincos(int pos, double freq, float magnitude, float* sn, float* cs) {
  const double a = (double)pos * freq;
  const double turns = rint(a * 0.15915494309189535);
  const float r = (float)fma(-turns, 6.283185307179586, a);
  sincosf(r, sn, cs);
  *sn *= magnitude;
  *cs *= magnitude;
}

// value e of a head after the rotation of its first rot_dim values; val(i) gives the head's value i before it
template <typename F>
__device__ __forceinline__ float turned(F val, int e, int rot_dim, int interleaved, const float* s_sincos) {
  if (e >= rot_dim) return val(e);
  const int rhalf = rot_dim >> 1;
  int pair, other;
  bool first;
  if (interleaved) { pair = e >> 1; first = (e & 1) == 0; other = first ? e + 1 : e - 1; }
  else { first = e < rhalf; pair = first ? e : e - rhalf; other = first ? e + rhalf : e - rhalf; }
  const float sn = s_sincos[pair], cs = s_sincos[rhalf + pair];
  const float me = val(e), ot = val(other);
  return first ? me * cs - ot * sn : me * cs + ot * sn;
}

// one or two neighbouring values (two: the address is a multiple of two values)
template <typename T> __device__ __forceinline__ void rb_store_values(T* dst, const float* y, int n);
template <> __device__ __forceinline__ void rb_store_values<float>(float* dst, const float* y, int n) {
  if (n == 2) *reinterpret_cast<float2*>(dst) = make_float2(y[0], y[1]);
  else dst[0] = y[0];
}
template <> __device__ __forceinline__ void rb_store_values<__nv_bfloat16>(__nv_bfloat16* dst, const float* y, int n) {
  if (n == 2) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(y[0], y[1]);
  else dst[0] = __float2bfloat16_rn(y[0]);
}

template <typename T>
__global__ void __launch_bounds__(256) round_rows_kernel(T* __restrict__ out, const float* __restrict__ x, int64_t n) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  // four values a thread and turn where the addresses allow 16-byte loads, the rest value by value
  const bool vec = ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % (4 * sizeof(T)) == 0);
  const int64_t n4 = vec ? n / 4 : 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(x + 4 * i);
    const float y[4] = {v.x, v.y, v.z, v.w};
    rb_store_values<T>(out + 4 * i, y, 2);
    rb_store_values<T>(out + 4 * i + 2, y + 2, 2);
  }
  for (int64_t i = 4 * n4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = rb_from_float<T>(x[i]);
}

// A block per row.  VEC: the row is read four values at a time (E a multiple of 4, aligned rows).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) norm_add_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                       const float* __restrict__ w, float eps, int E,
                                                       T* __restrict__ rounded) {
  rb_pdl_launch_dependents();
  __shared__ float scratch[33];
  rb_pdl_wait();
  const int64_t row = blockIdx.x;
  const float* yr = y + row * E;
  float* xr = x + row * E;
  float ss = 0.f;
  if (VEC) {
    for (int e = threadIdx.x * 4; e < E; e += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(yr + e);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int e = threadIdx.x; e < E; e += blockDim.x) ss += yr[e] * yr[e];
  }
  ss = rb_block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)E + eps);
  if (VEC) {
    for (int e = threadIdx.x * 4; e < E; e += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(yr + e);
      const float4 ww = *reinterpret_cast<const float4*>(w + e);
      float4 o = *reinterpret_cast<const float4*>(xr + e);
      o.x += v.x * r * ww.x; o.y += v.y * r * ww.y; o.z += v.z * r * ww.z; o.w += v.w * r * ww.w;
      *reinterpret_cast<float4*>(xr + e) = o;
      if (rounded != nullptr) {
        T* d = rounded + row * E + e;
        d[0] = rb_from_float<T>(o.x); d[1] = rb_from_float<T>(o.y); d[2] = rb_from_float<T>(o.z); d[3] = rb_from_float<T>(o.w);
      }
    }
  } else {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const float o = xr[e] + yr[e] * r * w[e];
      xr[e] = o;
      if (rounded != nullptr) rounded[row * E + e] = rb_from_float<T>(o);
    }
  }
}

__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T, typename TT>
__global__ void __launch_bounds__(256) token_gate_kernel(T* __restrict__ out, const float* __restrict__ a, int64_t lda,
                                                         const TT* __restrict__ table, const int* __restrict__ ids,
                                                         int64_t n, int dim) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / dim;
    const int j = (int)(i % dim);
    out[i] = rb_from_float<T>(gelu_tanh_(a[t * lda + j]) * rb_to_float<TT>(table[(int64_t)ids[t] * dim + j]));
  }
}

// A block per row.  add: the embedded rows are made; update: the run's last row leaves its token in `previous`.
// single: every row is a run of its own (a decode step; rows that pad a captured step may share a slot).  A step of
// runs of several rows takes two launches (add, then update), because a run's first row reads what its last row writes.
template <typename TT>
__global__ void __launch_bounds__(256) embed_pairs_kernel(float* __restrict__ out, const TT* __restrict__ table,
                                                          const TT* __restrict__ pairs, const int* __restrict__ ids,
                                                          const int* __restrict__ tok_pos, const int* __restrict__ tok_slot,
                                                          int* __restrict__ previous, int T, int E, int V, float scale,
                                                          int buckets, int mul_prev, int mul_cur, int add, int update,
                                                          int single) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int t = blockIdx.x;
  const int slot = tok_slot[t], pos = tok_pos[t];
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const bool first = single || t == 0 || tok_slot[t - 1] != slot;
  const bool last = single || t == T - 1 || tok_slot[t + 1] != slot;
  if (add) {
    int row = buckets;
    if (pos > 0) {
      int prev = first ? previous[slot] : ids[t - 1];
      prev = prev < 0 ? 0 : (prev >= V ? V - 1 : prev);
      row = (int)(((int64_t)prev * mul_prev + (int64_t)id * mul_cur) % buckets);
    }
    const TT* a = table + (int64_t)id * E;
    const TT* b = pairs + (int64_t)row * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      out[(int64_t)t * E + e] = rb_to_float<TT>(a[e]) * scale + rb_to_float<TT>(b[e]);
  }
  if (update && last) {
    __syncthreads();                 // every thread of a single row's block has read the old value
    if (threadIdx.x == 0) previous[slot] = id;
  }
}

struct QkParams {
  const float* proj; int64_t ld;
  const float* conv_w; int K; float* tail; const int* tok_first;     // taps [C, K]; ring [n_slots, K, C]; null: rows are runs
  int norm_mode;                                                     // 0 none, 1 whole projection, 2 per head, one weight
  const float* q_norm_w; const float* k_norm_w; float eps;
  const double* freq; float magnitude; int rot_dim; int interleaved;
  const int* tok_pos; const int* tok_slot;
  int H, D, Dv;
  int values_are_keys;
  const float* mix_rows; int64_t mix_ld; float mix_weight;           // another layer's values of the same rows, or null
  int gate_heads;
};

// A block per token.  Shared memory: rot_dim sines and cosines, the C = (H + Kh) D convolved q and k values, a factor
// per head.
template <typename T>
__global__ void __launch_bounds__(1024) qk_prepare_kernel(T* __restrict__ q_out, T* __restrict__ gates_out, QkParams p,
                                                         RbPagedLayer cache) {
  rb_pdl_launch_dependents();
  __shared__ float scratch[33];
  extern __shared__ float s_mem[];
  const int H = p.H, D = p.D, Dv = p.Dv, Kh = cache.n_kv_heads, Dc = cache.head_dim;
  const int C = (H + Kh) * D;
  float* s_sincos = s_mem;
  float* s_qk = s_mem + p.rot_dim;
  float* s_fac = s_qk + C;
  const int t = blockIdx.x;
  const int pos = p.tok_pos[t], slot = p.tok_slot[t];
  for (int i = threadIdx.x; i < p.rot_dim / 2; i += blockDim.x)
    angle_sincos(pos, p.freq[i], p.magnitude, &s_sincos[i], &s_sincos[p.rot_dim / 2 + i]);
  rb_pdl_wait();
  const float* row = p.proj + (int64_t)t * p.ld;
  if (p.conv_w != nullptr) {
    // tap by tap over all channels, so that a thread's loads of one pass do not wait for one another
    const int K = p.K;
    const int pos0 = p.tok_first != nullptr ? p.tok_pos[p.tok_first[t]] : pos;     // the run's first position
    for (int c = threadIdx.x; c < C; c += blockDim.x) s_qk[c] = p.conv_w[(int64_t)c * K + K - 1] * row[c];
    for (int back = 1; back < K && back <= pos; ++back) {
      const int at = pos - back;
      const float* src = at >= pos0 ? row - (int64_t)back * p.ld : p.tail + ((int64_t)slot * K + at % K) * C;
      for (int c = threadIdx.x; c < C; c += blockDim.x)
        s_qk[c] = fmaf(p.conv_w[(int64_t)c * K + K - 1 - back], src[c], s_qk[c]);
    }
    if (p.tok_first == nullptr && K > 1)                                           // a row that is its own run
      for (int c = threadIdx.x; c < C; c += blockDim.x) p.tail[((int64_t)slot * K + pos % K) * C + c] = row[c];
  } else {
    for (int c = threadIdx.x; c < C; c += blockDim.x) s_qk[c] = row[c];
  }
  __syncthreads();
  if (p.norm_mode == 1) {
    float ss = 0.f;
    for (int e = threadIdx.x; e < H * D; e += blockDim.x) ss += s_qk[e] * s_qk[e];
    ss = rb_block_sum(ss, scratch);
    const float rq = 1.0f / sqrtf(ss / (float)(H * D) + p.eps);
    ss = 0.f;
    for (int e = threadIdx.x; e < Kh * D; e += blockDim.x) ss += s_qk[H * D + e] * s_qk[H * D + e];
    ss = rb_block_sum(ss, scratch);
    const float rk = 1.0f / sqrtf(ss / (float)(Kh * D) + p.eps);
    for (int h = threadIdx.x; h < H + Kh; h += blockDim.x) s_fac[h] = h < H ? rq : rk;
  } else if (p.norm_mode == 2) {
    const int lane = threadIdx.x & 31;
    for (int h = threadIdx.x >> 5; h < H + Kh; h += blockDim.x >> 5) {
      float ss = 0.f;
      for (int e = lane; e < D; e += 32) ss += s_qk[h * D + e] * s_qk[h * D + e];
      ss = rb_warp_sum(ss);
      if (lane == 0) s_fac[h] = 1.0f / sqrtf(ss / (float)D + p.eps);
    }
  }
  __syncthreads();
  T* kdst = (T*)cache.k;
  T* vdst = (T*)cache.v;
  // a warp takes a head at a time (no division per value); a lane makes `step` neighbouring values of it at a time
  // (two where the cache rows have an even width)
  const int step = (Dc & 1) ? 1 : 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int mode = p.norm_mode;
  for (int head = warp; head < H + Kh; head += n_warps) {
    const bool is_q = head < H;
    T* dst = is_q ? q_out + ((int64_t)t * H + head) * Dc : kdst + rb_page_offset(cache, slot, pos, head - H);
    const float* src = s_qk + head * D;
    const float* nw = (is_q ? p.q_norm_w : p.k_norm_w) + (mode == 1 ? (is_q ? head : head - H) * D : 0);
    const float fac = mode ? s_fac[head] : 1.f;
    auto val = [&](int i) { return mode ? src[i] * fac * nw[i] : src[i]; };
    for (int e0 = lane * step; e0 < Dc; e0 += 32 * step) {
      float y[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int e = e0 + k;
        y[k] = (k < step && e < D) ? turned(val, e, p.rot_dim, p.interleaved, s_sincos) : 0.f;
      }
      rb_store_values<T>(dst + e0, y, step);
    }
  }
  const int v_at = C;                                        // own values follow the keys in a row
  for (int kvh = warp; kvh < Kh; kvh += n_warps) {
    T* dst = vdst + rb_page_offset(cache, slot, pos, kvh);
    const float* own = row + v_at + kvh * Dv;
    const float* other = p.mix_rows != nullptr ? p.mix_rows + (int64_t)t * p.mix_ld + kvh * Dv : nullptr;
    for (int e0 = lane * step; e0 < Dc; e0 += 32 * step) {
      float y[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int e = e0 + k;
        float v = 0.f;
        if (k < step && e < Dv) {
          if (p.values_are_keys) {
            v = s_qk[(H + kvh) * D + e];
          } else {
            v = own[e];
            if (other != nullptr) v = (1.0f - p.mix_weight) * v + p.mix_weight * other[e];
          }
        }
        y[k] = v;
      }
      rb_store_values<T>(dst + e0, y, step);
    }
  }
  if (p.gate_heads) {
    const int g_at = C + (p.values_are_keys ? 0 : Kh * Dv);
    for (int h = threadIdx.x; h < H; h += blockDim.x) gates_out[(int64_t)t * H + h] = rb_from_float<T>(row[g_at + h]);
  }
}

// A block per token.  rows: [H heads of (D + R) | C latent | R shared key part].  q_out [T, H (D + R)]; the cache row
// (one stream, one head, Dc wide) takes [c / rms(c) * w | turned key part | zeros].
template <typename T>
__global__ void __launch_bounds__(256) latent_rotate_append_kernel(
    T* __restrict__ q_out, const float* __restrict__ rows, int64_t ld, const float* __restrict__ w, float eps,
    const double* __restrict__ freq, float magnitude, int interleaved, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_slot, RbPagedLayer cache, int H, int D, int R, int C) {
  rb_pdl_launch_dependents();
  __shared__ float scratch[33];
  extern __shared__ float s_sincos[];
  const int t = blockIdx.x;
  const int pos = tok_pos[t], slot = tok_slot[t];
  for (int i = threadIdx.x; i < R / 2; i += blockDim.x) angle_sincos(pos, freq[i], magnitude, &s_sincos[i], &s_sincos[R / 2 + i]);
  rb_pdl_wait();
  const float* row = rows + (int64_t)t * ld;
  const int Dq = D + R, Dc = cache.head_dim;
  const float* lat = row + (int64_t)H * Dq;
  float ss = 0.f;
  for (int e = threadIdx.x; e < C; e += blockDim.x) ss += lat[e] * lat[e];
  ss = rb_block_sum(ss, scratch);                            // also the barrier after the table's writes
  const float r = 1.0f / sqrtf(ss / (float)C + eps);
  for (int idx = threadIdx.x; idx < H * Dq; idx += blockDim.x) {
    const int head = idx / Dq, e = idx - head * Dq;
    const float* src = row + (int64_t)head * Dq;
    float y;
    if (e < D) {
      y = src[e];
    } else {
      auto val = [&](int i) { return src[D + i]; };
      y = turned(val, e - D, R, interleaved, s_sincos);
    }
    q_out[(int64_t)t * H * Dq + idx] = rb_from_float<T>(y);
  }
  T* dst = (T*)cache.k + rb_page_offset(cache, slot, pos, 0);
  for (int e = threadIdx.x; e < Dc; e += blockDim.x) {
    float y = 0.f;
    if (e < C) {
      y = lat[e] * r * w[e];
    } else if (e < C + R) {
      auto val = [&](int i) { return lat[C + i]; };
      y = turned(val, e - C, R, interleaved, s_sincos);
    }
    dst[e] = rb_from_float<T>(y);
  }
}

// rows[t, col0 + head * D + e], head < n_heads: the first rot_dim values of every head turned by the row's position,
// in place.  A block per token; a thread owns whole pairs, so nothing is read after it was written.
__global__ void __launch_bounds__(256) rotate_rows_kernel(float* __restrict__ rows, int64_t ld, int col0, int n_heads, int D,
                                                          const double* __restrict__ freq, float magnitude, int rot_dim,
                                                          int interleaved, const int* __restrict__ tok_pos) {
  rb_pdl_launch_dependents();
  extern __shared__ float s_sincos[];
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int rhalf = rot_dim / 2;
  for (int i = threadIdx.x; i < rhalf; i += blockDim.x) angle_sincos(pos, freq[i], magnitude, &s_sincos[i], &s_sincos[rhalf + i]);
  __syncthreads();
  rb_pdl_wait();
  float* row = rows + (int64_t)t * ld + col0;
  for (int idx = threadIdx.x; idx < n_heads * rhalf; idx += blockDim.x) {
    const int head = idx / rhalf, pair = idx - head * rhalf;
    const int ia = interleaved ? 2 * pair : pair, ib = interleaved ? 2 * pair + 1 : pair + rhalf;
    float* hp = row + (int64_t)head * D;
    const float a = hp[ia], b = hp[ib];
    const float sn = s_sincos[pair], cs = s_sincos[rhalf + pair];
    hp[ia] = a * cs - b * sn;
    hp[ib] = b * cs + a * sn;
  }
}

inline int blocks_for(int64_t n, int threads) {
  const int64_t most = (int64_t)rb_sm_count() * 16;
  const int64_t b = (n + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b < most ? b : most));
}

}  // namespace

RB_EXPORT int rb_round_rows(void* out, int out_dtype, const float* x, int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  if (out_dtype == RB_BF16)
    RB_LAUNCH("round_rows_kernel", (round_rows_kernel<__nv_bfloat16>), blocks_for((n + 3) / 4, 256), 256, 0, stream, (__nv_bfloat16*)out, x, n);
  else if (out_dtype == RB_F32)
    RB_LAUNCH("round_rows_kernel", (round_rows_kernel<float>), blocks_for((n + 3) / 4, 256), 256, 0, stream, (float*)out, x, n);
  else
    RB_FAIL("rb_round_rows: unknown dtype %d", out_dtype);
  RB_CHECK_LAUNCH("rb_round_rows");
  return 0;
}

// x [T, E] += y / rms(y) * w; rounded (or null): the new x in rounded_dtype.
RB_EXPORT int rb_norm_add(float* x, const float* y, const float* w, float eps, int T, int E, void* rounded, int rounded_dtype,
                          cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(E > 0, "rb_norm_add: bad width %d", E);
  const bool vec = E % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)w % 16 == 0;
  const int threads = E >= 1024 ? 256 : 128;
#define GO(TT, V) RB_LAUNCH("norm_add_kernel", (norm_add_kernel<TT, V>), T, threads, 0, stream, x, y, w, eps, E, (TT*)rounded)
  if (rounded == nullptr || rounded_dtype == RB_F32) { if (vec) GO(float, true); else GO(float, false); }
  else if (rounded_dtype == RB_BF16) { if (vec) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false); }
  else RB_FAIL("rb_norm_add: unknown dtype %d", rounded_dtype);
#undef GO
  RB_CHECK_LAUNCH("rb_norm_add");
  return 0;
}

// out [T, dim] = gelu_tanh(a[t, :dim]) * table[ids[t], :dim]
RB_EXPORT int rb_token_gate(void* out, int out_dtype, const float* a, int64_t lda, const void* table, int table_dtype,
                            const int* ids, int T, int dim, cudaStream_t stream) {
  if (T == 0) return 0;
  const int64_t n = (int64_t)T * dim;
  const int blocks = blocks_for(n, 256);
#define GO(TO, TT) RB_LAUNCH("token_gate_kernel", (token_gate_kernel<TO, TT>), blocks, 256, 0, stream, (TO*)out, a, lda, (const TT*)table, ids, n, dim)
  if (out_dtype == RB_BF16 && table_dtype == RB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
  else if (out_dtype == RB_F32 && table_dtype == RB_F32) GO(float, float);
  else RB_FAIL("rb_token_gate: unsupported dtypes %d, %d", out_dtype, table_dtype);
#undef GO
  RB_CHECK_LAUNCH("rb_token_gate");
  return 0;
}

// single: every row is a sequence of its own (one launch); else one launch makes the rows and a second moves
// `previous` (int [n_slots]) on to each run's last token.
RB_EXPORT int rb_embed_pairs(float* out, const void* table, const void* pairs, int table_dtype, const int* ids,
                             const int* tok_pos, const int* tok_slot, int* previous, int T, int E, int V, float scale,
                             int buckets, int mul_prev, int mul_cur, int single, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(E > 0 && V > 0 && buckets > 0 && mul_prev >= 0 && mul_cur >= 0, "rb_embed_pairs: bad sizes E=%d V=%d buckets=%d", E, V, buckets);
  const int threads = E >= 1024 ? 256 : 128;
#define GO(TT, ADD, UPD, THREADS)                                                                                           \
  RB_LAUNCH("embed_pairs_kernel", (embed_pairs_kernel<TT>), T, THREADS, 0, stream, out, (const TT*)table, (const TT*)pairs, ids, \
            tok_pos, tok_slot, previous, T, E, V, scale, buckets, mul_prev, mul_cur, ADD, UPD, single)
  if (table_dtype == RB_BF16) {
    if (single) GO(__nv_bfloat16, 1, 1, threads); else { GO(__nv_bfloat16, 1, 0, threads); GO(__nv_bfloat16, 0, 1, 32); }
  } else if (table_dtype == RB_F32) {
    if (single) GO(float, 1, 1, threads); else { GO(float, 1, 0, threads); GO(float, 0, 1, 32); }
  } else {
    RB_FAIL("rb_embed_pairs: unknown dtype %d", table_dtype);
  }
#undef GO
  RB_CHECK_LAUNCH("rb_embed_pairs");
  return 0;
}

// proj: float32 rows [q (H D) | k (Kh D) | v (Kh Dv), unless values_are_keys | gates (H), if gate_heads].
// dtype: of q_out [T, H, Dc], gates_out [T, H] and the cache.  conv_w: [(H + Kh) D, K] or null; tail: the ring
// [n_slots, K, (H + Kh) D] of a sequence's last projected rows by position modulo K (a step of runs of several rows
// moves it on with rb_conv_tail_update afterwards; tok_first null: every row is its own run and moves it on here).
// norm_mode 1: q and k each under an RMS norm over the whole projection, weights [H D] and [Kh D]; 2: every head
// under its own, one weight [D] for all q heads and one for all k heads; both before the rotation.
RB_EXPORT int rb_qk_prepare(void* q_out, void* gates_out, int dtype, const float* proj, int64_t ld, const float* conv_w, int K,
                            float* tail, const int* tok_first, int norm_mode, const float* q_norm_w, const float* k_norm_w,
                            float eps, const double* freq, float magnitude, int rot_dim, int interleaved, const int* tok_pos,
                            const int* tok_slot, void* cache_k, void* cache_v, const int* page_table, int max_pages,
                            int page_size, int T, int H, int Kh, int D, int Dv, int Dc, int values_are_keys,
                            const float* mix_rows, int64_t mix_ld, float mix_weight, int gate_heads, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(H > 0 && Kh > 0 && D > 0 && Dv > 0 && Dc >= D && Dc >= Dv && page_size > 0,
             "rb_qk_prepare: bad sizes H=%d Kh=%d D=%d Dv=%d cache width %d", H, Kh, D, Dv, Dc);
  RB_REQUIRE(rot_dim >= 0 && rot_dim <= D && rot_dim % 2 == 0 && (rot_dim == 0 || freq != nullptr),
             "rb_qk_prepare: the rotated prefix %d must be even and at most the head size %d", rot_dim, D);
  RB_REQUIRE(norm_mode == 0 || (q_norm_w != nullptr && k_norm_w != nullptr), "rb_qk_prepare: norm %d without weights", norm_mode);
  RB_REQUIRE(!values_are_keys || Dv == D, "rb_qk_prepare: values that are the keys have the keys' size");
  RB_REQUIRE(conv_w == nullptr || K <= 1 || tail != nullptr, "rb_qk_prepare: a convolution of %d taps needs the ring", K);
  RB_REQUIRE(!gate_heads || gates_out != nullptr, "rb_qk_prepare: gates without a place for them");
  QkParams p{proj, ld, conv_w, K, tail, tok_first, norm_mode, q_norm_w, k_norm_w, eps, freq, magnitude, rot_dim, interleaved,
             tok_pos, tok_slot, H, D, Dv, values_are_keys, mix_rows, mix_ld, mix_weight, gate_heads};
  RbPagedLayer c{cache_k, cache_v, page_table, max_pages, page_size, Kh, Dc};
  const size_t smem = ((size_t)rot_dim + (size_t)(H + Kh) * D + (size_t)(H + Kh)) * sizeof(float);
  // few tokens (a decode step): a token's block is the whole chain, so it gets as many threads as it has pairs of
  // values to make; many tokens: blocks of 256, several of which share an SM
  int threads = 256;
  if (T <= 2 * rb_sm_count()) {
    const int pairs = (H + Kh) * Dc / 2;
    threads = pairs >= 1024 ? 1024 : (pairs >= 512 ? 512 : 256);
  }
  RB_REQUIRE(smem <= 200 * 1024, "rb_qk_prepare: %d q and k values per token do not fit shared memory", (H + Kh) * D);
#define GO(TT)                                                                                                          \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      RB_CUDA(cudaFuncSetAttribute(qk_prepare_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
    RB_LAUNCH("qk_prepare_kernel", (qk_prepare_kernel<TT>), T, threads, smem, stream, (TT*)q_out, (TT*)gates_out, p, c); \
  } while (0)
  if (dtype == RB_BF16) GO(__nv_bfloat16);
  else if (dtype == RB_F32) GO(float);
  else RB_FAIL("rb_qk_prepare: unknown dtype %d", dtype);
#undef GO
  RB_CHECK_LAUNCH("rb_qk_prepare");
  return 0;
}

RB_EXPORT int rb_latent_rotate_append(void* q_out, int dtype, const float* rows, int64_t ld, const float* w, float eps,
                                      const double* freq, float magnitude, int interleaved, const int* tok_pos,
                                      const int* tok_slot, void* cache, const int* page_table, int max_pages, int page_size,
                                      int Dc, int T, int H, int D, int R, int C, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(H > 0 && D > 0 && C > 0 && R >= 0 && R % 2 == 0 && Dc >= C + R && page_size > 0,
             "rb_latent_rotate_append: bad sizes H=%d D=%d R=%d C=%d cache width %d", H, D, R, C, Dc);
  RB_REQUIRE(R == 0 || freq != nullptr, "rb_latent_rotate_append: a turned part without frequencies");
  RbPagedLayer c{cache, cache, page_table, max_pages, page_size, 1, Dc};
  const size_t smem = (size_t)(R > 0 ? R : 1) * sizeof(float);
#define GO(TT) RB_LAUNCH("latent_rotate_append_kernel", (latent_rotate_append_kernel<TT>), T, 256, smem, stream, (TT*)q_out, rows, ld, w, eps, freq, magnitude, interleaved, tok_pos, tok_slot, c, H, D, R, C)
  if (dtype == RB_BF16) GO(__nv_bfloat16);
  else if (dtype == RB_F32) GO(float);
  else RB_FAIL("rb_latent_rotate_append: unknown dtype %d", dtype);
#undef GO
  RB_CHECK_LAUNCH("rb_latent_rotate_append");
  return 0;
}

RB_EXPORT int rb_rotate_rows(float* rows, int64_t ld, int col0, int n_heads, int D, const double* freq, float magnitude,
                             int rot_dim, int interleaved, const int* tok_pos, int T, cudaStream_t stream) {
  if (T == 0 || rot_dim == 0) return 0;
  RB_REQUIRE(n_heads > 0 && D > 0 && rot_dim % 2 == 0 && rot_dim <= D && freq != nullptr,
             "rb_rotate_rows: bad sizes heads=%d D=%d rotated %d", n_heads, D, rot_dim);
  RB_LAUNCH("rotate_rows_kernel", (rotate_rows_kernel), T, 256, (size_t)rot_dim * sizeof(float), stream, rows, ld, col0, n_heads,
            D, freq, magnitude, rot_dim, interleaved, tok_pos);
  RB_CHECK_LAUNCH("rb_rotate_rows");
  return 0;
}

RB_CHECK_READER(prepare)
