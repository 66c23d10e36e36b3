// Attention through latents: what stands between the down-projections and the attention kernels.
//
// rows: float32 [T, ...] of the stacked down-projections, holding the query latent (q_rank values at q_off) and
// the key/value latent (kv_rank values at kv_off).  Each is divided by its root mean square (eps inside the root) and
// multiplied by its weight, in float32.  The query latent leaves as a row of the compute dtype for the up-projection;
// the key/value latent is what the cache keeps per position: it goes to the sequence's page as one "head" of
// `width` values (kv_rank, padded with zeros).
#include "rb_common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) latent_norm_append_kernel(
    T* __restrict__ cq, const float* __restrict__ rows, int64_t ld, int q_off, int kv_off, int q_rank, int kv_rank,
    const float* __restrict__ wq, const float* __restrict__ wkv, float eps, RbPagedLayer cache, int width,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_slot) {
  rb_pdl_launch_dependents();
  __shared__ float scratch[33];
  rb_pdl_wait();
  const int t = blockIdx.x;
  const float* row = rows + (int64_t)t * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss = fmaf(row[q_off + i], row[q_off + i], ss);
  ss = rb_block_sum(ss, scratch);
  const float rq = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(int64_t)t * q_rank + i] = rb_from_float<T>(row[q_off + i] * rq * wq[i]);
  ss = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) ss = fmaf(row[kv_off + i], row[kv_off + i], ss);
  ss = rb_block_sum(ss, scratch);
  const float rk = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  T* dst = reinterpret_cast<T*>(cache.k) + rb_page_offset(cache, tok_slot[t], tok_pos[t], 0);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = rb_from_float<T>(i < kv_rank ? row[kv_off + i] * rk * wkv[i] : 0.f);
}

}  // namespace

RB_EXPORT int rb_latent_norm_append(void* cq, int dtype, const float* rows, int64_t ld, int q_off, int kv_off, int q_rank,
                                    int kv_rank, const float* wq, const float* wkv, float eps, void* pool,
                                    const int* page_table, int max_pages, int page_size, int width, const int* tok_pos,
                                    const int* tok_slot, int T, cudaStream_t stream) {
  if (T == 0) return 0;
  RB_REQUIRE(q_rank > 0 && kv_rank > 0 && width >= kv_rank, "rb_latent_norm_append: bad sizes q_rank=%d kv_rank=%d width=%d",
             q_rank, kv_rank, width);
  RbPagedLayer cache{pool, pool, page_table, max_pages, page_size, 1, width};
  const int threads = (q_rank > 512 || kv_rank > 512) ? 256 : 128;
  if (dtype == RB_F32)
    RB_LAUNCH("latent_norm_append_kernel", (latent_norm_append_kernel<float>), T, threads, 0, stream, (float*)cq, rows, ld, q_off, kv_off, q_rank, kv_rank, wq, wkv, eps, cache, width, tok_pos, tok_slot);
  else if (dtype == RB_BF16)
    RB_LAUNCH("latent_norm_append_kernel", (latent_norm_append_kernel<__nv_bfloat16>), T, threads, 0, stream, (__nv_bfloat16*)cq, rows, ld, q_off, kv_off, q_rank, kv_rank, wq, wkv, eps, cache, width, tok_pos, tok_slot);
  else
    RB_FAIL("rb_latent_norm_append: unknown dtype %d", dtype);
  RB_CHECK_LAUNCH("rb_latent_norm_append");
  return 0;
}

RB_CHECK_READER(latent)
