// Plain tiled matrix product on the CUDA cores: C[M,N] (+)= alpha * A[M,K] * W[N,K]^T.
//
// This is the true 32-bit path's product (FFMA with float32 accumulation, no
// tensor-core or reduced-precision mode) and the product for shapes that the
// tensor-core kernel refuses.  W is row-major [out, in], the layout the
// reference indexes as w[i + o*n_in] (crates/bitnet-core/src/llama/model.rs:67-91),
// so no weight is transposed at load.  Each output element is one sequential
// float32 sum over k in ascending order, whatever M is: a row's result does not
// depend on which other rows are in the batch.
#include "rb_common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

template <typename TA, typename TC>
__global__ void __launch_bounds__(256) gemm_simple_kernel(TC* __restrict__ C, int64_t ldc,
                                                         const TA* __restrict__ A, int64_t lda,
                                                         const TA* __restrict__ W, int64_t ldw, int M, int N,
                                                         int K, int accumulate, float alpha, int64_t batch_c,
                                                         int64_t batch_a, int64_t batch_w) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  // blockIdx.z: one of several independent products of equal sizes, their operands a fixed distance apart
  C += blockIdx.z * batch_c;
  A += blockIdx.z * batch_a;
  W += blockIdx.z * batch_w;
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64x16 elements of each operand, 256 threads -> 4 each
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? rb_to_float<TA>(A[(int64_t)gm * lda + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? rb_to_float<TA>(W[(int64_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      TC* p = C + (int64_t)gm * ldc + gn;
      float v = alpha == 1.0f ? acc[i][j] : acc[i][j] * alpha;
      if (accumulate) v += rb_to_float<TC>(*p);
      *p = rb_from_float<TC>(v);
    }
  }
}


// The same product with tiles of 128 x 128 and 8 x 8 outputs per thread, for many rows: every value read from shared
// memory feeds eight multiply-adds instead of four.  Each output element is still one sequential float32 sum over k in
// ascending order.
constexpr int LM = 128, LN = 128, LK = 16;

template <typename TA, typename TC>
__global__ void __launch_bounds__(256) gemm_simple_large_kernel(TC* __restrict__ C, int64_t ldc, const TA* __restrict__ A,
                                                               int64_t lda, const TA* __restrict__ W, int64_t ldw, int M,
                                                               int N, int K, int accumulate, float alpha, int64_t batch_c,
                                                               int64_t batch_a, int64_t batch_w) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  C += blockIdx.z * batch_c;
  A += blockIdx.z * batch_a;
  W += blockIdx.z * batch_w;
  __shared__ __align__(16) float As[LK][LM + 4];
  __shared__ __align__(16) float Ws[LK][LN + 4];
  const int m0 = blockIdx.y * LM, n0 = blockIdx.x * LN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;      // outputs: rows ty*4 + {0..3} and 64 + ty*4 + {0..3}, columns likewise with tx
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += LK) {
#pragma unroll
    for (int e = threadIdx.x; e < LM * LK; e += 256) {
      const int r = e / LK, c = e % LK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? rb_to_float<TA>(A[(int64_t)gm * lda + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? rb_to_float<TA>(W[(int64_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < LK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
      const float4 w0 = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float4 w1 = *reinterpret_cast<const float4*>(&Ws[kk][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (gn >= N) continue;
      TC* p = C + (int64_t)gm * ldc + gn;
      float v = alpha == 1.0f ? acc[i][j] : acc[i][j] * alpha;
      if (accumulate) v += rb_to_float<TC>(*p);
      *p = rb_from_float<TC>(v);
    }
  }
}

// Few rows (a decode step) times one matrix per head: a warp makes one output of one head for up to eight rows at a
// time, its lanes sharing K, so that the head's matrix is read once and 8 heads x N / 8 blocks are at work instead of
// a few tiles.  float32 sums (a lane's share in ascending order, then the lanes' shares added up).
constexpr int FEW_ROWS = 8;
template <typename TA, typename TC>
__global__ void __launch_bounds__(256) per_head_few_rows_kernel(TC* __restrict__ C, int64_t ldc, const TA* __restrict__ A,
                                                               int64_t lda, const TA* __restrict__ W, int M, int N, int K) {
  rb_pdl_launch_dependents();
  rb_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const TA* w = W + ((int64_t)h * N + n) * K;
  const TA* a = A + (int64_t)h * K;
  for (int m0 = 0; m0 < M; m0 += FEW_ROWS) {
    float acc[FEW_ROWS];
#pragma unroll
    for (int i = 0; i < FEW_ROWS; ++i) acc[i] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float wv = rb_to_float<TA>(w[k]);
#pragma unroll
      for (int i = 0; i < FEW_ROWS; ++i)
        if (m0 + i < M) acc[i] = fmaf(rb_to_float<TA>(a[(int64_t)(m0 + i) * lda + k]), wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < FEW_ROWS; ++i) {
      const float v = rb_warp_sum(acc[i]);
      if (lane == 0 && m0 + i < M) C[(int64_t)(m0 + i) * ldc + (int64_t)h * N + n] = rb_from_float<TC>(v);
    }
  }
}

}  // namespace

// C[m, h * N + n] = sum_k A[m, h * K + k] * W[h, n, k] for few rows m (any number is right; up to 16 is what it is for).
RB_EXPORT int rb_per_head_few_rows(void* C, int64_t ldc, int c_dtype, const void* A, int64_t lda, const void* W, int a_dtype,
                                   int M, int H, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0 || H == 0) return 0;
  RB_REQUIRE(M > 0 && N > 0 && K > 0 && H > 0 && H <= 65535, "rb_per_head_few_rows: bad sizes M=%d H=%d N=%d K=%d", M, H, N, K);
  const dim3 grid((N + 7) / 8, H);
#define LAUNCH(TA, TC)                                                                                                  \
  RB_LAUNCH("per_head_few_rows_kernel", (per_head_few_rows_kernel<TA, TC>), grid, 256, 0, stream, (TC*)C, ldc, (const TA*)A, \
            lda, (const TA*)W, M, N, K)
  if (a_dtype == RB_F32 && c_dtype == RB_F32) LAUNCH(float, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_F32) LAUNCH(__nv_bfloat16, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else RB_FAIL("rb_per_head_few_rows: unsupported dtypes a=%d c=%d", a_dtype, c_dtype);
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_per_head_few_rows");
  return 0;
}

// a_dtype: dtype of A and W; c_dtype: dtype of C.  accumulate: C += instead of C =.
// alpha multiplies the finished sum (1.0 leaves it as it is).
// n_batch products at once: product z reads A + z*batch_a and W + z*batch_w and writes C + z*batch_c
// (distances in elements); block-diagonal matrices are the use.
RB_EXPORT int rb_gemm_simple_batched(void* C, int64_t ldc, int c_dtype, const void* A, int64_t lda, const void* W,
                                     int64_t ldw, int a_dtype, int M, int N, int K, int accumulate, float alpha,
                                     int n_batch, int64_t batch_c, int64_t batch_a, int64_t batch_w,
                                     cudaStream_t stream) {
  if (M == 0 || N == 0 || n_batch == 0) return 0;
  RB_REQUIRE(M > 0 && N > 0 && K > 0, "rb_gemm_simple: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M >= 256 && N >= LN) {
    // many rows: the larger tiles
    dim3 lgrid((N + LN - 1) / LN, (M + LM - 1) / LM, n_batch);
    RB_REQUIRE(lgrid.y <= 65535 && n_batch >= 1 && n_batch <= 65535, "rb_gemm_simple: M=%d, %d products: too large for one launch", M, n_batch);
#define LLAUNCH(TA, TC)                                                                                            \
  RB_LAUNCH("gemm_simple_large_kernel", (gemm_simple_large_kernel<TA, TC>), lgrid, 256, 0, stream, (TC*)C, ldc,     \
            (const TA*)A, lda, (const TA*)W, ldw, M, N, K, accumulate, alpha, batch_c, batch_a, batch_w)
    if (a_dtype == RB_F32 && c_dtype == RB_F32) LLAUNCH(float, float);
    else if (a_dtype == RB_BF16 && c_dtype == RB_F32) LLAUNCH(__nv_bfloat16, float);
    else if (a_dtype == RB_BF16 && c_dtype == RB_BF16) LLAUNCH(__nv_bfloat16, __nv_bfloat16);
    else RB_FAIL("rb_gemm_simple: unsupported dtypes a=%d c=%d", a_dtype, c_dtype);
#undef LLAUNCH
    RB_CHECK_LAUNCH("rb_gemm_simple");
    return 0;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, n_batch);
  RB_REQUIRE(grid.y <= 65535 && n_batch >= 1 && n_batch <= 65535, "rb_gemm_simple: M=%d, %d products: too large for one launch", M, n_batch);
#define LAUNCH(TA, TC)                                                                                     \
  RB_LAUNCH("gemm_simple_kernel", (gemm_simple_kernel<TA, TC>), grid, 256, 0, stream, (TC*)C, ldc, (const TA*)A, \
            lda, (const TA*)W, ldw, M, N, K, accumulate, alpha, batch_c, batch_a, batch_w)
  if (a_dtype == RB_F32 && c_dtype == RB_F32) LAUNCH(float, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_F32) LAUNCH(__nv_bfloat16, float);
  else if (a_dtype == RB_BF16 && c_dtype == RB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else RB_FAIL("rb_gemm_simple: unsupported dtypes a=%d c=%d", a_dtype, c_dtype);
#undef LAUNCH
  RB_CHECK_LAUNCH("rb_gemm_simple");
  return 0;
}

RB_EXPORT int rb_gemm_simple(void* C, int64_t ldc, int c_dtype, const void* A, int64_t lda, const void* W,
                             int64_t ldw, int a_dtype, int M, int N, int K, int accumulate,
                             float alpha, cudaStream_t stream) {
  return rb_gemm_simple_batched(C, ldc, c_dtype, A, lda, W, ldw, a_dtype, M, N, K, accumulate, alpha, 1, 0, 0, 0, stream);
}
