// C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]) with 32-bit FMA on the CUDA cores.
//
// This is the matrix product of the true 32-bit path: no tensor cores, no reduced
// precision mode.  Every output element is summed in the same order whatever the tile shape
// or M is, so a row's result does not depend on what else is in the batch: k runs in order,
// in chains of fmaf over SUM_BLOCK = 64 consecutive k, and the chains' results are added in
// order.  (One chain over all of K loses about sqrt(K) roundings of the running sum; two levels
// lose sqrt(64) + sqrt(K / 64): at K = 4,096 an eighth of the error, which 36 layers of four
// products each need to stay within 1e-4 of a float64 reference.)  Inputs may also be bfloat16
// (products and sums still 32-bit).
// tinyserve uses cuBLAS through nn.Linear for all of these (serve.py:828-829, 912-913, 1263).
#include "common.cuh"

TS_DEFINE_LAST_ERROR()

namespace {

constexpr int BK = 16;
constexpr int SUM_BLOCK = 64;        // k of one fmaf chain
constexpr int THREADS = 256;

template <typename T> struct Load4;
template <> struct Load4<float> {
  static __device__ __forceinline__ void run(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
};
template <> struct Load4<__nv_bfloat16> {
  static __device__ __forceinline__ void run(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&q.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
    v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
  }
};

// rows x BK tile of a [rows_total, K] matrix (leading dimension ld) -> smem[k][row]
template <typename T, int ROWS, bool VEC>
__device__ __forceinline__ void load_tile(const T* __restrict__ src, int row0, int rows_total, int k0,
                                          int K, size_t ld, float (*dst)[ROWS + 4]) {
  if (VEC) {
    for (int i = threadIdx.x; i < ROWS * (BK / 4); i += THREADS) {
      const int r = i / (BK / 4), kq = (i % (BK / 4)) * 4;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (row0 + r < rows_total && k0 + kq < K) Load4<T>::run(src + (size_t)(row0 + r) * ld + k0 + kq, v);
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[kq + j][r] = v[j];
    }
  } else {
    for (int i = threadIdx.x; i < ROWS * BK; i += THREADS) {
      const int r = i / BK, k = i % BK;
      dst[k][r] = (row0 + r < rows_total && k0 + k < K)
                      ? to_f32<T>(src[(size_t)(row0 + r) * ld + k0 + k]) : 0.f;
    }
  }
}

// index of the j-th of a thread's TX values along a tile edge of length B: chunks of 4
// spread over the edge so that shared-memory reads of neighbouring threads do not collide
template <int B, int TX>
__device__ __forceinline__ int spread(int t, int j) {
  return (j / 4) * (B / (TX / 4)) + t * 4 + (j % 4);
}

template <typename TI, typename TO, int BM, int BN, int TM, int TN, bool VEC>
__global__ void __launch_bounds__(THREADS)
gemm_nt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, const TI* __restrict__ bias,
               TO* __restrict__ C, int M, int N, int K, size_t lda, size_t ldw, size_t ldc) {
  static_assert((BM / TM) * (BN / TN) == THREADS, "tile does not match the block");
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_trigger();
  pdl_wait();
  const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN], part[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = part[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    load_tile<TI, BM, VEC>(A, m0, M, k0, K, lda, As);
    load_tile<TI, BN, VEC>(W, n0, N, k0, K, ldw, Ws);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][spread<BM, TM>(ty, i)];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[k][spread<BN, TN>(tx, j)];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
    }
    if ((k0 + BK) % SUM_BLOCK == 0 || k0 + BK >= K) {
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] += part[i][j];
          part[i][j] = 0.f;
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + spread<BM, TM>(ty, i);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + spread<BN, TN>(tx, j);
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_f32<TI>(bias[n]);
      C[(size_t)m * ldc + n] = from_f32<TO>(v);
    }
  }
}

template <typename TI, typename TO>
int launch(const void* A, const void* W, const void* bias, void* C, int M, int N, int K, size_t lda,
           size_t ldw, size_t ldc, cudaStream_t stream) {
  const size_t align = 4 * sizeof(TI);
  const bool vec = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 &&
                   reinterpret_cast<uintptr_t>(A) % align == 0 && reinterpret_cast<uintptr_t>(W) % align == 0;
  const TI* a = static_cast<const TI*>(A);
  const TI* w = static_cast<const TI*>(W);
  const TI* b = static_cast<const TI*>(bias);
  TO* c = static_cast<TO*>(C);
  if (M > 64) {
    dim3 grid((N + 127) / 128, (M + 127) / 128);
    if (grid.y > 65535) return ts_fail("gemm: M = %d is too large", M);
    if (vec) TS_LAUNCH("gemm_simt", (gemm_nt_kernel<TI, TO, 128, 128, 8, 8, true>), grid, THREADS, 0, stream, a, w, b, c, M, N, K, lda, ldw, ldc);
    else TS_LAUNCH("gemm_simt", (gemm_nt_kernel<TI, TO, 128, 128, 8, 8, false>), grid, THREADS, 0, stream, a, w, b, c, M, N, K, lda, ldw, ldc);
  } else {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (vec) TS_LAUNCH("gemm_simt", (gemm_nt_kernel<TI, TO, 64, 64, 4, 4, true>), grid, THREADS, 0, stream, a, w, b, c, M, N, K, lda, ldw, ldc);
    else TS_LAUNCH("gemm_simt", (gemm_nt_kernel<TI, TO, 64, 64, 4, 4, false>), grid, THREADS, 0, stream, a, w, b, c, M, N, K, lda, ldw, ldc);
  }
  return 0;
}

}  // namespace

// in_dtype: element type of A, W and bias; out_dtype: element type of C
TS_EXPORT int ts_gemm_simt(int in_dtype, int out_dtype, const void* A, const void* W,
                           const void* bias, void* C, int M, int N, int K, long long lda,
                           long long ldw, long long ldc, cudaStream_t stream) {
  TS_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty operand (M=%d N=%d K=%d)", M, N, K);
  TS_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: a leading dimension is smaller than its row");
  if (in_dtype == TS_F32 && out_dtype == TS_F32)
    return launch<float, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream);
  if (in_dtype == TS_BF16 && out_dtype == TS_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream);
  if (in_dtype == TS_BF16 && out_dtype == TS_F32)
    return launch<__nv_bfloat16, float>(A, W, bias, C, M, N, K, lda, ldw, ldc, stream);
  return ts_fail("gemm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}
