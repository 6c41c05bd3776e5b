// General matmul / linear on CUDA cores: any shape, any transpose, f32 / bf16 / f16 operands,
// f32 FFMA accumulation in ascending-k order.  It serves (a) f32 graphs, where the tensor
// cores' TF32 path cannot meet the 1e-4 tolerance against the reference's f32 CPU matmul
// (tosa.matmul with f32 accumulation, lib/Conversion/TTIRToLinalg/TTIRToLinalg.cpp:542-549),
// (b) shapes the tcgen05 kernel does not take, and (c) as the in-library cross-check of the
// tensor-core kernel.  64x64 tile per 256-thread block, 4x4 outputs per thread, k-step 16.
#include "common.cuh"
#include "epilogue.cuh"

namespace ttb {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T, typename TC>
__global__ void __launch_bounds__(256)
    gemmSimtKernel(const T *__restrict__ a, const T *__restrict__ b, const void *__restrict__ bias, int biasDt,
                   TC *__restrict__ c, int64_t M, int64_t N, int64_t K, int64_t asM, int64_t asK, int64_t bsK,
                   int64_t bsN, int64_t aBatch, int64_t bBatch, int act, int roundSteps) {
  __shared__ float sa[BK][BM + 1];
  __shared__ float sb[BK][BN + 1];
  int64_t batch = blockIdx.z;
  const T *A = a + batch * aBatch;
  const T *B = b + batch * bBatch;
  TC *C = c + batch * M * N;
  int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
  int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += BK) {
    // 64x16 elements per operand, 256 threads -> 4 each.  Index so that the fastest-varying
    // thread index follows the contiguous global dimension of each operand.
    for (int i = threadIdx.x; i < BM * BK; i += 256) {
      int mm, kk;
      if (asK == 1) { kk = i % BK; mm = i / BK; } else { mm = i % BM; kk = i / BM; }
      int64_t gm = m0 + mm, gk = k0 + kk;
      sa[kk][mm] = (gm < M && gk < K) ? toF32(A[gm * asM + gk * asK]) : 0.0f;
    }
    for (int i = threadIdx.x; i < BN * BK; i += 256) {
      int nn, kk;
      if (bsN == 1) { nn = i % BN; kk = i / BN; } else { kk = i % BK; nn = i / BK; }
      int64_t gn = n0 + nn, gk = k0 + kk;
      sb[kk][nn] = (gn < N && gk < K) ? toF32(B[gk * bsK + gn * bsN]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float bz = bias ? loadBias(bias, biasDt, gn) : 0.0f;
      C[gm * N + gn] = epilogue<TC>(acc[i][j], bias != nullptr, bz, act, roundSteps);
    }
  }
}

template <typename T, typename TC>
static int launchSimt(const void *a, const void *b, const void *bias, int biasDt, void *c, int64_t batch, int64_t m,
                      int64_t n, int64_t k, int ta, int tb, int64_t aBatch, int64_t bBatch, int act, int roundSteps,
                      cudaStream_t st) {
  dim3 grid(static_cast<unsigned>((n + BN - 1) / BN), static_cast<unsigned>((m + BM - 1) / BM),
            static_cast<unsigned>(batch));
  int64_t asM = ta ? 1 : k, asK = ta ? m : 1;
  int64_t bsK = tb ? 1 : n, bsN = tb ? k : 1;
  ProfScope prof("gemm_simt", 2.0 * double(batch) * m * n * k, double(batch) * (double(m) * k + double(n) * k) * sizeof(T) + double(batch) * m * n * sizeof(TC), st);
  gemmSimtKernel<T, TC><<<grid, 256, 0, st>>>(static_cast<const T *>(a), static_cast<const T *>(b), bias, biasDt,
                                              static_cast<TC *>(c), m, n, k, asM, asK, bsK, bsN, aBatch, bBatch, act,
                                              roundSteps);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // namespace ttb

using namespace ttb;

extern "C" int ttb_gemm_simt(const void *a, const void *b, const void *bias, void *c, int ab_dtype, int bias_dtype,
                             int c_dtype, int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                             int64_t a_batch_stride, int64_t b_batch_stride, int act, int round_steps,
                             void *stream) {
  TTB_CHECK(a && b && c, "null tensor");
  TTB_CHECK(batch >= 0 && m >= 0 && n >= 0 && k >= 0, "negative dimension");
  TTB_CHECK(batch <= 65535 && (m + BM - 1) / BM <= 65535, "grid too large");
  if (batch * m * n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
#define TTB_SIMT(T, TC) return launchSimt<T, TC>(a, b, bias, bias_dtype, c, batch, m, n, k, trans_a, trans_b, a_batch_stride, b_batch_stride, act, round_steps, st)
  if (ab_dtype == kF32 && c_dtype == kF32) TTB_SIMT(float, float);
  if (ab_dtype == kBF16 && c_dtype == kBF16) TTB_SIMT(__nv_bfloat16, __nv_bfloat16);
  if (ab_dtype == kBF16 && c_dtype == kF32) TTB_SIMT(__nv_bfloat16, float);
  if (ab_dtype == kF16 && c_dtype == kF16) TTB_SIMT(__half, __half);
  if (ab_dtype == kF16 && c_dtype == kF32) TTB_SIMT(__half, float);
  if (ab_dtype == kF32 && c_dtype == kBF16) TTB_SIMT(float, __nv_bfloat16);
#undef TTB_SIMT
  setLastError("gemm: unsupported dtype combination");
  return TTB_ERR_UNSUPPORTED;
}
