// Quantized contractions: C = A B with 8-bit integer operands and exact 32-bit integer accumulation.
//
// In tt-mlir a matmul / conv2d whose operands were quantized runs on the quantized values and is
// followed by a dequantize whose scale is the product of the operands' scales, per tensor or per output
// channel (lib/Dialect/TTIR/Transforms/QuantDequantConversion.cpp commutes the dequantize below the op;
// lib/Dialect/TTIR/IR/TTIROps.cpp:1492-1577 builds the quantized convolution with an i32 accumulator
// type; the runtime then sees an ordinary MatmulOp / Conv2dOp on integer tensors,
// runtime/lib/ttnn/operations/matmul/matmul.cpp:47-83).  Here that is tcgen05.mma kind::i8 for the
// weight layout B[N, K] (gemm_tcgen05.cu) and a CUDA-core kernel for every other layout and for shapes
// the tensor-core kernel does not take.  Integer results are exact, so both kernels agree bit for bit
// with each other and with an integer matmul on the CPU.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace ttb {

int gemmTcgen05I8Try(const void *a, const void *b, void *c, int aDtype, int bDtype, int cDtype, int64_t m, int64_t n,
                     int64_t k, const float *deqScale, float deqScalar, const void *bias, int biasDtype, cudaStream_t stream);

constexpr int I8_TILE = 32, I8_K = 32;

template <typename TA, typename TB> struct I8Ops {
  __device__ static int a(const void *p, int64_t i) { return static_cast<int>(static_cast<const TA *>(p)[i]); }
  __device__ static int b(const void *p, int64_t i) { return static_cast<int>(static_cast<const TB *>(p)[i]); }
};

template <typename TC> __device__ __forceinline__ TC storeI8(int acc, int deq, float scalar, const float *scale, int64_t col);
template <> __device__ __forceinline__ int32_t storeI8<int32_t>(int acc, int, float, const float *, int64_t) { return acc; }
template <> __device__ __forceinline__ float storeI8<float>(int acc, int deq, float scalar, const float *scale, int64_t col) {
  return __fmul_rn(__int2float_rn(acc), deq == 2 ? scale[col] : scalar);
}
template <> __device__ __forceinline__ __nv_bfloat16 storeI8<__nv_bfloat16>(int acc, int deq, float scalar, const float *scale, int64_t col) {
  return __float2bfloat16_rn(__fmul_rn(__int2float_rn(acc), deq == 2 ? scale[col] : scalar));
}
template <> __device__ __forceinline__ __half storeI8<__half>(int acc, int deq, float scalar, const float *scale, int64_t col) {
  return __float2half_rn(__fmul_rn(__int2float_rn(acc), deq == 2 ? scale[col] : scalar));
}

// 32 x 32 outputs per 256-thread block (a 2 x 2 patch per thread), k in steps of 32 through shared memory;
// operands addressed through element strides, so every transpose combination is the same code.
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256)
    gemmI8SimtKernel(const TA *__restrict__ a, const TB *__restrict__ b, TC *__restrict__ c, int64_t M, int64_t N, int64_t K,
                     int64_t asM, int64_t asK, int64_t bsK, int64_t bsN, int64_t aBatch, int64_t bBatch, int deq, float scalar,
                     const float *__restrict__ scale) {
  __shared__ int sa[I8_K][I8_TILE + 1];
  __shared__ int sb[I8_K][I8_TILE + 1];
  const TA *A = a + static_cast<int64_t>(blockIdx.z) * aBatch;
  const TB *B = b + static_cast<int64_t>(blockIdx.z) * bBatch;
  TC *C = c + static_cast<int64_t>(blockIdx.z) * M * N;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * I8_TILE, n0 = static_cast<int64_t>(blockIdx.x) * I8_TILE;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  int acc[2][2] = {};
  for (int64_t k0 = 0; k0 < K; k0 += I8_K) {
    for (int i = threadIdx.x; i < I8_K * I8_TILE; i += 256) {
      const int kk = i % I8_K, r = i / I8_K;
      const int64_t gk = k0 + kk;
      sa[kk][r] = (gk < K && m0 + r < M) ? static_cast<int>(A[(m0 + r) * asM + gk * asK]) : 0;
      sb[kk][r] = (gk < K && n0 + r < N) ? static_cast<int>(B[gk * bsK + (n0 + r) * bsN]) : 0;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < I8_K; ++kk) {
      const int a0 = sa[kk][ty * 2], a1 = sa[kk][ty * 2 + 1], b0 = sb[kk][tx * 2], b1 = sb[kk][tx * 2 + 1];
      acc[0][0] += a0 * b0;
      acc[0][1] += a0 * b1;
      acc[1][0] += a1 * b0;
      acc[1][1] += a1 * b1;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t gm = m0 + ty * 2 + i, gn = n0 + tx * 2 + j;
      if (gm < M && gn < N) C[gm * N + gn] = storeI8<TC>(acc[i][j], deq, scalar, scale, gn);
    }
  }
}

template <typename TA, typename TB, typename TC>
static int launchI8Simt(const void *a, const void *b, void *c, int64_t batch, int64_t m, int64_t n, int64_t k, int ta, int tb,
                        int64_t aBatch, int64_t bBatch, int deq, float scalar, const float *scale, cudaStream_t st) {
  const int64_t asM = ta ? 1 : k, asK = ta ? m : 1, bsK = tb ? 1 : n, bsN = tb ? k : 1;
  dim3 grid(static_cast<unsigned>((n + I8_TILE - 1) / I8_TILE), static_cast<unsigned>((m + I8_TILE - 1) / I8_TILE),
            static_cast<unsigned>(batch));
  ProfScope prof("gemm_i8_simt", 2.0 * double(batch) * m * n * k, double(batch) * (double(m) * k + double(n) * k + double(m) * n * sizeof(TC)), st);
  gemmI8SimtKernel<TA, TB, TC><<<grid, 256, 0, st>>>(static_cast<const TA *>(a), static_cast<const TB *>(b), static_cast<TC *>(c), m, n,
                                                     k, asM, asK, bsK, bsN, aBatch, bBatch, deq, scalar, scale);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

template <typename TA, typename TB>
static int dispatchI8Out(const void *a, const void *b, void *c, int cDtype, int64_t batch, int64_t m, int64_t n, int64_t k, int ta,
                         int tb, int64_t aBatch, int64_t bBatch, int deq, float scalar, const float *scale, cudaStream_t st) {
  switch (cDtype) {
  case kI32: return launchI8Simt<TA, TB, int32_t>(a, b, c, batch, m, n, k, ta, tb, aBatch, bBatch, 0, 0.0f, nullptr, st);
  case kF32: return launchI8Simt<TA, TB, float>(a, b, c, batch, m, n, k, ta, tb, aBatch, bBatch, deq, scalar, scale, st);
  case kBF16: return launchI8Simt<TA, TB, __nv_bfloat16>(a, b, c, batch, m, n, k, ta, tb, aBatch, bBatch, deq, scalar, scale, st);
  case kF16: return launchI8Simt<TA, TB, __half>(a, b, c, batch, m, n, k, ta, tb, aBatch, bBatch, deq, scalar, scale, st);
  default: setLastError("gemm_i8: result must be Int32 or a float type"); return TTB_ERR_UNSUPPORTED;
  }
}

} // namespace ttb

using namespace ttb;

static bool i8TensorCoreOff() {
  static const bool off = [] {
    const char *e = std::getenv("TTB_DISABLE_TCGEN05");
    return e && e[0] && std::strcmp(e, "0") != 0;
  }();
  return off;
}

extern "C" int ttb_gemm_i8(const void *a, const void *b, void *c, int a_dtype, int b_dtype, int c_dtype, int64_t batch,
                           int64_t m, int64_t n, int64_t k, int trans_a, int trans_b, int64_t a_batch_stride,
                           int64_t b_batch_stride, const float *deq_scale, float deq_scalar, void *stream) {
  TTB_CHECK(a && b && c, "null tensor");
  TTB_CHECK(batch >= 0 && m >= 0 && n >= 0 && k >= 0, "negative dimension");
  TTB_CHECK((a_dtype == kI8 || a_dtype == kU8) && (b_dtype == kI8 || b_dtype == kU8), "gemm_i8 takes Int8 / UInt8 operands");
  TTB_CHECK(batch <= 65535 && (m + I8_TILE - 1) / I8_TILE <= 65535, "grid too large");
  if (batch * m * n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  if (!i8TensorCoreOff() && batch == 1 && !trans_a && trans_b) {
    int rc = gemmTcgen05I8Try(a, b, c, a_dtype, b_dtype, c_dtype, m, n, k, deq_scale, deq_scalar, nullptr, 0, st);
    if (rc != -1) return rc;
  }
  const int deq = c_dtype == kI32 ? 0 : (deq_scale ? 2 : 1);
#define TTB_I8(TA, TB) return dispatchI8Out<TA, TB>(a, b, c, c_dtype, batch, m, n, k, trans_a, trans_b, a_batch_stride, b_batch_stride, deq, deq_scalar, deq_scale, st)
  if (a_dtype == kI8 && b_dtype == kI8) TTB_I8(int8_t, int8_t);
  if (a_dtype == kU8 && b_dtype == kI8) TTB_I8(uint8_t, int8_t);
  if (a_dtype == kI8 && b_dtype == kU8) TTB_I8(int8_t, uint8_t);
  TTB_I8(uint8_t, uint8_t);
#undef TTB_I8
}

// The same contraction forced onto the CUDA-core kernel (the in-library cross-check of the tensor-core path).
extern "C" int ttb_gemm_i8_simt(const void *a, const void *b, void *c, int a_dtype, int b_dtype, int c_dtype, int64_t batch,
                                int64_t m, int64_t n, int64_t k, int trans_a, int trans_b, int64_t a_batch_stride,
                                int64_t b_batch_stride, const float *deq_scale, float deq_scalar, void *stream) {
  TTB_CHECK(a && b && c, "null tensor");
  TTB_CHECK((a_dtype == kI8 || a_dtype == kU8) && (b_dtype == kI8 || b_dtype == kU8), "gemm_i8 takes Int8 / UInt8 operands");
  TTB_CHECK(batch >= 0 && m >= 0 && n >= 0 && k >= 0 && batch <= 65535 && (m + I8_TILE - 1) / I8_TILE <= 65535, "bad dimensions");
  if (batch * m * n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  const int deq = c_dtype == kI32 ? 0 : (deq_scale ? 2 : 1);
#define TTB_I8(TA, TB) return dispatchI8Out<TA, TB>(a, b, c, c_dtype, batch, m, n, k, trans_a, trans_b, a_batch_stride, b_batch_stride, deq, deq_scalar, deq_scale, st)
  if (a_dtype == kI8 && b_dtype == kI8) TTB_I8(int8_t, int8_t);
  if (a_dtype == kU8 && b_dtype == kI8) TTB_I8(uint8_t, int8_t);
  if (a_dtype == kI8 && b_dtype == kU8) TTB_I8(int8_t, uint8_t);
  TTB_I8(uint8_t, uint8_t);
#undef TTB_I8
}

// ttb_gemm_i8 followed by `+ bias` (a row vector of n values in a float type): what a quantized linear
// layer is after the compiler has moved the dequantize below the contraction -- matmul on the 8-bit
// values, dequantize, add.  The dequantized value is rounded to the result type before the bias is added
// and the sum rounded again, as the two separate ops round.  On the tensor-core kernel one launch;
// elsewhere the contraction and a broadcast add.
extern "C" int ttb_gemm_i8_bias(const void *a, const void *b, void *c, int a_dtype, int b_dtype, int c_dtype, int64_t batch,
                                int64_t m, int64_t n, int64_t k, int trans_a, int trans_b, int64_t a_batch_stride,
                                int64_t b_batch_stride, const float *deq_scale, float deq_scalar, const void *bias,
                                int bias_dtype, void *stream) {
  if (!bias) {
    return ttb_gemm_i8(a, b, c, a_dtype, b_dtype, c_dtype, batch, m, n, k, trans_a, trans_b, a_batch_stride, b_batch_stride,
                       deq_scale, deq_scalar, stream);
  }
  TTB_CHECK(a && b && c, "null tensor");
  TTB_CHECK(c_dtype != kI32, "a bias needs a dequantized (float) result");
  if (batch * m * n == 0) return TTB_OK;
  if (!i8TensorCoreOff() && batch == 1 && !trans_a && trans_b) {
    int rc = gemmTcgen05I8Try(a, b, c, a_dtype, b_dtype, c_dtype, m, n, k, deq_scale, deq_scalar, bias, bias_dtype, asStream(stream));
    if (rc != -1) return rc;
  }
  int rc = ttb_gemm_i8(a, b, c, a_dtype, b_dtype, c_dtype, batch, m, n, k, trans_a, trans_b, a_batch_stride, b_batch_stride,
                       deq_scale, deq_scalar, stream);
  if (rc) return rc;
  int64_t shape[2] = {batch * m, n}, cs[2] = {n, 1}, bs[2] = {0, 1};
  return ttb_eltwise_binary(0 /* EltwiseBinaryOpType::Add */, c, c_dtype, bias, bias_dtype, c, c_dtype, 2, shape, cs, bs, stream);
}
