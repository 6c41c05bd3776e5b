// Elementwise kernels: unary, binary (with broadcasting), where, clamp, typecast, fill, arange.
//
// Numerics follow the reference's CPU path for these ops: operands are widened to f32 (i32 for
// integer tensors), the op is applied once, and the result is rounded once to the output
// dtype (lib/Dialect/TTIR/Transforms/HoistCPUOps/HoistCPUOps.cpp:78-93 widens, the torch
// functions in tools/tt-alchemist/templates/python/local/ttir_cpu.py:94-330 define each op).
// All kernels are HBM-bound: dense same-dtype cases use 16-byte streaming accesses, the
// general broadcasting case falls back to per-element index arithmetic.
#include "common.cuh"

#include <cmath>
#include <type_traits>

namespace ttb {

// EltwiseUnaryOpType (include/ttmlir/Target/TTNN/operations/eltwise.fbs:133-166)
enum UnaryOp {
  uAbs, uCeil, uCos, uFloor, uGelu, uIsFinite, uLogicalNot, uNeg, uRelu, uSqrt, uRsqrt, uSigmoid, uSin,
  uReciprocal, uSign, uTan, uTanh, uAtan, uExp, uErf, uErfc, uLog, uExpm1, uLeakyRelu, uBitwiseNot,
  uRelu6, uSilu, uHardsigmoid, uMish, uAcos, uAsin, uAsinh, uCount
};
// Composite unary ops handled by the same kernel (EltwiseUnaryCompositeOpType :177-182).
// ... and EltwiseBinaryCompositeScalarOpType::PowScalar (:56-58): x to the power of the op's scalar parameter.
enum { uCbrt = 200, uLog1p = 201, uPowScalar = 202 };

// EltwiseBinaryOpType (:11-26) and, from 100 up, EltwiseBinaryCompositeOpType (:37-47).
enum BinaryOp {
  bAdd, bMultiply, bLogicalRightShift, bSubtract, bEqual, bNotEqual, bGreaterEqual, bGreaterThan,
  bLessEqual, bLessThan, bDivide, bLogicalAnd, bLogicalOr, bLogicalXor,
  bMaximum = TTB_BINARY_COMPOSITE_BASE, bMinimum, bRemainder, bPow, bAtan2, bBitwiseAnd, bBitwiseOr,
  bBitwiseXor, bLogicalLeftShift
};

__device__ __forceinline__ float applyUnary(int op, float x, float p) {
  switch (op) {
  case uAbs: return fabsf(x);
  case uCeil: return ceilf(x);
  case uCos: return cosf(x);
  case uFloor: return floorf(x);
  case uGelu: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
  case uIsFinite: return isfinite(x) ? 1.0f : 0.0f;
  case uLogicalNot: return x == 0.0f ? 1.0f : 0.0f;
  case uNeg: return -x;
  case uRelu: return x > 0.0f ? x : (x != x ? x : 0.0f);
  case uSqrt: return sqrtf(x);
  case uRsqrt: return 1.0f / sqrtf(x);
  case uSigmoid: return 1.0f / (1.0f + expf(-x));
  case uSin: return sinf(x);
  case uReciprocal: return 1.0f / x;
  case uSign: return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : x);
  case uTan: return tanf(x);
  case uTanh: return tanhf(x);
  case uAtan: return atanf(x);
  case uExp: return expf(x);
  case uErf: return erff(x);
  case uErfc: return erfcf(x);
  case uLog: return logf(x);
  case uExpm1: return expm1f(x);
  case uLeakyRelu: return x > 0.0f ? x : x * p;
  case uRelu6: return fminf(fmaxf(x, 0.0f), 6.0f);
  case uSilu: return x / (1.0f + expf(-x));
  case uHardsigmoid: return fminf(fmaxf(x * (1.0f / 6.0f) + 0.5f, 0.0f), 1.0f);
  case uMish: return x * tanhf(log1pf(expf(x)));
  case uAcos: return acosf(x);
  case uAsin: return asinf(x);
  case uAsinh: return asinhf(x);
  case uCbrt: return cbrtf(x);
  case uLog1p: return log1pf(x);
  case uPowScalar: return powf(x, p);
  default: return x;
  }
}

__device__ __forceinline__ long long applyUnaryInt(int op, long long x) {
  switch (op) {
  case uAbs: return x < 0 ? -x : x;
  case uNeg: return -x;
  case uRelu: return x > 0 ? x : 0;
  case uSign: return (x > 0) - (x < 0);
  case uLogicalNot: return x == 0;
  case uBitwiseNot: return ~x;
  case uRelu6: return x < 0 ? 0 : (x > 6 ? 6 : x);
  default: return x;
  }
}

__device__ __forceinline__ float applyBinary(int op, float a, float b) {
  switch (op) {
  case bAdd: return a + b;
  case bMultiply: return a * b;
  case bSubtract: return a - b;
  case bDivide: return a / b;
  case bEqual: return a == b ? 1.0f : 0.0f;
  case bNotEqual: return a != b ? 1.0f : 0.0f;
  case bGreaterEqual: return a >= b ? 1.0f : 0.0f;
  case bGreaterThan: return a > b ? 1.0f : 0.0f;
  case bLessEqual: return a <= b ? 1.0f : 0.0f;
  case bLessThan: return a < b ? 1.0f : 0.0f;
  case bLogicalAnd: return (a != 0.0f && b != 0.0f) ? 1.0f : 0.0f;
  case bLogicalOr: return (a != 0.0f || b != 0.0f) ? 1.0f : 0.0f;
  case bLogicalXor: return ((a != 0.0f) != (b != 0.0f)) ? 1.0f : 0.0f;
  case bMaximum: return (a != a || b != b) ? NAN : fmaxf(a, b);
  case bMinimum: return (a != a || b != b) ? NAN : fminf(a, b);
  case bRemainder: { float r = fmodf(a, b); return (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) ? r + b : r; }
  case bPow: return powf(a, b);
  case bAtan2: return atan2f(a, b);
  default: return a;
  }
}

__device__ __forceinline__ long long applyBinaryInt(int op, long long a, long long b) {
  switch (op) {
  case bAdd: return a + b;
  case bMultiply: return a * b;
  case bSubtract: return a - b;
  case bDivide: return b == 0 ? 0 : a / b;
  case bEqual: return a == b;
  case bNotEqual: return a != b;
  case bGreaterEqual: return a >= b;
  case bGreaterThan: return a > b;
  case bLessEqual: return a <= b;
  case bLessThan: return a < b;
  case bLogicalAnd: return a != 0 && b != 0;
  case bLogicalOr: return a != 0 || b != 0;
  case bLogicalXor: return (a != 0) != (b != 0);
  case bLogicalRightShift: return static_cast<long long>(static_cast<uint32_t>(a) >> (b & 31));
  case bLogicalLeftShift: return static_cast<long long>(static_cast<uint32_t>(a) << (b & 31));
  case bMaximum: return a > b ? a : b;
  case bMinimum: return a < b ? a : b;
  case bRemainder: { if (b == 0) return 0; long long r = a % b; return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r; }
  case bBitwiseAnd: return a & b;
  case bBitwiseOr: return a | b;
  case bBitwiseXor: return a ^ b;
  default: return a;
  }
}

__host__ __device__ inline bool isIntDtype(int dt) { return dt == kI32 || dt == kU32 || dt == kU16 || dt == kU8 || dt == kI8; }

// Runtime-typed element access, used by the general (non-vectorised) kernels.
__device__ __forceinline__ float loadF(const void *p, int dt, size_t i) {
  switch (dt) {
  case kF32: return static_cast<const float *>(p)[i];
  case kBF16: return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
  case kF16: return __half2float(static_cast<const __half *>(p)[i]);
  case kI32: return static_cast<float>(static_cast<const int32_t *>(p)[i]);
  case kU32: return static_cast<float>(static_cast<const uint32_t *>(p)[i]);
  case kU16: return static_cast<float>(static_cast<const uint16_t *>(p)[i]);
  case kU8: return static_cast<float>(static_cast<const uint8_t *>(p)[i]);
  case kI8: return static_cast<float>(static_cast<const int8_t *>(p)[i]);
  default: return 0.0f;
  }
}
__device__ __forceinline__ long long loadI(const void *p, int dt, size_t i) {
  switch (dt) {
  case kI32: return static_cast<const int32_t *>(p)[i];
  case kU32: return static_cast<const uint32_t *>(p)[i];
  case kU16: return static_cast<const uint16_t *>(p)[i];
  case kU8: return static_cast<const uint8_t *>(p)[i];
  case kI8: return static_cast<const int8_t *>(p)[i];
  case kF32: return static_cast<long long>(static_cast<const float *>(p)[i]);
  case kBF16: return static_cast<long long>(__bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]));
  case kF16: return static_cast<long long>(__half2float(static_cast<const __half *>(p)[i]));
  default: return 0;
  }
}
__device__ __forceinline__ void storeF(void *p, int dt, size_t i, float v) {
  switch (dt) {
  case kF32: static_cast<float *>(p)[i] = v; break;
  case kBF16: static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v); break;
  case kF16: static_cast<__half *>(p)[i] = __float2half_rn(v); break;
  case kI32: static_cast<int32_t *>(p)[i] = fromF32<int32_t>(v); break;
  case kU32: static_cast<uint32_t *>(p)[i] = fromF32<uint32_t>(v); break;
  case kU16: static_cast<uint16_t *>(p)[i] = fromF32<uint16_t>(v); break;
  case kU8: static_cast<uint8_t *>(p)[i] = fromF32<uint8_t>(v); break;
  case kI8: static_cast<int8_t *>(p)[i] = fromF32<int8_t>(v); break;
  default: break;
  }
}
__device__ __forceinline__ void storeI(void *p, int dt, size_t i, long long v) {
  switch (dt) {
  case kI32: static_cast<int32_t *>(p)[i] = static_cast<int32_t>(v); break;
  case kU32: static_cast<uint32_t *>(p)[i] = static_cast<uint32_t>(v); break;
  case kU16: static_cast<uint16_t *>(p)[i] = static_cast<uint16_t>(v); break;
  case kU8: static_cast<uint8_t *>(p)[i] = static_cast<uint8_t>(v); break;
  case kI8: static_cast<int8_t *>(p)[i] = static_cast<int8_t>(v); break;
  case kF32: static_cast<float *>(p)[i] = static_cast<float>(v); break;
  case kBF16: static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(static_cast<float>(v)); break;
  case kF16: static_cast<__half *>(p)[i] = __float2half_rn(static_cast<float>(v)); break;
  default: break;
  }
}

constexpr int kVec = 16;

// ---- unary -----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) unaryVecKernel(int op, const T *__restrict__ in, T *__restrict__ out,
                                                      size_t n, float p) {
  size_t nvec = n / kVec;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<T, kVec> x, y;
    loadPack(x, in + i * kVec);
#pragma unroll
    for (int j = 0; j < kVec; ++j) y.v[j] = fromF32<T>(applyUnary(op, toF32(x.v[j]), p));
    storePack(out + i * kVec, y);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n) out[tail] = fromF32<T>(applyUnary(op, toF32(in[tail]), p));
}

__global__ void __launch_bounds__(256) unaryGenericKernel(int op, const void *in, int inDt, void *out, int outDt,
                                                          size_t n, float p) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  bool intPath = isIntDtype(inDt) && isIntDtype(outDt);
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (intPath) storeI(out, outDt, i, applyUnaryInt(op, loadI(in, inDt, i)));
    else storeF(out, outDt, i, applyUnary(op, loadF(in, inDt, i), p));
  }
}

// ---- binary ----------------------------------------------------------------------------
// Dense fast path: a has n elements; b has bMod elements and is indexed i % bMod (bMod == n
// means same shape, bMod == cols means a row vector broadcast over rows).  bMod % kVec == 0.
template <typename T>
__global__ void __launch_bounds__(256) binaryVecKernel(int op, const T *__restrict__ a, const T *__restrict__ b,
                                                       T *__restrict__ out, size_t n, size_t aMod, size_t bMod) {
  size_t nvec = n / kVec;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<T, kVec> x, y, z;
    size_t e = i * kVec;
    loadPack(x, a + (aMod == n ? e : e % aMod));
    loadPack(y, b + (bMod == n ? e : e % bMod));
#pragma unroll
    for (int j = 0; j < kVec; ++j) z.v[j] = fromF32<T>(applyBinary(op, toF32(x.v[j]), toF32(y.v[j])));
    storePack(out + e, z);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n) out[tail] = fromF32<T>(applyBinary(op, toF32(a[tail % aMod]), toF32(b[tail % bMod])));
}

struct BcastDims {
  int rank;
  int64_t shape[8];
  int64_t sa[8];
  int64_t sb[8];
  int64_t sc[8];
};

__global__ void __launch_bounds__(256)
    binaryGenericKernel(int op, const void *a, int aDt, const void *b, int bDt, void *out, int oDt, size_t n,
                        BcastDims d) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  bool intPath = isIntDtype(aDt) && isIntDtype(bDt);
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    size_t r = i, ia = 0, ib = 0;
    for (int k = d.rank - 1; k >= 0; --k) {
      size_t c = r % d.shape[k];
      r /= d.shape[k];
      ia += c * d.sa[k];
      ib += c * d.sb[k];
    }
    if (intPath) {
      long long v = applyBinaryInt(op, loadI(a, aDt, ia), loadI(b, bDt, ib));
      if (isIntDtype(oDt)) storeI(out, oDt, i, v);
      else storeF(out, oDt, i, static_cast<float>(v));
    } else {
      storeF(out, oDt, i, applyBinary(op, loadF(a, aDt, ia), loadF(b, bDt, ib)));
    }
  }
}

__global__ void __launch_bounds__(256)
    whereKernel(const void *c, int cDt, const void *a, const void *b, int dt, void *out, size_t n, BcastDims d) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t es = dt == kF32 || dt == kI32 || dt == kU32 ? 4 : (dt == kU8 || dt == kI8 ? 1 : 2);
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    size_t r = i, ia = 0, ib = 0, ic = 0;
    for (int k = d.rank - 1; k >= 0; --k) {
      size_t x = r % d.shape[k];
      r /= d.shape[k];
      ia += x * d.sa[k];
      ib += x * d.sb[k];
      ic += x * d.sc[k];
    }
    bool pick = loadF(c, cDt, ic) != 0.0f;
    const char *src = static_cast<const char *>(pick ? a : b) + (pick ? ia : ib) * es;
    char *dst = static_cast<char *>(out) + i * es;
    for (size_t k = 0; k < es; ++k) dst[k] = src[k];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) clampKernel(const T *__restrict__ in, T *__restrict__ out, size_t n,
                                                   float lo, float hi) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float x = toF32(in[i]);
    out[i] = fromF32<T>(x != x ? x : fminf(fmaxf(x, lo), hi));
  }
}

// ---- typecast --------------------------------------------------------------------------
template <typename TI, typename TO> __device__ __forceinline__ TO convertElem(TI v) {
  constexpr bool inInt = std::is_integral<TI>::value, outInt = std::is_integral<TO>::value;
  if constexpr (inInt && outInt) {
    return static_cast<TO>(v); // two's-complement wrap, as torch's integer casts
  } else if constexpr (outInt) {
    // float -> integer truncates toward zero; out-of-range values wrap through int64 like torch on x86
    float f = toF32(v);
    long long w = (f != f) ? 0 : static_cast<long long>(f);
    return static_cast<TO>(w);
  } else {
    return fromF32<TO>(toF32(v));
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) typecastKernel(const TI *__restrict__ in, TO *__restrict__ out, size_t n) {
  size_t nvec = n / kVec;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<TI, kVec> x;
    Pack<TO, kVec> y;
    loadPack(x, in + i * kVec);
#pragma unroll
    for (int j = 0; j < kVec; ++j) y.v[j] = convertElem<TI, TO>(x.v[j]);
    storePack(out + i * kVec, y);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n) out[tail] = convertElem<TI, TO>(in[tail]);
}

template <typename T> __global__ void __launch_bounds__(256) fillKernel(T *out, size_t n, T v) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = v;
}

template <typename T>
__global__ void __launch_bounds__(256) arangeKernel(T *out, size_t n, double start, double step) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    double v = start + step * static_cast<double>(i);
    if constexpr (std::is_integral<T>::value) out[i] = static_cast<T>(static_cast<long long>(v));
    else out[i] = fromF32<T>(static_cast<float>(v));
  }
}

// silu(g) rounded to T, times u, rounded to T: the two roundings of the unfused op pair.
template <typename T>
__global__ void __launch_bounds__(256) siluMulKernel(const T *__restrict__ g, const T *__restrict__ u,
                                                     T *__restrict__ out, size_t n) {
  size_t nvec = n / kVec;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<T, kVec> x, y, z;
    loadPack(x, g + i * kVec);
    loadPack(y, u + i * kVec);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      float s = toF32(fromF32<T>(applyUnary(uSilu, toF32(x.v[j]), 0.0f)));
      z.v[j] = fromF32<T>(s * toF32(y.v[j]));
    }
    storePack(out + i * kVec, z);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n) {
    float s = toF32(fromF32<T>(applyUnary(uSilu, toF32(g[tail]), 0.0f)));
    out[tail] = fromF32<T>(s * toF32(u[tail]));
  }
}

static int fillDims(BcastDims &d, int rank, const int64_t *shape, const int64_t *sa, const int64_t *sb,
                    const int64_t *sc, size_t &n) {
  TTB_CHECK(rank >= 0 && rank <= 8, "rank must be <= 8");
  d.rank = rank;
  n = 1;
  for (int i = 0; i < rank; ++i) {
    TTB_CHECK(shape[i] >= 0, "negative dimension");
    d.shape[i] = shape[i];
    d.sa[i] = sa ? sa[i] : 0;
    d.sb[i] = sb ? sb[i] : 0;
    d.sc[i] = sc ? sc[i] : 0;
    n *= static_cast<size_t>(shape[i]);
  }
  return TTB_OK;
}

// If `strides` index a dense tensor that is broadcast over leading dims only, returns its
// element count (so that element i of the output reads i % count); 0 otherwise.
static size_t trailingDenseCount(int rank, const int64_t *shape, const int64_t *strides) {
  size_t expect = 1;
  int k = rank - 1;
  for (; k >= 0; --k) {
    if (shape[k] == 1) continue;
    if (strides[k] != static_cast<int64_t>(expect)) break;
    expect *= static_cast<size_t>(shape[k]);
  }
  for (; k >= 0; --k) {
    if (shape[k] != 1 && strides[k] != 0) return 0;
  }
  return expect;
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_eltwise_unary(int op, const void *in, int in_dtype, void *out, int out_dtype, size_t n, float param,
                      void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK((op >= 0 && op < uCount) || op == uCbrt || op == uLog1p || op == uPowScalar, "unknown unary op");
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("eltwise_unary", 0, double(n) * (dtypeSize(in_dtype) + dtypeSize(out_dtype)), st);
  bool vec = in_dtype == out_dtype && aligned16(in) && aligned16(out) && op != uBitwiseNot;
  if (vec && in_dtype == kBF16) {
    unaryVecKernel<__nv_bfloat16><<<gridFor((n + kVec - 1) / kVec, 256), 256, 0, st>>>(
        op, static_cast<const __nv_bfloat16 *>(in), static_cast<__nv_bfloat16 *>(out), n, param);
  } else if (vec && in_dtype == kF32) {
    unaryVecKernel<float><<<gridFor((n + kVec - 1) / kVec, 256), 256, 0, st>>>(
        op, static_cast<const float *>(in), static_cast<float *>(out), n, param);
  } else {
    TTB_CHECK(dtypeSize(in_dtype) && dtypeSize(out_dtype), "unsupported dtype");
    unaryGenericKernel<<<gridFor(n, 256), 256, 0, st>>>(op, in, in_dtype, out, out_dtype, n, param);
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_eltwise_binary(int op, const void *a, int a_dtype, const void *b, int b_dtype, void *out, int out_dtype,
                       int rank, const int64_t *out_shape, const int64_t *a_strides, const int64_t *b_strides,
                       void *stream) {
  TTB_CHECK(a && b && out, "null tensor");
  TTB_CHECK(dtypeSize(a_dtype) && dtypeSize(b_dtype) && dtypeSize(out_dtype), "unsupported dtype");
  BcastDims d;
  size_t n;
  if (int rc = fillDims(d, rank, out_shape, a_strides, b_strides, nullptr, n)) return rc;
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  bool floatOp = op == bAdd || op == bMultiply || op == bSubtract || op == bDivide || op == bMaximum ||
                 op == bMinimum || (op >= bEqual && op <= bLessThan);
  ProfScope prof("eltwise_binary", 0, double(n) * (dtypeSize(a_dtype) + dtypeSize(b_dtype) + dtypeSize(out_dtype)), st);
  size_t aCnt = trailingDenseCount(rank, out_shape, a_strides);
  size_t bCnt = trailingDenseCount(rank, out_shape, b_strides);
  bool vec = floatOp && a_dtype == b_dtype && a_dtype == out_dtype && (a_dtype == kBF16 || a_dtype == kF32) &&
             aCnt && bCnt && aCnt % kVec == 0 && bCnt % kVec == 0 && (aCnt == n || bCnt == n) &&
             aligned16(a) && aligned16(b) && aligned16(out);
  if (vec && a_dtype == kBF16) {
    binaryVecKernel<__nv_bfloat16><<<gridFor((n + kVec - 1) / kVec, 256), 256, 0, st>>>(
        op, static_cast<const __nv_bfloat16 *>(a), static_cast<const __nv_bfloat16 *>(b),
        static_cast<__nv_bfloat16 *>(out), n, aCnt, bCnt);
  } else if (vec) {
    binaryVecKernel<float><<<gridFor((n + kVec - 1) / kVec, 256), 256, 0, st>>>(
        op, static_cast<const float *>(a), static_cast<const float *>(b), static_cast<float *>(out), n, aCnt, bCnt);
  } else {
    binaryGenericKernel<<<gridFor(n, 256), 256, 0, st>>>(op, a, a_dtype, b, b_dtype, out, out_dtype, n, d);
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_where(const void *cond, int cond_dtype, const void *a, const void *b, int dtype, void *out, int rank,
              const int64_t *out_shape, const int64_t *c_strides, const int64_t *a_strides,
              const int64_t *b_strides, void *stream) {
  TTB_CHECK(cond && a && b && out, "null tensor");
  TTB_CHECK(dtypeSize(cond_dtype) && dtypeSize(dtype), "unsupported dtype");
  BcastDims d;
  size_t n;
  if (int rc = fillDims(d, rank, out_shape, a_strides, b_strides, c_strides, n)) return rc;
  if (n == 0) return TTB_OK;
  whereKernel<<<gridFor(n, 256), 256, 0, asStream(stream)>>>(cond, cond_dtype, a, b, dtype, out, n, d);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_clamp(const void *in, int dtype, void *out, size_t n, float lo, float hi, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (n == 0) return TTB_OK;
  TTB_DISPATCH_DTYPE(dtype, T, {
    clampKernel<T><<<gridFor(n, 256), 256, 0, asStream(stream)>>>(static_cast<const T *>(in),
                                                                  static_cast<T *>(out), n, lo, hi);
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_typecast(const void *in, int in_dtype, void *out, int out_dtype, size_t n, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(aligned16(in) && aligned16(out), "tensors must be 16-byte aligned");
  if (n == 0) return TTB_OK;
  if (in_dtype == out_dtype) {
    return ttb_memcpy_d2d(out, in, n * dtypeSize(in_dtype), stream);
  }
  int grid = gridFor((n + kVec - 1) / kVec, 256);
  ProfScope prof("typecast", 0, double(n) * (dtypeSize(in_dtype) + dtypeSize(out_dtype)), asStream(stream));
  TTB_DISPATCH_DTYPE(in_dtype, TI, TTB_DISPATCH_DTYPE(out_dtype, TO, {
    typecastKernel<TI, TO><<<grid, 256, 0, asStream(stream)>>>(static_cast<const TI *>(in),
                                                               static_cast<TO *>(out), n);
  }));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_fill(void *out, int dtype, size_t n, double value, void *stream) {
  TTB_CHECK(out, "null tensor");
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  int grid = gridFor(n, 256);
  switch (dtype) {
  case kF32: fillKernel<float><<<grid, 256, 0, st>>>(static_cast<float *>(out), n, static_cast<float>(value)); break;
  case kBF16: fillKernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<__nv_bfloat16 *>(out), n, __float2bfloat16_rn(static_cast<float>(value))); break;
  case kF16: fillKernel<__half><<<grid, 256, 0, st>>>(static_cast<__half *>(out), n, __float2half_rn(static_cast<float>(value))); break;
  case kI32: fillKernel<int32_t><<<grid, 256, 0, st>>>(static_cast<int32_t *>(out), n, static_cast<int32_t>(value)); break;
  case kU32: fillKernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<uint32_t *>(out), n, static_cast<uint32_t>(value)); break;
  case kU16: fillKernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<uint16_t *>(out), n, static_cast<uint16_t>(value)); break;
  case kU8: fillKernel<uint8_t><<<grid, 256, 0, st>>>(static_cast<uint8_t *>(out), n, static_cast<uint8_t>(value)); break;
  case kI8: fillKernel<int8_t><<<grid, 256, 0, st>>>(static_cast<int8_t *>(out), n, static_cast<int8_t>(value)); break;
  default: setLastError("fill: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_arange(void *out, int dtype, size_t n, double start, double step, void *stream) {
  TTB_CHECK(out, "null tensor");
  if (n == 0) return TTB_OK;
  TTB_DISPATCH_DTYPE(dtype, T, {
    arangeKernel<T><<<gridFor(n, 256), 256, 0, asStream(stream)>>>(static_cast<T *>(out), n, start, step);
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_silu_mul(const void *gate, const void *up, void *out, int dtype, size_t n, void *stream) {
  TTB_CHECK(gate && up && out, "null tensor");
  TTB_CHECK(aligned16(gate) && aligned16(up) && aligned16(out), "tensors must be 16-byte aligned");
  if (n == 0) return TTB_OK;
  int grid = gridFor((n + kVec - 1) / kVec, 256);
  ProfScope prof("silu_mul", 0, double(n) * 3 * dtypeSize(dtype), asStream(stream));
  TTB_DISPATCH_FLOAT(dtype, T, {
    siluMulKernel<T><<<grid, 256, 0, asStream(stream)>>>(static_cast<const T *>(gate), static_cast<const T *>(up),
                                                         static_cast<T *>(out), n);
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
