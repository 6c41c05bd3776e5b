// quantize / dequantize / requantize and the fused chain: HBM-bound streaming kernels.
//
// Arithmetic (bit-exact with torch.quantize_per_tensor / torch.dequantize, which are the
// goldens the reference checks these ops against, tools/golden/mapping.py:2534-2582):
//   q  = clamp(rne(x * inv_scale) + zp)   with inv_scale = 1.0f / scale computed once in f32
//   x' = float(q - zp) * scale
//   requantize = quantize(dequantize(q)) with both f32 roundings kept.
// Each thread moves 16 elements per iteration with 16-byte streaming loads and stores, so a
// warp touches 512 contiguous elements; the grid is a few waves of the SM count and strides.
#include "common.cuh"

#include <climits>

namespace ttb {

struct QRange {
  int lo, hi;
};

template <typename TQ> __host__ __device__ inline QRange qrangeOf(int clampI8) {
  if (sizeof(TQ) == 1) {
    return (TQ(-1) < TQ(0)) ? QRange{-128, 127} : QRange{0, 255};
  }
  if (sizeof(TQ) == 2) {
    return QRange{0, 65535};
  }
  if (clampI8) {
    return QRange{-128, 127};
  }
  return (TQ(-1) < TQ(0)) ? QRange{INT_MIN, INT_MAX} : QRange{0, INT_MAX};
}

// Narrow ranges (int8 / uint8 / uint16 containers, or int32 holding int8 values) never leave the
// float pipe: rint, float->int and int->float all issue on the quarter-rate conversion unit, and
// six of them per element made the fused chain issue-bound at half the HBM rate.  Instead:
// round half to even with the 1.5 * 2^23 trick (exact for |t| < 2^22; t is clamped to that first,
// which cannot change the result because the final range is far narrower), clamp in float, and
// carry q - zp as an integer-valued float.
struct QNarrow {
  float lo, hi; // range of q - zp
  int zp;
  bool ok;
};
__host__ __device__ inline QNarrow narrowOf(QRange r, int zp) {
  QNarrow n;
  n.ok = (static_cast<long long>(r.hi) - r.lo) <= 65535ll && zp > -(1 << 20) && zp < (1 << 20);
  n.lo = static_cast<float>(static_cast<long long>(r.lo) - zp);
  n.hi = static_cast<float>(static_cast<long long>(r.hi) - zp);
  n.zp = zp;
  return n;
}
// Clamping first and rounding second gives what rounding first gives (the bounds are integers, rounding is
// monotonic and leaves integers alone) and keeps the magic-number rounding inside its exact range without a
// second clamp: min / max issue on the half-rate ALU pipe, which is what bounded the fused chain.
// MAYBE_NAN = false: x is known to be a number (a dequantized integer), so the NaN -> 0 step is dropped.
template <bool MAYBE_NAN = true> __device__ __forceinline__ float roundClampNarrow(float x, float inv, QNarrow n) {
  float t = __fmul_rn(x, inv);
  if (MAYBE_NAN) t = (t != t) ? 0.0f : t;
  t = fminf(fmaxf(t, n.lo), n.hi);
  return __fsub_rn(__fadd_rn(t, 12582912.0f), 12582912.0f); // nearest integer, ties to even
}
// integer-valued float in (-2^22, 2^22) -> int without a conversion instruction
__device__ __forceinline__ int floatIntBits(float r) { return __float_as_int(__fadd_rn(r, 12582912.0f)) - 0x4B400000; }

__device__ __forceinline__ int quantOne(float x, float inv, int zp, QRange r) {
  QNarrow n = narrowOf(r, zp);
  if (n.ok) return floatIntBits(roundClampNarrow(x, inv, n)) + zp;
  // Full 32-bit range: the conversion saturates, the 64-bit add cannot wrap.
  float t = rintf(__fmul_rn(x, inv));
  long long q = static_cast<long long>(__float2int_rn(t)) + zp;
  q = q < r.lo ? r.lo : q;
  q = q > r.hi ? r.hi : q;
  return static_cast<int>(q);
}

__device__ __forceinline__ float dequantOne(int q, float scale, int zp) {
  return __fmul_rn(static_cast<float>(q - zp), scale);
}

constexpr int kVec = 16;

// ---- per-tensor ------------------------------------------------------------------------
template <typename TI, typename TQ>
__global__ void __launch_bounds__(256) quantizeKernel(const TI *__restrict__ in, TQ *__restrict__ out,
                                                      size_t n, float inv, int zp, QRange r) {
  size_t nvec = n / kVec;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<TI, kVec> x;
    Pack<TQ, kVec> q;
    loadPack(x, in + i * kVec);
#pragma unroll
    for (int j = 0; j < kVec; ++j) q.v[j] = static_cast<TQ>(quantOne(toF32(x.v[j]), inv, zp, r));
    storePack(out + i * kVec, q);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n) out[tail] = static_cast<TQ>(quantOne(toF32(in[tail]), inv, zp, r));
}

template <typename TQ, typename TO>
__global__ void __launch_bounds__(256) dequantizeKernel(const TQ *__restrict__ in, TO *__restrict__ out,
                                                        size_t n, float scale, int zp) {
  size_t nvec = n / kVec;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<TQ, kVec> q;
    Pack<TO, kVec> x;
    loadPack(q, in + i * kVec);
#pragma unroll
    for (int j = 0; j < kVec; ++j) x.v[j] = fromF32<TO>(dequantOne(static_cast<int>(q.v[j]), scale, zp));
    storePack(out + i * kVec, x);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n) out[tail] = fromF32<TO>(dequantOne(static_cast<int>(in[tail]), scale, zp));
}

template <typename TA, typename TB>
__global__ void __launch_bounds__(256) requantizeKernel(const TA *__restrict__ in, TB *__restrict__ out,
                                                        size_t n, float sIn, int zpIn, float invOut,
                                                        int zpOut, QRange r) {
  size_t nvec = n / kVec;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<TA, kVec> a;
    Pack<TB, kVec> b;
    loadPack(a, in + i * kVec);
#pragma unroll
    for (int j = 0; j < kVec; ++j)
      b.v[j] = static_cast<TB>(quantOne(dequantOne(static_cast<int>(a.v[j]), sIn, zpIn), invOut, zpOut, r));
    storePack(out + i * kVec, b);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n)
    out[tail] = static_cast<TB>(quantOne(dequantOne(static_cast<int>(in[tail]), sIn, zpIn), invOut, zpOut, r));
}

// quantize -> requantize -> dequantize, one read of x and one write of the result; the two
// integer intermediates are written only when the caller wants them.
template <typename TI, typename T1, typename T2, typename TO, bool W1, bool W2>
__global__ void __launch_bounds__(256)
    quantChainKernel(const TI *__restrict__ in, T1 *__restrict__ q1, T2 *__restrict__ q2,
                     TO *__restrict__ out, size_t n, float inv1, float s1, int zp1, float inv2, float s2,
                     int zp2, QRange r1, QRange r2) {
  // Eight elements per thread and iteration (one 16-byte load for 16-bit input): with one
  // resident wave of blocks every thread then runs ~7 iterations on the benchmark's 16.7 M
  // elements, so the ragged last iteration costs 1 % instead of the 13 % it cost with 16.
  // (16 when byte-wide intermediates are written, whose vectors must still be 16 bytes).
  constexpr int kVec = ((W1 && sizeof(T1) == 1) || (W2 && sizeof(T2) == 1)) ? 16 : 8;
  size_t nvec = n / kVec;
  const QNarrow n1 = narrowOf(r1, zp1), n2 = narrowOf(r2, zp2);
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<TI, kVec> x;
    Pack<T1, kVec> a;
    Pack<T2, kVec> b;
    Pack<TO, kVec> y;
    loadPack(x, in + i * kVec);
    if (n1.ok && n2.ok) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        float ra = roundClampNarrow(toF32(x.v[j]), inv1, n1);             // q1 - zp1
        float rb = roundClampNarrow<false>(__fmul_rn(ra, s1), inv2, n2);   // q2 - zp2
        if (W1) a.v[j] = static_cast<T1>(floatIntBits(ra) + zp1);
        if (W2) b.v[j] = static_cast<T2>(floatIntBits(rb) + zp2);
        y.v[j] = fromF32<TO>(__fmul_rn(rb, s2));
      }
    } else {
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        int qa = quantOne(toF32(x.v[j]), inv1, zp1, r1);
        int qb = quantOne(dequantOne(qa, s1, zp1), inv2, zp2, r2);
        a.v[j] = static_cast<T1>(qa);
        b.v[j] = static_cast<T2>(qb);
        y.v[j] = fromF32<TO>(dequantOne(qb, s2, zp2));
      }
    }
    if constexpr (W1) storePack(q1 + i * kVec, a);
    if constexpr (W2) storePack(q2 + i * kVec, b);
    storePack(out + i * kVec, y);
  }
  size_t tail = nvec * kVec + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tail < n) {
    int qa = quantOne(toF32(in[tail]), inv1, zp1, r1);
    int qb = quantOne(dequantOne(qa, s1, zp1), inv2, zp2, r2);
    if (W1) q1[tail] = static_cast<T1>(qa);
    if (W2) q2[tail] = static_cast<T2>(qb);
    out[tail] = fromF32<TO>(dequantOne(qb, s2, zp2));
  }
}

// ---- per-axis: tensor viewed as [outer, axisLen, inner] ------------------------------------
template <typename TI, typename TQ>
__global__ void __launch_bounds__(256)
    quantizeAxisKernel(const TI *__restrict__ in, TQ *__restrict__ out, size_t n, size_t axisLen, size_t inner,
                       const float *__restrict__ scales, const int *__restrict__ zps, QRange r) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    size_t c = (i / inner) % axisLen;
    float inv = __fdiv_rn(1.0f, scales[c]);
    int zp = zps ? zps[c] : 0;
    out[i] = static_cast<TQ>(quantOne(toF32(in[i]), inv, zp, r));
  }
}

template <typename TQ, typename TO>
__global__ void __launch_bounds__(256)
    dequantizeAxisKernel(const TQ *__restrict__ in, TO *__restrict__ out, size_t n, size_t axisLen, size_t inner,
                         const float *__restrict__ scales, const int *__restrict__ zps) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    size_t c = (i / inner) % axisLen;
    int zp = zps ? zps[c] : 0;
    out[i] = fromF32<TO>(dequantOne(static_cast<int>(in[i]), scales[c], zp));
  }
}

// inner % 16 == 0: a 16-element pack never straddles two channels, so it shares one scale.
template <typename TQ, typename TO>
__global__ void __launch_bounds__(256)
    dequantizeAxisVecKernel(const TQ *__restrict__ in, TO *__restrict__ out, size_t nvec, size_t axisLen, size_t innerVec,
                            const float *__restrict__ scales, const int *__restrict__ zps) {
  size_t per = (nvec + gridDim.x - 1) / gridDim.x;
  size_t first = per * blockIdx.x, last = first + per < nvec ? first + per : nvec;
  for (size_t i = first + threadIdx.x; i < last; i += blockDim.x) {
    size_t c = (i / innerVec) % axisLen;
    float sc = __ldg(scales + c);
    int zp = zps ? __ldg(zps + c) : 0;
    Pack<TQ, kVec> q;
    Pack<TO, kVec> x;
    loadPack(q, in + i * kVec);
#pragma unroll
    for (int j = 0; j < kVec; ++j) x.v[j] = fromF32<TO>(dequantOne(static_cast<int>(q.v[j]), sc, zp));
    storePack(out + i * kVec, x);
  }
}

template <typename TA, typename TB>
__global__ void __launch_bounds__(256)
    requantizeAxisKernel(const TA *__restrict__ in, TB *__restrict__ out, size_t n, size_t axisLen, size_t inner,
                         const float *__restrict__ sIn, const int *__restrict__ zIn,
                         const float *__restrict__ sOut, const int *__restrict__ zOut, QRange r) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    size_t c = (i / inner) % axisLen;
    float inv = __fdiv_rn(1.0f, sOut[c]);
    float x = dequantOne(static_cast<int>(in[i]), sIn[c], zIn ? zIn[c] : 0);
    out[i] = static_cast<TB>(quantOne(x, inv, zOut ? zOut[c] : 0, r));
  }
}

static bool vecOk(const void *a, const void *b) { return aligned16(a) && aligned16(b); }

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_quantize(const void *in, int in_dtype, void *out, int out_dtype, size_t n, float scale,
                 int32_t zero_point, int clamp_i8, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(scale > 0.0f, "scale must be positive");
  TTB_CHECK(vecOk(in, out), "tensors must be 16-byte aligned");
  if (n == 0) return TTB_OK;
  float inv = 1.0f / scale;
  int grid = gridFor((n + kVec - 1) / kVec, 256);
  ProfScope prof("quantize", 0, double(n) * (dtypeSize(in_dtype) + dtypeSize(out_dtype)), asStream(stream));
  TTB_DISPATCH_FLOAT(in_dtype, TI, TTB_DISPATCH_INT(out_dtype, TQ, {
    quantizeKernel<TI, TQ><<<grid, 256, 0, asStream(stream)>>>(
        static_cast<const TI *>(in), static_cast<TQ *>(out), n, inv, zero_point, qrangeOf<TQ>(clamp_i8));
  }));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_dequantize(const void *in, int in_dtype, void *out, int out_dtype, size_t n, float scale,
                   int32_t zero_point, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(vecOk(in, out), "tensors must be 16-byte aligned");
  if (n == 0) return TTB_OK;
  int grid = gridFor((n + kVec - 1) / kVec, 256);
  ProfScope prof("dequantize", 0, double(n) * (dtypeSize(in_dtype) + dtypeSize(out_dtype)), asStream(stream));
  TTB_DISPATCH_INT(in_dtype, TQ, TTB_DISPATCH_FLOAT(out_dtype, TO, {
    dequantizeKernel<TQ, TO><<<grid, 256, 0, asStream(stream)>>>(
        static_cast<const TQ *>(in), static_cast<TO *>(out), n, scale, zero_point);
  }));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_requantize(const void *in, int in_dtype, void *out, int out_dtype, size_t n, float in_scale,
                   int32_t in_zp, float out_scale, int32_t out_zp, int clamp_i8, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(out_scale > 0.0f, "scale must be positive");
  TTB_CHECK(vecOk(in, out), "tensors must be 16-byte aligned");
  if (n == 0) return TTB_OK;
  float inv = 1.0f / out_scale;
  int grid = gridFor((n + kVec - 1) / kVec, 256);
  ProfScope prof("requantize", 0, double(n) * (dtypeSize(in_dtype) + dtypeSize(out_dtype)), asStream(stream));
  TTB_DISPATCH_INT(in_dtype, TA, TTB_DISPATCH_INT(out_dtype, TB, {
    requantizeKernel<TA, TB><<<grid, 256, 0, asStream(stream)>>>(
        static_cast<const TA *>(in), static_cast<TB *>(out), n, in_scale, in_zp, inv, out_zp,
        qrangeOf<TB>(clamp_i8));
  }));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_quantize_per_axis(const void *in, int in_dtype, void *out, int out_dtype, size_t outer,
                          size_t axis_len, size_t inner, const float *scales, const int32_t *zero_points,
                          int clamp_i8, void *stream) {
  TTB_CHECK(in && out && scales, "null tensor");
  size_t n = outer * axis_len * inner;
  if (n == 0) return TTB_OK;
  int grid = gridFor(n, 256);
  TTB_DISPATCH_FLOAT(in_dtype, TI, TTB_DISPATCH_INT(out_dtype, TQ, {
    quantizeAxisKernel<TI, TQ><<<grid, 256, 0, asStream(stream)>>>(
        static_cast<const TI *>(in), static_cast<TQ *>(out), n, axis_len, inner, scales, zero_points,
        qrangeOf<TQ>(clamp_i8));
  }));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_dequantize_per_axis(const void *in, int in_dtype, void *out, int out_dtype, size_t outer,
                            size_t axis_len, size_t inner, const float *scales, const int32_t *zero_points,
                            void *stream) {
  TTB_CHECK(in && out && scales, "null tensor");
  size_t n = outer * axis_len * inner;
  if (n == 0) return TTB_OK;
  ProfScope prof("dequantize_per_axis", 0, double(n) * (dtypeSize(in_dtype) + dtypeSize(out_dtype)), asStream(stream));
  if (inner % kVec == 0 && vecOk(in, out)) {
    int grid = gridFor(n / kVec, 256, 8);
    TTB_DISPATCH_INT(in_dtype, TQ, TTB_DISPATCH_FLOAT(out_dtype, TO, {
      dequantizeAxisVecKernel<TQ, TO><<<grid, 256, 0, asStream(stream)>>>(
          static_cast<const TQ *>(in), static_cast<TO *>(out), n / kVec, axis_len, inner / kVec, scales, zero_points);
    }));
  } else {
    int grid = gridFor(n, 256);
    TTB_DISPATCH_INT(in_dtype, TQ, TTB_DISPATCH_FLOAT(out_dtype, TO, {
      dequantizeAxisKernel<TQ, TO><<<grid, 256, 0, asStream(stream)>>>(
          static_cast<const TQ *>(in), static_cast<TO *>(out), n, axis_len, inner, scales, zero_points);
    }));
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_requantize_per_axis(const void *in, int in_dtype, void *out, int out_dtype, size_t outer,
                            size_t axis_len, size_t inner, const float *in_scales, const int32_t *in_zps,
                            const float *out_scales, const int32_t *out_zps, int clamp_i8, void *stream) {
  TTB_CHECK(in && out && in_scales && out_scales, "null tensor");
  size_t n = outer * axis_len * inner;
  if (n == 0) return TTB_OK;
  int grid = gridFor(n, 256);
  TTB_DISPATCH_INT(in_dtype, TA, TTB_DISPATCH_INT(out_dtype, TB, {
    requantizeAxisKernel<TA, TB><<<grid, 256, 0, asStream(stream)>>>(
        static_cast<const TA *>(in), static_cast<TB *>(out), n, axis_len, inner, in_scales, in_zps,
        out_scales, out_zps, qrangeOf<TB>(clamp_i8));
  }));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"

namespace {
template <typename TI, typename T1, typename T2, typename TO>
int launchChain(const void *in, void *q1, void *q2, void *out, size_t n, float s1, int zp1, float s2, int zp2,
                int clampI8, cudaStream_t st) {
  float inv1 = 1.0f / s1, inv2 = 1.0f / s2;
  const int vec = ((q1 && sizeof(T1) == 1) || (q2 && sizeof(T2) == 1)) ? 16 : 8;
  int grid = gridFor((n + vec - 1) / vec, 256, 8); // 8 blocks of 256 threads per SM: one resident wave
  QRange r1 = qrangeOf<T1>(clampI8), r2 = qrangeOf<T2>(clampI8);
  auto I = static_cast<const TI *>(in);
  auto A = static_cast<T1 *>(q1);
  auto B = static_cast<T2 *>(q2);
  auto O = static_cast<TO *>(out);
  ProfScope prof("quant_chain", 0, double(n) * (sizeof(TI) + sizeof(TO) + (q1 ? sizeof(T1) : 0) + (q2 ? sizeof(T2) : 0)), st);
  if (q1 && q2)
    quantChainKernel<TI, T1, T2, TO, true, true><<<grid, 256, 0, st>>>(I, A, B, O, n, inv1, s1, zp1, inv2, s2, zp2, r1, r2);
  else if (q1)
    quantChainKernel<TI, T1, T2, TO, true, false><<<grid, 256, 0, st>>>(I, A, B, O, n, inv1, s1, zp1, inv2, s2, zp2, r1, r2);
  else if (q2)
    quantChainKernel<TI, T1, T2, TO, false, true><<<grid, 256, 0, st>>>(I, A, B, O, n, inv1, s1, zp1, inv2, s2, zp2, r1, r2);
  else
    quantChainKernel<TI, T1, T2, TO, false, false><<<grid, 256, 0, st>>>(I, A, B, O, n, inv1, s1, zp1, inv2, s2, zp2, r1, r2);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}
} // namespace

extern "C" {

int ttb_quant_chain(const void *in, int in_dtype, void *q1, int q1_dtype, void *q2, int q2_dtype, void *out,
                    int out_dtype, size_t n, float scale1, int32_t zp1, float scale2, int32_t zp2,
                    int clamp_i8, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(scale1 > 0.0f && scale2 > 0.0f && scale1 <= 3.0e38f && scale2 <= 3.0e38f, "scale must be positive and finite");
  TTB_CHECK(vecOk(in, out) && aligned16(q1) && aligned16(q2), "tensors must be 16-byte aligned");
  TTB_CHECK(q1_dtype == q2_dtype, "intermediate dtypes must match");
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  // The chain the compiler emits is float -> int -> int -> float; instantiate the dtype
  // combinations that occur (bf16/f32 in, i8/u8/i32 intermediates, f32/bf16 out).
#define TTB_CHAIN(TI, TQ, TO) return launchChain<TI, TQ, TQ, TO>(in, q1, q2, out, n, scale1, zp1, scale2, zp2, clamp_i8, st)
#define TTB_CHAIN_Q(TI, TO)                                                                                  \
  switch (q1_dtype) {                                                                                        \
  case kI8: TTB_CHAIN(TI, int8_t, TO);                                                                       \
  case kU8: TTB_CHAIN(TI, uint8_t, TO);                                                                      \
  case kI32: TTB_CHAIN(TI, int32_t, TO);                                                                     \
  default: break;                                                                                            \
  }
  if (in_dtype == kBF16 && out_dtype == kF32) { TTB_CHAIN_Q(__nv_bfloat16, float) }
  else if (in_dtype == kBF16 && out_dtype == kBF16) { TTB_CHAIN_Q(__nv_bfloat16, __nv_bfloat16) }
  else if (in_dtype == kF32 && out_dtype == kF32) { TTB_CHAIN_Q(float, float) }
  else if (in_dtype == kF32 && out_dtype == kBF16) { TTB_CHAIN_Q(float, __nv_bfloat16) }
#undef TTB_CHAIN_Q
#undef TTB_CHAIN
  setLastError("quant chain: unsupported dtype combination");
  return TTB_ERR_UNSUPPORTED;
}

} // extern "C"
