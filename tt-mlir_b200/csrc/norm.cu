// softmax, rms_norm (+ fused residual add) and reductions.  All are HBM-bound row kernels:
// 16-byte loads, f32 accumulation, warp-shuffle + shared-memory reductions.
//
// Reference semantics:
//  softmax  exp(x - max) * (1 / sum)   lib/Conversion/TTIRToLinalg/TTIRToLinalg.cpp:956-1017,
//           torch twin tools/tt-alchemist/templates/python/local/ttir_cpu.py:585
//  rms_norm x * rsqrt(mean(x^2) + eps) * w (+ b), computed in f32, rounded once
//           include/ttmlir/Dialect/TTIR/IR/TTIROps.td:2300-2336, golden tools/golden/mapping.py:1221-1290
//  reduce   sum / mean / max / min over a dimension, f32 accumulation  ttir_cpu.py:374-397
#include "common.cuh"

#include <cfloat>
#include <type_traits>

namespace ttb {

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warpMin(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum across a block of up to 1024 threads; every thread gets the result.
__device__ __forceinline__ float blockSum(float v, float *scratch /* 33 floats */) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warpSum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.0f;
    t = warpSum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  float r = scratch[32];
  __syncthreads();
  return r;
}

// ---- softmax ---------------------------------------------------------------------------
// inner == 1: one warp per row.
template <typename T>
__global__ void __launch_bounds__(256) softmaxRowKernel(const T *__restrict__ in, T *__restrict__ out, size_t rows,
                                                        size_t len) {
  size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T *x = in + row * len;
  T *y = out + row * len;
  float m = -INFINITY;
  for (size_t i = lane; i < len; i += 32) m = fmaxf(m, toF32(x[i]));
  m = warpMax(m);
  float s = 0.0f;
  for (size_t i = lane; i < len; i += 32) s += expf(toF32(x[i]) - m);
  s = warpSum(s);
  float inv = 1.0f / s;
  for (size_t i = lane; i < len; i += 32) y[i] = fromF32<T>(expf(toF32(x[i]) - m) * inv);
}

// inner > 1: one thread per (outer, inner) column; neighbouring threads read neighbouring addresses.
template <typename T>
__global__ void __launch_bounds__(256) softmaxColKernel(const T *__restrict__ in, T *__restrict__ out, size_t outer,
                                                        size_t len, size_t inner) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < outer * inner; c += stride) {
    size_t base = (c / inner) * len * inner + (c % inner);
    float m = -INFINITY;
    for (size_t i = 0; i < len; ++i) m = fmaxf(m, toF32(in[base + i * inner]));
    float s = 0.0f;
    for (size_t i = 0; i < len; ++i) s += expf(toF32(in[base + i * inner]) - m);
    float inv = 1.0f / s;
    for (size_t i = 0; i < len; ++i) out[base + i * inner] = fromF32<T>(expf(toF32(in[base + i * inner]) - m) * inv);
  }
}

// ---- rms_norm --------------------------------------------------------------------------
// One block per row.  The row is held in registers (P packs of 16 elements per thread) so the
// input is read from HBM exactly once.  RES: x = round(a + b) first (fused residual add).
template <typename T, int P, bool RES>
__global__ void __launch_bounds__(256)
    rmsNormKernel(const T *__restrict__ a, const T *__restrict__ b, const T *__restrict__ w,
                  const T *__restrict__ bias, T *__restrict__ sumOut, T *__restrict__ out, size_t cols, float eps) {
  constexpr int V = 16;
  __shared__ float scratch[33];
  size_t row = blockIdx.x;
  const T *x = a + row * cols;
  Pack<T, V> r[P];
  float ss = 0.0f;
  size_t nvec = cols / V;
#pragma unroll
  for (int p = 0; p < P; ++p) {
    size_t v = threadIdx.x + static_cast<size_t>(p) * blockDim.x;
    if (v < nvec) {
      loadPack(r[p], x + v * V);
      if (RES) {
        Pack<T, V> q;
        loadPack(q, b + row * cols + v * V);
#pragma unroll
        for (int j = 0; j < V; ++j) r[p].v[j] = fromF32<T>(toF32(r[p].v[j]) + toF32(q.v[j]));
        if (sumOut) storePack(sumOut + row * cols + v * V, r[p]);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float f = toF32(r[p].v[j]);
        ss += f * f;
      }
    }
  }
  ss = blockSum(ss, scratch);
  float rstd = rsqrtf(ss / static_cast<float>(cols) + eps);
#pragma unroll
  for (int p = 0; p < P; ++p) {
    size_t v = threadIdx.x + static_cast<size_t>(p) * blockDim.x;
    if (v < nvec) {
      Pack<T, V> y;
      Pack<T, V> wv;
      if (w) loadPack(wv, w + v * V); // weights are re-read by every row: L2 resident
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float f = toF32(r[p].v[j]) * rstd;
        if (w) f *= toF32(wv.v[j]);
        if (bias) f += toF32(bias[v * V + j]);
        y.v[j] = fromF32<T>(f);
      }
      storePack(out + row * cols + v * V, y);
    }
  }
}

// Any width: two passes over the row (second one hits L1/L2).
template <typename T, bool RES>
__global__ void __launch_bounds__(256)
    rmsNormGenericKernel(const T *__restrict__ a, const T *__restrict__ b, const T *__restrict__ w,
                         const T *__restrict__ bias, T *__restrict__ sumOut, T *__restrict__ out, size_t cols,
                         float eps) {
  __shared__ float scratch[33];
  size_t row = blockIdx.x;
  float ss = 0.0f;
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float f = toF32(a[row * cols + i]);
    if (RES) {
      f = toF32(fromF32<T>(f + toF32(b[row * cols + i])));
      if (sumOut) sumOut[row * cols + i] = fromF32<T>(f);
    }
    ss += f * f;
  }
  ss = blockSum(ss, scratch);
  float rstd = rsqrtf(ss / static_cast<float>(cols) + eps);
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float f = toF32(a[row * cols + i]);
    if (RES) f = toF32(fromF32<T>(f + toF32(b[row * cols + i])));
    f *= rstd;
    if (w) f *= toF32(w[i]);
    if (bias) f += toF32(bias[i]);
    out[row * cols + i] = fromF32<T>(f);
  }
}

template <typename T, bool RES>
int launchRms(const void *a, const void *b, const void *w, const void *bias, void *sumOut, void *out, size_t rows,
              size_t cols, float eps, cudaStream_t st) {
  auto A = static_cast<const T *>(a), B = static_cast<const T *>(b), W = static_cast<const T *>(w),
       Bi = static_cast<const T *>(bias);
  auto S = static_cast<T *>(sumOut), O = static_cast<T *>(out);
  bool al = aligned16(a) && aligned16(b) && aligned16(w) && aligned16(out) && aligned16(sumOut);
  int grid = static_cast<int>(rows);
  ProfScope prof(RES ? "add_rms_norm" : "rms_norm", 0, double(rows) * cols * sizeof(T) * ((RES ? 3 : 2) + (sumOut ? 1 : 0)), st);
  if (al && cols % 16 == 0 && cols <= 256 * 16) {
    rmsNormKernel<T, 1, RES><<<grid, 256, 0, st>>>(A, B, W, Bi, S, O, cols, eps);
  } else if (al && cols % 16 == 0 && cols <= 256 * 16 * 2) {
    rmsNormKernel<T, 2, RES><<<grid, 256, 0, st>>>(A, B, W, Bi, S, O, cols, eps);
  } else {
    rmsNormGenericKernel<T, RES><<<grid, 256, 0, st>>>(A, B, W, Bi, S, O, cols, eps);
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// ---- reductions ------------------------------------------------------------------------
enum { rSum, rMean, rMax, rMin };

template <typename T> __device__ __forceinline__ T finishReduce(int op, float acc, size_t len) {
  if (op == rMean) acc = acc / static_cast<float>(len);
  return fromF32<T>(acc);
}

// inner == 1: warp per output element.
template <typename T>
__global__ void __launch_bounds__(256) reduceRowKernel(int op, const T *__restrict__ in, T *__restrict__ out,
                                                       size_t rows, size_t len) {
  size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T *x = in + row * len;
  float acc = op == rMax ? -INFINITY : (op == rMin ? INFINITY : 0.0f);
  for (size_t i = lane; i < len; i += 32) {
    float f = toF32(x[i]);
    acc = op == rMax ? fmaxf(acc, f) : (op == rMin ? fminf(acc, f) : acc + f);
  }
  acc = op == rMax ? warpMax(acc) : (op == rMin ? warpMin(acc) : warpSum(acc));
  if (lane == 0) out[row] = finishReduce<T>(op, acc, len);
}

template <typename T>
__global__ void __launch_bounds__(256) reduceColKernel(int op, const T *__restrict__ in, T *__restrict__ out,
                                                       size_t outer, size_t len, size_t inner) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < outer * inner; c += stride) {
    size_t base = (c / inner) * len * inner + (c % inner);
    float acc = op == rMax ? -INFINITY : (op == rMin ? INFINITY : 0.0f);
    for (size_t i = 0; i < len; ++i) {
      float f = toF32(in[base + i * inner]);
      acc = op == rMax ? fmaxf(acc, f) : (op == rMin ? fminf(acc, f) : acc + f);
    }
    out[c] = finishReduce<T>(op, acc, len);
  }
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_softmax(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (outer * len * inner == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("softmax", 0, double(outer) * len * inner * 2 * dtypeSize(dtype), st);
  TTB_DISPATCH_FLOAT(dtype, T, {
    if (inner == 1) {
      int grid = static_cast<int>((outer + 7) / 8);
      softmaxRowKernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), outer, len);
    } else {
      softmaxColKernel<T><<<gridFor(outer * inner, 256), 256, 0, st>>>(static_cast<const T *>(in),
                                                                       static_cast<T *>(out), outer, len, inner);
    }
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_rms_norm(const void *in, const void *weight, const void *bias, void *out, int dtype, size_t rows,
                 size_t cols, float eps, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (rows * cols == 0) return TTB_OK;
  TTB_DISPATCH_FLOAT(dtype, T, {
    return launchRms<T, false>(in, nullptr, weight, bias, nullptr, out, rows, cols, eps, asStream(stream));
  });
  return TTB_OK;
}

int ttb_add_rms_norm(const void *a, const void *b, const void *weight, void *sum_out, void *out, int dtype,
                     size_t rows, size_t cols, float eps, void *stream) {
  TTB_CHECK(a && b && out, "null tensor");
  if (rows * cols == 0) return TTB_OK;
  TTB_DISPATCH_FLOAT(dtype, T, {
    return launchRms<T, true>(a, b, weight, nullptr, sum_out, out, rows, cols, eps, asStream(stream));
  });
  return TTB_OK;
}

int ttb_reduce(int op, const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(op >= 0 && op <= 3, "unknown reduction op");
  if (outer * inner == 0) return TTB_OK;
  TTB_CHECK(len > 0, "reduction over an empty dimension");
  cudaStream_t st = asStream(stream);
  TTB_DISPATCH_DTYPE(dtype, T, {
    if (inner == 1) {
      int grid = static_cast<int>((outer + 7) / 8);
      reduceRowKernel<T><<<grid, 256, 0, st>>>(op, static_cast<const T *>(in), static_cast<T *>(out), outer, len);
    } else {
      reduceColKernel<T><<<gridFor(outer * inner, 256), 256, 0, st>>>(op, static_cast<const T *>(in),
                                                                      static_cast<T *>(out), outer, len, inner);
    }
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
