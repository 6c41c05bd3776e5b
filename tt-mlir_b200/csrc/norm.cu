// softmax, rms_norm (+ fused residual add) and reductions.  All are HBM-bound row kernels:
// 16-byte loads, f32 accumulation, warp-shuffle + shared-memory reductions.
//
// Reference semantics:
//  softmax  exp(x - max) * (1 / sum)   lib/Conversion/TTIRToLinalg/TTIRToLinalg.cpp:956-1017,
//           torch twin tools/tt-alchemist/templates/python/local/ttir_cpu.py:585
//  rms_norm x * rsqrt(mean(x^2) + eps) * w (+ b), computed in f32, rounded once
//           include/ttmlir/Dialect/TTIR/IR/TTIROps.td:2300-2336, golden tools/golden/mapping.py:1221-1290
//  reduce   sum / mean / max / min over a dimension, f32 accumulation  ttir_cpu.py:374-397
//  layer_norm (x - mean) * rsqrt(var + eps) * w + b over the trailing dimensions the weight
//           covers, biased variance, f32   ttir_cpu.py layer_norm (torch F.layer_norm);
//           call site runtime/lib/ttnn/operations/normalization/layer_norm.cpp
//  argmax   index of the first maximum (a NaN counts as the maximum), Int32   ttir_cpu.py argmax;
//           call site runtime/lib/ttnn/operations/reduction/argmax.cpp
//  cumsum   running sum along a dimension, f32 accumulation for floats, every prefix rounded
//           to the element type   ttir_cpu.py cumsum; call site operations/cumsum/cumsum.cpp
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
  pdlLaunchDependents();
  pdlWait();
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
  pdlLaunchDependents();
  pdlWait();
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
  pdlLaunchDependents();
  pdlWait();
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
    TTB_CUDA(launchPdl(rmsNormKernel<T, 1, RES>, dim3(grid), dim3(256), 0, st, A, B, W, Bi, S, O, cols, eps));
  } else if (al && cols % 16 == 0 && cols <= 256 * 16 * 2) {
    TTB_CUDA(launchPdl(rmsNormKernel<T, 2, RES>, dim3(grid), dim3(256), 0, st, A, B, W, Bi, S, O, cols, eps));
  } else {
    TTB_CUDA(launchPdl(rmsNormGenericKernel<T, RES>, dim3(grid), dim3(256), 0, st, A, B, W, Bi, S, O, cols, eps));
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// ---- layer_norm ------------------------------------------------------------------------
// One block per row, two passes over the row for the statistics (mean first, then the centred
// sum of squares: the numerically safe form) and one for the result; passes two and three hit
// L1 / L2.  The row's bytes cross HBM once in, once out.
template <typename T>
__global__ void __launch_bounds__(256)
    layerNormKernel(const T *__restrict__ in, const T *__restrict__ w, const T *__restrict__ bias, T *__restrict__ out,
                    size_t cols, float eps) {
  __shared__ float scratch[33];
  const T *x = in + static_cast<size_t>(blockIdx.x) * cols;
  T *y = out + static_cast<size_t>(blockIdx.x) * cols;
  float s = 0.0f;
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) s += toF32(x[i]);
  const float mean = blockSum(s, scratch) / static_cast<float>(cols);
  float ss = 0.0f;
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const float d = toF32(x[i]) - mean;
    ss += d * d;
  }
  const float rstd = rsqrtf(blockSum(ss, scratch) / static_cast<float>(cols) + eps);
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float f = (toF32(x[i]) - mean) * rstd;
    if (w) f *= toF32(w[i]);
    if (bias) f += toF32(bias[i]);
    y[i] = fromF32<T>(f);
  }
}

// ---- argmax ----------------------------------------------------------------------------
// `better(a, ia, b, ib)`: does candidate b replace a?  A NaN beats every number; among equals
// (and among NaNs) the smaller index stays.
__device__ __forceinline__ bool argBetter(float a, long long ia, float b, long long ib) {
  const bool an = a != a, bn = b != b;
  if (an || bn) return bn && (!an || ib < ia);
  return b > a || (b == a && ib < ia);
}

// inner == 1: one warp per row.
template <typename T>
__global__ void __launch_bounds__(256) argmaxRowKernel(const T *__restrict__ in, int32_t *__restrict__ out, size_t rows,
                                                       size_t len) {
  size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T *x = in + row * len;
  float best = -INFINITY;
  long long at = 0x7fffffffffffffffll;
  for (size_t i = lane; i < len; i += 32) {
    const float f = toF32(x[i]);
    if (at == 0x7fffffffffffffffll || argBetter(best, at, f, static_cast<long long>(i))) {
      best = f;
      at = static_cast<long long>(i);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const long long oa = __shfl_xor_sync(0xffffffffu, at, o);
    if (oa != 0x7fffffffffffffffll && (at == 0x7fffffffffffffffll || argBetter(best, at, ob, oa))) {
      best = ob;
      at = oa;
    }
  }
  if (lane == 0) out[row] = static_cast<int32_t>(at);
}

// inner > 1: one thread per (outer, inner) column.
template <typename T>
__global__ void __launch_bounds__(256) argmaxColKernel(const T *__restrict__ in, int32_t *__restrict__ out, size_t outer,
                                                       size_t len, size_t inner) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < outer * inner; c += stride) {
    size_t base = (c / inner) * len * inner + (c % inner);
    float best = toF32(in[base]);
    long long at = 0;
    for (size_t i = 1; i < len; ++i) {
      const float f = toF32(in[base + i * inner]);
      if (argBetter(best, at, f, static_cast<long long>(i))) {
        best = f;
        at = static_cast<long long>(i);
      }
    }
    out[c] = static_cast<int32_t>(at);
  }
}

// ---- cumsum ----------------------------------------------------------------------------
// One thread per (outer, inner) line, sequential along the scanned dimension (the order of a
// sequential sum, which is what the reference computes).  ACC: float for floats, int64 for ints.
template <typename T, typename ACC>
__global__ void __launch_bounds__(256) cumsumKernel(const T *__restrict__ in, T *__restrict__ out, size_t outer, size_t len,
                                                    size_t inner) {
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < outer * inner; c += stride) {
    size_t base = (c / inner) * len * inner + (c % inner);
    ACC acc = 0;
    for (size_t i = 0; i < len; ++i) {
      if constexpr (std::is_same<ACC, float>::value) {
        acc += toF32(in[base + i * inner]);
        out[base + i * inner] = fromF32<T>(acc);
      } else {
        acc += static_cast<ACC>(in[base + i * inner]);
        out[base + i * inner] = static_cast<T>(acc);
      }
    }
  }
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
      TTB_CUDA(launchPdl(softmaxRowKernel<T>, dim3(grid), dim3(256), 0, st, static_cast<const T *>(in), static_cast<T *>(out), outer, len));
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

int ttb_layer_norm(const void *in, const void *weight, const void *bias, void *out, int dtype, size_t rows, size_t cols,
                   float eps, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (rows * cols == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("layer_norm", 0, double(rows) * cols * 2 * dtypeSize(dtype), st);
  TTB_DISPATCH_FLOAT(dtype, T, {
    layerNormKernel<T><<<static_cast<unsigned>(rows), 256, 0, st>>>(static_cast<const T *>(in), static_cast<const T *>(weight),
                                                                    static_cast<const T *>(bias), static_cast<T *>(out),
                                                                    cols, eps);
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_argmax(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (outer * inner == 0) return TTB_OK;
  TTB_CHECK(len > 0 && len <= 0x7fffffffull, "argmax needs between 1 and 2^31-1 candidates");
  cudaStream_t st = asStream(stream);
  ProfScope prof("argmax", 0, double(outer) * len * inner * dtypeSize(dtype) + double(outer) * inner * 4, st);
  TTB_DISPATCH_DTYPE(dtype, T, {
    if (inner == 1) {
      int grid = static_cast<int>((outer + 7) / 8);
      argmaxRowKernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<int32_t *>(out), outer, len);
    } else {
      argmaxColKernel<T><<<gridFor(outer * inner, 256), 256, 0, st>>>(static_cast<const T *>(in),
                                                                      static_cast<int32_t *>(out), outer, len, inner);
    }
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_cumsum(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (outer * len * inner == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("cumsum", 0, double(outer) * len * inner * 2 * dtypeSize(dtype), st);
  const int grid = gridFor(outer * inner, 256);
  switch (dtype) {
  case kF32: cumsumKernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float *>(in), static_cast<float *>(out), outer, len, inner); break;
  case kBF16: cumsumKernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(in), static_cast<__nv_bfloat16 *>(out), outer, len, inner); break;
  case kF16: cumsumKernel<__half, float><<<grid, 256, 0, st>>>(static_cast<const __half *>(in), static_cast<__half *>(out), outer, len, inner); break;
  case kI32: cumsumKernel<int32_t, long long><<<grid, 256, 0, st>>>(static_cast<const int32_t *>(in), static_cast<int32_t *>(out), outer, len, inner); break;
  case kU32: cumsumKernel<uint32_t, long long><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(in), static_cast<uint32_t *>(out), outer, len, inner); break;
  default: setLastError("cumsum: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
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
