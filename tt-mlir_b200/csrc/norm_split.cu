// Normalisations whose statistics and whose application are separate steps, as tensor-parallel graphs with the
// hidden dimension split over the mesh use them: every device reduces its slice of each row, the per-row statistics
// cross the mesh (a few bytes per row), and every device normalises its own slice with the combined statistics.
//
//   rms_norm_pre_all_gather    operations/normalization/rms_norm_pre_all_gather.cpp; golden tools/golden/mapping.py:7800-7826
//   layer_norm_pre_all_gather  operations/normalization/layer_norm_pre_all_gather.cpp; mapping.py:7852-7888
//   layer_norm_post_all_gather operations/normalization/layer_norm_post_all_gather.cpp; mapping.py:7891-7921
//   distributed_rms_norm       operations/normalization/distributed_rms_norm.cpp (::ttnn::fused_rms_minimal);
//                              mapping.py:1329-1415 (RMS norm of the concatenated shards, chunked back)
//   dit_rms_norm_unary_fused   operations/normalization/dit_rms_norm_unary_fused.cpp; mapping.py:1291-1326
//
// The statistics tensors keep the reference's tile layout, because graphs slice and gather them by it: 32 columns per
// statistic with the value in column 0 and zeros behind it.  rms pre: [rows, 32] holding E(x^2) of the local slice;
// layer-norm pre: [rows, 64] holding sum(x^2) in column 0 and sum(x) in column 32; after the all-gather along the last
// dimension the post op sees one such block per device.
//
// All kernels: one block per row, f32 arithmetic, one rounding per stored value; the row is read twice by the apply
// kernels (the second read comes from L1 / L2).  HBM-bound: 2 (pre) or 2-3 (apply) bytes-per-element passes.
#include "common.cuh"

namespace ttb {

__device__ __forceinline__ float splitBlockSum(float v, float *scratch /* 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  const float r = scratch[32];
  __syncthreads();
  return r;
}

enum SplitAct { aNone, aRelu, aRelu6, aSilu, aMish, aSigmoid, aHardsigmoid, aTanh, aLog, aSoftplus, aGelu, aSqrt, aCount };

__device__ __forceinline__ float splitAct(int act, float x) {
  switch (act) {
  case aRelu: return x > 0.0f ? x : (x != x ? x : 0.0f);
  case aRelu6: return fminf(fmaxf(x, 0.0f), 6.0f);
  case aSilu: return x / (1.0f + expf(-x));
  case aMish: return x * tanhf(log1pf(expf(x)));
  case aSigmoid: return 1.0f / (1.0f + expf(-x));
  case aHardsigmoid: return fminf(fmaxf(x * (1.0f / 6.0f) + 0.5f, 0.0f), 1.0f);
  case aTanh: return tanhf(x);
  case aLog: return logf(x);
  case aSoftplus: return x > 20.0f ? x : log1pf(expf(x)); // torch's threshold
  case aGelu: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
  case aSqrt: return sqrtf(x);
  default: return x;
  }
}

// mode 0: out[row, 0] = mean(x^2) over the local columns, 31 zeros behind it      (S, 32 columns)
// mode 1: out[row, 0] = sum(x^2), out[row, 32] = sum(x), zeros elsewhere          (S, 64 columns)
// mode 2: out[row] = sum(x^2)                                                     (S = float, 1 column)
template <typename T, typename S>
__global__ void __launch_bounds__(256) rowStatsKernel(const T *__restrict__ x, const T *__restrict__ res, S *__restrict__ out, size_t cols,
                                                      int mode) {
  __shared__ float scratch[33];
  const size_t row = blockIdx.x;
  const T *xr = x + row * cols;
  const T *rr = res ? res + row * cols : nullptr;
  float s = 0.0f, ss = 0.0f;
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = toF32(xr[i]);
    if (rr) v += toF32(rr[i]);
    s += v;
    ss += v * v;
  }
  ss = splitBlockSum(ss, scratch);
  if (mode == 1) s = splitBlockSum(s, scratch);
  if (mode == 2) {
    if (threadIdx.x == 0) out[row] = fromF32<S>(ss);
    return;
  }
  const int width = mode == 0 ? 32 : 64;
  if (threadIdx.x < width) {
    float v = 0.0f;
    if (threadIdx.x == 0) v = mode == 0 ? ss / static_cast<float>(cols) : ss;
    if (mode == 1 && threadIdx.x == 32) v = s;
    out[row * width + threadIdx.x] = fromF32<S>(v);
  }
}

// y = act(((x + res) * rsqrt(sumsq / n + eps)) * weight + bias).  `totals` (nullable) holds the row's sum of squares
// over ALL `totalCols` columns of the distributed row; without it the block computes its own over `cols`.
template <typename T>
__global__ void __launch_bounds__(256) rmsApplyKernel(const T *__restrict__ x, const T *__restrict__ res, const T *__restrict__ weight,
                                                      const T *__restrict__ bias, const float *__restrict__ totals, T *__restrict__ y,
                                                      size_t cols, size_t totalCols, float eps, int act) {
  __shared__ float scratch[33];
  const size_t row = blockIdx.x;
  const T *xr = x + row * cols;
  const T *rr = res ? res + row * cols : nullptr;
  float ss;
  if (totals) {
    ss = totals[row];
  } else {
    float p = 0.0f;
    for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
      float v = toF32(xr[i]);
      if (rr) v += toF32(rr[i]);
      p += v * v;
    }
    ss = splitBlockSum(p, scratch);
  }
  const float scale = rsqrtf(ss / static_cast<float>(totalCols) + eps);
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = toF32(xr[i]);
    if (rr) v += toF32(rr[i]);
    v *= scale;
    if (weight) v *= toF32(weight[i]);
    if (bias) v += toF32(bias[i]);
    y[row * cols + i] = fromF32<T>(splitAct(act, v));
  }
}

// stats: [rows, 64 * blocks] as the all-gather of layer-norm pre statistics leaves them.
template <typename T, typename S>
__global__ void __launch_bounds__(256) layerNormPostKernel(const T *__restrict__ x, const S *__restrict__ stats, const T *__restrict__ weight,
                                                           const T *__restrict__ bias, T *__restrict__ y, size_t cols, size_t blocks,
                                                           float eps) {
  const size_t row = blockIdx.x;
  float sumsq = 0.0f, sum = 0.0f;
  for (size_t k = 0; k < blocks; ++k) {
    sumsq += toF32(stats[(row * blocks + k) * 64]);
    sum += toF32(stats[(row * blocks + k) * 64 + 32]);
  }
  const float n = static_cast<float>(cols * blocks);
  const float mean = sum / n;
  const float var = fmaxf(sumsq / n - mean * mean, 0.0f);
  const float rstd = rsqrtf(var + eps);
  for (size_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = (toF32(x[row * cols + i]) - mean) * rstd;
    if (weight) v *= toF32(weight[i]);
    if (bias) v += toF32(bias[i]);
    y[row * cols + i] = fromF32<T>(v);
  }
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_norm_row_stats(const void *x, const void *residual, void *stats, int dtype, int stats_dtype, size_t rows, size_t cols, int mode,
                       void *stream) {
  TTB_CHECK(x && stats, "null tensor");
  TTB_CHECK(mode >= 0 && mode <= 2, "unknown statistics layout");
  TTB_CHECK(mode != 2 || stats_dtype == kF32, "raw sums of squares are f32");
  if (rows == 0 || cols == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("norm_row_stats", 0, double(rows) * cols * dtypeSize(dtype) * (residual ? 2 : 1), st);
#define TTB_STATS(S)                                                                                                        \
  TTB_DISPATCH_FLOAT(dtype, T,                                                                                              \
                     (rowStatsKernel<T, S><<<static_cast<unsigned>(rows), 256, 0, st>>>(                                    \
                         static_cast<const T *>(x), static_cast<const T *>(residual), static_cast<S *>(stats), cols, mode)))
  switch (stats_dtype) {
  case kF32: TTB_STATS(float); break;
  case kBF16: TTB_STATS(__nv_bfloat16); break;
  case kF16: TTB_STATS(__half); break;
  default: setLastError("norm statistics must be a floating-point tensor"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_STATS
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_rms_norm_apply(const void *x, const void *residual, const void *weight, const void *bias, const float *row_sumsq, void *y,
                       int dtype, size_t rows, size_t cols, size_t total_cols, float eps, int act, void *stream) {
  TTB_CHECK(x && y, "null tensor");
  TTB_CHECK(act >= 0 && act < aCount, "unknown activation");
  TTB_CHECK(total_cols >= cols && (row_sumsq || total_cols == cols), "row length of the whole distributed row is missing");
  if (rows == 0 || cols == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("rms_norm_apply", 0, double(rows) * cols * dtypeSize(dtype) * (residual ? 3 : 2), st);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (rmsApplyKernel<T><<<static_cast<unsigned>(rows), 256, 0, st>>>(
                         static_cast<const T *>(x), static_cast<const T *>(residual), static_cast<const T *>(weight),
                         static_cast<const T *>(bias), row_sumsq, static_cast<T *>(y), cols, total_cols, eps, act)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_layer_norm_post_all_gather(const void *x, const void *stats, const void *weight, const void *bias, void *y, int dtype,
                                   int stats_dtype, size_t rows, size_t cols, size_t blocks, float eps, void *stream) {
  TTB_CHECK(x && stats && y, "null tensor");
  TTB_CHECK(blocks >= 1, "statistics of at least one device are needed");
  if (rows == 0 || cols == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("layer_norm_post_all_gather", 0, double(rows) * cols * dtypeSize(dtype) * 2, st);
#define TTB_POST(S)                                                                                                         \
  TTB_DISPATCH_FLOAT(dtype, T,                                                                                              \
                     (layerNormPostKernel<T, S><<<static_cast<unsigned>(rows), 256, 0, st>>>(                               \
                         static_cast<const T *>(x), static_cast<const S *>(stats), static_cast<const T *>(weight),          \
                         static_cast<const T *>(bias), static_cast<T *>(y), cols, blocks, eps)))
  switch (stats_dtype) {
  case kF32: TTB_POST(float); break;
  case kBF16: TTB_POST(__nv_bfloat16); break;
  case kF16: TTB_POST(__half); break;
  default: setLastError("norm statistics must be a floating-point tensor"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_POST
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
