// Ops beyond the benchmark graphs that real model flatbuffers carry: cumprod, prod reduction, batch-norm inference
// and 2-D upsampling.  All are HBM- or latency-bound element work: coalesced accesses along the contiguous dimension,
// f32 arithmetic per element, one rounding to the element type per result.
//
// Reference call sites and goldens:
//   cumprod     operations/cumprod/cumprod.cpp (::ttnn::cumprod); tools/golden/mapping.py:4308-4314 (torch.cumprod)
//   prod        operations/reduction/prod.cpp (::ttnn::prod);     mapping.py:2858-2900 (torch.prod, dims one at a time)
//   batch norm  operations/normalization/batch_norm.cpp (::ttnn::batch_norm, training = false);
//               mapping.py:4948-4976 (torch.nn.functional.batch_norm over the channel dimension)
//   upsample    operations/pool/upsample.cpp (::ttnn::upsample, NHWC); mapping.py:3552-3578
//               (torch.nn.functional.interpolate, "nearest" or "bilinear" with align_corners = False)
#include "common.cuh"

#include <type_traits>

namespace ttb {

// One thread per (outer, inner) line, sequential along the scanned dimension.  The running product is kept one step
// wider than the elements, as torch's CPU scan keeps it (float for 16-bit types, double for f32), and every prefix is
// rounded to the element type; integers wrap like torch's (64-bit running product truncated to the element type).
template <typename T, typename ACC>
__global__ void __launch_bounds__(256) cumprodKernel(const T *__restrict__ in, T *__restrict__ out, size_t outer, size_t len,
                                                     size_t inner) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < outer * inner; c += stride) {
    const size_t base = (c / inner) * len * inner + (c % inner);
    ACC acc = 1;
    for (size_t i = 0; i < len; ++i) {
      if constexpr (std::is_same<ACC, float>::value) {
        acc = __fmul_rn(acc, toF32(in[base + i * inner]));
        out[base + i * inner] = fromF32<T>(acc);
      } else if constexpr (std::is_same<ACC, double>::value) {
        acc = __dmul_rn(acc, static_cast<double>(in[base + i * inner]));
        out[base + i * inner] = static_cast<T>(acc);
      } else {
        acc *= static_cast<ACC>(in[base + i * inner]);
        out[base + i * inner] = static_cast<T>(acc);
      }
    }
  }
}

// Product over the middle dimension of [outer, len, inner]: one warp per output when the reduced dimension is the
// contiguous one (lanes stride the row, partial products combined by shuffles), one thread per output otherwise.
template <typename T> __global__ void __launch_bounds__(256) prodRowKernel(const T *__restrict__ in, T *__restrict__ out, size_t rows, size_t len) {
  const size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T *x = in + row * len;
  float acc = 1.0f;
  for (size_t i = lane; i < len; i += 32) acc *= toF32(x[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc *= __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[row] = fromF32<T>(acc);
}
template <typename T> __global__ void __launch_bounds__(256) prodColKernel(const T *__restrict__ in, T *__restrict__ out, size_t outer, size_t len, size_t inner) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < outer * inner; c += stride) {
    const size_t base = (c / inner) * len * inner + (c % inner);
    float acc = 1.0f;
    for (size_t i = 0; i < len; ++i) acc *= toF32(in[base + i * inner]);
    out[c] = fromF32<T>(acc);
  }
}
__global__ void __launch_bounds__(256) prodIntKernel(const int32_t *__restrict__ in, int32_t *__restrict__ out, size_t outer, size_t len, size_t inner) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t c = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < outer * inner; c += stride) {
    const size_t base = (c / inner) * len * inner + (c % inner);
    long long acc = 1;
    for (size_t i = 0; i < len; ++i) acc *= static_cast<long long>(in[base + i * inner]); // wraps like torch's int64 product
    out[c] = static_cast<int32_t>(acc);
  }
}

// y = (x - mean[c]) * rsqrt-free scale + shift, written the way torch's inference batch norm evaluates it in f32:
//   invstd = 1 / sqrt(var[c] + eps);  y = (x - mean[c]) * invstd * weight[c] + bias[c]
// over [outer, channels, inner] (NCHW: inner = H * W).  The per-channel factors are recomputed per element: they are
// four cached loads and one reciprocal square root, and the kernel stays bound by x and y.
template <typename T>
__global__ void __launch_bounds__(256) batchNormInferenceKernel(const T *__restrict__ x, const T *__restrict__ mean, const T *__restrict__ var,
                                                                const T *__restrict__ weight, const T *__restrict__ bias, T *__restrict__ y,
                                                                size_t total, size_t channels, size_t inner, float eps) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t c = (i / inner) % channels;
    const float invstd = 1.0f / sqrtf(toF32(var[c]) + eps);
    float f = (toF32(x[i]) - toF32(mean[c])) * invstd;
    if (weight) f *= toF32(weight[c]);
    if (bias) f += toF32(bias[c]);
    y[i] = fromF32<T>(f);
  }
}

// NHWC upsampling by integer factors.  Nearest: out[n, y, x, :] = in[n, y / sy, x / sx, :].  Bilinear: the source
// coordinate of output pixel y is (y + 0.5) / sy - 0.5, clamped below at 0 (align_corners = False), blended from the
// two neighbouring rows and columns in f32.  One thread per 16-byte piece of a pixel's channels when the channel count
// allows, else per element.
template <typename T>
__global__ void __launch_bounds__(256) upsampleKernel(const T *__restrict__ in, T *__restrict__ out, size_t n, size_t h, size_t w, size_t c,
                                                      int sy, int sx, int bilinear) {
  const size_t ho = h * sy, wo = w * sx, total = n * ho * wo * c;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t ch = i % c, px = (i / c) % wo, py = (i / c / wo) % ho, img = i / c / wo / ho;
    const T *src = in + img * h * w * c;
    if (!bilinear) {
      out[i] = src[((py / sy) * w + px / sx) * c + ch];
      continue;
    }
    float fy = (static_cast<float>(py) + 0.5f) / static_cast<float>(sy) - 0.5f;
    float fx = (static_cast<float>(px) + 0.5f) / static_cast<float>(sx) - 0.5f;
    fy = fy < 0.0f ? 0.0f : fy;
    fx = fx < 0.0f ? 0.0f : fx;
    const size_t y0 = static_cast<size_t>(fy), x0 = static_cast<size_t>(fx);
    const size_t y1 = y0 + 1 < h ? y0 + 1 : h - 1, x1 = x0 + 1 < w ? x0 + 1 : w - 1;
    const float ly = fy - static_cast<float>(y0), lx = fx - static_cast<float>(x0);
    const float v00 = toF32(src[(y0 * w + x0) * c + ch]), v01 = toF32(src[(y0 * w + x1) * c + ch]);
    const float v10 = toF32(src[(y1 * w + x0) * c + ch]), v11 = toF32(src[(y1 * w + x1) * c + ch]);
    const float top = v00 * (1.0f - lx) + v01 * lx, bot = v10 * (1.0f - lx) + v11 * lx;
    out[i] = fromF32<T>(top * (1.0f - ly) + bot * ly);
  }
}

// group_norm on channels-last tensors [N, 1, H*W, C] (::ttnn::group_norm, operations/normalization/group_norm.cpp;
// golden tools/golden/mapping.py:1541-1574: torch group_norm on the NCHW view): a group is C / G consecutive channels,
// its statistics run over all pixels of one image.  One block per (image, group): mean, then the centred sum of
// squares (the numerically safe form), then the normalised values scaled and shifted per channel; passes two and
// three hit L1 / L2.
__device__ __forceinline__ float extraBlockSum(float v, float *scratch /* 33 floats */) {
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

template <typename T>
__global__ void __launch_bounds__(256) groupNormKernel(const T *__restrict__ x, const T *__restrict__ weight, const T *__restrict__ bias,
                                                       T *__restrict__ y, size_t pixels, size_t channels, size_t groups, float eps) {
  __shared__ float scratch[33];
  const size_t img = blockIdx.x / groups, g = blockIdx.x % groups, cg = channels / groups;
  const T *xi = x + img * pixels * channels + g * cg;
  T *yi = y + img * pixels * channels + g * cg;
  const size_t count = pixels * cg;
  float s = 0.0f;
  for (size_t i = threadIdx.x; i < count; i += blockDim.x) s += toF32(xi[(i / cg) * channels + i % cg]);
  const float mean = extraBlockSum(s, scratch) / static_cast<float>(count);
  float ss = 0.0f;
  for (size_t i = threadIdx.x; i < count; i += blockDim.x) {
    const float d = toF32(xi[(i / cg) * channels + i % cg]) - mean;
    ss += d * d;
  }
  const float rstd = rsqrtf(extraBlockSum(ss, scratch) / static_cast<float>(count) + eps);
  for (size_t i = threadIdx.x; i < count; i += blockDim.x) {
    const size_t c = i % cg, at = (i / cg) * channels + c;
    float f = (toF32(xi[at]) - mean) * rstd;
    if (weight) f *= toF32(weight[g * cg + c]);
    if (bias) f += toF32(bias[g * cg + c]);
    yi[at] = fromF32<T>(f);
  }
}

// Transposed convolution, NHWC, weights [C_in, C_out / groups, kH, kW] (::ttnn::conv_transpose2d,
// operations/conv/conv_transpose2d.cpp; golden tools/golden/mapping.py:804-893, torch conv_transpose2d).  One thread
// per output value gathers the input pixels that reach it: output (oy, ox) receives x[iy, ix] * w[ky, kx] where
// oy = iy * stride - pad + ky * dilation.  f32 accumulation over (ky, kx, c) in that order, one rounding.  A CUDA-core
// kernel: the op is rare in the graphs this runtime is measured on.
template <typename T>
__global__ void __launch_bounds__(256) convTranspose2dKernel(const T *__restrict__ x, const T *__restrict__ w, const T *__restrict__ bias,
                                                             T *__restrict__ y, int n, int h, int wd, int c, int o, int kh, int kw, int sh,
                                                             int sw, int pt, int pl, int dh, int dw, int groups, int ho, int wo) {
  const size_t total = static_cast<size_t>(n) * ho * wo * o, stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const int cg = c / groups, og = o / groups;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int oc = static_cast<int>(i % o), ox = static_cast<int>((i / o) % wo), oy = static_cast<int>((i / o / wo) % ho);
    const int img = static_cast<int>(i / o / wo / ho), g = oc / og, ocg = oc % og;
    float acc = 0.0f;
    for (int ky = 0; ky < kh; ++ky) {
      const int ty = oy + pt - ky * dh;
      if (ty < 0 || ty % sh != 0 || ty / sh >= h) continue;
      for (int kx = 0; kx < kw; ++kx) {
        const int tx = ox + pl - kx * dw;
        if (tx < 0 || tx % sw != 0 || tx / sw >= wd) continue;
        const T *xp = x + ((static_cast<size_t>(img) * h + ty / sh) * wd + tx / sw) * c + g * cg;
        for (int ic = 0; ic < cg; ++ic)
          acc += toF32(xp[ic]) * toF32(w[((static_cast<size_t>(g * cg + ic) * og + ocg) * kh + ky) * kw + kx]);
      }
    }
    if (bias) acc += toF32(bias[oc]);
    y[i] = fromF32<T>(acc);
  }
}


// Training-mode batch norm over the channel dimension of [N, C, inner] (::ttnn::batch_norm with training = true,
// operations/normalization/batch_norm.cpp; golden tools/golden/mapping.py:4979-5063): the batch mean and the biased
// batch variance of every channel normalise the input, and the running statistics move towards them in place:
// running = momentum * batch + (1 - momentum) * running.  One block per channel, three passes over its N * inner
// values (the second and third come from L2).
template <typename T>
__global__ void __launch_bounds__(256) batchNormTrainingKernel(const T *__restrict__ x, T *__restrict__ runMean, T *__restrict__ runVar,
                                                               const T *__restrict__ weight, const T *__restrict__ bias, T *__restrict__ y,
                                                               size_t outer, size_t channels, size_t inner, float eps, float momentum) {
  __shared__ float scratch[33];
  const size_t c = blockIdx.x, count = outer * inner;
  auto at = [&](size_t i) { return ((i / inner) * channels + c) * inner + i % inner; };
  float s = 0.0f;
  for (size_t i = threadIdx.x; i < count; i += blockDim.x) s += toF32(x[at(i)]);
  const float mean = extraBlockSum(s, scratch) / static_cast<float>(count);
  float ss = 0.0f;
  for (size_t i = threadIdx.x; i < count; i += blockDim.x) {
    const float d = toF32(x[at(i)]) - mean;
    ss += d * d;
  }
  const float var = extraBlockSum(ss, scratch) / static_cast<float>(count);
  const float sd = sqrtf(var + eps);
  const float w = weight ? toF32(weight[c]) : 1.0f, b = bias ? toF32(bias[c]) : 0.0f;
  for (size_t i = threadIdx.x; i < count; i += blockDim.x) {
    const size_t j = at(i);
    y[j] = fromF32<T>((toF32(x[j]) - mean) / sd * w + b);
  }
  if (threadIdx.x == 0) {
    runMean[c] = fromF32<T>(mean * momentum + toF32(runMean[c]) * (1.0f - momentum));
    runVar[c] = fromF32<T>(var * momentum + toF32(runVar[c]) * (1.0f - momentum));
  }
}

// max_pool2d that also returns where each maximum came from (::ttnn::max_pool2d with return_indices,
// operations/pool/pool2d.cpp; golden tools/golden/mapping.py:5339-5378, torch max_pool2d(return_indices = True)):
// the index is the position iy * W + ix inside the image's H x W plane, the first maximum wins, a NaN wins over
// everything.  NHWC, one thread per output value.
template <typename T, typename I>
__global__ void __launch_bounds__(256) maxPoolIndicesKernel(const T *__restrict__ in, T *__restrict__ out, I *__restrict__ idx, int n, int h,
                                                            int w, int c, int ho, int wo, int kh, int kw, int sh, int sw, int pt, int pl,
                                                            int dh, int dw) {
  const size_t total = static_cast<size_t>(n) * ho * wo * c;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int ch = static_cast<int>(i % c);
    size_t p = i / c;
    const int ox = static_cast<int>(p % wo);
    p /= wo;
    const int oy = static_cast<int>(p % ho);
    const int img = static_cast<int>(p / ho);
    float best = -INFINITY;
    int where = -1;
    for (int ky = 0; ky < kh; ++ky) {
      const int iy = oy * sh - pt + ky * dh;
      if (iy < 0 || iy >= h) continue;
      for (int kx = 0; kx < kw; ++kx) {
        const int ix = ox * sw - pl + kx * dw;
        if (ix < 0 || ix >= w) continue;
        const float f = toF32(in[((static_cast<size_t>(img) * h + iy) * w + ix) * c + ch]);
        if (where < 0 || f > best || (f != f && best == best)) {
          best = f;
          where = iy * w + ix;
        }
      }
    }
    out[i] = fromF32<T>(best);
    idx[i] = static_cast<I>(where < 0 ? 0 : where);
  }
}

// rotary_embedding_llama (::ttnn::experimental::rotary_embedding_llama, operations/transformer/
// rotary_embedding_llama.cpp): y = x * cos + (x @ T) * sin, where the 32 x 32 matrix T multiplies every 32-wide
// piece of the head dimension on its own (Llama passes the matrix that maps pairs (a, b) to (-b, a)).  One block per
// row; the row and T sit in shared memory; f32 throughout, one rounding.  `cosRows` says how rows of x map to rows
// of the caches: prefill caches are [seq, D] and x rows cycle through them; decode caches are [batch, D] (or one row
// per (batch, head)) and x rows [batch, heads] share their batch's row.
template <typename T>
__global__ void __launch_bounds__(256) rotaryLlamaKernel(const T *__restrict__ x, const T *__restrict__ cosT, const T *__restrict__ sinT,
                                                         const T *__restrict__ trans, T *__restrict__ y, size_t rows, int d, size_t cosMod,
                                                         size_t cosDiv) {
  __shared__ float tm[32][33];
  __shared__ float row[256];
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) tm[i >> 5][i & 31] = toF32(trans[i]);
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    __syncthreads();
    for (int j = threadIdx.x; j < d; j += blockDim.x) row[j] = toF32(x[r * d + j]);
    __syncthreads();
    const size_t cr = (r / cosDiv) % cosMod;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
      const int base = j & ~31, col = j & 31;
      float rot = 0.0f;
#pragma unroll 8
      for (int i = 0; i < 32; ++i) rot = fmaf(row[base + i], tm[i][col], rot);
      y[r * d + j] = fromF32<T>(row[j] * toF32(cosT[cr * d + j]) + rot * toF32(sinT[cr * d + j]));
    }
  }
}

// Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011): a counter-based generator, so
// element i's random bits depend only on (seed, i) and every launch geometry gives the same tensor.
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}

// dropout (::ttnn::experimental::dropout, operations/eltwise/unary/dropout.cpp; golden mapping.py:4365-4376,
// torch.dropout in training mode): every element is zeroed with probability `prob`, the others are multiplied by
// `scale`.  The stream is this generator's, not the Tensix one: which elements fall is a property of (seed, index).
template <typename T>
__global__ void __launch_bounds__(256) dropoutKernel(const T *__restrict__ x, T *__restrict__ y, size_t n, float prob, float scale, uint32_t seed,
                                                     uint32_t stream) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t q = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; q * 4 < n; q += stride) {
    const uint4 r = philox4x32(make_uint4(static_cast<uint32_t>(q), static_cast<uint32_t>(q >> 32), stream, 0), make_uint2(seed, 0x64726F70u));
    const uint32_t bits[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t i = q * 4 + j;
      if (i >= n) break;
      const float u = static_cast<float>(bits[j] >> 8) * (1.0f / 16777216.0f); // [0, 1)
      y[i] = u < prob ? fromF32<T>(0.0f) : fromF32<T>(toF32(x[i]) * scale);
    }
  }
}

// rand (::ttnn::rand, operations/rand/rand.cpp; golden mapping.py:4340-4362): uniform in [low, high).  As the golden
// draws its base values in bf16, 16-bit results take u = k / 2^m with m the type's significand width (8 for bf16, 11
// for f16), so that u * (high - low) + low stays below `high`; f32 takes 24 bits.
template <typename T>
__global__ void __launch_bounds__(256) randKernel(T *__restrict__ y, size_t n, float low, float high, uint32_t seed, uint32_t stream, int bitsUsed) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const float unit = 1.0f / static_cast<float>(1u << bitsUsed);
  for (size_t q = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; q * 4 < n; q += stride) {
    const uint4 r = philox4x32(make_uint4(static_cast<uint32_t>(q), static_cast<uint32_t>(q >> 32), stream, 0), make_uint2(seed, 0x72616E64u));
    const uint32_t bits[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t i = q * 4 + j;
      if (i >= n) break;
      const float u = static_cast<float>(bits[j] >> (32 - bitsUsed)) * unit;
      y[i] = fromF32<T>(u * (high - low) + low);
    }
  }
}


// conv3d on NDHWC activations (::ttnn::experimental::conv3d, operations/conv/conv3d.cpp; golden
// tools/golden/mapping.py:714-801, torch conv3d with symmetric padding, "zeros" or "replicate").  The weight is read
// through element strides over (o, c, kd, kh, kw), so both the framework layout [O, C/g, kD, kH, kW] and TTNN's
// prepared [kD*kH*kW*C/g, O] matrix are taken as they are.  One thread per output value, f32 accumulation, one
// rounding.  A CUDA-core kernel: the op is rare in the graphs this runtime is measured on.
struct Conv3dGeom {
  int n, d, h, w, c, o, kd, kh, kw, sd, sh, sw, pd, ph, pw, od, oh, ow, groups, replicate;
  long long wo, wc, wkd, wkh, wkw; // weight strides in elements
};

template <typename T>
__global__ void __launch_bounds__(256) conv3dKernel(const T *__restrict__ x, const T *__restrict__ wgt, const T *__restrict__ bias,
                                                    T *__restrict__ y, Conv3dGeom g) {
  const size_t total = static_cast<size_t>(g.n) * g.od * g.oh * g.ow * g.o;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const int cg = g.c / g.groups, og = g.o / g.groups;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int oc = static_cast<int>(i % g.o);
    size_t p = i / g.o;
    const int ox = static_cast<int>(p % g.ow);
    p /= g.ow;
    const int oy = static_cast<int>(p % g.oh);
    p /= g.oh;
    const int oz = static_cast<int>(p % g.od);
    const int img = static_cast<int>(p / g.od);
    const int c0 = (oc / og) * cg;
    float acc = bias ? toF32(bias[oc]) : 0.0f;
    for (int kz = 0; kz < g.kd; ++kz) {
      int iz = oz * g.sd - g.pd + kz;
      if (g.replicate) iz = min(max(iz, 0), g.d - 1);
      if (iz < 0 || iz >= g.d) continue;
      for (int ky = 0; ky < g.kh; ++ky) {
        int iy = oy * g.sh - g.ph + ky;
        if (g.replicate) iy = min(max(iy, 0), g.h - 1);
        if (iy < 0 || iy >= g.h) continue;
        for (int kx = 0; kx < g.kw; ++kx) {
          int ix = ox * g.sw - g.pw + kx;
          if (g.replicate) ix = min(max(ix, 0), g.w - 1);
          if (ix < 0 || ix >= g.w) continue;
          const T *xp = x + (((static_cast<size_t>(img) * g.d + iz) * g.h + iy) * g.w + ix) * g.c + c0;
          const T *wp = wgt + oc * g.wo + kz * g.wkd + ky * g.wkh + kx * g.wkw;
          for (int c = 0; c < cg; ++c) acc = fmaf(toF32(xp[c]), toF32(wp[c * g.wc]), acc);
        }
      }
    }
    y[i] = fromF32<T>(acc);
  }
}

// gelu_bw (::ttnn::experimental::gelu_bw, operations/eltwise/binary/experimental_binary_backward.cpp; golden
// mapping.py:4379-4383, aten.gelu_backward): grad * d/dx gelu(x), exact (erf) or the tanh approximation.
template <typename T>
__global__ void __launch_bounds__(256) geluBackwardKernel(const T *__restrict__ grad, const T *__restrict__ x, T *__restrict__ y, size_t n,
                                                          int tanhApprox) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = toF32(x[i]);
    float d;
    if (tanhApprox) {
      const float kBeta = 0.79788456080286535588f * 0.044715f, kAlpha = 0.79788456080286535588f; // sqrt(2 / pi)
      const float inner = kAlpha * v + kBeta * v * v * v;
      const float t = tanhf(inner);
      d = 0.5f * (1.0f + t) + 0.5f * v * (1.0f - t * t) * (kAlpha + 3.0f * kBeta * v * v);
    } else {
      const float cdf = 0.5f * (1.0f + erff(v * 0.70710678118654752440f));
      const float pdf = 0.39894228040143267794f * expf(-0.5f * v * v);
      d = cdf + v * pdf;
    }
    y[i] = fromF32<T>(toF32(grad[i]) * d);
  }
}

// embedding_bw (::ttnn::embedding_bw, operations/embedding/embedding_backward.cpp; golden mapping.py:5875-5912,
// index_add_ of the gradient rows into a zero table): rows are accumulated in f32 (atomics, so the order of equal
// indices is not fixed) and rounded to the result type once.
template <typename T, typename I>
__global__ void __launch_bounds__(256) embeddingBackwardAccumulate(const I *__restrict__ idx, const T *__restrict__ grad, float *__restrict__ acc,
                                                                   size_t rows, size_t dim, size_t vocab) {
  const size_t total = rows * dim, stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = static_cast<long long>(idx[i / dim]);
    if (r < 0 || static_cast<size_t>(r) >= vocab) continue;
    atomicAdd(acc + static_cast<size_t>(r) * dim + i % dim, toF32(grad[i]));
  }
}
template <typename T> __global__ void __launch_bounds__(256) roundFromF32Kernel(const float *__restrict__ in, T *__restrict__ out, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = fromF32<T>(in[i]);
}

// adamw (ttml::metal::adamw, operations/ttml/adamw.cpp; golden mapping.py:1155-1218, tt-train's CPUAdamW), in place:
//   m = b1 m + (1 - b1) g;  v = b2 v + (1 - b2) g^2;  [vmax = max(vmax, v)]
//   p = p - lr (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps) - lr wd p
// f32 arithmetic; the parameter is stored with round-to-nearest or, with stochastic rounding, by adding 16 random bits
// below a bf16's last place and truncating (Philox keyed by seed and element).
template <typename P, typename G, typename M>
__global__ void __launch_bounds__(256) adamwKernel(P *__restrict__ param, const G *__restrict__ grad, M *__restrict__ m, M *__restrict__ v,
                                                   M *__restrict__ vmax, size_t n, float lr, float b1, float b2, float b1pow, float b2pow,
                                                   float eps, float wd, int stochastic, uint32_t seed) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const float c1 = 1.0f - b1pow, c2 = 1.0f - b2pow;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float g = toF32(grad[i]), p = toF32(param[i]);
    const float mi = toF32(m[i]) * b1 + g * (1.0f - b1);
    const float vi = toF32(v[i]) * b2 + (g * g) * (1.0f - b2);
    m[i] = fromF32<M>(mi);
    v[i] = fromF32<M>(vi);
    float vv = vi;
    if (vmax) {
      vv = fmaxf(toF32(vmax[i]), vi);
      vmax[i] = fromF32<M>(vv);
    }
    const float denom = sqrtf(vv / c2) + eps;
    const float r = (p - (mi / c1) / denom * lr) - p * (lr * wd);
    if (stochastic && std::is_same<P, __nv_bfloat16>::value) {
      const uint4 rnd = philox4x32(make_uint4(static_cast<uint32_t>(i), static_cast<uint32_t>(i >> 32), 0, 0), make_uint2(seed, 0x6164616Du));
      const uint32_t bits = __float_as_uint(r) + (rnd.x & 0xffffu);
      param[i] = fromF32<P>(__uint_as_float(bits & 0xffff0000u));
    } else {
      param[i] = fromF32<P>(r);
    }
  }
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_cumprod(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (outer * len * inner == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("cumprod", 0, double(outer) * len * inner * 2 * dtypeSize(dtype), st);
  const int grid = gridFor(outer * inner, 256);
  switch (dtype) {
  case kF32: cumprodKernel<float, double><<<grid, 256, 0, st>>>(static_cast<const float *>(in), static_cast<float *>(out), outer, len, inner); break;
  case kBF16: cumprodKernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(in), static_cast<__nv_bfloat16 *>(out), outer, len, inner); break;
  case kF16: cumprodKernel<__half, float><<<grid, 256, 0, st>>>(static_cast<const __half *>(in), static_cast<__half *>(out), outer, len, inner); break;
  case kI32: cumprodKernel<int32_t, long long><<<grid, 256, 0, st>>>(static_cast<const int32_t *>(in), static_cast<int32_t *>(out), outer, len, inner); break;
  default: setLastError("cumprod: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_prod(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  if (outer * inner == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("prod", 0, double(outer) * len * inner * dtypeSize(dtype), st);
#define TTB_PROD(T)                                                                                                        \
  if (inner == 1) {                                                                                                        \
    prodRowKernel<T><<<static_cast<unsigned>((outer + 7) / 8), 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), outer, len); \
  } else {                                                                                                                 \
    prodColKernel<T><<<gridFor(outer * inner, 256), 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), outer, len, inner);    \
  }
  switch (dtype) {
  case kF32: TTB_PROD(float) break;
  case kBF16: TTB_PROD(__nv_bfloat16) break;
  case kF16: TTB_PROD(__half) break;
  case kI32:
    prodIntKernel<<<gridFor(outer * inner, 256), 256, 0, st>>>(static_cast<const int32_t *>(in), static_cast<int32_t *>(out), outer, len, inner);
    break;
  default: setLastError("prod: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_PROD
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_batch_norm_inference(const void *x, const void *mean, const void *var, const void *weight, const void *bias, void *y,
                             int dtype, size_t outer, size_t channels, size_t inner, float eps, void *stream) {
  TTB_CHECK(x && mean && var && y, "null tensor");
  const size_t total = outer * channels * inner;
  if (total == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("batch_norm", 0, double(total) * 2 * dtypeSize(dtype), st);
  const int grid = gridFor(total, 256);
#define TTB_BN(T)                                                                                                          \
  batchNormInferenceKernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(x), static_cast<const T *>(mean), static_cast<const T *>(var), \
                                                    static_cast<const T *>(weight), static_cast<const T *>(bias), static_cast<T *>(y), \
                                                    total, channels, inner, eps)
  switch (dtype) {
  case kF32: TTB_BN(float); break;
  case kBF16: TTB_BN(__nv_bfloat16); break;
  case kF16: TTB_BN(__half); break;
  default: setLastError("batch_norm: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_BN
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_upsample2d(const void *in, void *out, int dtype, size_t n, size_t h, size_t w, size_t c, int scale_h, int scale_w,
                   int bilinear, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(scale_h >= 1 && scale_w >= 1, "scale factors must be positive");
  const size_t total = n * h * scale_h * w * scale_w * c;
  if (total == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("upsample", 0, double(total + n * h * w * c) * dtypeSize(dtype), st);
  const int grid = gridFor(total, 256);
#define TTB_UP(T) upsampleKernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), n, h, w, c, scale_h, scale_w, bilinear)
  switch (dtype) {
  case kF32: TTB_UP(float); break;
  case kBF16: TTB_UP(__nv_bfloat16); break;
  case kF16: TTB_UP(__half); break;
  default: setLastError("upsample: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_UP
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_group_norm(const void *x, const void *weight, const void *bias, void *y, int dtype, size_t images, size_t pixels,
                   size_t channels, size_t groups, float eps, void *stream) {
  TTB_CHECK(x && y, "null tensor");
  TTB_CHECK(groups >= 1 && channels % groups == 0, "the channel count must divide by the number of groups");
  if (images * pixels * channels == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("group_norm", 0, double(images) * pixels * channels * 2 * dtypeSize(dtype), st);
  const unsigned grid = static_cast<unsigned>(images * groups);
#define TTB_GN(T)                                                                                                          \
  groupNormKernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(x), static_cast<const T *>(weight), static_cast<const T *>(bias), \
                                           static_cast<T *>(y), pixels, channels, groups, eps)
  switch (dtype) {
  case kF32: TTB_GN(float); break;
  case kBF16: TTB_GN(__nv_bfloat16); break;
  case kF16: TTB_GN(__half); break;
  default: setLastError("group_norm: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_GN
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_conv_transpose2d(const void *x, const void *weight, const void *bias, void *out, int dtype, int64_t n, int64_t h, int64_t w,
                         int64_t c, int64_t o, int kh, int kw, int stride_h, int stride_w, int pad_top, int pad_left, int out_pad_h,
                         int out_pad_w, int dil_h, int dil_w, int groups, void *stream) {
  TTB_CHECK(x && weight && out, "null tensor");
  TTB_CHECK(n > 0 && h > 0 && w > 0 && c > 0 && o > 0 && kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0 &&
                groups > 0 && c % groups == 0 && o % groups == 0 && pad_top >= 0 && pad_left >= 0 && out_pad_h >= 0 && out_pad_w >= 0,
            "bad convolution extents");
  const int64_t ho = (h - 1) * stride_h - 2 * pad_top + dil_h * (kh - 1) + out_pad_h + 1;
  const int64_t wo = (w - 1) * stride_w - 2 * pad_left + dil_w * (kw - 1) + out_pad_w + 1;
  TTB_CHECK(ho > 0 && wo > 0 && n * ho * wo * o < (1ll << 40) && h < (1 << 30) && w < (1 << 30) && ho < (1 << 30) && wo < (1 << 30),
            "bad output extents");
  cudaStream_t st = asStream(stream);
  ProfScope prof("conv_transpose2d", 2.0 * double(n) * h * w * c * (o / groups) * kh * kw,
                 (double(n) * h * w * c + double(n) * ho * wo * o) * dtypeSize(dtype), st);
  const int grid = gridFor(static_cast<size_t>(n * ho * wo * o), 256);
#define TTB_CT(T)                                                                                                          \
  convTranspose2dKernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(x), static_cast<const T *>(weight), static_cast<const T *>(bias), \
                                                 static_cast<T *>(out), static_cast<int>(n), static_cast<int>(h), static_cast<int>(w), \
                                                 static_cast<int>(c), static_cast<int>(o), kh, kw, stride_h, stride_w, pad_top, pad_left, \
                                                 dil_h, dil_w, groups, static_cast<int>(ho), static_cast<int>(wo))
  switch (dtype) {
  case kF32: TTB_CT(float); break;
  case kBF16: TTB_CT(__nv_bfloat16); break;
  case kF16: TTB_CT(__half); break;
  default: setLastError("conv_transpose2d: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_CT
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_batch_norm_training(const void *x, void *running_mean, void *running_var, const void *weight, const void *bias, void *y,
                            int dtype, size_t outer, size_t channels, size_t inner, float eps, float momentum, void *stream) {
  TTB_CHECK(x && running_mean && running_var && y, "null tensor");
  if (outer * channels * inner == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("batch_norm_training", 0, double(outer) * channels * inner * 2 * dtypeSize(dtype), st);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (batchNormTrainingKernel<T><<<static_cast<unsigned>(channels), 256, 0, st>>>(
                         static_cast<const T *>(x), static_cast<T *>(running_mean), static_cast<T *>(running_var),
                         static_cast<const T *>(weight), static_cast<const T *>(bias), static_cast<T *>(y), outer, channels, inner, eps,
                         momentum)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_max_pool2d_with_indices(const void *in, void *out, void *indices, int dtype, int index_dtype, int n, int h, int w, int c,
                                int ho, int wo, int kh, int kw, int sh, int sw, int pt, int pl, int dh, int dw, void *stream) {
  TTB_CHECK(in && out && indices, "null tensor");
  TTB_CHECK(kh > 0 && kw > 0 && sh > 0 && sw > 0 && dh > 0 && dw > 0 && pt >= 0 && pl >= 0, "bad pooling window");
  TTB_CHECK(index_dtype != kU16 || static_cast<long long>(h) * w <= 65536, "image too large for 16-bit indices");
  const size_t total = static_cast<size_t>(n) * ho * wo * c;
  if (total == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("max_pool2d_with_indices", 0, double(total) * (dtypeSize(dtype) + dtypeSize(index_dtype)) + double(n) * h * w * c * dtypeSize(dtype), st);
  const int grid = gridFor(total, 256);
#define TTB_POOL_IDX(I)                                                                                                     \
  TTB_DISPATCH_FLOAT(dtype, T,                                                                                              \
                     (maxPoolIndicesKernel<T, I><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out),   \
                                                                       static_cast<I *>(indices), n, h, w, c, ho, wo, kh, kw, sh, sw, pt, \
                                                                       pl, dh, dw)))
  switch (index_dtype) {
  case kI32: TTB_POOL_IDX(int32_t); break;
  case kU32: TTB_POOL_IDX(uint32_t); break;
  case kU16: TTB_POOL_IDX(uint16_t); break;
  default: setLastError("max_pool2d_with_indices: indices must be Int32, UInt32 or UInt16"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_POOL_IDX
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_rotary_embedding_llama(const void *x, const void *cos_cache, const void *sin_cache, const void *trans_mat, void *y, int dtype,
                               size_t rows, size_t head_dim, size_t cos_mod, size_t cos_div, void *stream) {
  TTB_CHECK(x && cos_cache && sin_cache && trans_mat && y, "null tensor");
  TTB_CHECK(head_dim > 0 && head_dim <= 256 && head_dim % 32 == 0, "head dimension must be a multiple of 32, at most 256");
  TTB_CHECK(cos_mod > 0 && cos_div > 0, "bad cache row mapping");
  if (rows == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("rotary_embedding_llama", 0, double(rows) * head_dim * 2 * dtypeSize(dtype), st);
  const int grid = static_cast<int>(rows < static_cast<size_t>(smCount()) * 8 ? rows : static_cast<size_t>(smCount()) * 8);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (rotaryLlamaKernel<T><<<grid, static_cast<unsigned>(head_dim < 64 ? 64 : head_dim), 0, st>>>(
                         static_cast<const T *>(x), static_cast<const T *>(cos_cache), static_cast<const T *>(sin_cache),
                         static_cast<const T *>(trans_mat), static_cast<T *>(y), rows, static_cast<int>(head_dim), cos_mod, cos_div)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_dropout(const void *x, void *y, int dtype, size_t n, float prob, float scale, uint32_t seed, uint32_t stream_id, void *stream) {
  TTB_CHECK(x && y, "null tensor");
  TTB_CHECK(prob >= 0.0f && prob <= 1.0f, "dropout probability outside [0, 1]");
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("dropout", 0, double(n) * 2 * dtypeSize(dtype), st);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (dropoutKernel<T><<<gridFor((n + 3) / 4, 256), 256, 0, st>>>(static_cast<const T *>(x), static_cast<T *>(y), n, prob, scale,
                                                                                 seed, stream_id)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_rand_uniform(void *y, int dtype, size_t n, float low, float high, uint32_t seed, uint32_t stream_id, void *stream) {
  TTB_CHECK(y, "null tensor");
  TTB_CHECK(low <= high, "rand: low above high");
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("rand", 0, double(n) * dtypeSize(dtype), st);
  const int bitsUsed = dtype == kF32 ? 24 : (dtype == kBF16 ? 8 : 11);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (randKernel<T><<<gridFor((n + 3) / 4, 256), 256, 0, st>>>(static_cast<T *>(y), n, low, high, seed, stream_id, bitsUsed)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_conv3d(const void *x, const void *weight, const void *bias, void *y, int dtype, int n, int d, int h, int w, int c, int o, int kd,
               int kh, int kw, int sd, int sh, int sw, int pd, int ph, int pw, int groups, int replicate, const int64_t *weight_strides5,
               void *stream) {
  TTB_CHECK(x && weight && y && weight_strides5, "null tensor");
  TTB_CHECK(kd > 0 && kh > 0 && kw > 0 && sd > 0 && sh > 0 && sw > 0 && pd >= 0 && ph >= 0 && pw >= 0, "bad convolution window");
  TTB_CHECK(groups > 0 && c % groups == 0 && o % groups == 0, "channels do not divide into the groups");
  Conv3dGeom g;
  g.n = n; g.d = d; g.h = h; g.w = w; g.c = c; g.o = o; g.kd = kd; g.kh = kh; g.kw = kw; g.sd = sd; g.sh = sh; g.sw = sw;
  g.pd = pd; g.ph = ph; g.pw = pw; g.groups = groups; g.replicate = replicate;
  g.od = (d + 2 * pd - kd) / sd + 1;
  g.oh = (h + 2 * ph - kh) / sh + 1;
  g.ow = (w + 2 * pw - kw) / sw + 1;
  TTB_CHECK(g.od > 0 && g.oh > 0 && g.ow > 0, "the kernel does not fit the padded input");
  g.wo = weight_strides5[0]; g.wc = weight_strides5[1]; g.wkd = weight_strides5[2]; g.wkh = weight_strides5[3]; g.wkw = weight_strides5[4];
  const size_t total = static_cast<size_t>(n) * g.od * g.oh * g.ow * o;
  if (total == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("conv3d", 2.0 * double(total) * kd * kh * kw * (c / groups), double(total) * dtypeSize(dtype), st);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (conv3dKernel<T><<<gridFor(total, 256), 256, 0, st>>>(static_cast<const T *>(x), static_cast<const T *>(weight),
                                                                          static_cast<const T *>(bias), static_cast<T *>(y), g)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_gelu_backward(const void *grad, const void *x, void *y, int dtype, size_t n, int tanh_approx, void *stream) {
  TTB_CHECK(grad && x && y, "null tensor");
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("gelu_backward", 0, double(n) * 3 * dtypeSize(dtype), st);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (geluBackwardKernel<T><<<gridFor(n, 256), 256, 0, st>>>(static_cast<const T *>(grad), static_cast<const T *>(x),
                                                                            static_cast<T *>(y), n, tanh_approx)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

size_t ttb_embedding_backward_workspace_bytes(size_t vocab, size_t dim) { return vocab * dim * sizeof(float); }

int ttb_embedding_backward(const void *indices, const void *grad, void *out, int index_dtype, int dtype, size_t rows, size_t vocab,
                           size_t dim, void *workspace, void *stream) {
  TTB_CHECK(indices && grad && out && workspace, "null tensor");
  if (vocab * dim == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("embedding_backward", 0, double(rows) * dim * dtypeSize(dtype) + double(vocab) * dim * (8 + dtypeSize(dtype)), st);
  float *acc = static_cast<float *>(workspace);
  TTB_CUDA(cudaMemsetAsync(acc, 0, vocab * dim * sizeof(float), st));
  if (rows != 0 && dim != 0) {
#define TTB_EMB_BW(I)                                                                                                        \
    TTB_DISPATCH_FLOAT(dtype, T,                                                                                             \
                       (embeddingBackwardAccumulate<T, I><<<gridFor(rows * dim, 256), 256, 0, st>>>(                         \
                           static_cast<const I *>(indices), static_cast<const T *>(grad), acc, rows, dim, vocab)))
    switch (index_dtype) {
    case kI32: TTB_EMB_BW(int32_t); break;
    case kU32: TTB_EMB_BW(uint32_t); break;
    case kU16: TTB_EMB_BW(uint16_t); break;
    default: setLastError("embedding_backward: indices must be Int32, UInt32 or UInt16"); return TTB_ERR_UNSUPPORTED;
    }
#undef TTB_EMB_BW
    countLaunch();
  }
  TTB_DISPATCH_FLOAT(dtype, T, (roundFromF32Kernel<T><<<gridFor(vocab * dim, 256), 256, 0, st>>>(acc, static_cast<T *>(out), vocab * dim)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_adamw(void *param, const void *grad, void *exp_avg, void *exp_avg_sq, void *max_exp_avg_sq, int param_dtype, int grad_dtype,
              int moment_dtype, size_t n, float lr, float beta1, float beta2, float beta1_pow, float beta2_pow, float eps,
              float weight_decay, int stochastic_rounding, uint32_t seed, void *stream) {
  TTB_CHECK(param && grad && exp_avg && exp_avg_sq, "null tensor");
  TTB_CHECK(beta1_pow != 1.0f && beta2_pow != 1.0f, "bias corrections of step 0 divide by zero");
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("adamw", 0, double(n) * (2 * dtypeSize(param_dtype) + dtypeSize(grad_dtype) + 4 * dtypeSize(moment_dtype)), st);
  const int grid = gridFor(n, 256);
#define TTB_ADAMW(P, G, M)                                                                                                   \
  adamwKernel<P, G, M><<<grid, 256, 0, st>>>(static_cast<P *>(param), static_cast<const G *>(grad), static_cast<M *>(exp_avg),        \
                                             static_cast<M *>(exp_avg_sq), static_cast<M *>(max_exp_avg_sq), n, lr, beta1, beta2,    \
                                             beta1_pow, beta2_pow, eps, weight_decay, stochastic_rounding, seed)
  if (param_dtype == kBF16 && grad_dtype == kBF16 && moment_dtype == kF32) TTB_ADAMW(__nv_bfloat16, __nv_bfloat16, float);
  else if (param_dtype == kBF16 && grad_dtype == kBF16 && moment_dtype == kBF16) TTB_ADAMW(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (param_dtype == kF32 && grad_dtype == kF32 && moment_dtype == kF32) TTB_ADAMW(float, float, float);
  else if (param_dtype == kF32 && grad_dtype == kBF16 && moment_dtype == kF32) TTB_ADAMW(float, __nv_bfloat16, float);
  else { setLastError("adamw: unsupported combination of parameter / gradient / moment types"); return TTB_ERR_UNSUPPORTED; }
#undef TTB_ADAMW
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
