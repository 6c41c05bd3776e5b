// 2-D pooling over NHWC activations (Pool2dOp: MaxPool2d / AvgPool2d).  HBM-bound: one thread per
// (output pixel, 16-byte channel vector), the window's taps are read through L1/L2, f32
// accumulation for the average, one rounding.
//
// Reference semantics: runtime/lib/ttnn/operations/pool/pool2d.cpp:20-139 (argument decoding: the
// 4-element padding is [top, left, bottom, right]) and the torch twin the CPU-hoist path runs,
// tools/tt-alchemist/templates/python/local/ttir_cpu.py (max_pool2d, avg_pool2d, _pool_padding):
//  * max: padding counts as -inf, a NaN in the window wins, ties keep the first tap;
//  * avg: the divisor is the window clipped to the padded extent (count_include_pad) or to the
//    input (otherwise); 4-element paddings are applied as real data first, so with them -- or with
//    a 2-element padding larger than half the kernel, which torch refuses and the reference
//    therefore also pads by hand -- `count_include_pad = false` only discounts padding when the
//    padding is asymmetric (the reference's sum / count formulation);
//  * output extent: floor or ceil of (in + pads - dilation * (k - 1) - 1) / stride + 1, and in
//    ceil mode the last window must start inside the input or its leading padding (torch's rule;
//    hand-applied padding counts as input for it).
#include "common.cuh"

#include <cfloat>

namespace ttb {

struct PoolGeom {
  int n, h, w, c, ho, wo, kh, kw, sh, sw, pt, pl, pb, pr, dh, dw;
  int includePad; // divisor = window clipped to the padded extent
};

template <typename T, int V, bool MAX>
__global__ void __launch_bounds__(256) pool2dKernel(const T *__restrict__ in, T *__restrict__ out, PoolGeom g) {
  const size_t cv = static_cast<size_t>(g.c / V);
  const size_t total = static_cast<size_t>(g.n) * g.ho * g.wo * cv;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c0 = static_cast<int>(i % cv) * V;
    size_t p = i / cv;
    const int ox = static_cast<int>(p % g.wo);
    p /= g.wo;
    const int oy = static_cast<int>(p % g.ho);
    const int img = static_cast<int>(p / g.ho);
    const int y0 = oy * g.sh - g.pt, x0 = ox * g.sw - g.pl;
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = MAX ? -INFINITY : 0.0f;
    int count = 0;
    for (int ky = 0; ky < g.kh; ++ky) {
      const int iy = y0 + ky * g.dh;
      if (iy < 0 || iy >= g.h) continue;
      for (int kx = 0; kx < g.kw; ++kx) {
        const int ix = x0 + kx * g.dw;
        if (ix < 0 || ix >= g.w) continue;
        const T *src = in + ((static_cast<size_t>(img) * g.h + iy) * g.w + ix) * g.c + c0;
        T v[V];
        if (V * sizeof(T) == 16) {
          *reinterpret_cast<uint4 *>(v) = __ldg(reinterpret_cast<const uint4 *>(src));
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) v[j] = src[j];
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float f = toF32(v[j]);
          if (MAX) {
            if (f > acc[j] || f != f) acc[j] = f; // strict: the first maximum stays; NaN wins
          } else {
            acc[j] += f;
          }
        }
        ++count;
      }
    }
    if (!MAX) {
      int div = count;
      if (g.includePad) {
        const int y1 = min(y0 + g.kh, g.h + g.pb), x1 = min(x0 + g.kw, g.w + g.pr);
        div = (y1 - y0) * (x1 - x0);
      }
      const float d = static_cast<float>(div > 0 ? div : 1);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = acc[j] / d;
    }
    T r[V];
#pragma unroll
    for (int j = 0; j < V; ++j) r[j] = fromF32<T>(acc[j]);
    T *dst = out + ((static_cast<size_t>(img) * g.ho + oy) * g.wo + ox) * g.c + c0;
    if (V * sizeof(T) == 16) {
      *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(r);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) dst[j] = r[j];
    }
  }
}

// torch's pooling_output_shape: `padLo` / `padHi` are what the pooling call itself is given (zero
// when the padding was applied by hand, in which case `in` already contains it).
static int poolOutExtent(int in, int k, int padLo, int padHi, int stride, int dil, bool ceilMode) {
  const int num = in + padLo + padHi - dil * (k - 1) - 1 + (ceilMode ? stride - 1 : 0);
  int out = (num >= 0 ? num / stride : -((-num + stride - 1) / stride)) + 1;
  if (ceilMode && (out - 1) * stride >= in + padLo) --out;
  return out;
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_pool2d_out_shape(int is_max, int h, int w, int kh, int kw, int sh, int sw, int pt, int pl, int pb, int pr,
                         int dh, int dw, int ceil_mode, int padding_has_four, int *ho, int *wo) {
  TTB_CHECK(ho && wo, "null result");
  TTB_CHECK(kh > 0 && kw > 0 && sh > 0 && sw > 0 && dh > 0 && dw > 0, "kernel, stride and dilation must be positive");
  TTB_CHECK(pt >= 0 && pl >= 0 && pb >= 0 && pr >= 0, "negative padding");
  // Which paddings the reference applies by hand before calling torch's pooling.
  bool byHand = padding_has_four != 0;
  if (!is_max) {
    const bool symmetric = pt == pb && pl == pr, exceeds = pt > kh / 2 || pl > kw / 2;
    byHand = !(symmetric && !exceeds);
  }
  if (byHand) {
    *ho = poolOutExtent(h + pt + pb, kh, 0, 0, sh, dh, ceil_mode != 0);
    *wo = poolOutExtent(w + pl + pr, kw, 0, 0, sw, dw, ceil_mode != 0);
  } else {
    *ho = poolOutExtent(h, kh, pt, pb, sh, dh, ceil_mode != 0);
    *wo = poolOutExtent(w, kw, pl, pr, sw, dw, ceil_mode != 0);
  }
  TTB_CHECK(*ho > 0 && *wo > 0, "pooling window does not fit the input");
  return TTB_OK;
}

int ttb_pool2d(const void *in, void *out, int dtype, int is_max, int n, int h, int w, int c, int kh, int kw, int sh,
               int sw, int pt, int pl, int pb, int pr, int dh, int dw, int ceil_mode, int count_include_pad,
               int padding_has_four, void *stream) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(n > 0 && h > 0 && w > 0 && c > 0, "empty activation");
  PoolGeom g;
  g.n = n; g.h = h; g.w = w; g.c = c;
  g.kh = kh; g.kw = kw; g.sh = sh; g.sw = sw;
  g.pt = pt; g.pl = pl; g.pb = pb; g.pr = pr;
  g.dh = is_max ? dh : 1; g.dw = is_max ? dw : 1;
  int rc = ttb_pool2d_out_shape(is_max, h, w, kh, kw, sh, sw, pt, pl, pb, pr, g.dh, g.dw, ceil_mode, padding_has_four,
                                &g.ho, &g.wo);
  if (rc) return rc;
  const bool symmetric = pt == pb && pl == pr, exceeds = pt > kh / 2 || pl > kw / 2;
  g.includePad = (count_include_pad || (symmetric && exceeds)) ? 1 : 0;
  cudaStream_t st = asStream(stream);
  const size_t outElems = static_cast<size_t>(n) * g.ho * g.wo * c, inElems = static_cast<size_t>(n) * h * w * c;
  ProfScope prof(is_max ? "max_pool2d" : "avg_pool2d", 0, double(outElems + inElems) * dtypeSize(dtype), st);
  TTB_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = 16 / static_cast<int>(sizeof(T));
    const bool vec = c % V == 0 && aligned16(in) && aligned16(out);
    const size_t items = outElems / (vec ? V : 1);
    const int grid = gridFor(items, 256);
    if (is_max) {
      if (vec) pool2dKernel<T, V, true><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), g);
      else pool2dKernel<T, 1, true><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), g);
    } else {
      if (vec) pool2dKernel<T, V, false><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), g);
      else pool2dKernel<T, 1, false><<<grid, 256, 0, st>>>(static_cast<const T *>(in), static_cast<T *>(out), g);
    }
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
