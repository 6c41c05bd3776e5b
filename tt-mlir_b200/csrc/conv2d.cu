// conv2d on NHWC activations as a GEMM: M = N*Ho*Wo output pixels, N = O output channels,
// K = kH*kW*C (reference semantics: include/ttmlir/Dialect/TTIR/IR/TTIROps.td:3959-4033; the
// CPU path lowers it to tosa.conv2d with f32 accumulation,
// lib/Conversion/TTIRToLinalg/TTIRToLinalg.cpp:576-787).
//
// 1x1 / stride 1 / no padding convolutions are already in GEMM layout (activations [P, C],
// weights [O, C]) and go straight to the contraction kernel.  Everything else gathers the
// receptive fields into a [P, K] operand (16-byte vectors along C, zero fill outside the
// image) and reorders the weights from [O, C, kH, kW] to [O, kH, kW, C] in a workspace.
#include "common.cuh"

#include <cstdlib>
#include <mutex>

namespace ttb {

// Implicit GEMM on the tensor-core kernel (gemm_tcgen05.cu); -1 = not taken.
int convTcgen05Try(const void *x, const void *wre, const void *bias, void *out, int dtype, int biasDtype, int64_t n,
                   int64_t h, int64_t w, int64_t c, int64_t o, int64_t ho, int64_t wo, int kh, int kw, int sh, int sw,
                   int pt, int pl, int dh, int dw, int act, const void *extra, int extraOp, cudaStream_t stream);

// Scratch for ttb_conv2d_static: lives in the library's device image, so every GPU that loads
// the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_convStaticScratch[TTB_CONV2D_STATIC_SCRATCH_BYTES];

struct ConvGeom {
  int64_t N, H, W, C, Ho, Wo;
  int kh, kw, sh, sw, pt, pl, dh, dw;
};

// One thread per V channels of one (pixel, ky, kx) tap.
template <typename T, int V>
__global__ void __launch_bounds__(256) im2colKernel(const T *__restrict__ x, T *__restrict__ col, ConvGeom g) {
  int64_t cv = g.C / V;
  int64_t K = static_cast<int64_t>(g.kh) * g.kw * g.C;
  int64_t total = g.N * g.Ho * g.Wo * g.kh * g.kw * cv;
  int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    int64_t c = (i % cv) * V;
    int64_t r = i / cv;
    int kx = static_cast<int>(r % g.kw);
    r /= g.kw;
    int ky = static_cast<int>(r % g.kh);
    int64_t p = r / g.kh;
    int64_t ox = p % g.Wo, oy = (p / g.Wo) % g.Ho, n = p / (g.Wo * g.Ho);
    int64_t iy = oy * g.sh + ky * g.dh - g.pt, ix = ox * g.sw + kx * g.dw - g.pl;
    T *dst = col + p * K + (static_cast<int64_t>(ky) * g.kw + kx) * g.C + c;
    bool inside = iy >= 0 && iy < g.H && ix >= 0 && ix < g.W;
    const T *src = x + ((n * g.H + iy) * g.W + ix) * g.C + c;
    if (V * sizeof(T) == 16) {
      uint4 v = inside ? __ldg(reinterpret_cast<const uint4 *>(src)) : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4 *>(dst) = v;
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) dst[j] = inside ? src[j] : T(0);
    }
  }
}

static int64_t outDim(int64_t in, int k, int s, int p0, int p1, int d) {
  return (in + p0 + p1 - static_cast<int64_t>(d) * (k - 1) - 1) / s + 1;
}

static bool isPointwise(int kh, int kw, int sh, int sw, const int *pad, int groups) {
  return kh == 1 && kw == 1 && sh == 1 && sw == 1 && pad[0] == 0 && pad[1] == 0 && pad[2] == 0 && pad[3] == 0 &&
         groups == 1;
}

static size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

static bool im2colForced() {
  static const bool forced = [] {
    const char *e = std::getenv("TTB_CONV_IM2COL");
    return e && e[0] == '1';
  }();
  return forced;
}

// Shapes the tensor-core kernel convolves without an im2col operand in memory (it gathers the
// receptive fields itself): 16-bit data, whole 64-channel blocks.  Decides the workspace size, so
// it depends on the shape only; operands are then required to be 16-byte aligned.
static bool implicitGemmShape(int dtype, int64_t c, int64_t o) {
  return !im2colForced() && (dtype == kBF16 || dtype == kF16) && c % 64 == 0 && o >= 8 && o % 8 == 0;
}

} // namespace ttb

using namespace ttb;

extern "C" {

size_t ttb_conv2d_workspace_bytes(int dtype, int64_t n, int64_t h, int64_t w, int64_t c, int64_t o, int kh, int kw,
                                  int stride_h, int stride_w, const int *padding4, int dil_h, int dil_w, int groups) {
  // Sizes that make no sense, or whose byte count does not fit size_t, come back as SIZE_MAX: no
  // allocation of that size succeeds and ttb_conv2d_static refuses it.
  if (n == 0) return 0;
  if (!padding4 || n < 0 || h <= 0 || w <= 0 || c <= 0 || o <= 0 || kh <= 0 || kw <= 0 || stride_h <= 0 || stride_w <= 0 ||
      dil_h <= 0 || dil_w <= 0 || padding4[0] < 0 || padding4[1] < 0 || padding4[2] < 0 || padding4[3] < 0)
    return SIZE_MAX;
  if (isPointwise(kh, kw, stride_h, stride_w, padding4, groups)) return 0;
  int64_t ho = outDim(h, kh, stride_h, padding4[0], padding4[2], dil_h);
  int64_t wo = outDim(w, kw, stride_w, padding4[1], padding4[3], dil_w);
  if (ho <= 0 || wo <= 0) return 0;
  size_t es = dtypeSize(dtype);
  if (es == 0) return SIZE_MAX;
  size_t K = 0, weights = 0, pixels = 0, col = 0;
  if (__builtin_mul_overflow(static_cast<size_t>(kh) * static_cast<size_t>(kw), static_cast<size_t>(c), &K) ||
      __builtin_mul_overflow(static_cast<size_t>(o), K, &weights) || __builtin_mul_overflow(weights, es, &weights) ||
      weights > SIZE_MAX - 512)
    return SIZE_MAX;
  weights = alignUp(weights, 256);
  if (implicitGemmShape(dtype, c, o)) return weights; // only the reordered weights
  if (__builtin_mul_overflow(static_cast<size_t>(n), static_cast<size_t>(ho), &pixels) ||
      __builtin_mul_overflow(pixels, static_cast<size_t>(wo), &pixels) || __builtin_mul_overflow(pixels, K, &col) ||
      __builtin_mul_overflow(col, es, &col) || col > SIZE_MAX - 512 - weights)
    return SIZE_MAX;
  return alignUp(col, 256) + weights;
}

int ttb_conv2d(const void *x, const void *weight, const void *bias, void *out, int dtype, int bias_dtype, int64_t n,
               int64_t h, int64_t w, int64_t c, int64_t o, int kh, int kw, int stride_h, int stride_w,
               const int *padding4, int dil_h, int dil_w, int groups, int act, void *workspace, void *stream) {
  return ttb_conv2d_fused(x, weight, bias, out, dtype, bias_dtype, n, h, w, c, o, kh, kw, stride_h, stride_w, padding4,
                          dil_h, dil_w, groups, act, nullptr, TTB_EXTRA_NONE, workspace, stream);
}

int ttb_conv2d_fused(const void *x, const void *weight, const void *bias, void *out, int dtype, int bias_dtype, int64_t n,
                     int64_t h, int64_t w, int64_t c, int64_t o, int kh, int kw, int stride_h, int stride_w,
                     const int *padding4, int dil_h, int dil_w, int groups, int act, const void *extra, int extra_op,
                     void *workspace, void *stream) {
  TTB_CHECK(x && weight && out && padding4, "null argument");
  TTB_CHECK(groups == 1, "grouped convolution is not supported");
  TTB_CHECK(kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0, "bad convolution geometry");
  if (n == 0) return TTB_OK; // an empty batch: nothing to compute
  TTB_CHECK(n > 0 && h > 0 && w > 0 && c > 0 && o > 0, "convolution extents must be positive");
  TTB_CHECK(padding4[0] >= 0 && padding4[1] >= 0 && padding4[2] >= 0 && padding4[3] >= 0, "negative padding");
  size_t es = dtypeSize(dtype);
  TTB_CHECK(dtype == kBF16 || dtype == kF32 || dtype == kF16, "conv2d needs a float dtype");
  if (isPointwise(kh, kw, stride_h, stride_w, padding4, groups)) {
    return ttb_gemm_fused(x, weight, bias, out, dtype, bias_dtype, dtype, 1, n * h * w, o, c, 0, 1, 0, 0, act, 0, extra, extra_op,
                          stream);
  }
  ConvGeom g;
  g.N = n; g.H = h; g.W = w; g.C = c;
  g.kh = kh; g.kw = kw; g.sh = stride_h; g.sw = stride_w; g.pt = padding4[0]; g.pl = padding4[1];
  g.dh = dil_h; g.dw = dil_w;
  g.Ho = outDim(h, kh, stride_h, padding4[0], padding4[2], dil_h);
  g.Wo = outDim(w, kw, stride_w, padding4[1], padding4[3], dil_w);
  TTB_CHECK(g.Ho > 0 && g.Wo > 0, "convolution output is empty");
  TTB_CHECK(workspace != nullptr, "conv2d needs its workspace");
  int64_t P = n * g.Ho * g.Wo, K = static_cast<int64_t>(kh) * kw * c;
  const bool implicit = implicitGemmShape(dtype, c, o);
  char *col = static_cast<char *>(workspace);
  char *wre = implicit ? col : col + alignUp(static_cast<size_t>(P) * K * es, 256);
  cudaStream_t st = asStream(stream);
  // weights [O, C, kH, kW] -> [O, kH, kW, C]
  {
    int64_t shape[4] = {o, kh, kw, c};
    int64_t strides[4] = {c * kh * kw, kw, 1, static_cast<int64_t>(kh) * kw};
    int rc = ttb_strided_copy(weight, wre, static_cast<int>(es), 4, shape, strides, 0, stream);
    if (rc) return rc;
  }
  // The tensor-core kernel gathers the receptive fields itself when the channel count allows.
  if (implicit) {
    int rc = convTcgen05Try(x, wre, bias, out, dtype, bias_dtype, n, h, w, c, o, g.Ho, g.Wo, kh, kw, stride_h, stride_w,
                            padding4[0], padding4[1], dil_h, dil_w, act, extra, extra_op, st);
    if (rc != -1) return rc;
    setLastError("conv2d: this shape runs without an im2col workspace, but the tensor-core path declined it (operand alignment or extents)");
    return TTB_ERR_INVALID;
  }
  int vec = static_cast<int>(16 / es);
  ProfScope prof("conv2d_im2col", 0, double(P) * K * es + double(n) * h * w * c * es, st);
  if (c % vec == 0 && aligned16(x) && aligned16(col)) {
    int64_t total = P * kh * kw * (c / vec);
    int grid = gridFor(static_cast<size_t>(total), 256);
    if (es == 2) im2colKernel<uint16_t, 8><<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(x), reinterpret_cast<uint16_t *>(col), g);
    else im2colKernel<uint32_t, 4><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(x), reinterpret_cast<uint32_t *>(col), g);
  } else {
    int64_t total = P * kh * kw * c;
    int grid = gridFor(static_cast<size_t>(total), 256);
    if (es == 2) im2colKernel<uint16_t, 1><<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(x), reinterpret_cast<uint16_t *>(col), g);
    else im2colKernel<uint32_t, 1><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(x), reinterpret_cast<uint32_t *>(col), g);
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return ttb_gemm_fused(col, wre, bias, out, dtype, bias_dtype, dtype, 1, P, o, K, 0, 1, 0, 0, act, 0, extra, extra_op, stream);
}

// Convolution on quantized operands (8-bit integers, exact 32-bit accumulation): the integer conv2d the
// compiler builds when input and weight are quantized (lib/Dialect/TTIR/IR/TTIROps.cpp:1492-1577), with the
// dequantize that follows it optionally fused (out_dtype a float type: result = float(acc) * scale, scale
// per output channel or one scalar).  Pointwise convolutions are the contraction itself; others gather the
// receptive fields into the workspace (ttb_conv2d_workspace_bytes with the input's dtype) first.
int ttb_conv2d_i8(const void *x, const void *weight, void *out, int x_dtype, int w_dtype, int out_dtype, int64_t n, int64_t h,
                  int64_t w, int64_t c, int64_t o, int kh, int kw, int stride_h, int stride_w, const int *padding4, int dil_h,
                  int dil_w, int groups, const float *deq_scale, float deq_scalar, void *workspace, void *stream) {
  TTB_CHECK(x && weight && out && padding4, "null argument");
  TTB_CHECK(groups == 1, "grouped convolution is not supported");
  TTB_CHECK((x_dtype == kI8 || x_dtype == kU8) && (w_dtype == kI8 || w_dtype == kU8), "conv2d_i8 takes Int8 / UInt8 operands");
  TTB_CHECK(kh > 0 && kw > 0 && stride_h > 0 && stride_w > 0 && dil_h > 0 && dil_w > 0, "bad convolution geometry");
  if (n == 0) return TTB_OK;
  TTB_CHECK(n > 0 && h > 0 && w > 0 && c > 0 && o > 0, "convolution extents must be positive");
  TTB_CHECK(padding4[0] >= 0 && padding4[1] >= 0 && padding4[2] >= 0 && padding4[3] >= 0, "negative padding");
  if (isPointwise(kh, kw, stride_h, stride_w, padding4, groups)) {
    return ttb_gemm_i8(x, weight, out, x_dtype, w_dtype, out_dtype, 1, n * h * w, o, c, 0, 1, 0, 0, deq_scale, deq_scalar, stream);
  }
  ConvGeom g;
  g.N = n; g.H = h; g.W = w; g.C = c;
  g.kh = kh; g.kw = kw; g.sh = stride_h; g.sw = stride_w; g.pt = padding4[0]; g.pl = padding4[1];
  g.dh = dil_h; g.dw = dil_w;
  g.Ho = outDim(h, kh, stride_h, padding4[0], padding4[2], dil_h);
  g.Wo = outDim(w, kw, stride_w, padding4[1], padding4[3], dil_w);
  TTB_CHECK(g.Ho > 0 && g.Wo > 0, "convolution output is empty");
  TTB_CHECK(workspace != nullptr, "conv2d needs its workspace");
  const int64_t P = n * g.Ho * g.Wo, K = static_cast<int64_t>(kh) * kw * c;
  char *col = static_cast<char *>(workspace);
  char *wre = col + alignUp(static_cast<size_t>(P) * K, 256);
  cudaStream_t st = asStream(stream);
  {
    int64_t shape[4] = {o, kh, kw, c};
    int64_t strides[4] = {c * kh * kw, kw, 1, static_cast<int64_t>(kh) * kw};
    int rc = ttb_strided_copy(weight, wre, 1, 4, shape, strides, 0, stream);
    if (rc) return rc;
  }
  {
    ProfScope prof("conv2d_im2col", 0, double(P) * K + double(n) * h * w * c, st);
    if (c % 16 == 0 && aligned16(x) && aligned16(col)) {
      int grid = gridFor(static_cast<size_t>(P * kh * kw * (c / 16)), 256);
      im2colKernel<uint8_t, 16><<<grid, 256, 0, st>>>(static_cast<const uint8_t *>(x), reinterpret_cast<uint8_t *>(col), g);
    } else {
      int grid = gridFor(static_cast<size_t>(P * kh * kw * c), 256);
      im2colKernel<uint8_t, 1><<<grid, 256, 0, st>>>(static_cast<const uint8_t *>(x), reinterpret_cast<uint8_t *>(col), g);
    }
    countLaunch();
    TTB_LAUNCH_CHECK();
  }
  return ttb_gemm_i8(col, wre, out, x_dtype, w_dtype, out_dtype, 1, P, o, K, 0, 1, 0, 0, deq_scale, deq_scalar, stream);
}

int ttb_conv2d_static(const void *x, const void *weight, const void *bias, void *out, int dtype, int bias_dtype,
                      int64_t n, int64_t h, int64_t w, int64_t c, int64_t o, int kh, int kw, int stride_h, int stride_w,
                      const int *padding4, int dil_h, int dil_w, int groups, int act, void *stream) {
  TTB_CHECK(padding4 != nullptr, "null argument");
  // The built-in buffer is split in two: the convolution's workspace in front, and a fixed tail for the
  // partial sums of the CUDA-core contraction's split-K mode (what it would otherwise allocate).
  constexpr size_t kGemmTail = TTB_CONV2D_STATIC_GEMM_BYTES;
  constexpr size_t kConvPart = TTB_CONV2D_STATIC_SCRATCH_BYTES - kGemmTail;
  size_t need = ttb_conv2d_workspace_bytes(dtype, n, h, w, c, o, kh, kw, stride_h, stride_w, padding4, dil_h, dil_w, groups);
  if (need > kConvPart) {
    setLastError(need == SIZE_MAX
                     ? std::string("conv2d_static: bad convolution extents")
                     : "conv2d_static: this convolution needs " + std::to_string(need) + " bytes of scratch, the built-in buffer has " +
                           std::to_string(kConvPart) + "; use ttb_conv2d with a caller-provided workspace");
    return TTB_ERR_INVALID;
  }
  // The array's name is only a host-side handle; the kernels need its device address, which
  // differs per GPU.  It is looked up once per device, with that device current, and kept for the
  // life of the process (the library does not outlive a cudaDeviceReset of a device it ran on).
  static std::mutex mu;
  static void *scratchOf[64] = {};
  int dev = -1;
  TTB_CUDA(cudaGetDevice(&dev));
  TTB_CHECK(dev >= 0 && dev < 64, "device ordinal out of range");
  void *scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!scratchOf[dev]) {
      void *p = nullptr;
      TTB_CUDA(cudaGetSymbolAddress(&p, g_convStaticScratch));
      TTB_CHECK(p != nullptr, "scratch symbol has no device address");
      scratchOf[dev] = p;
    }
    scratch = scratchOf[dev];
  }
  // Every contraction below this call takes its split-K scratch from the tail (or runs unsplit).
  GemmScratchScope noAlloc(static_cast<char *>(scratch) + kConvPart, kGemmTail);
  return ttb_conv2d(x, weight, bias, out, dtype, bias_dtype, n, h, w, c, o, kh, kw, stride_h, stride_w, padding4, dil_h,
                    dil_w, groups, act, need ? scratch : nullptr, stream);
}

} // extern "C"
