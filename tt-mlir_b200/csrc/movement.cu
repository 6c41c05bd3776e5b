// Data-movement kernels: one strided gather (permute / transpose / slice / repeat / head
// split), one strided scatter (concat pieces, head merge) and rotary embedding.
//
// The launchers coalesce what they can on the host: when the innermost dimension is
// contiguous on both sides and everything is 16-byte aligned, the copy runs in 16-byte units,
// so a permute such as [1,S,H,D] -> [1,H,S,D] moves D*2 bytes per (s,h) with full-width
// accesses.  Reference call sites: runtime/lib/ttnn/operations/data_movement/*.cpp.
#include "common.cuh"

#include <cstring>

namespace ttb {

struct CopyDims {
  int rank;
  int64_t shape[8];
  int64_t stride[8];
};

template <typename U, bool SCATTER>
__global__ void __launch_bounds__(256)
    stridedCopyKernel(const U *__restrict__ in, U *__restrict__ out, size_t n, CopyDims d, int64_t offset) {
  size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) {
    size_t r = i;
    int64_t at = offset;
    for (int k = d.rank - 1; k >= 0; --k) {
      size_t c = r % d.shape[k];
      r /= d.shape[k];
      at += static_cast<int64_t>(c) * d.stride[k];
    }
    if (SCATTER) out[at] = in[i];
    else out[i] = in[at];
  }
}

// Shared host logic: merge dimensions, pick the widest unit, launch.
template <bool SCATTER>
static int launchStrided(const void *in, void *out, int elemSize, int rank, const int64_t *shape,
                         const int64_t *strides, int64_t offset, cudaStream_t st) {
  TTB_CHECK(in && out, "null tensor");
  TTB_CHECK(rank >= 0 && rank <= 8, "rank must be <= 8");
  TTB_CHECK(elemSize == 1 || elemSize == 2 || elemSize == 4 || elemSize == 8, "element size must be 1, 2, 4 or 8");
  // drop size-1 dims, merge neighbours that are contiguous with respect to each other
  int64_t sh[8], sd[8];
  int r = 0;
  size_t n = 1;
  for (int i = 0; i < rank; ++i) {
    TTB_CHECK(shape[i] >= 0, "negative dimension");
    n *= static_cast<size_t>(shape[i]);
    if (shape[i] == 1) continue;
    if (r > 0 && sd[r - 1] == strides[i] * shape[i]) {
      sh[r - 1] *= shape[i];
      sd[r - 1] = strides[i];
    } else {
      sh[r] = shape[i];
      sd[r] = strides[i];
      ++r;
    }
  }
  if (n == 0) return TTB_OK;
  if (r == 0) {
    sh[0] = 1;
    sd[0] = 1;
    r = 1;
  }
  // widen the unit while the innermost run, all other strides, the offset and both bases allow it
  int unit = elemSize;
  const char *src = static_cast<const char *>(in);
  char *dst = static_cast<char *>(out);
  if (sd[r - 1] == 1) {
    while (unit < 16) {
      int f = 2;
      bool ok = sh[r - 1] % f == 0 && offset % f == 0;
      for (int i = 0; i < r - 1 && ok; ++i) ok = sd[i] % f == 0;
      ok = ok && (reinterpret_cast<uintptr_t>(src) % (unit * f) == 0) &&
           (reinterpret_cast<uintptr_t>(dst) % (unit * f) == 0);
      if (!ok) break;
      sh[r - 1] /= f;
      for (int i = 0; i < r - 1; ++i) sd[i] /= f;
      offset /= f;
      unit *= f;
      n /= f;
    }
  }
  CopyDims d;
  d.rank = r;
  for (int i = 0; i < r; ++i) {
    d.shape[i] = sh[i];
    d.stride[i] = sd[i];
  }
  int grid = gridFor(n, 256);
  ProfScope prof(SCATTER ? "strided_scatter" : "strided_copy", 0, 2.0 * double(n) * unit, st);
  switch (unit) {
  case 1: stridedCopyKernel<uint8_t, SCATTER><<<grid, 256, 0, st>>>(static_cast<const uint8_t *>(in), static_cast<uint8_t *>(out), n, d, offset); break;
  case 2: stridedCopyKernel<uint16_t, SCATTER><<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(in), static_cast<uint16_t *>(out), n, d, offset); break;
  case 4: stridedCopyKernel<uint32_t, SCATTER><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(in), static_cast<uint32_t *>(out), n, d, offset); break;
  case 8: stridedCopyKernel<uint2, SCATTER><<<grid, 256, 0, st>>>(static_cast<const uint2 *>(in), static_cast<uint2 *>(out), n, d, offset); break;
  default: stridedCopyKernel<uint4, SCATTER><<<grid, 256, 0, st>>>(static_cast<const uint4 *>(in), static_cast<uint4 *>(out), n, d, offset); break;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// out = x*cos + rotate_half(x)*sin, rotate_half(x) = concat(-x[D/2:], x[:D/2]).
// One thread handles 8 elements of the first half and the matching 8 of the second half.
// x is read as [batch, heads, seq, dim] through element strides (dim contiguous), so a head
// split that is only a permutation of a [batch, seq, heads, dim] tensor costs no extra pass;
// out is dense.
template <typename T>
__global__ void __launch_bounds__(256) ropeKernel(const T *__restrict__ x, const T *__restrict__ cs,
                                                  const T *__restrict__ sn, T *__restrict__ out, size_t batch,
                                                  size_t heads, size_t seq, size_t dim, int64_t sb, int64_t sh, int64_t ss) {
  constexpr int V = 16 / sizeof(T);
  pdlLaunchDependents();
  pdlWait();
  size_t half = dim / 2;
  size_t perRow = half / V;
  size_t total = batch * heads * seq * perRow;
  size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    size_t c = (i % perRow) * V;
    size_t row = i / perRow; // (b, h, s)
    size_t s = row % seq;
    size_t bh = row / seq;
    size_t h = bh % heads, b = bh / heads;
    const T *xr = x + static_cast<int64_t>(b) * sb + static_cast<int64_t>(h) * sh + static_cast<int64_t>(s) * ss;
    const T *cr = cs + s * dim;
    const T *sr = sn + s * dim;
    Vec16<T> x1 = ldcs16(xr + c), x2 = ldcs16(xr + half + c);
    Vec16<T> c1 = ldg16(cr + c), c2 = ldg16(cr + half + c);
    Vec16<T> s1 = ldg16(sr + c), s2 = ldg16(sr + half + c);
    Vec16<T> o1, o2;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float a = toF32(x1.v[j]), b2 = toF32(x2.v[j]);
      o1.v[j] = fromF32<T>(__fadd_rn(__fmul_rn(a, toF32(c1.v[j])), __fmul_rn(-b2, toF32(s1.v[j]))));
      o2.v[j] = fromF32<T>(__fadd_rn(__fmul_rn(b2, toF32(c2.v[j])), __fmul_rn(a, toF32(s2.v[j]))));
    }
    stcs16(out + row * dim + c, o1);
    stcs16(out + row * dim + half + c, o2);
  }
}

// ---- embedding -------------------------------------------------------------------------
// out[r, :] = table[index[r], :]  (EmbeddingOp, runtime/lib/ttnn/operations/embedding/embedding.cpp;
// torch twin ttir_cpu.py embedding = F.embedding).  One warp per row, `unit`-byte accesses.
// Indices may be stored as integers or as floats (TTNN accepts bf16 index tensors).  An index
// outside the table sets the error word instead of reading out of bounds.
template <typename I> __device__ __forceinline__ long long indexValue(I v) { return static_cast<long long>(v); }
template <> __device__ __forceinline__ long long indexValue<float>(float v) { return static_cast<long long>(v); }
template <> __device__ __forceinline__ long long indexValue<__nv_bfloat16>(__nv_bfloat16 v) {
  return static_cast<long long>(__bfloat162float(v));
}
template <> __device__ __forceinline__ long long indexValue<__half>(__half v) {
  return static_cast<long long>(__half2float(v));
}

__device__ int g_embeddingBadIndex; // set when a kernel saw an index outside its table; cleared when read

template <typename I, typename U>
__global__ void __launch_bounds__(256) embeddingKernel(const I *__restrict__ idx, const U *__restrict__ table,
                                                       U *__restrict__ out, size_t rows, size_t vocab, size_t unitsPerRow) {
  size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  long long t = indexValue(idx[row]);
  if (t < 0 || static_cast<size_t>(t) >= vocab) {
    if (lane == 0) g_embeddingBadIndex = 1;
    t = 0;
  }
  const U *src = table + static_cast<size_t>(t) * unitsPerRow;
  U *dst = out + row * unitsPerRow;
  for (size_t i = lane; i < unitsPerRow; i += 32) dst[i] = src[i];
}

// ---- pad -------------------------------------------------------------------------------
// Constant padding in front of and behind every dimension (PadOp,
// runtime/lib/ttnn/operations/data_movement/pad.cpp: `padding` holds (low, high) per dimension;
// torch twin ttir_cpu.py pad).  One thread per output element.
struct PadDims {
  int rank;
  int64_t outShape[8], inShape[8], lo[8];
};

template <typename U>
__global__ void __launch_bounds__(256) padKernel(const U *__restrict__ in, U *__restrict__ out, size_t n, PadDims d, U fill) {
  size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) {
    size_t r = i;
    int64_t at = 0, mul = 1;
    bool inside = true;
    for (int k = d.rank - 1; k >= 0; --k) {
      const int64_t c = static_cast<int64_t>(r % d.outShape[k]) - d.lo[k];
      r /= d.outShape[k];
      inside = inside && c >= 0 && c < d.inShape[k];
      at += c * mul;
      mul *= d.inShape[k];
    }
    out[i] = inside ? in[at] : fill;
  }
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_embedding(const void *indices, const void *table, void *out, int index_dtype, int dtype, size_t rows,
                  size_t vocab, size_t dim, void *stream) {
  TTB_CHECK(indices && table && out, "null tensor");
  if (rows * dim == 0) return TTB_OK;
  TTB_CHECK(vocab > 0, "empty embedding table");
  cudaStream_t st = asStream(stream);
  const size_t rowBytes = dim * dtypeSize(dtype);
  TTB_CHECK(rowBytes > 0, "unsupported table dtype");
  int unit = 16;
  while (unit > 1 && (rowBytes % unit != 0 || reinterpret_cast<uintptr_t>(table) % unit != 0 ||
                      reinterpret_cast<uintptr_t>(out) % unit != 0)) {
    unit /= 2;
  }
  ProfScope prof("embedding", 0, double(rows) * rowBytes * 2 + double(rows) * dtypeSize(index_dtype), st);
  const int grid = static_cast<int>((rows + 7) / 8);
#define TTB_EMB(I)                                                                                                   \
  switch (unit) {                                                                                                    \
  case 16: embeddingKernel<I, uint4><<<grid, 256, 0, st>>>(static_cast<const I *>(indices), static_cast<const uint4 *>(table), static_cast<uint4 *>(out), rows, vocab, rowBytes / 16); break; \
  case 8: embeddingKernel<I, uint2><<<grid, 256, 0, st>>>(static_cast<const I *>(indices), static_cast<const uint2 *>(table), static_cast<uint2 *>(out), rows, vocab, rowBytes / 8); break;    \
  case 4: embeddingKernel<I, uint32_t><<<grid, 256, 0, st>>>(static_cast<const I *>(indices), static_cast<const uint32_t *>(table), static_cast<uint32_t *>(out), rows, vocab, rowBytes / 4); break; \
  case 2: embeddingKernel<I, uint16_t><<<grid, 256, 0, st>>>(static_cast<const I *>(indices), static_cast<const uint16_t *>(table), static_cast<uint16_t *>(out), rows, vocab, rowBytes / 2); break; \
  default: embeddingKernel<I, uint8_t><<<grid, 256, 0, st>>>(static_cast<const I *>(indices), static_cast<const uint8_t *>(table), static_cast<uint8_t *>(out), rows, vocab, rowBytes); break;      \
  }
  switch (index_dtype) {
  case kI32: TTB_EMB(int32_t) break;
  case kU32: TTB_EMB(uint32_t) break;
  case kU16: TTB_EMB(uint16_t) break;
  case kF32: TTB_EMB(float) break;
  case kBF16: TTB_EMB(__nv_bfloat16) break;
  case kF16: TTB_EMB(__half) break;
  default: setLastError("embedding: unsupported index dtype"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_EMB
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_embedding_status(int *bad_index_seen) {
  TTB_CHECK(bad_index_seen != nullptr, "null result");
  TTB_CUDA(cudaDeviceSynchronize());
  TTB_CUDA(cudaMemcpyFromSymbol(bad_index_seen, g_embeddingBadIndex, sizeof(int)));
  if (*bad_index_seen) { // reported once
    const int zero = 0;
    TTB_CUDA(cudaMemcpyToSymbol(g_embeddingBadIndex, &zero, sizeof(int)));
  }
  return TTB_OK;
}

int ttb_pad(const void *in, void *out, int dtype, int rank, const int64_t *in_shape, const int64_t *low,
            const int64_t *high, double value, void *stream) {
  TTB_CHECK(in && out && in_shape && low && high, "null argument");
  TTB_CHECK(rank >= 1 && rank <= 8, "rank must be between 1 and 8");
  PadDims d;
  d.rank = rank;
  size_t n = 1, nin = 1;
  for (int i = 0; i < rank; ++i) {
    TTB_CHECK(in_shape[i] >= 0 && low[i] >= 0 && high[i] >= 0, "negative extent or padding");
    d.inShape[i] = in_shape[i];
    d.lo[i] = low[i];
    d.outShape[i] = in_shape[i] + low[i] + high[i];
    n *= static_cast<size_t>(d.outShape[i]);
    nin *= static_cast<size_t>(in_shape[i]);
  }
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("pad", 0, double(n + nin) * dtypeSize(dtype), st);
  const int grid = gridFor(n, 256);
  switch (dtype) {
  case kF32: { float f = static_cast<float>(value); uint32_t u; memcpy(&u, &f, 4);
    padKernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(in), static_cast<uint32_t *>(out), n, d, u); break; }
  case kBF16: { __nv_bfloat16 b = __float2bfloat16_rn(static_cast<float>(value)); uint16_t u; memcpy(&u, &b, 2);
    padKernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(in), static_cast<uint16_t *>(out), n, d, u); break; }
  case kF16: { __half b = __float2half_rn(static_cast<float>(value)); uint16_t u; memcpy(&u, &b, 2);
    padKernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(in), static_cast<uint16_t *>(out), n, d, u); break; }
  case kI32: padKernel<int32_t><<<grid, 256, 0, st>>>(static_cast<const int32_t *>(in), static_cast<int32_t *>(out), n, d, static_cast<int32_t>(value)); break;
  case kU32: padKernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t *>(in), static_cast<uint32_t *>(out), n, d, static_cast<uint32_t>(value)); break;
  case kU16: padKernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(in), static_cast<uint16_t *>(out), n, d, static_cast<uint16_t>(value)); break;
  case kU8: padKernel<uint8_t><<<grid, 256, 0, st>>>(static_cast<const uint8_t *>(in), static_cast<uint8_t *>(out), n, d, static_cast<uint8_t>(value)); break;
  case kI8: padKernel<int8_t><<<grid, 256, 0, st>>>(static_cast<const int8_t *>(in), static_cast<int8_t *>(out), n, d, static_cast<int8_t>(value)); break;
  default: setLastError("pad: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_strided_copy(const void *in, void *out, int elem_size, int rank, const int64_t *out_shape,
                     const int64_t *in_strides, int64_t in_offset, void *stream) {
  return launchStrided<false>(in, out, elem_size, rank, out_shape, in_strides, in_offset, asStream(stream));
}

int ttb_strided_scatter(const void *in, void *out, int elem_size, int rank, const int64_t *in_shape,
                        const int64_t *out_strides, int64_t out_offset, void *stream) {
  return launchStrided<true>(in, out, elem_size, rank, in_shape, out_strides, out_offset, asStream(stream));
}

int ttb_rotary_embedding(const void *x, const void *cos, const void *sin, void *out, int dtype, size_t batch_heads,
                         size_t seq, size_t head_dim, void *stream) {
  int64_t strides[3] = {static_cast<int64_t>(batch_heads * seq * head_dim), static_cast<int64_t>(seq * head_dim),
                        static_cast<int64_t>(head_dim)};
  return ttb_rotary_embedding_strided(x, cos, sin, out, dtype, 1, batch_heads, seq, head_dim, strides, stream);
}

int ttb_rotary_embedding_strided(const void *x, const void *cos, const void *sin, void *out, int dtype, size_t batch,
                                 size_t heads, size_t seq, size_t head_dim, const int64_t *x_strides3, void *stream) {
  TTB_CHECK(x && cos && sin && out && x_strides3, "null tensor");
  TTB_CHECK(aligned16(x) && aligned16(cos) && aligned16(sin) && aligned16(out), "tensors must be 16-byte aligned");
  size_t es = dtypeSize(dtype);
  TTB_CHECK(es == 2 || es == 4, "rotary embedding needs a float dtype");
  TTB_CHECK(head_dim % (2 * (16 / es)) == 0, "head_dim/2 must be a multiple of 16 bytes");
  for (int i = 0; i < 3; ++i) {
    TTB_CHECK(x_strides3[i] >= 0 && (x_strides3[i] * es) % 16 == 0, "input strides must be multiples of 16 bytes");
  }
  size_t total = batch * heads * seq * (head_dim / 2 / (16 / es));
  if (total == 0) return TTB_OK;
  ProfScope prof("rotary_embedding", 0, 2.0 * double(batch * heads) * seq * head_dim * es, asStream(stream));
  TTB_DISPATCH_FLOAT(dtype, T, {
    TTB_CUDA(launchPdl(ropeKernel<T>, dim3(gridFor(total, 256)), dim3(256), 0, asStream(stream), static_cast<const T *>(x),
                       static_cast<const T *>(cos), static_cast<const T *>(sin), static_cast<T *>(out), batch, heads, seq,
                       head_dim, x_strides3[0], x_strides3[1], x_strides3[2]));
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
