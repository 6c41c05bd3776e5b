// Indexing ops: gather, scatter, sort, top-k and sampling.
//
// Reference call sites: runtime/lib/ttnn/operations/data_movement/{gather,scatter,sort}.cpp and
// operations/reduction/{topk,sampling}.cpp (::ttnn::gather / scatter / sort / topk / sampling); semantics
// from the goldens tools/golden/mapping.py:5384-5437 (torch.gather, torch.scatter / scatter_reduce),
// :5624-5640 (torch.sort, stable), :5927-5958 (torch.topk, always sorted) and :5994-6019 (softmax of
// values / temperature, then a multinomial draw among the candidates).
//
// All of them are HBM- or latency-bound integer / index work: coalesced loads along the contiguous
// dimension, no tensor cores.  Sorting is a bitonic network over 64-bit (order key, position) pairs --
// the position in the low half makes every key unique, which is what makes the result stable and the
// same on every run -- with all exchange distances below a tile done in shared memory.
#include "common.cuh"

#include <cfloat>
#include <type_traits>

namespace ttb {

__device__ int g_indexBad; // an index outside its dimension was seen (the element was skipped / read as 0); cleared when read

struct IdxDims {
  int rank;
  int dim;
  int64_t idxShape[8];  // shape of the index tensor (= of gather's result, of scatter's source window)
  int64_t xStrides[8];  // dense strides of the data tensor that is indexed along `dim`
  int64_t srcStrides[8]; // scatter: dense strides of the source tensor
  int64_t dimSize;      // extent of the indexed dimension
};

template <typename I> __device__ __forceinline__ long long indexOf(I v) { return static_cast<long long>(v); }
template <> __device__ __forceinline__ long long indexOf<float>(float v) { return static_cast<long long>(v); }

// out[i] = x[..., index[i], ...]: one thread per element of the index tensor.
template <typename U, typename I>
__global__ void __launch_bounds__(256) gatherKernel(const U *__restrict__ x, const I *__restrict__ index, U *__restrict__ out,
                                                    size_t n, IdxDims d) {
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) {
    size_t r = i;
    int64_t at = 0;
    for (int k = d.rank - 1; k >= 0; --k) {
      const int64_t c = static_cast<int64_t>(r % d.idxShape[k]);
      r /= d.idxShape[k];
      if (k != d.dim) at += c * d.xStrides[k];
    }
    long long t = indexOf(index[i]);
    if (t < 0) t += d.dimSize; // torch accepts negative indices
    if (t < 0 || t >= d.dimSize) {
      g_indexBad = 1;
      out[i] = U{};
      continue;
    }
    out[i] = x[at + t * d.xStrides[d.dim]];
  }
}

// Arithmetic of scatter's reduce modes in the tensor's own type: every step rounds, as torch's does.
template <typename T> __device__ __forceinline__ T scatterCombine(T cur, T v, int mode) {
  const float a = toF32(cur), b = toF32(v);
  switch (mode) {
  case 0: return fromF32<T>(a + b);                 // Sum
  case 2: return (b > a || b != b) ? v : cur;       // Max (NaN propagates)
  case 3: return (b < a || b != b) ? v : cur;       // Min
  case 6: return fromF32<T>(a * b);                 // Prod
  default: return v;                                // plain scatter: the last write wins
  }
}
template <> __device__ __forceinline__ int32_t scatterCombine<int32_t>(int32_t cur, int32_t v, int mode) {
  switch (mode) {
  case 0: return cur + v;
  case 2: return v > cur ? v : cur;
  case 3: return v < cur ? v : cur;
  case 6: return cur * v;
  default: return v;
  }
}

// out (already a copy of the input) [..., index[i], ...] (op)= src[i].  One thread owns one line of the
// result along `dim` -- all positions that share the other coordinates -- and walks the index tensor
// along `dim` in order, so that duplicates are applied in the order torch's CPU loop applies them and
// no two threads touch the same element.  A is the type the running value is kept in: T itself, or
// float for sums and products of 16-bit tensors, which torch accumulates in f32 and rounds once at the end
// (`out` is then an f32 image of the result that scatterFinishKernel rounds).
template <typename T, typename A, typename I>
__global__ void __launch_bounds__(256) scatterKernel(A *__restrict__ out, const I *__restrict__ index, const T *__restrict__ src,
                                                     size_t lines, IdxDims d, int mode) {
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t line = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; line < lines; line += step) {
    // coordinates of the line over the index shape without `dim`
    size_t r = line;
    int64_t atOut = 0, atIdx = 0, atSrc = 0, idxStride = 1, mul = 1;
    for (int k = d.rank - 1; k >= 0; --k) {
      if (k == d.dim) {
        idxStride = mul;
        mul *= d.idxShape[k];
        continue;
      }
      const int64_t c = static_cast<int64_t>(r % d.idxShape[k]);
      r /= d.idxShape[k];
      atOut += c * d.xStrides[k];
      atSrc += c * d.srcStrides[k];
      atIdx += c * mul;
      mul *= d.idxShape[k];
    }
    for (int64_t j = 0; j < d.idxShape[d.dim]; ++j) {
      long long t = indexOf(index[atIdx + j * idxStride]);
      if (t < 0) t += d.dimSize;
      if (t < 0 || t >= d.dimSize) {
        g_indexBad = 1;
        continue;
      }
      A *p = out + atOut + t * d.xStrides[d.dim];
      const T v = src[atSrc + j * d.srcStrides[d.dim]];
      if constexpr (std::is_same<A, T>::value) *p = scatterCombine<T>(*p, v, mode);
      else *p = scatterCombine<float>(*p, toF32(v), mode);
    }
  }
}

template <typename T> __global__ void __launch_bounds__(256) scatterWidenKernel(const T *__restrict__ x, float *__restrict__ acc, size_t n) {
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) acc[i] = toF32(x[i]);
}
template <typename T> __global__ void __launch_bounds__(256) scatterFinishKernel(const float *__restrict__ acc, T *__restrict__ out, size_t n) {
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += step) out[i] = fromF32<T>(acc[i]);
}

// ---- sort ------------------------------------------------------------------------------------------------
// Order key: a 32-bit unsigned integer whose natural order is the wanted order of the values (NaN after
// everything, as torch sorts it); descending order inverts it.  The position goes in the low 32 bits.
template <typename T> __device__ __forceinline__ uint32_t orderKey(T v);
template <> __device__ __forceinline__ uint32_t orderKey<float>(float v) {
  if (v != v) return 0xffffffffu;
  uint32_t b = __float_as_uint(v);
  if (b == 0x80000000u) b = 0; // -0 and +0 compare equal
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
template <> __device__ __forceinline__ uint32_t orderKey<__nv_bfloat16>(__nv_bfloat16 v) { return orderKey<float>(__bfloat162float(v)); }
template <> __device__ __forceinline__ uint32_t orderKey<__half>(__half v) { return orderKey<float>(__half2float(v)); }
template <> __device__ __forceinline__ uint32_t orderKey<int32_t>(int32_t v) { return static_cast<uint32_t>(v) ^ 0x80000000u; }
template <> __device__ __forceinline__ uint32_t orderKey<uint32_t>(uint32_t v) { return v; }

constexpr int SORT_TILE = 2048; // pairs per shared-memory tile (16 KiB)
constexpr uint64_t SORT_PAD = ~0ull;

template <typename T>
__global__ void __launch_bounds__(256) sortLoadKernel(const T *__restrict__ x, uint64_t *__restrict__ keys, size_t rows, size_t n,
                                                      size_t padded, int descending) {
  const size_t total = rows * padded, step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const size_t row = i / padded, j = i % padded;
    uint64_t k = SORT_PAD;
    if (j < n) {
      uint32_t o = orderKey<T>(x[row * n + j]);
      // NaN stays last in ascending order and comes first in descending order, as torch has it
      if (descending) o = ~o;
      k = (static_cast<uint64_t>(o) << 32) | static_cast<uint32_t>(j);
    }
    keys[i] = k;
  }
}

__device__ __forceinline__ void bitonicExchange(uint64_t &a, uint64_t &b, bool up) {
  if ((a > b) == up) {
    const uint64_t t = a;
    a = b;
    b = t;
  }
}

// All steps of the network whose exchange distance is below the tile: a full sort of each tile
// (kFrom = 2), or the tail of a merge of size k > tile (kFrom = kTo = k, distances tile/2 .. 1).
__global__ void __launch_bounds__(SORT_TILE / 2) sortTileKernel(uint64_t *__restrict__ keys, size_t padded, uint32_t kFrom, uint32_t kTo) {
  __shared__ uint64_t s[SORT_TILE];
  const size_t base = static_cast<size_t>(blockIdx.x) * SORT_TILE; // tiles of all rows back to back; padded is a multiple of the tile
  const size_t inRow = base % padded;
  for (int i = threadIdx.x; i < SORT_TILE; i += blockDim.x) s[i] = keys[base + i];
  __syncthreads();
  for (uint32_t k = kFrom; k <= kTo; k <<= 1) {
    for (uint32_t j = (k > SORT_TILE ? SORT_TILE : k) >> 1; j > 0; j >>= 1) {
      const uint32_t t = threadIdx.x;
      const uint32_t lo = 2 * t - (t & (j - 1)); // index of the lower element of pair t at distance j
      const bool up = (((inRow + lo) & k) == 0);
      bitonicExchange(s[lo], s[lo + j], up);
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < SORT_TILE; i += blockDim.x) keys[base + i] = s[i];
}

// One step of the network at distance j >= tile.
__global__ void __launch_bounds__(256) sortGlobalKernel(uint64_t *__restrict__ keys, size_t rows, size_t padded, uint32_t k, uint32_t j) {
  const size_t pairs = rows * (padded / 2), step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < pairs; i += step) {
    const size_t row = i / (padded / 2), t = i % (padded / 2);
    const size_t lo = 2 * t - (t & (j - 1));
    uint64_t *p = keys + row * padded;
    uint64_t a = p[lo], b = p[lo + j];
    const bool up = ((lo & k) == 0);
    if ((a > b) == up) {
      p[lo] = b;
      p[lo + j] = a;
    }
  }
}

// Writes the first `take` entries of every sorted row: the value is fetched from the input by position
// (its exact bits), the position is stored in the index tensor's type.
template <typename T, typename I>
__global__ void __launch_bounds__(256) sortStoreKernel(const T *__restrict__ x, const uint64_t *__restrict__ keys, T *__restrict__ values,
                                                       I *__restrict__ indices, size_t rows, size_t n, size_t padded, size_t take) {
  const size_t total = rows * take, step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const size_t row = i / take, j = i % take;
    const uint32_t pos = static_cast<uint32_t>(keys[row * padded + j]);
    if (values) values[i] = x[row * n + pos];
    if (indices) indices[i] = static_cast<I>(pos);
  }
}

static size_t sortPadded(size_t n) {
  size_t p = SORT_TILE;
  while (p < n) p <<= 1;
  return p;
}

template <typename T>
static int sortRows(const void *x, void *values, void *indices, int indexDtype, size_t rows, size_t n, size_t take, int descending,
                    void *workspace, cudaStream_t st) {
  const size_t padded = sortPadded(n);
  uint64_t *keys = static_cast<uint64_t *>(workspace);
  sortLoadKernel<T><<<gridFor(rows * padded, 256), 256, 0, st>>>(static_cast<const T *>(x), keys, rows, n, padded, descending);
  const unsigned tiles = static_cast<unsigned>(rows * padded / SORT_TILE);
  sortTileKernel<<<tiles, SORT_TILE / 2, 0, st>>>(keys, padded, 2, SORT_TILE);
  int launches = 2;
  for (size_t k = 2 * static_cast<size_t>(SORT_TILE); k <= padded; k <<= 1) {
    for (size_t j = k >> 1; j >= SORT_TILE; j >>= 1) {
      sortGlobalKernel<<<gridFor(rows * padded / 2, 256), 256, 0, st>>>(keys, rows, padded, static_cast<uint32_t>(k), static_cast<uint32_t>(j));
      ++launches;
    }
    sortTileKernel<<<tiles, SORT_TILE / 2, 0, st>>>(keys, padded, static_cast<uint32_t>(k), static_cast<uint32_t>(k));
    ++launches;
  }
  const int grid = gridFor(rows * take, 256);
#define TTB_STORE(I)                                                                                                            \
  sortStoreKernel<T, I><<<grid, 256, 0, st>>>(static_cast<const T *>(x), keys, static_cast<T *>(values), static_cast<I *>(indices), \
                                              rows, n, padded, take)
  switch (indices ? indexDtype : kI32) {
  case kI32: TTB_STORE(int32_t); break;
  case kU32: TTB_STORE(uint32_t); break;
  case kU16: TTB_STORE(uint16_t); break;
  default: setLastError("sort: the index tensor must be Int32, UInt32 or UInt16"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_STORE
  countLaunch(launches + 1);
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// ---- sampling ----------------------------------------------------------------------------------------------
// Counter-based generator (a 64-bit mix of seed, row and draw number): the same (seed, row) gives the
// same draw on every run and every launch geometry.
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t row) {
  uint64_t z = seed * 0x9E3779B97F4A7C15ull + (row + 1) * 0xBF58476D1CE4E5B9ull;
  z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27; z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f); // 24 random bits: [0, 1)
}

constexpr int SAMPLE_MAX = 4096; // candidates per row

// One block per row: softmax(values / temperature) over the candidates, the k most probable kept, of
// those the smallest prefix (in order of probability) whose mass reaches p, one draw from what is left,
// and the candidate's entry of `indices` as the result.  k <= 0 or k > candidates keeps all; p >= 1 or
// p <= 0 switches the nucleus cut off.
template <typename T, typename I, typename O>
__global__ void __launch_bounds__(256)
    samplingKernel(const T *__restrict__ values, const I *__restrict__ indices, const uint32_t *__restrict__ topK, const T *__restrict__ topP,
                   const T *__restrict__ temp, O *__restrict__ out, int candidates, int padded, uint64_t seed) {
  __shared__ uint64_t keys[SAMPLE_MAX];
  __shared__ float red[256];
  const int row = blockIdx.x, tid = threadIdx.x;
  const T *v = values + static_cast<size_t>(row) * candidates;
  const float invT = 1.0f / fmaxf(toF32(temp[row]), 1e-6f);
  // candidates in descending order of their logit (ties: the earlier candidate first)
  for (int i = tid; i < padded; i += 256) {
    uint64_t k = SORT_PAD;
    if (i < candidates) k = (static_cast<uint64_t>(~orderKey<float>(toF32(v[i]) * invT)) << 32) | static_cast<uint32_t>(i);
    keys[i] = k;
  }
  __syncthreads();
  for (int k = 2; k <= padded; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = tid; t < padded / 2; t += 256) {
        const int lo = 2 * t - (t & (j - 1));
        bitonicExchange(keys[lo], keys[lo + j], (lo & k) == 0);
      }
      __syncthreads();
    }
  }
  int keep = candidates;
  const uint32_t kk = topK[row];
  if (kk > 0 && kk < static_cast<uint32_t>(candidates)) keep = static_cast<int>(kk);
  // softmax over the kept candidates, relative to the largest logit (position 0 after the sort)
  const float top = toF32(v[static_cast<uint32_t>(keys[0])]) * invT;
  float part = 0.0f;
  for (int i = tid; i < keep; i += 256) part += __expf(toF32(v[static_cast<uint32_t>(keys[i])]) * invT - top);
  red[tid] = part;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (tid < s) red[tid] += red[tid + s];
    __syncthreads();
  }
  if (tid == 0) {
    const float total = red[0];
    const float p = toF32(topP[row]);
    // nucleus: the shortest prefix whose probability mass reaches p (always at least one candidate)
    float mass = total;
    int last = keep;
    if (p > 0.0f && p < 1.0f) {
      float run = 0.0f;
      for (int i = 0; i < keep; ++i) {
        run += __expf(toF32(v[static_cast<uint32_t>(keys[i])]) * invT - top);
        if (run >= p * total) {
          last = i + 1;
          mass = run;
          break;
        }
      }
    }
    // inverse CDF
    const float u = uniform01(seed, static_cast<uint64_t>(row)) * mass;
    float run = 0.0f;
    int pick = last - 1;
    for (int i = 0; i < last; ++i) {
      run += __expf(toF32(v[static_cast<uint32_t>(keys[i])]) * invT - top);
      if (u < run) {
        pick = i;
        break;
      }
    }
    out[row] = static_cast<O>(indices[static_cast<size_t>(row) * candidates + static_cast<uint32_t>(keys[pick])]);
  }
}

static bool fillIdxDims(IdxDims &d, int rank, int dim, const int64_t *idxShape, const int64_t *xShape, const int64_t *srcShape) {
  if (rank < 1 || rank > 8 || dim < 0 || dim >= rank) return false;
  d.rank = rank;
  d.dim = dim;
  int64_t xs = 1, ss = 1;
  for (int k = rank - 1; k >= 0; --k) {
    d.idxShape[k] = idxShape[k];
    d.xStrides[k] = xs;
    xs *= xShape[k];
    d.srcStrides[k] = ss;
    ss *= srcShape ? srcShape[k] : idxShape[k];
    if (k != dim && idxShape[k] > xShape[k]) return false;            // torch's rule for gather and scatter
    if (srcShape && idxShape[k] > srcShape[k]) return false;
  }
  d.dimSize = xShape[dim];
  return true;
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_gather(const void *x, const void *index, void *out, int dtype, int index_dtype, int rank, const int64_t *x_shape,
               const int64_t *index_shape, int dim, void *stream) {
  TTB_CHECK(x && index && out && x_shape && index_shape, "null argument");
  IdxDims d;
  TTB_CHECK(fillIdxDims(d, rank, dim, index_shape, x_shape, nullptr), "gather: bad rank, dim or an index extent larger than the input's");
  size_t n = 1;
  for (int k = 0; k < rank; ++k) n *= static_cast<size_t>(index_shape[k]);
  if (n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  const size_t es = dtypeSize(dtype);
  ProfScope prof("gather", 0, double(n) * (2.0 * es + dtypeSize(index_dtype)), st);
  const int grid = gridFor(n, 256);
#define TTB_G(U, I) gatherKernel<U, I><<<grid, 256, 0, st>>>(static_cast<const U *>(x), static_cast<const I *>(index), static_cast<U *>(out), n, d)
#define TTB_GI(U)                                                                        \
  switch (index_dtype) {                                                                 \
  case kI32: TTB_G(U, int32_t); break;                                                   \
  case kU32: TTB_G(U, uint32_t); break;                                                  \
  case kU16: TTB_G(U, uint16_t); break;                                                  \
  default: setLastError("gather: the index must be Int32, UInt32 or UInt16"); return TTB_ERR_UNSUPPORTED; \
  }
  switch (es) {
  case 1: TTB_GI(uint8_t) break;
  case 2: TTB_GI(uint16_t) break;
  case 4: TTB_GI(uint32_t) break;
  default: setLastError("gather: unsupported element size"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_GI
#undef TTB_G
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

size_t ttb_scatter_workspace_bytes(int dtype, int reduce_type, size_t elements) {
  const bool wide = (dtype == kBF16 || dtype == kF16) && (reduce_type == 0 || reduce_type == 6);
  return wide ? elements * sizeof(float) : 0;
}

int ttb_scatter(const void *x, const void *index, const void *src, void *out, int dtype, int index_dtype, int rank,
                const int64_t *x_shape, const int64_t *index_shape, const int64_t *src_shape, int dim, int reduce_type,
                void *workspace, size_t workspace_bytes, void *stream) {
  TTB_CHECK(x && index && src && out && x_shape && index_shape && src_shape, "null argument");
  TTB_CHECK(reduce_type == 0 || reduce_type == 2 || reduce_type == 3 || reduce_type == 6 || reduce_type == 7,
            "scatter: reduce type must be Sum (0), Max (2), Min (3), Prod (6) or Invalid (7, plain scatter)");
  IdxDims d;
  TTB_CHECK(fillIdxDims(d, rank, dim, index_shape, x_shape, src_shape), "scatter: bad rank, dim or an index extent larger than the input's / source's");
  size_t total = 1, lines = 1;
  for (int k = 0; k < rank; ++k) {
    total *= static_cast<size_t>(x_shape[k]);
    if (k != dim) lines *= static_cast<size_t>(index_shape[k]);
  }
  cudaStream_t st = asStream(stream);
  const size_t es = dtypeSize(dtype);
  const size_t need = ttb_scatter_workspace_bytes(dtype, reduce_type, total);
  TTB_CHECK(need == 0 || (workspace && workspace_bytes >= need), "scatter: workspace too small (see ttb_scatter_workspace_bytes)");
  const bool empty = lines == 0 || index_shape[dim] == 0;
  if ((need == 0 || empty) && out != x && total) TTB_CUDA(cudaMemcpyAsync(out, x, total * es, cudaMemcpyDeviceToDevice, st));
  if (empty || total == 0) return TTB_OK;
  ProfScope prof("scatter", 0, double(total) * es * 2 + double(lines) * index_shape[dim] * (es + dtypeSize(index_dtype)), st);
  const int grid = gridFor(lines, 256), gridAll = gridFor(total, 256);
  float *acc = static_cast<float *>(workspace);
#define TTB_S(T, A, I, dst) scatterKernel<T, A, I><<<grid, 256, 0, st>>>(dst, static_cast<const I *>(index), static_cast<const T *>(src), lines, d, reduce_type)
#define TTB_SI(T, A, dst)                                                                \
  switch (index_dtype) {                                                                 \
  case kI32: TTB_S(T, A, int32_t, dst); break;                                           \
  case kU32: TTB_S(T, A, uint32_t, dst); break;                                          \
  case kU16: TTB_S(T, A, uint16_t, dst); break;                                          \
  default: setLastError("scatter: the index must be Int32, UInt32 or UInt16"); return TTB_ERR_UNSUPPORTED; \
  }
#define TTB_S16(T)                                                                       \
  if (need) {                                                                            \
    scatterWidenKernel<T><<<gridAll, 256, 0, st>>>(static_cast<const T *>(x), acc, total); \
    TTB_SI(T, float, acc)                                                                \
    scatterFinishKernel<T><<<gridAll, 256, 0, st>>>(acc, static_cast<T *>(out), total);  \
    countLaunch(2);                                                                      \
  } else {                                                                               \
    TTB_SI(T, T, static_cast<T *>(out))                                                  \
  }
  switch (dtype) {
  case kF32: TTB_SI(float, float, static_cast<float *>(out)) break;
  case kBF16: TTB_S16(__nv_bfloat16) break;
  case kF16: TTB_S16(__half) break;
  case kI32: TTB_SI(int32_t, int32_t, static_cast<int32_t *>(out)) break;
  default: setLastError("scatter: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_S16
#undef TTB_SI
#undef TTB_S
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_index_status(int *bad_index_seen) {
  TTB_CHECK(bad_index_seen != nullptr, "null result");
  TTB_CUDA(cudaDeviceSynchronize());
  TTB_CUDA(cudaMemcpyFromSymbol(bad_index_seen, g_indexBad, sizeof(int)));
  if (*bad_index_seen) { // reported once
    const int zero = 0;
    TTB_CUDA(cudaMemcpyToSymbol(g_indexBad, &zero, sizeof(int)));
  }
  return TTB_OK;
}

size_t ttb_sort_workspace_bytes(size_t rows, size_t n) { return rows * sortPadded(n) * sizeof(uint64_t); }

int ttb_sort(const void *x, void *values, void *indices, int dtype, int index_dtype, size_t rows, size_t n, size_t take,
             int descending, void *workspace, size_t workspace_bytes, void *stream) {
  TTB_CHECK(x && (values || indices), "null tensor");
  TTB_CHECK(take <= n, "cannot take more entries than a row has");
  if (rows * take == 0) return TTB_OK;
  TTB_CHECK(n <= 0x7fffffffull, "row too long");
  TTB_CHECK(workspace && workspace_bytes >= ttb_sort_workspace_bytes(rows, n), "workspace too small (see ttb_sort_workspace_bytes)");
  cudaStream_t st = asStream(stream);
  ProfScope prof("sort", 0, double(rows) * n * dtypeSize(dtype) + double(rows) * take * (dtypeSize(dtype) + dtypeSize(index_dtype)), st);
  switch (dtype) {
  case kF32: return sortRows<float>(x, values, indices, index_dtype, rows, n, take, descending, workspace, st);
  case kBF16: return sortRows<__nv_bfloat16>(x, values, indices, index_dtype, rows, n, take, descending, workspace, st);
  case kF16: return sortRows<__half>(x, values, indices, index_dtype, rows, n, take, descending, workspace, st);
  case kI32: return sortRows<int32_t>(x, values, indices, index_dtype, rows, n, take, descending, workspace, st);
  case kU32: return sortRows<uint32_t>(x, values, indices, index_dtype, rows, n, take, descending, workspace, st);
  default: setLastError("sort: unsupported dtype"); return TTB_ERR_UNSUPPORTED;
  }
}

int ttb_sampling(const void *values, const void *indices, const void *k, const void *p, const void *temp, void *out, int dtype,
                 int index_dtype, int out_dtype, int rows, int candidates, uint64_t seed, void *stream) {
  TTB_CHECK(values && indices && k && p && temp && out, "null tensor");
  TTB_CHECK(rows >= 0 && candidates >= 1, "bad extents");
  TTB_CHECK(candidates <= SAMPLE_MAX, "sampling takes at most 4096 candidates per row");
  if (rows == 0) return TTB_OK;
  int padded = 2;
  while (padded < candidates) padded <<= 1;
  cudaStream_t st = asStream(stream);
  ProfScope prof("sampling", 0, double(rows) * candidates * (dtypeSize(dtype) + dtypeSize(index_dtype)), st);
#define TTB_SMP(T, I, O)                                                                                                       \
  samplingKernel<T, I, O><<<rows, 256, 0, st>>>(static_cast<const T *>(values), static_cast<const I *>(indices),              \
                                                static_cast<const uint32_t *>(k), static_cast<const T *>(p),                   \
                                                static_cast<const T *>(temp), static_cast<O *>(out), candidates, padded, seed)
#define TTB_SMP_O(T, I)                                                                  \
  if (out_dtype == kI32) TTB_SMP(T, I, int32_t);                                         \
  else if (out_dtype == kU32) TTB_SMP(T, I, uint32_t);                                   \
  else { setLastError("sampling: the result must be Int32 or UInt32"); return TTB_ERR_UNSUPPORTED; }
#define TTB_SMP_I(T)                                                                     \
  if (index_dtype == kI32) { TTB_SMP_O(T, int32_t) }                                     \
  else if (index_dtype == kU32) { TTB_SMP_O(T, uint32_t) }                               \
  else { setLastError("sampling: candidate indices must be Int32 or UInt32"); return TTB_ERR_UNSUPPORTED; }
  switch (dtype) {
  case kBF16: TTB_SMP_I(__nv_bfloat16) break;
  case kF32: TTB_SMP_I(float) break;
  case kF16: TTB_SMP_I(__half) break;
  default: setLastError("sampling: values, p and temp must share a float type"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_SMP_I
#undef TTB_SMP_O
#undef TTB_SMP
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
