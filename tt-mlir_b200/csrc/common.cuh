// Shared helpers for the sm_100a kernels: dtype tags, error reporting, vector access.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>
#include <utility>

#include "../../include/ttb_kernels.h"

namespace ttb {

// Numeric values follow tt::target::DataType (include/ttmlir/Target/Common/types.fbs:19-42).
enum DType : int {
  kF32 = TTB_DTYPE_FLOAT32,
  kF16 = TTB_DTYPE_FLOAT16,
  kBF16 = TTB_DTYPE_BFLOAT16,
  kU32 = TTB_DTYPE_UINT32,
  kU16 = TTB_DTYPE_UINT16,
  kU8 = TTB_DTYPE_UINT8,
  kI32 = TTB_DTYPE_INT32,
  kI8 = TTB_DTYPE_INT8,
};

inline size_t dtypeSize(int dt) {
  switch (dt) {
  case kF32: case kU32: case kI32: return 4;
  case kF16: case kBF16: case kU16: return 2;
  case kU8: case kI8: return 1;
  default: return 0;
  }
}

void setLastError(const std::string &msg);
int cudaFail(cudaError_t e, const char *what, const char *file, int line);

#define TTB_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      return ::ttb::cudaFail(_e, #expr, __FILE__, __LINE__);                             \
    }                                                                                    \
  } while (0)

#define TTB_CHECK(cond, msg)                                                             \
  do {                                                                                   \
    if (!(cond)) {                                                                       \
      ::ttb::setLastError(std::string(msg) + " (" #cond ")");                            \
      return TTB_ERR_INVALID;                                                            \
    }                                                                                    \
  } while (0)

// After a launch: report configuration errors without synchronising.
#define TTB_LAUNCH_CHECK() TTB_CUDA(cudaGetLastError())

inline cudaStream_t asStream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// While a GemmScratchScope is alive on the calling thread, the CUDA-core GEMM takes the scratch of its
// split-K mode from [ptr, ptr + bytes) instead of the memory pool, and runs without split-K when that
// is too small: nothing below the scope allocates.  Used by the entry points that promise not to.
struct GemmScratchScope {
  GemmScratchScope(void *ptr, size_t bytes);
  ~GemmScratchScope();
  // Active scope of this thread, if any: true and its range.
  static bool current(void **ptr, size_t *bytes);
};

// Number of SMs of the current device (148 on B200); cached per device.
int smCount();
// Adds to the process-wide count of kernels launched by this library.
void countLaunch(uint64_t n = 1);

// Optional per-launch timing.  When profiling is on (ttb_prof_enable), a ProfScope around a
// launch records a CUDA event pair on the launching stream together with the algorithmic work
// of that launch; ttb_prof_summary aggregates them per tag.  Off: one relaxed atomic load.
struct ProfScope {
  ProfScope(const char *tag, double flops, double bytes, cudaStream_t stream);
  ~ProfScope();
  int slot;
  cudaStream_t stream;
};

// ---- programmatic dependent launch ---------------------------------------------------------
// A kernel launched through launchPdl may start (be scheduled, run its prologue) while the kernel
// before it on the stream is still finishing; it calls pdlWait() before it touches global memory,
// which returns once that kernel has completed and its writes are visible.  A kernel calls
// pdlLaunchDependents() to let its successor be scheduled early.  Every kernel launched this way
// MUST execute pdlWait(): its own successor relies on "this kernel is done" implying "everything
// before it is done".  Without the launch attribute both calls do nothing.  TTB_DISABLE_PDL=1
// launches everything the ordinary way.
__device__ __forceinline__ void pdlWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdlLaunchDependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool pdlEnabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launchPdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdlEnabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Grid for a grid-stride kernel: enough blocks for `items`, capped at a few waves of the GPU.
inline int gridFor(size_t items, int block, int blocksPerSm = 16) {
  size_t need = (items + block - 1) / block;
  size_t cap = static_cast<size_t>(smCount()) * blocksPerSm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

// N elements of T moved with 16-byte accesses (N * sizeof(T) must be a multiple of 16).
template <typename T, int N> struct alignas(16) Pack {
  T v[N];
};
template <typename T, int N>
__device__ __forceinline__ void loadPack(Pack<T, N> &r, const T *p) {
  static_assert((N * sizeof(T)) % 16 == 0, "pack must be a multiple of 16 bytes");
  constexpr int Q = N * sizeof(T) / 16;
  uint4 *d = reinterpret_cast<uint4 *>(r.v);
  const uint4 *s = reinterpret_cast<const uint4 *>(p);
#pragma unroll
  for (int i = 0; i < Q; ++i) d[i] = __ldcs(s + i);
}
template <typename T, int N>
__device__ __forceinline__ void storePack(T *p, const Pack<T, N> &r) {
  static_assert((N * sizeof(T)) % 16 == 0, "pack must be a multiple of 16 bytes");
  constexpr int Q = N * sizeof(T) / 16;
  const uint4 *s = reinterpret_cast<const uint4 *>(r.v);
  uint4 *d = reinterpret_cast<uint4 *>(p);
#pragma unroll
  for (int i = 0; i < Q; ++i) __stcs(d + i, s[i]);
}

// ---- element conversion --------------------------------------------------------------
template <typename T> __device__ __forceinline__ float toF32(T v);
template <> __device__ __forceinline__ float toF32<float>(float v) { return v; }
template <> __device__ __forceinline__ float toF32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float toF32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float toF32<int32_t>(int32_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float toF32<uint32_t>(uint32_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float toF32<uint16_t>(uint16_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float toF32<uint8_t>(uint8_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float toF32<int8_t>(int8_t v) { return static_cast<float>(v); }

// Float -> T with round-to-nearest-even; integers saturate like a C++ cast after clamping.
template <typename T> __device__ __forceinline__ T fromF32(float v);
template <> __device__ __forceinline__ float fromF32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 fromF32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half fromF32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ int32_t fromF32<int32_t>(float v) { return __float2int_rz(v); }
template <> __device__ __forceinline__ uint32_t fromF32<uint32_t>(float v) { return __float2uint_rz(v); }
template <> __device__ __forceinline__ uint16_t fromF32<uint16_t>(float v) { return static_cast<uint16_t>(min(max(__float2int_rz(v), 0), 65535)); }
template <> __device__ __forceinline__ uint8_t fromF32<uint8_t>(float v) { return static_cast<uint8_t>(min(max(__float2int_rz(v), 0), 255)); }
template <> __device__ __forceinline__ int8_t fromF32<int8_t>(float v) { return static_cast<int8_t>(min(max(__float2int_rz(v), -128), 127)); }

// 16-byte vector of T.
template <typename T> struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ldg16(const T *p) {
  Vec16<T> r;
  *reinterpret_cast<uint4 *>(&r) = __ldg(reinterpret_cast<const uint4 *>(p));
  return r;
}
// Streaming variants: data touched once should not displace reusable lines in L2/L1.
template <typename T>
__device__ __forceinline__ Vec16<T> ldcs16(const T *p) {
  Vec16<T> r;
  *reinterpret_cast<uint4 *>(&r) = __ldcs(reinterpret_cast<const uint4 *>(p));
  return r;
}
template <typename T>
__device__ __forceinline__ void stcs16(T *p, const Vec16<T> &r) {
  __stcs(reinterpret_cast<uint4 *>(p), *reinterpret_cast<const uint4 *>(&r));
}
template <typename T>
__device__ __forceinline__ void st16(T *p, const Vec16<T> &r) {
  *reinterpret_cast<uint4 *>(p) = *reinterpret_cast<const uint4 *>(&r);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Dispatch a callable templated on the C++ element type of a dtype tag.
#define TTB_DISPATCH_DTYPE(dt, T, ...)                                                   \
  switch (dt) {                                                                          \
  case ::ttb::kF32: { using T = float; __VA_ARGS__; } break;                             \
  case ::ttb::kBF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;                    \
  case ::ttb::kF16: { using T = __half; __VA_ARGS__; } break;                            \
  case ::ttb::kI32: { using T = int32_t; __VA_ARGS__; } break;                           \
  case ::ttb::kU32: { using T = uint32_t; __VA_ARGS__; } break;                          \
  case ::ttb::kU16: { using T = uint16_t; __VA_ARGS__; } break;                          \
  case ::ttb::kU8: { using T = uint8_t; __VA_ARGS__; } break;                            \
  case ::ttb::kI8: { using T = int8_t; __VA_ARGS__; } break;                             \
  default: ::ttb::setLastError("unsupported dtype"); return TTB_ERR_UNSUPPORTED;         \
  }

#define TTB_DISPATCH_FLOAT(dt, T, ...)                                                   \
  switch (dt) {                                                                          \
  case ::ttb::kF32: { using T = float; __VA_ARGS__; } break;                             \
  case ::ttb::kBF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;                    \
  case ::ttb::kF16: { using T = __half; __VA_ARGS__; } break;                            \
  default: ::ttb::setLastError("unsupported float dtype"); return TTB_ERR_UNSUPPORTED;   \
  }

#define TTB_DISPATCH_INT(dt, T, ...)                                                     \
  switch (dt) {                                                                          \
  case ::ttb::kI32: { using T = int32_t; __VA_ARGS__; } break;                           \
  case ::ttb::kU32: { using T = uint32_t; __VA_ARGS__; } break;                          \
  case ::ttb::kU16: { using T = uint16_t; __VA_ARGS__; } break;                          \
  case ::ttb::kU8: { using T = uint8_t; __VA_ARGS__; } break;                            \
  case ::ttb::kI8: { using T = int8_t; __VA_ARGS__; } break;                             \
  default: ::ttb::setLastError("unsupported integer dtype"); return TTB_ERR_UNSUPPORTED; \
  }

} // namespace ttb
