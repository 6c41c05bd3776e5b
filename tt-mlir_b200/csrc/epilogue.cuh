// Epilogue shared by the SIMT and tcgen05 GEMM kernels: bias, activation and the rounding
// points that make a fused launch equal to the unfused op chain it replaces.
#pragma once

#include "common.cuh"

namespace ttb {

__device__ __forceinline__ float loadBias(const void *bias, int dt, int64_t i) {
  switch (dt) {
  case kF32: return static_cast<const float *>(bias)[i];
  case kBF16: return __bfloat162float(static_cast<const __nv_bfloat16 *>(bias)[i]);
  case kF16: return __half2float(static_cast<const __half *>(bias)[i]);
  default: return 0.0f;
  }
}

__device__ __forceinline__ float applyAct(int act, float x) {
  switch (act) {
  case TTB_ACT_RELU: return x > 0.0f ? x : (x != x ? x : 0.0f);
  case TTB_ACT_SILU: return x / (1.0f + expf(-x));
  case TTB_ACT_GELU: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
  case TTB_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
  default: return x;
  }
}

// roundSteps bit 0: round to TC after the product (a separate matmul op wrote its result);
// bit 1: round after the bias add (a separate add op wrote its result).
template <typename TC>
__device__ __forceinline__ TC epilogue(float acc, bool hasBias, float bias, int act, int roundSteps) {
  if (roundSteps & 1) acc = toF32(fromF32<TC>(acc));
  if (hasBias) {
    acc = __fadd_rn(acc, bias);
    if (roundSteps & 2) acc = toF32(fromF32<TC>(acc));
  }
  if (act) acc = applyAct(act, acc);
  return fromF32<TC>(acc);
}

// Same rounding points, result left in f32 (the caller rounds pairs with one packed convert).
template <typename TC>
__device__ __forceinline__ float epilogueF32(float acc, bool hasBias, float bias, int act, int roundSteps) {
  if (roundSteps & 1) acc = toF32(fromF32<TC>(acc));
  if (hasBias) {
    acc = __fadd_rn(acc, bias);
    if (roundSteps & 2) acc = toF32(fromF32<TC>(acc));
  }
  if (act) acc = applyAct(act, acc);
  return acc;
}

} // namespace ttb
