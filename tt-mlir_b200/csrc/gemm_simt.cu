// General matmul / linear on CUDA cores: any shape, any transpose, f32 / bf16 / f16 operands,
// f32 FFMA accumulation in ascending-k order.  It serves (a) f32 graphs, where the tensor
// cores' TF32 path cannot meet the 1e-4 tolerance against the reference's f32 CPU matmul
// (tosa.matmul with f32 accumulation, lib/Conversion/TTIRToLinalg/TTIRToLinalg.cpp:542-549),
// (b) shapes the tcgen05 kernel does not take, and (c) as the in-library cross-check of the
// tensor-core kernel.  64x64 tile per 256-thread block, 4x4 outputs per thread, k-step 16.
// Problems with few output tiles and a long K (the f32 MLP layers: 8 tiles, K = 784) are split
// along K over gridDim.z: every block writes its partial tile to a scratch buffer, and the block
// that arrives last at a tile adds the partials in split order (the same order every run) and
// applies the epilogue.
#include "common.cuh"
#include "epilogue.cuh"

namespace ttb {

constexpr int BM = 64, BN = 64, BK = 16;

namespace {
thread_local void *t_scratchPtr = nullptr;
thread_local size_t t_scratchBytes = 0;
thread_local bool t_scratchActive = false;
} // namespace

GemmScratchScope::GemmScratchScope(void *ptr, size_t bytes) {
  t_scratchPtr = ptr;
  t_scratchBytes = bytes;
  t_scratchActive = true;
}
GemmScratchScope::~GemmScratchScope() {
  t_scratchActive = false;
  t_scratchPtr = nullptr;
  t_scratchBytes = 0;
}
bool GemmScratchScope::current(void **ptr, size_t *bytes) {
  if (!t_scratchActive) return false;
  *ptr = t_scratchPtr;
  *bytes = t_scratchBytes;
  return true;
}

template <typename T, typename TC>
__global__ void __launch_bounds__(256)
    gemmSimtKernel(const T *__restrict__ a, const T *__restrict__ b, const void *__restrict__ bias, int biasDt,
                   TC *__restrict__ c, int64_t M, int64_t N, int64_t K, int64_t asM, int64_t asK, int64_t bsK,
                   int64_t bsN, int64_t aBatch, int64_t bBatch, int act, int roundSteps, int splitK, int64_t kPer,
                   float *__restrict__ partials, unsigned *__restrict__ arrivals) {
  __shared__ float sa[BK][BM + 1];
  __shared__ float sb[BK][BN + 1];
  __shared__ bool lastBlock;
  pdlLaunchDependents();
  pdlWait();
  const int split = splitK > 1 ? static_cast<int>(blockIdx.z) : 0;
  int64_t batch = splitK > 1 ? 0 : blockIdx.z;
  const T *A = a + batch * aBatch;
  const T *B = b + batch * bBatch;
  TC *C = c + batch * M * N;
  int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
  int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  const int64_t kBegin = splitK > 1 ? split * kPer : 0;
  const int64_t kEnd = splitK > 1 ? (kBegin + kPer < K ? kBegin + kPer : K) : K;
  // Register prefetch: the global loads of k-step i+1 are issued before the products of k-step
  // i, so their latency overlaps the arithmetic (each thread holds 4 + 4 operand values).
  // The element a thread fetches: index i = threadIdx.x + 256 j, laid out so that the
  // fastest-varying thread index follows the contiguous global dimension of each operand.
  int aM[4], aK[4], bN[4], bK[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + 256 * j;
    if (asK == 1) { aK[j] = i % BK; aM[j] = i / BK; } else { aM[j] = i % BM; aK[j] = i / BM; }
    if (bsN == 1) { bN[j] = i % BN; bK[j] = i / BN; } else { bK[j] = i % BK; bN[j] = i / BK; }
  }
  float ra[4], rb[4];
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gm = m0 + aM[j], gka = k0 + aK[j], gn = n0 + bN[j], gkb = k0 + bK[j];
      ra[j] = (gm < M && gka < kEnd) ? toF32(A[gm * asM + gka * asK]) : 0.0f;
      rb[j] = (gn < N && gkb < kEnd) ? toF32(B[gkb * bsK + gn * bsN]) : 0.0f;
    }
  };
  if (kBegin < kEnd) fetch(kBegin);
  for (int64_t k0 = kBegin; k0 < kEnd; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sa[aK[j]][aM[j]] = ra[j];
      sb[bK[j]][bN[j]] = rb[j];
    }
    __syncthreads();
    if (k0 + BK < kEnd) fetch(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  if (splitK > 1) {
    const size_t tile = static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x;
    float *mine = partials + (tile * splitK + split) * (BM * BN);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) mine[(i * 4 + j) * 256 + threadIdx.x] = acc[i][j];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) lastBlock = atomicAdd(&arrivals[tile], 1u) == static_cast<unsigned>(splitK - 1);
    __syncthreads();
    if (!lastBlock) return;
    __threadfence();
    // Every element is summed in split order, but the loads of four splits (64 per thread) are
    // in flight together: one element at a time, the loop would pay an L2 round trip per load.
    const float *all = partials + tile * splitK * (BM * BN) + threadIdx.x;
    float sum[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) sum[e] = 0.0f;
    for (int sp = 0; sp < splitK; sp += 4) {
      float v[4][16];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (sp + u < splitK) {
#pragma unroll
          for (int e = 0; e < 16; ++e) v[u][e] = __ldcg(all + (sp + u) * (BM * BN) + e * 256);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (sp + u < splitK) {
#pragma unroll
          for (int e = 0; e < 16; ++e) sum[e] += v[u][e];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = sum[i * 4 + j];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float bz = bias ? loadBias(bias, biasDt, gn) : 0.0f;
      C[gm * N + gn] = epilogue<TC>(acc[i][j], bias != nullptr, bz, act, roundSteps);
    }
  }
}

template <typename T, typename TC>
static int launchSimt(const void *a, const void *b, const void *bias, int biasDt, void *c, int64_t batch, int64_t m,
                      int64_t n, int64_t k, int ta, int tb, int64_t aBatch, int64_t bBatch, int act, int roundSteps,
                      cudaStream_t st) {
  const int64_t tilesN = (n + BN - 1) / BN, tilesM = (m + BM - 1) / BM;
  int64_t asM = ta ? 1 : k, asK = ta ? m : 1;
  int64_t bsK = tb ? 1 : n, bsN = tb ? k : 1;
  // Split K when the tiles alone leave most SMs idle and each split still has a few k-steps.
  int splitK = 1;
  if (batch == 1 && tilesM * tilesN * 2 <= smCount() && k >= 8 * BK) {
    int64_t want = smCount() / (tilesM * tilesN);
    int64_t most = k / (2 * BK);
    splitK = static_cast<int>(want < most ? want : most);
    if (splitK > 32) splitK = 32;
    if (splitK < 2) splitK = 1;
  }
  int64_t kPer = k;
  float *partials = nullptr;
  unsigned *arrivals = nullptr;
  void *scratch = nullptr;
  if (splitK > 1) {
    kPer = ((k + splitK - 1) / splitK + BK - 1) / BK * BK;
    splitK = static_cast<int>((k + kPer - 1) / kPer);
  }
  bool ownScratch = false;
  if (splitK > 1) {
    const size_t counters = (static_cast<size_t>(tilesM * tilesN) * sizeof(unsigned) + 255) / 256 * 256;
    const size_t bytes = counters + static_cast<size_t>(tilesM * tilesN) * splitK * BM * BN * sizeof(float);
    void *given = nullptr;
    size_t givenBytes = 0;
    if (GemmScratchScope::current(&given, &givenBytes)) {
      // the caller forbids allocation: its buffer, or no split at all
      if (given && givenBytes >= bytes) {
        scratch = given;
      } else {
        splitK = 1;
        kPer = k;
      }
    } else {
      int rc = ttb_malloc(&scratch, bytes, st);
      if (rc) return rc;
      ownScratch = true;
    }
    if (scratch) {
      TTB_CUDA(cudaMemsetAsync(scratch, 0, counters, st));
      arrivals = static_cast<unsigned *>(scratch);
      partials = reinterpret_cast<float *>(static_cast<char *>(scratch) + counters);
    }
  }
  dim3 grid(static_cast<unsigned>(tilesN), static_cast<unsigned>(tilesM), static_cast<unsigned>(splitK > 1 ? splitK : batch));
  {
    ProfScope prof("gemm_simt", 2.0 * double(batch) * m * n * k, double(batch) * (double(m) * k + double(n) * k) * sizeof(T) + double(batch) * m * n * sizeof(TC), st);
    TTB_CUDA(launchPdl(gemmSimtKernel<T, TC>, grid, dim3(256), 0, st, static_cast<const T *>(a), static_cast<const T *>(b), bias,
                       biasDt, static_cast<TC *>(c), m, n, k, asM, asK, bsK, bsN, aBatch, bBatch, act, roundSteps, splitK, kPer,
                       partials, arrivals));
  }
  if (ownScratch) {
    int rc = ttb_free(scratch, st); // stream-ordered: released once the kernel has run
    if (rc) return rc;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // namespace ttb

using namespace ttb;

extern "C" int ttb_gemm_simt(const void *a, const void *b, const void *bias, void *c, int ab_dtype, int bias_dtype,
                             int c_dtype, int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                             int64_t a_batch_stride, int64_t b_batch_stride, int act, int round_steps,
                             void *stream) {
  TTB_CHECK(a && b && c, "null tensor");
  TTB_CHECK(batch >= 0 && m >= 0 && n >= 0 && k >= 0, "negative dimension");
  TTB_CHECK(batch <= 65535 && (m + BM - 1) / BM <= 65535, "grid too large");
  if (batch * m * n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
#define TTB_SIMT(T, TC) return launchSimt<T, TC>(a, b, bias, bias_dtype, c, batch, m, n, k, trans_a, trans_b, a_batch_stride, b_batch_stride, act, round_steps, st)
  if (ab_dtype == kF32 && c_dtype == kF32) TTB_SIMT(float, float);
  if (ab_dtype == kBF16 && c_dtype == kBF16) TTB_SIMT(__nv_bfloat16, __nv_bfloat16);
  if (ab_dtype == kBF16 && c_dtype == kF32) TTB_SIMT(__nv_bfloat16, float);
  if (ab_dtype == kF16 && c_dtype == kF16) TTB_SIMT(__half, __half);
  if (ab_dtype == kF16 && c_dtype == kF32) TTB_SIMT(__half, float);
  if (ab_dtype == kF32 && c_dtype == kBF16) TTB_SIMT(float, __nv_bfloat16);
#undef TTB_SIMT
  setLastError("gemm: unsupported dtype combination");
  return TTB_ERR_UNSUPPORTED;
}
