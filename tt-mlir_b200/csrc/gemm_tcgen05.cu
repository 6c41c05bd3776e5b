// bf16 / f16 GEMM on the Blackwell tensor cores: C[M,N] = act(A[M,K] * B[N,K]^T + bias).
//
// This is the contraction behind ttnn.matmul / ttnn.linear / 1x1 and im2col'd conv2d for 16-bit
// operands (reference call sites: runtime/lib/ttnn/operations/matmul/matmul.cpp:75-80,117-122).
// Structure (one persistent CTA per SM, 192 threads, warp specialised):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of a 128 x 64 A tile and a BN x 64 B
//               tile per k-step into a ring of 128-byte-swizzled shared-memory stages
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16, f32 accumulate)
//               straight from shared-memory descriptors into TMEM; owns the TMEM allocation
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM lanes), add bias,
//               apply the activation / rounding points, stage 32 x 128 B blocks in shared
//               memory and write them out with TMA stores (full lines, tails clipped)
// The accumulator is double buffered in TMEM (2 x BN columns of the 512), so the epilogue of
// tile i overlaps the main loop of tile i+1.  Stages and accumulators are handed over through
// mbarriers; tcgen05.commit arrives on them when the MMAs that read a stage have retired.
// Every wait is bounded: on a timeout the CTA raises a status word, drains and exits instead
// of hanging the GPU.  No cluster launch and no multicast: every CTA fetches its own tiles.
#include "common.cuh"
#include "epilogue.cuh"
#include "tcgen05.cuh"

#include <cstdlib>

namespace ttb {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64; // 64 x 2 bytes = one 128-byte swizzle row
constexpr int TC_THREADS = 192;
constexpr int TC_TMEM_COLS = 512;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;
constexpr int TC_OUT_BYTES = 4 * 2 * 4096; // epilogue staging: 4 warps, double buffered, 32 rows x 128 B

template <int BN> struct TcCfg {
  static constexpr int kBBytes = BN * TC_BK * 2;
  static constexpr int kStageBytes = TC_A_BYTES + kBBytes;
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kSmem = kStages * kStageBytes + TC_OUT_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the
// 128-byte swizzle TMA applied: 8-row groups are 1024 bytes apart (stride byte offset), the
// leading byte offset is not used for this layout, descriptor version 1 (sm_100), layout type
// 2 (SWIZZLE_128B).  Stepping 16 elements along K inside the row adds 32 bytes to the start.
__device__ __forceinline__ uint64_t smemDesc(uint32_t addr) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

// kind::f16 instruction descriptor: f32 accumulator, A/B format (1 = bf16, 0 = f16), both
// operands K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instrDesc(int fmt, int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

template <typename TC> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<float>(float a, float) { return __float_as_uint(a); }

struct TcParams {
  int64_t M, N, K;
  const void *bias;
  int biasDt;
  int act;
  int roundSteps;
  const void *extra; // optional [M, N] operand in the output type, combined after bias / activation
  int extraOp;       // TTB_EXTRA_*
  int fmt; // 1 bf16, 0 f16
  int debug; // diagnostic: 1 = epilogue loads TMEM but skips math and stores, 2 = epilogue only hands the buffer back
};

template <int BN, typename TC, bool PLAIN>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemmTcgen05Kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                      const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapE,
                      TC *__restrict__ c, TcParams p) {
  using Cfg = TcCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smemRaw[];
  // 1024-byte alignment: required by the 128-byte swizzle pattern
  const uint32_t base = (smemU32(smemRaw) + 1023u) & ~1023u;
  const uint32_t outBase = base + STAGES * Cfg::kStageBytes; // 4 warps x 2 x 4 KB epilogue staging
  const uint32_t barBase = outBase + TC_OUT_BYTES;
  auto fullBar = [&](int s) { return barBase + 8u * s; };
  auto emptyBar = [&](int s) { return barBase + 8u * (STAGES + s); };
  auto tmemFullBar = [&](int a) { return barBase + 8u * (2 * STAGES + a); };
  auto tmemEmptyBar = [&](int a) { return barBase + 8u * (2 * STAGES + 2 + a); };
  __shared__ uint32_t tmemBaseSlot;
  __shared__ int abortFlagS;
  volatile int *abortFlag = &abortFlagS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tilesM = (p.M + TC_BM - 1) / TC_BM, tilesN = (p.N + BN - 1) / BN;
  const int64_t numTiles = tilesM * tilesN;
  const int kBlocks = static_cast<int>((p.K + TC_BK - 1) / TC_BK);

  if (threadIdx.x == 0) {
    abortFlagS = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbarInit(fullBar(s), 1);
      mbarInit(emptyBar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(tmemFullBar(a), 1);
      mbarInit(tmemEmptyBar(a), 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetchTensorMap(&mapA);
    prefetchTensorMap(&mapB);
    prefetchTensorMap(&mapC);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&tmemBaseSlot)), "r"(TC_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = tmemBaseSlot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < numTiles && alive; tile += gridDim.x) {
        const int m0 = static_cast<int>(tile % tilesM) * TC_BM, n0 = static_cast<int>(tile / tilesM) * BN;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1u;
          if (!mbarWait(emptyBar(s), phase ^ 1u, abortFlag, 1)) { alive = false; break; }
          const uint32_t sa = base + s * Cfg::kStageBytes, sb = sa + TC_A_BYTES;
          mbarArriveExpectTx(fullBar(s), Cfg::kStageBytes);
          tmaLoad2d(sa, &mapA, fullBar(s), kb * TC_BK, m0);
          tmaLoad2d(sb, &mapB, fullBar(s), kb * TC_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = instrDesc(p.fmt, TC_BM, BN);
      uint32_t it = 0, accIt = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < numTiles && alive; tile += gridDim.x, ++accIt) {
        const int acc = accIt & 1;
        const uint32_t accPhase = (accIt >> 1) & 1u;
        if (!mbarWait(tmemEmptyBar(acc), accPhase ^ 1u, abortFlag, 2)) break;
        tcFenceAfter();
        const uint32_t tmemD = tmemBase + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1u;
          if (!mbarWait(fullBar(s), phase, abortFlag, 3)) { alive = false; break; }
          tcFenceAfter();
          const uint32_t sa = base + s * Cfg::kStageBytes, sb = sa + TC_A_BYTES;
          const uint64_t da = smemDesc(sa), db = smemDesc(sb);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            // +32 bytes per 16-element k-step = +2 in the descriptor's 16-byte address units
            tcMma(tmemD, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tcCommit(emptyBar(s)); // frees the stage once these MMAs have read it
        }
        if (alive) tcCommit(tmemFullBar(acc)); // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 ----------------
    // Each warp owns 32 rows of the tile.  Per chunk of CH columns (one 128-byte output row
    // segment) it reads its TMEM lanes, applies the epilogue, writes the 32 x 128 B block to a
    // swizzled staging buffer and hands it to a TMA store, which writes full lines and clips
    // rows / columns that fall outside the matrix.  Two staging buffers per warp let the next
    // chunk be prepared while the previous store drains.
    constexpr int CH = 128 / static_cast<int>(sizeof(TC));
    constexpr int NLD = CH / 32;
    const int quarter = warp & 3; // TMEM lanes this warp may read
    const uint32_t stageOut = outBase + static_cast<uint32_t>(warp - 2) * 2u * 4096u;
    uint32_t accIt = 0, chunkIt = 0;
    // The extra operand is read row by row (one 128-byte segment per thread and chunk), which
    // would expose DRAM latency in every chunk.  Its 32-row x CH-column blocks are therefore
    // pulled into L2 one whole tile ahead: lanes 0 .. BN/CH-1 prefetch one block each.
    auto prefetchExtra = [&](int64_t t) {
      if constexpr (!PLAIN && sizeof(TC) == 2) {
        if (p.extraOp && lane < BN / CH && t < numTiles) {
          const int64_t col = (t / tilesM) * BN + lane * CH, row = (t % tilesM) * TC_BM + quarter * 32;
          if (col < p.N && row < p.M) {
            asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
                         ::"l"(reinterpret_cast<uint64_t>(&mapE)), "r"(static_cast<int>(col)), "r"(static_cast<int>(row)) : "memory");
          }
        }
      }
    };
    prefetchExtra(blockIdx.x);
    for (int64_t tile = blockIdx.x; tile < numTiles; tile += gridDim.x, ++accIt) {
      const int acc = accIt & 1;
      const uint32_t accPhase = (accIt >> 1) & 1u;
      prefetchExtra(tile + gridDim.x);
      if (!mbarWait(tmemFullBar(acc), accPhase, abortFlag, 4)) break;
      tcFenceAfter();
      const int64_t m0 = (tile % tilesM) * TC_BM, n0 = (tile / tilesM) * BN;
      const uint32_t taddrRow = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int cc = 0; cc < BN / CH; ++cc) {
        const int64_t col0 = n0 + cc * CH;
        if (col0 >= p.N || p.debug == 2) break; // warp-uniform
        // The extra operand's 128-byte row segment is fetched first so that it is in flight
        // while the accumulator is read.
        uint4 ev[sizeof(TC) == 2 && !PLAIN ? CH / 8 : 1] = {};
        if constexpr (!PLAIN && sizeof(TC) == 2) {
          if (p.extraOp && p.debug != 3) {
            const int64_t row = m0 + quarter * 32 + lane;
            const TC *erow = static_cast<const TC *>(p.extra) + row * p.N + col0;
#pragma unroll
            for (int g = 0; g < CH / 8; ++g) {
              ev[g] = (row < p.M && col0 + g * 8 < p.N) ? __ldg(reinterpret_cast<const uint4 *>(erow + g * 8))
                                                       : make_uint4(0, 0, 0, 0);
            }
          }
        }
        uint32_t r[CH];
#pragma unroll
        for (int l = 0; l < NLD; ++l) {
          tcLoad32(taddrRow + static_cast<uint32_t>(cc * CH + l * 32), *reinterpret_cast<uint32_t(*)[32]>(&r[l * 32]));
        }
        tcWaitLd();
        if (p.debug == 1) {
          if (r[0] == 0x7fc12345u && r[CH - 1] == 0x7fc54321u) c[0] = TC(0); // keeps the loads alive
          continue;
        }
        if constexpr (!PLAIN) {
          // Whole-chunk passes keep each activation's code in one straight run (a per-element
          // switch would interleave all of them and thrash the instruction cache).
          // bias of this chunk's columns: lane l holds columns l, l + 32, ...; broadcast by shuffle
          float biasReg[NLD];
#pragma unroll
          for (int l = 0; l < NLD; ++l) {
            const int64_t col = col0 + l * 32 + lane;
            biasReg[l] = (p.bias && col < p.N) ? loadBias(p.bias, p.biasDt, col) : 0.0f;
          }
          const bool hasBias = p.bias != nullptr, round1 = (p.roundSteps & 1) != 0, round2 = (p.roundSteps & 2) != 0;
#pragma unroll
          for (int e = 0; e < CH; ++e) {
            float f = __uint_as_float(r[e]);
            float bz = __shfl_sync(0xffffffffu, biasReg[e / 32], e & 31);
            if (round1) f = toF32(fromF32<TC>(f));
            if (hasBias) f = __fadd_rn(f, bz);
            if (hasBias && round2) f = toF32(fromF32<TC>(f));
            r[e] = __float_as_uint(f);
          }
          switch (p.act) {
          case TTB_ACT_RELU:
#pragma unroll
            for (int e = 0; e < CH; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(f > 0.0f ? f : (f != f ? f : 0.0f)); }
            break;
          case TTB_ACT_SILU:
#pragma unroll
            for (int e = 0; e < CH; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(f / (1.0f + expf(-f))); }
            break;
          case TTB_ACT_GELU:
#pragma unroll
            for (int e = 0; e < CH; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(applyAct(TTB_ACT_GELU, f)); }
            break;
          case TTB_ACT_SIGMOID:
#pragma unroll
            for (int e = 0; e < CH; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(1.0f / (1.0f + expf(-f))); }
            break;
          default: break;
          }
          if constexpr (sizeof(TC) == 2) {
            // A separate op consumed the (rounded) result of the chain so far.
            if (p.extraOp == TTB_EXTRA_ADD) {
#pragma unroll
              for (int e = 0; e < CH; ++e) {
                const TC *x = reinterpret_cast<const TC *>(&ev[e / 8]) + (e & 7);
                r[e] = __float_as_uint(__fadd_rn(toF32(fromF32<TC>(__uint_as_float(r[e]))), toF32(*x)));
              }
            } else if (p.extraOp == TTB_EXTRA_SILU_MUL) {
#pragma unroll
              for (int e = 0; e < CH; ++e) {
                const TC *x = reinterpret_cast<const TC *>(&ev[e / 8]) + (e & 7);
                const float g = toF32(*x);
                const float sg = toF32(fromF32<TC>(__fdividef(g, 1.0f + __expf(-g))));
                r[e] = __float_as_uint(__fmul_rn(sg, toF32(fromF32<TC>(__uint_as_float(r[e])))));
              }
            }
          }
        }
        const uint32_t buf = stageOut + (chunkIt & 1u) * 4096u;
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); // buffer free again
        __syncwarp();
        const uint32_t rowAddr = buf + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
        for (int v = 0; v < 8; ++v) { // eight 16-byte pieces of this lane's 128-byte row
          uint32_t w[4];
          if constexpr (sizeof(TC) == 2) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int e = v * 8 + q * 2;
              float f0 = __uint_as_float(r[e]), f1 = __uint_as_float(r[e + 1]);
              w[q] = pack2<TC>(f0, f1); // one cvt.rn for the pair
            }
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int e = v * 4 + q;
              float f0 = __uint_as_float(r[e]);
              w[q] = __float_as_uint(f0);
            }
          }
          // 128-byte swizzle (what the tensor map of C expects): 16-byte piece v of row `lane`
          // lives at piece v ^ (lane % 8); this also spreads the lanes over the banks
          const uint32_t addr = rowAddr + (static_cast<uint32_t>(v ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                       ::"l"(reinterpret_cast<uint64_t>(&mapC)), "r"(buf), "r"(static_cast<int>(col0)),
                         "r"(static_cast<int>(m0 + quarter * 32)) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        ++chunkIt;
      }
      tcFenceBefore();
      mbarArrive(tmemEmptyBar(acc)); // all 128 epilogue threads arrive: the accumulator may be overwritten
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); // stores done before smem goes away
  }

  // ---------------- teardown ----------------
  if (*abortFlag) {
    // give bulk copies that may still be in flight time to land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) { __nanosleep(1000); }
  }
  tcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcFenceAfter();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(TC_TMEM_COLS) : "memory");
  }
}

} // namespace ttb

// ---- host side ------------------------------------------------------------------------------
namespace ttb {

// The driver entry point is looked up through the runtime so that the library does not link libcuda.
EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return static_cast<EncodeTiledFn>(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Row-major [rows, cols] matrix, box = boxCols x boxRows (boxCols spans 128 bytes), 128-byte
// swizzle; out-of-bounds elements read as zero and are not written, which is what makes ragged
// M / N / K tails work.
static bool makeMap(CUtensorMap *map, const void *ptr, int dtype, int64_t rows, int64_t cols, int boxRows) {
  EncodeTiledFn fn = encodeTiled();
  if (!fn) return false;
  size_t es = dtypeSize(dtype);
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * es};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(boxRows)};
  cuuint32_t elemStrides[2] = {1, 1};
  CUtensorMapDataType dt = dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : (dtype == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
  CUresult r = fn(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, typename TC, bool PLAIN>
static int launchTc(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc, const CUtensorMap &me, void *c, const TcParams &p,
                    cudaStream_t st) {
  using Cfg = TcCfg<BN>;
  // Function attributes belong to a device: set the shared-memory limit once on each.
  static bool attrSet[64] = {};
  int dev = 0;
  TTB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attrSet[dev]) {
    TTB_CUDA(cudaFuncSetAttribute(gemmTcgen05Kernel<BN, TC, PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
    attrSet[dev] = true;
  }
  int64_t tiles = ((p.M + TC_BM - 1) / TC_BM) * ((p.N + BN - 1) / BN);
  int grid = static_cast<int>(tiles < smCount() ? tiles : smCount());
  gemmTcgen05Kernel<BN, TC, PLAIN><<<grid, TC_THREADS, Cfg::kSmem, st>>>(ma, mb, mc, me, static_cast<TC *>(c), p);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int gemmTcgen05Try(const void *a, const void *b, const void *bias, void *c, int abDtype, int biasDtype, int cDtype,
                   int64_t batch, int64_t m, int64_t n, int64_t k, int transA, int transB, int64_t, int64_t, int act,
                   int roundSteps, const void *extra, int extraOp, cudaStream_t stream) {
  // What this kernel takes: one 16-bit A[M,K] and B[N,K] (the "transpose_b" weight layout),
  // rows 16-byte aligned, output in a 16- or 32-bit float type.
  if (batch != 1 || transA || !transB) return -1;
  if (abDtype != kBF16 && abDtype != kF16) return -1;
  if (cDtype != abDtype && cDtype != kF32) return -1;
  if (k % 8 != 0 || m < 1 || n < 8 || k < 8) return -1;
  if ((n * static_cast<int64_t>(dtypeSize(cDtype))) % 16 != 0) return -1; // row pitch of C for the TMA store
  if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return -1;
  if (extraOp && (!extra || cDtype == kF32 || !aligned16(extra))) return -1;
  if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return -1;
  // Tiny problems are launch-bound either way; keep them on the simple kernel.
  if (m * n * k < (1ll << 18)) return -1;
  // Tile width: fewest (waves x per-tile cost); the +64 stands for the A tile every CTA loads
  // whatever its width, which makes narrow tiles less efficient per column.
  int bn = 64;
  {
    int64_t best = -1;
    for (int w : {256, 128, 64}) {
      if (w > 64 && n < w) continue;
      int64_t tiles = ((m + TC_BM - 1) / TC_BM) * ((n + w - 1) / w);
      int64_t waves = (tiles + smCount() - 1) / smCount();
      int64_t cost = waves * (w + 64);
      if (best < 0 || cost < best) {
        best = cost;
        bn = w;
      }
    }
  }
  CUtensorMap ma, mb, mc, me;
  if (!makeMap(&ma, a, abDtype, m, k, TC_BM) || !makeMap(&mb, b, abDtype, n, k, bn) ||
      !makeMap(&mc, c, cDtype, m, n, 32))
    return -1;
  if (extraOp) {
    if (!makeMap(&me, extra, cDtype, m, n, 32)) return -1;
  } else {
    me = mc; // not used
  }
  TcParams p;
  p.M = m; p.N = n; p.K = k;
  p.bias = bias; p.biasDt = biasDtype; p.act = act; p.roundSteps = roundSteps;
  p.extra = extraOp ? extra : nullptr;
  p.extraOp = extra ? extraOp : 0;
  p.fmt = abDtype == kBF16 ? 1 : 0;
  {
    const char *dbg = std::getenv("TTB_TC_DEBUG");
    p.debug = dbg ? std::atoi(dbg) : 0;
  }
  double flops = 2.0 * double(m) * double(n) * double(k);
  double bytes = (double(m) * k + double(n) * k) * 2 + double(m) * n * dtypeSize(cDtype) * (extraOp ? 2 : 1);
  ProfScope prof("gemm_tcgen05", flops, bytes, stream);
  const bool plain = !bias && act == TTB_ACT_NONE && roundSteps == 0 && !extraOp;
#define TTB_TC(BNv, TCv)                                                                 \
  return plain ? launchTc<BNv, TCv, true>(ma, mb, mc, me, c, p, stream) : launchTc<BNv, TCv, false>(ma, mb, mc, me, c, p, stream)
#define TTB_TC_BN(TCv)                                                                   \
  switch (bn) {                                                                          \
  case 256: TTB_TC(256, TCv);                                                            \
  case 128: TTB_TC(128, TCv);                                                            \
  default: TTB_TC(64, TCv);                                                              \
  }
  if (cDtype == kBF16) { TTB_TC_BN(__nv_bfloat16) }
  if (cDtype == kF16) { TTB_TC_BN(__half) }
  TTB_TC_BN(float)
#undef TTB_TC_BN
#undef TTB_TC
}

} // namespace ttb

// 0 when no tensor-core GEMM launch of this process has hit a wait timeout; otherwise
// (role << 8) | 1 with role 1 = loader, 2 / 3 = MMA issuer, 4 = epilogue.  Synchronises the device.
extern "C" int ttb_gemm_tcgen05_status(int *status) {
  TTB_CHECK(status != nullptr, "status is null");
  TTB_CUDA(cudaDeviceSynchronize());
  TTB_CUDA(cudaMemcpyFromSymbol(status, ttb::g_tcStatus, sizeof(int)));
  return TTB_OK;
}
