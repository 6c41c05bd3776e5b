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
//               memory (two buffers per warp) and write them out with TMA stores (full lines,
//               tails clipped); kernels with a non-trivial epilogue run warps 2..9 in two groups
// The accumulator is double buffered in TMEM (2 x BN columns of the 512), so the epilogue of
// tile i overlaps the main loop of tile i+1.  Stages and accumulators are handed over through
// mbarriers; tcgen05.commit arrives on them when the MMAs that read a stage have retired.
// Every wait is bounded: on a timeout the CTA raises a status word, drains and exits instead
// of hanging the GPU.  No cluster launch and no multicast: every CTA fetches its own tiles.
#include "common.cuh"
#include "epilogue.cuh"
#include "tcgen05.cuh"

#include <cstdlib>
#include <type_traits>

namespace ttb {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64; // 64 x 2 bytes = one 128-byte swizzle row
constexpr int TC_THREADS = 192;      // producer warp, MMA warp, four epilogue warps
constexpr int TC_THREADS_EPI8 = 320; // eight epilogue warps (kernels with a non-trivial epilogue)
constexpr int TC_TMEM_COLS = 512;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;
constexpr int TC_SMEM_LIMIT = 227 * 1024; // dynamic shared memory a CTA may have

// PAIR: two CTAs of a cluster share one 256 x BN tile (tcgen05 cta_group::2): each holds 128 rows of A and
// BN / 2 rows of B per stage, so a stage is smaller and more of them fit.
// Epilogue staging: two 32-row x 128-byte buffers per epilogue warp (four warps in the plain kernel, eight
// otherwise), so that a warp fills one while the TMA store of the other is still reading it; the operand ring
// gets the stages that fit beside it (at most eight).
template <int BN, bool PAIR = false, bool PLAIN = true> struct TcCfg {
  static constexpr int kBRows = PAIR ? BN / 2 : BN;
  static constexpr int kBBytes = kBRows * TC_BK * 2;
  static constexpr int kStageBytes = TC_A_BYTES + kBBytes;
  static constexpr int kOutBytes = (PLAIN ? 4 : 8) * 2 * 4096;
  static constexpr int kFixed = kOutBytes + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int kFit = (TC_SMEM_LIMIT - kFixed) / kStageBytes;
  static constexpr int kStages = kFit > 8 ? 8 : kFit;
  static constexpr int kSmem = kStages * kStageBytes + kFixed;
  static_assert(kStages >= 3, "operand ring too short");
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

// relu on a packed pair (NaN stays NaN); relu commutes with the rounding before it.
template <typename TC> __device__ __forceinline__ uint32_t relu2(uint32_t v);
template <> __device__ __forceinline__ uint32_t relu2<__nv_bfloat16>(uint32_t v) {
  __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162 *>(&v);
  x = __hmax2_nan(x, __floats2bfloat162_rn(0.0f, 0.0f));
  return *reinterpret_cast<uint32_t *>(&x);
}
template <> __device__ __forceinline__ uint32_t relu2<__half>(uint32_t v) {
  __half2 x = *reinterpret_cast<__half2 *>(&v);
  x = __hmax2_nan(x, __floats2half2_rn(0.0f, 0.0f));
  return *reinterpret_cast<uint32_t *>(&x);
}
template <> __device__ __forceinline__ uint32_t relu2<float>(uint32_t v) { return v; }

// A row segment of 32 bias values in the 16-bit output type, fetched as four 16-byte loads from the same address in
// every lane (one broadcast transaction each) instead of one value per lane handed round with 32 shuffles: the
// shuffle unit takes one warp instruction per cycle per SM, which made it the busiest unit of the short-reduction
// epilogues.  Element e is converted where it is used.
template <typename TC> struct BiasRow {
  uint4 raw[4];
  __device__ __forceinline__ void load(const void *bias, int64_t col) {
    const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const TC *>(bias) + col);
#pragma unroll
    for (int v = 0; v < 4; ++v) raw[v] = __ldg(p + v);
  }
  __device__ __forceinline__ float at(int e) const {
    const uint32_t w = reinterpret_cast<const uint32_t *>(raw)[e >> 1];
    if constexpr (sizeof(TC) == 2 && std::is_same<TC, __nv_bfloat16>::value) {
      return __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
    } else {
      const __half2 h = *reinterpret_cast<const __half2 *>(&w);
      return (e & 1) ? __high2float(h) : __low2float(h);
    }
  }
};

struct TcParams {
  int64_t M, N, K;
  const void *bias;
  int biasDt;
  int act;
  int roundSteps;
  // Grouped launch: up to three problems that share A, M and K run as one tile list; n-tile
  // indices [segCum[i-1], segCum[i]) belong to problem i, whose width is segN[i] (B and C maps
  // mapB/mapC, mapB1/mapC1, mapB2/mapC2).  An ordinary launch is one segment.
  int segCum[3];
  int64_t segN[3];
  // Push mode (the GEMM that feeds an all-reduce over peer memory): row block [o * pushRows,
  // (o + 1) * pushRows) of C is stored through pushMaps.m[o], a [pushRows, N] matrix in rank o's
  // workspace, instead of through mapC.  pushRows is a multiple of the tile height; 0 = off.
  int pushRows;
  // SwiGLU mode (BN = 256 only): the B tile of a stage is 128 rows of the gate weights (mapB) on
  // top of the matching 128 rows of the up weights (mapB1), so accumulator columns 0..127 hold the
  // gate projection and 128..255 the up projection of the same 128 output columns; the epilogue
  // stores silu(gate) * up, rounding where the chain of separate ops rounds.  N counts output columns.
  int dual;
  const void *extra; // optional [M, N] operand in the output type, combined after bias / activation
  int extraOp;       // TTB_EXTRA_*
  // Implicit-GEMM convolution: A is not a matrix in memory but the receptive fields of an NHWC
  // tensor; row p of A is output pixel p, k-block kb is channels [64*(kb % cb), +64) of filter tap
  // kb / cb, cb = C / 64.  convX null = plain GEMM.
  const void *convX;
  int cH, cW, cC, cHo, cWo, ckw, csh, csw, cpt, cpl, cdh, cdw;
  // Patch mode (stride-1 convolutions): a tile's 128 rows are a cTw x 128/cTw patch of output
  // pixels of one image, which makes the A tile of a filter tap one 4-D TMA box of the input
  // (zero fill outside the image = the padding) and the C tile a 4-D TMA box of the output.
  // cTw = 0: rows are 128 consecutive pixels and the producer warp gathers them with cp.async.
  int cTw, cTilesX, cTilesY;
  int64_t cTilesM; // images x cTilesY x cTilesX
  int fmt; // 1 bf16, 0 f16, 2 8-bit integers (kind::i8, 32-bit integer accumulator)
  int kElems; // elements in the 128 bytes of a k-block: 64 for 16-bit operands, 128 for 8-bit
  int aSigned, bSigned; // fmt 2: signedness of the operands
  // fmt 2 with a float output: the accumulator is converted to f32 and multiplied by a scale (the
  // dequantize op that follows a quantized contraction: per tensor, or per output column).
  int deq;               // 0 off (the integer accumulator is stored), 1 scalar, 2 per column
  float deqScalar;
  const float *deqScale; // [N] f32
  // Rotary embedding in the epilogue (plain 16-bit launches, BN >= 128): the columns of segment i (bit i of
  // ropeMask) are heads of 128 values; the product is rounded to the output type, as the separate linear op
  // stores it, and then rotated as rotary_embedding does: out = x cos + rotate_half(x) sin with the tables
  // ropeCos / ropeSin [ropeSeq, 128] in the output type and position = row mod ropeSeq.
  int ropeMask = 0;
  int ropeSeq = 1;
  const void *ropeCos = nullptr, *ropeSin = nullptr;
  // Two products into one result (BN <= 128, 16-bit output): C = act(round(A B^T + bias) + round(A2 B2^T + bias2)) --
  // a convolution and the projection convolution of its residual branch, each rounded as its own op rounds it, the sum
  // rounded as the add that follows them.  A2 [M, K2] comes through mapE, B2 [N, K2] through mapB1; a tile's k-blocks
  // are those of the first product followed by those of the second, which accumulates BN columns further on in TMEM.
  int dualA = 0;
  int64_t K2 = 0;
  const void *bias2 = nullptr;
  int bias2Dt = 0;
  // The biases are in the output's 16-bit type and 16-byte aligned: their values are fetched as broadcast vectors
  // (set by the launcher).
  int biasVec = 0;
};

struct PushMaps {
  CUtensorMap m[8];
};

template <int BN, typename TC, bool PLAIN, bool PAIR, bool I8, bool DUALA>
__global__ void __launch_bounds__(PLAIN ? TC_THREADS : TC_THREADS_EPI8, 1)
    gemmTcgen05Kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                      const __grid_constant__ CUtensorMap mapC, const __grid_constant__ CUtensorMap mapE,
                      const __grid_constant__ CUtensorMap mapB1, const __grid_constant__ CUtensorMap mapC1,
                      const __grid_constant__ CUtensorMap mapB2, const __grid_constant__ CUtensorMap mapC2,
                      const __grid_constant__ PushMaps pushMaps, TC *__restrict__ c, TcParams p) {
  using Cfg = TcCfg<BN, PAIR, PLAIN>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int TILE_M = PAIR ? 2 * TC_BM : TC_BM; // rows of C per tile (per CTA always TC_BM)
  extern __shared__ uint8_t smemRaw[];
  // 1024-byte alignment: required by the 128-byte swizzle pattern
  const uint32_t base = (smemU32(smemRaw) + 1023u) & ~1023u;
  const uint32_t outBase = base + STAGES * Cfg::kStageBytes; // 4 warps x 2 x 4 KB epilogue staging
  const uint32_t barBase = outBase + Cfg::kOutBytes;
  auto fullBar = [&](int s) { return barBase + 8u * s; };
  auto emptyBar = [&](int s) { return barBase + 8u * (STAGES + s); };
  auto tmemFullBar = [&](int a) { return barBase + 8u * (2 * STAGES + a); };
  auto tmemEmptyBar = [&](int a) { return barBase + 8u * (2 * STAGES + 2 + a); };
  auto extraBar = [&](int w) { return barBase + 8u * (2 * STAGES + 4 + w); }; // one per epilogue warp
  __shared__ uint32_t tmemBaseSlot;
  __shared__ int abortFlagS;
  volatile int *abortFlag = &abortFlagS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A pair works through the tile list as one worker; rank 0 of the pair issues the MMAs.
  const uint32_t ctaRank = PAIR ? clusterCtaRank() : 0u;
  const bool leader = ctaRank == 0;
  const int64_t worker = PAIR ? blockIdx.x / 2 : blockIdx.x, workers = PAIR ? gridDim.x / 2 : gridDim.x;
  const int64_t tilesM = p.cTw ? p.cTilesM : (p.M + TILE_M - 1) / TILE_M, tilesN = p.segCum[2];
  const int64_t numTiles = tilesM * tilesN;
  // n-tile index -> (segment, first column inside the segment)
  auto segmentOf = [&](int64_t nt, int &n0) {
    const int seg = nt < p.segCum[0] ? 0 : (nt < p.segCum[1] ? 1 : 2);
    n0 = static_cast<int>(nt - (seg == 0 ? 0 : p.segCum[seg - 1])) * (p.dual ? BN / 2 : BN);
    return seg;
  };
  // Elements in the 128 bytes of a k-block.  The 8-bit integer form is a template parameter, not a launch parameter: as
  // runtime branches, its issue path and its dequantizing epilogue cost the 16-bit kernels 12 % (measured).
  constexpr int K_ELEMS = I8 ? 128 : TC_BK; // (the two-product mode, DUALA, is a template parameter for the same reason: 1-2 %)
  const int kBlocks1 = static_cast<int>((p.K + K_ELEMS - 1) / K_ELEMS);
  const int kBlocks = kBlocks1 + (DUALA ? static_cast<int>((p.K2 + K_ELEMS - 1) / K_ELEMS) : 0);
  const uint32_t accCols = DUALA ? 2u * BN : static_cast<uint32_t>(BN); // TMEM columns of one accumulator buffer

  if (threadIdx.x == 0) {
    abortFlagS = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbarInit(fullBar(s), (p.convX && !p.cTw) ? 2 : 1); // gathering convolution: the weights' TMA and the pixels arrive separately
      mbarInit(emptyBar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(tmemFullBar(a), 1);
      mbarInit(tmemEmptyBar(a), PAIR ? 256 : 128); // pair: the epilogue threads of both CTAs arrive at rank 0's barrier
    }
    for (int w = 0; w < 8; ++w) mbarInit(extraBar(w), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetchTensorMap(&mapA);
    prefetchTensorMap(&mapB);
    prefetchTensorMap(&mapC);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&tmemBaseSlot)), "r"(TC_TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&tmemBaseSlot)), "r"(TC_TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  // Pair: neither CTA may signal the other's barriers before both have initialised them.
  if constexpr (PAIR) clusterSync();
  const uint32_t tmemBase = tmemBaseSlot;
  // Everything above touched only this CTA's shared memory, TMEM and the kernel parameters, so it
  // may run while the kernel before this one on the stream is still finishing; from here on
  // global memory is read and written.
  pdlLaunchDependents();
  pdlWait();

  if (warp == 0 && p.convX && !p.cTw) {
    // ---------------- convolution producer: the whole warp gathers A, lane 0 also loads B ----------------
    // One cp.async instruction of the warp copies four tile rows: eight consecutive lanes fetch
    // the eight 16-byte pieces of one pixel's 64 channels (one full 128-byte line), zero-filled
    // outside the image, to where the 128-byte swizzle of the operand layout puts them.  Per tile
    // every lane keeps, for its 32 (row, piece) slots, the element offset of the pixel at tap
    // (0, 0) and that pixel's coordinates; a k-block then costs a few integer operations per copy.
    // Up to kInFlight stages of copies are in flight; a stage is handed to the MMA warp when its
    // copies have landed and are visible to the async proxy.
    constexpr int kInFlight = STAGES > 3 ? 3 : STAGES - 1; // fewer than there are stages: a stage is handed over before its slot comes round again
    const uint16_t *x = static_cast<const uint16_t *>(p.convX);
    const int cb = p.cC / TC_BK;
    const int piece = lane & 7, rowInGroup = lane >> 3;
    uint32_t it = 0, handed = 0;
    bool alive = true;
    auto hand = [&](uint32_t item) { // copies of `item` are complete
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbarArrive(fullBar(item % STAGES));
    };
    for (int64_t tile = worker; tile < numTiles && alive; tile += workers) {
      const int64_t m0 = (tile % tilesM) * TC_BM;
      int n0;
      (void)segmentOf(tile / tilesM, n0);
      int off[32];      // element offset of (pixel at tap 0, piece), or of x itself for rows past the end
      uint32_t yx[32];  // (y0 + 0x4000) << 16 | (x0 + 0x4000); rows past the end get coordinates that never pass
#pragma unroll
      for (int q = 0; q < 32; ++q) {
        const int64_t pix = m0 + q * 4 + rowInGroup;
        if (pix < p.M) {
          const int64_t img = pix / (static_cast<int64_t>(p.cHo) * p.cWo);
          const int rem = static_cast<int>(pix - img * p.cHo * p.cWo);
          const int y0 = (rem / p.cWo) * p.csh - p.cpt, x0 = (rem % p.cWo) * p.csw - p.cpl;
          off[q] = static_cast<int>(((img * p.cH + y0) * p.cW + x0) * p.cC) + piece * 8;
          yx[q] = (static_cast<uint32_t>(y0 + 0x4000) << 16) | static_cast<uint32_t>(x0 + 0x4000);
        } else {
          off[q] = 0;
          yx[q] = 0; // y0 = x0 = -16384: outside for every tap
        }
      }
      for (int kb = 0; kb < kBlocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t phase = (it / STAGES) & 1u;
        if (!__all_sync(0xffffffffu, mbarWait(emptyBar(s), phase ^ 1u, abortFlag, 1))) { alive = false; break; }
        const uint32_t sa = base + s * Cfg::kStageBytes, sb = sa + TC_A_BYTES;
        if (lane == 0) {
          mbarArriveExpectTx(fullBar(s), BN * TC_BK * 2);
          tmaLoad2d(sb, &mapB, fullBar(s), kb * TC_BK, n0);
        }
        const int tap = kb / cb, c0 = (kb - tap * cb) * TC_BK;
        const int ky = tap / p.ckw, kx = tap - ky * p.ckw;
        const int dy = ky * p.cdh, dx = kx * p.cdw;
        const int tapOff = (dy * p.cW + dx) * p.cC + c0;
        // destination of this lane's piece in row q*4 + rowInGroup: rows are 128 bytes, the piece
        // index is XORed with the row's low three bits (rowInGroup + 4*(q & 1))
        const uint32_t dstLane = sa + static_cast<uint32_t>(rowInGroup) * 128u;
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          const int y = static_cast<int>(yx[q] >> 16) - 0x4000 + dy, xx = static_cast<int>(yx[q] & 0xffffu) - 0x4000 + dx;
          const bool inside = static_cast<unsigned>(y) < static_cast<unsigned>(p.cH) &&
                              static_cast<unsigned>(xx) < static_cast<unsigned>(p.cW);
          const uint16_t *src = x + (inside ? off[q] + tapOff : 0);
          const uint32_t bytes = inside ? 16u : 0u; // 0 source bytes = the 16 destination bytes are zero-filled
          const uint32_t row7 = static_cast<uint32_t>((rowInGroup + 4 * (q & 1)) & 7);
          const uint32_t dst = dstLane + static_cast<uint32_t>(q) * 512u + ((static_cast<uint32_t>(piece) ^ row7) << 4);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (it - handed >= static_cast<uint32_t>(kInFlight)) {
          asm volatile("cp.async.wait_group %0;" ::"n"(kInFlight) : "memory");
          hand(handed++);
        }
      }
    }
    // drain: everything issued has to land (also when leaving early) before its stage is handed over
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    while (handed < it) hand(handed++);
  } else if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int64_t tile = worker; tile < numTiles && alive; tile += workers) {
        const int mt = static_cast<int>(tile % tilesM);
        const int m0 = mt * TILE_M + static_cast<int>(ctaRank) * TC_BM;
        int n0;
        const int seg = segmentOf(tile / tilesM, n0);
        const CUtensorMap *mb = seg == 0 ? &mapB : (seg == 1 ? &mapB1 : &mapB2);
        int img = 0, oy0 = 0, ox0 = 0, cb = 1;
        if (p.cTw) {
          const int perImg = p.cTilesX * p.cTilesY, rem = mt % perImg;
          img = mt / perImg;
          oy0 = (rem / p.cTilesX) * (TC_BM / p.cTw);
          ox0 = (rem % p.cTilesX) * p.cTw;
          cb = p.cC / TC_BK;
        }
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1u;
          if (!mbarWait(emptyBar(s), phase ^ 1u, abortFlag, 1)) { alive = false; break; }
          const uint32_t sa = base + s * Cfg::kStageBytes, sb = sa + TC_A_BYTES;
          if constexpr (PAIR) {
            // Both CTAs' loads complete on rank 0's barrier, which expects the bytes of both; each CTA
            // fetches its own 128 rows of A and its own half of the B tile (in SwiGLU mode rank 0 the gate
            // rows and rank 1 the up rows of the same output columns).
            const uint32_t bar = mapToCta(fullBar(s), 0);
            if (leader) mbarArriveExpectTx(fullBar(s), 2 * Cfg::kStageBytes);
            const bool second = DUALA && kb >= kBlocks1; // k-blocks of the second product
            const int kc = (second ? kb - kBlocks1 : kb) * K_ELEMS;
            tmaLoad2dPair(sa, second ? &mapE : &mapA, bar, kc, m0);
            if (p.dual) tmaLoad2dPair(sb, leader ? &mapB : &mapB1, bar, kc, n0);
            else tmaLoad2dPair(sb, second ? &mapB1 : mb, bar, kc, n0 + static_cast<int>(ctaRank) * (BN / 2));
            continue;
          }
          mbarArriveExpectTx(fullBar(s), Cfg::kStageBytes);
          if (p.cTw) {
            // the input patch of this filter tap; coordinates left of / above the image read zeros
            const int tap = kb / cb, ky = tap / p.ckw, kx = tap - ky * p.ckw;
            tmaLoad4d(sa, &mapA, fullBar(s), (kb - tap * cb) * TC_BK, ox0 + kx * p.cdw - p.cpl, oy0 + ky * p.cdh - p.cpt, img);
          } else if (DUALA && kb >= kBlocks1) {
            tmaLoad2d(sa, &mapE, fullBar(s), (kb - kBlocks1) * K_ELEMS, m0);
          } else {
            tmaLoad2d(sa, &mapA, fullBar(s), kb * K_ELEMS, m0);
          }
          if (p.dual) {
            tmaLoad2d(sb, &mapB, fullBar(s), kb * TC_BK, n0);
            tmaLoad2d(sb + (BN / 2) * TC_BK * 2, &mapB1, fullBar(s), kb * TC_BK, n0);
          } else if (DUALA && kb >= kBlocks1) {
            tmaLoad2d(sb, &mapB1, fullBar(s), (kb - kBlocks1) * K_ELEMS, n0);
          } else {
            tmaLoad2d(sb, mb, fullBar(s), kb * K_ELEMS, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && leader) {
      constexpr bool ints = I8;
      const uint32_t idesc = ints ? instrDescI8(p.aSigned, p.bSigned, TILE_M, BN) : instrDesc(p.fmt, TILE_M, BN);
      uint32_t it = 0, accIt = 0;
      bool alive = true;
      for (int64_t tile = worker; tile < numTiles && alive; tile += workers, ++accIt) {
        const int acc = accIt & 1;
        const uint32_t accPhase = (accIt >> 1) & 1u;
        if (!mbarWait(tmemEmptyBar(acc), accPhase ^ 1u, abortFlag, 2)) break;
        tcFenceAfter();
        const uint32_t tmemD0 = tmemBase + static_cast<uint32_t>(acc) * accCols;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const bool second = DUALA && kb >= kBlocks1;
          const uint32_t tmemD = tmemD0 + (second ? static_cast<uint32_t>(BN) : 0u);
          const int kbIn = second ? kb - kBlocks1 : kb; // the first MMA of a product overwrites the accumulator
          const int s = it % STAGES;
          const uint32_t phase = (it / STAGES) & 1u;
          if (!mbarWait(fullBar(s), phase, abortFlag, 3)) { alive = false; break; }
          tcFenceAfter();
          const uint32_t sa = base + s * Cfg::kStageBytes, sb = sa + TC_A_BYTES;
          const uint64_t da = smemDesc(sa), db = smemDesc(sb);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            // +32 bytes per k-step (16 two-byte or 32 one-byte elements) = +2 in the descriptor's 16-byte address units
            if constexpr (PAIR) {
              if constexpr (ints) tcMmaPairI8(tmemD, da + 2u * k, db + 2u * k, idesc, (kbIn | k) != 0 ? 1u : 0u);
              else tcMmaPair(tmemD, da + 2u * k, db + 2u * k, idesc, (kbIn | k) != 0 ? 1u : 0u);
            } else {
              if constexpr (ints) tcMmaI8(tmemD, da + 2u * k, db + 2u * k, idesc, (kbIn | k) != 0 ? 1u : 0u);
              else tcMma(tmemD, da + 2u * k, db + 2u * k, idesc, (kbIn | k) != 0 ? 1u : 0u);
            }
          }
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if constexpr (PAIR) tcCommitPair(emptyBar(s));
          else tcCommit(emptyBar(s));
        }
        if (alive) { // accumulator complete
          if constexpr (PAIR) tcCommitPair(tmemFullBar(acc));
          else tcCommit(tmemFullBar(acc));
        }
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
    constexpr int EPW = PLAIN ? 4 : 8; // epilogue warps
    const int quarter = warp & 3; // TMEM lanes this warp may read
    // A relu that is the last step of a 16-bit epilogue is applied to the packed pairs.
    const bool reluPacked = !PLAIN && sizeof(TC) == 2 && p.act == TTB_ACT_RELU && p.extraOp == 0;
    // PLAIN: four warps, two staging buffers each.  Otherwise eight warps in two groups: group g
    // drains accumulator buffer g (every other tile), one staging buffer per warp; two warps per
    // scheduler hide each other's instruction latencies in the longer epilogues.
    const int group = (warp - 2) / 4;
    const uint32_t stageOut = outBase + static_cast<uint32_t>(warp - 2) * 2u * 4096u; // two buffers per warp
    uint32_t chunkIt = 0, extraPhase = 0;
    bool alive = true;
    // Tiles of this CTA are numbered 0 .. myTiles-1 (tile index = blockIdx.x + number * gridDim.x,
    // accumulator = number & 1).  With two groups, group g drains the tiles with number = g mod 2.
    // The last tile has no successor whose main loop could hide its epilogue, so there both groups
    // work on it: its owner takes the even column chunks, the other group the odd ones.
    const int64_t myTiles = worker < numTiles ? (numTiles - worker + workers - 1) / workers : 0;
    const int64_t lastNo = myTiles - 1;
    bool helped = false;
    for (int64_t no = group;; no += EPW / 4) {
      bool helper = false;
      if (no >= myTiles) {
        if (EPW == 8 && BN / CH >= 2 && lastNo >= 0 && (lastNo & 1) != group && !helped) {
          no = lastNo;
          helper = helped = true;
        } else {
          break;
        }
      }
      const bool shared = EPW == 8 && BN / CH >= 2 && no == lastNo;
      const int64_t tile = worker + no * workers;
      const uint32_t accIt = static_cast<uint32_t>(no);
      const int acc = accIt & 1;
      const uint32_t accPhase = (accIt >> 1) & 1u;
      const int64_t m0 = (tile % tilesM) * TILE_M + static_cast<int64_t>(ctaRank) * TC_BM;
      int n0i;
      const int seg = segmentOf(tile / tilesM, n0i);
      // Rotary embedding: this row's 128 cosines and 128 sines (the same for every head of the tile) are fetched
      // now, so that their latency passes while the main loop is still filling the accumulator.
      uint4 ropeTab[PLAIN && sizeof(TC) == 2 && BN >= 128 ? 32 : 1];
      bool ropeTile = false;
      if constexpr (PLAIN && sizeof(TC) == 2 && BN >= 128) {
        ropeTile = ((p.ropeMask >> seg) & 1) != 0;
        if (ropeTile) {
          const int64_t row = m0 + quarter * 32 + lane;
          const int64_t pos = row < p.M ? row % p.ropeSeq : 0;
          const uint4 *cosRow = reinterpret_cast<const uint4 *>(static_cast<const TC *>(p.ropeCos) + pos * 128);
          const uint4 *sinRow = reinterpret_cast<const uint4 *>(static_cast<const TC *>(p.ropeSin) + pos * 128);
#pragma unroll
          for (int v = 0; v < 16; ++v) {
            ropeTab[v] = __ldg(cosRow + v);
            ropeTab[16 + v] = __ldg(sinRow + v);
          }
        }
      }
      if (!mbarWait(tmemFullBar(acc), accPhase, abortFlag, 4)) break;
      tcFenceAfter();
      const int64_t n0 = n0i, segN = p.segN[seg];
      const CUtensorMap *mc = seg == 0 ? &mapC : (seg == 1 ? &mapC1 : &mapC2);
      int rowBase = static_cast<int>(m0) + quarter * 32; // first row of this warp's block in the 2-D store
      if (p.pushRows) {
        const int owner = static_cast<int>(m0) / p.pushRows;
        mc = &pushMaps.m[owner];
        rowBase -= owner * p.pushRows;
      }
      // patch mode: this warp's 32 rows are 32 / cTw rows of the patch, starting at (pOy, pOx) of image pImg
      int pImg = 0, pOy = 0, pOx = 0;
      if (p.cTw) {
        const int mt = static_cast<int>(tile % tilesM), perImg = p.cTilesX * p.cTilesY, rem = mt % perImg;
        pImg = mt / perImg;
        pOy = (rem / p.cTilesX) * (TC_BM / p.cTw) + quarter * (32 / p.cTw);
        pOx = (rem % p.cTilesX) * p.cTw;
      }
      const uint32_t taddrRow = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc) * accCols;
      // SwiGLU mode: two chunks of 64 output columns; gate in accumulator columns [0, 128), up in [128, 256).
      bool dualDone = false;
      if constexpr (!PLAIN && sizeof(TC) == 2 && BN == 256) {
        if (p.dual) {
          dualDone = true;
#pragma unroll 1
          for (int cc = (shared && helper) ? 1 : 0; cc < 2; cc += shared ? 2 : 1) {
            const int64_t col0 = n0 + cc * CH;
            if (col0 >= segN) break; // warp-uniform
            const uint32_t buf = stageOut + (chunkIt & 1u) * 4096u;
            const uint32_t rowAddr = buf + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
            for (int l = 0; l < 2; ++l) {
              uint32_t g[32], u[32];
              tcLoad32(taddrRow + static_cast<uint32_t>(cc * CH + l * 32), g);
              tcLoad32(taddrRow + static_cast<uint32_t>(BN / 2 + cc * CH + l * 32), u);
              tcWaitLd();
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                // every value the chain of separate ops would have stored is rounded here as well
                const float gv = toF32(fromF32<TC>(__uint_as_float(g[e])));
                const float sg = toF32(fromF32<TC>(__fdividef(gv, 1.0f + __expf(-gv))));
                g[e] = __float_as_uint(__fmul_rn(sg, toF32(fromF32<TC>(__uint_as_float(u[e])))));
              }
              if (l == 0) {
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); // the store before the last has read this buffer
                __syncwarp();
              }
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int e = v * 8 + q * 2;
                  w[q] = pack2<TC>(__uint_as_float(g[e]), __uint_as_float(g[e + 1]));
                }
                const int pieceIdx = l * 4 + v;
                const uint32_t addr = rowAddr + (static_cast<uint32_t>(pieceIdx ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(reinterpret_cast<uint64_t>(mc)), "r"(buf), "r"(static_cast<int>(col0)), "r"(rowBase)
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            ++chunkIt;
          }
        }
      }
      if constexpr (!PLAIN && sizeof(TC) == 2 && BN <= 128) {
        if constexpr (DUALA) {
          // Two products: columns [0, BN) and [BN, 2 BN) of the buffer; each gets its bias and its own rounding, the
          // sum is rounded again, relu (if any) commutes with that rounding and is applied to the packed pairs.
          dualDone = true;
          const bool relu = p.act == TTB_ACT_RELU;
#pragma unroll 1
          for (int cc = (shared && helper) ? 1 : 0; cc < BN / CH; cc += shared ? 2 : 1) {
            const int64_t col0 = n0 + cc * CH;
            if (col0 >= segN) break; // warp-uniform
            const uint32_t buf = stageOut + (chunkIt & 1u) * 4096u;
            const uint32_t rowAddr = buf + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
            for (int l = 0; l < 2; ++l) {
              const int64_t colH = col0 + l * 32;
              // both biases as broadcast vectors when the pass lies inside the matrix, one value per lane otherwise
              const bool wide = p.biasVec && p.bias && p.bias2 && colH + 32 <= p.N;
              float b1 = 0.0f, b2 = 0.0f;
              BiasRow<TC> row1, row2;
              if (wide) {
                row1.load(p.bias, colH);
                row2.load(p.bias2, colH);
              } else if (colH + lane < p.N) {
                if (p.bias) b1 = loadBias(p.bias, p.biasDt, colH + lane);
                if (p.bias2) b2 = loadBias(p.bias2, p.bias2Dt, colH + lane);
              }
              uint32_t r1[32], r2[32];
              tcLoad32(taddrRow + static_cast<uint32_t>(cc * CH + l * 32), r1);
              tcLoad32(taddrRow + static_cast<uint32_t>(BN + cc * CH + l * 32), r2);
              tcWaitLd();
              if (wide) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const float v1 = toF32(fromF32<TC>(__fadd_rn(__uint_as_float(r1[e]), row1.at(e))));
                  const float v2 = toF32(fromF32<TC>(__fadd_rn(__uint_as_float(r2[e]), row2.at(e))));
                  r1[e] = __float_as_uint(__fadd_rn(v1, v2));
                }
              } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const float v1 = toF32(fromF32<TC>(__fadd_rn(__uint_as_float(r1[e]), __shfl_sync(0xffffffffu, b1, e))));
                  const float v2 = toF32(fromF32<TC>(__fadd_rn(__uint_as_float(r2[e]), __shfl_sync(0xffffffffu, b2, e))));
                  r1[e] = __float_as_uint(__fadd_rn(v1, v2));
                }
              }
              if (l == 0) {
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); // the store before the last has read this buffer
                __syncwarp();
              }
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const int e = v * 8 + q * 2;
                  w[q] = pack2<TC>(__uint_as_float(r1[e]), __uint_as_float(r1[e + 1]));
                  if (relu) w[q] = relu2<TC>(w[q]);
                }
                const uint32_t addr = rowAddr + (static_cast<uint32_t>((l * 4 + v) ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(reinterpret_cast<uint64_t>(mc)), "r"(buf), "r"(static_cast<int>(col0)), "r"(rowBase)
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            ++chunkIt;
          }
        }
      }
      if constexpr (PLAIN && sizeof(TC) == 2 && BN >= 128) {
        if (ropeTile) {
          // Rotary embedding: chunks cc and cc + 1 hold the two halves of one head's 128 values of this row.
          dualDone = true;
          const uint32_t rowA = stageOut + static_cast<uint32_t>(lane) * 128u, rowB = rowA + 4096u;
#pragma unroll 1
          for (int cc = 0; cc < BN / CH; cc += 2) {
            const int64_t col0 = n0 + cc * CH;
            if (col0 >= segN) break; // warp-uniform
#pragma unroll
            for (int l = 0; l < 2; ++l) {
              uint32_t x1[32], x2[32];
              tcLoad32(taddrRow + static_cast<uint32_t>(cc * CH + l * 32), x1);
              tcLoad32(taddrRow + static_cast<uint32_t>((cc + 1) * CH + l * 32), x2);
              tcWaitLd();
              if (l == 0) {
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); // both staging buffers are free
                __syncwarp();
              }
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint32_t wA[4], wB[4];
                // 16-byte unit u of a table row holds columns [8u, 8u + 8): first half l * 4 + v, second half 8 more
                const TC *c1e = reinterpret_cast<const TC *>(&ropeTab[l * 4 + v]), *c2e = reinterpret_cast<const TC *>(&ropeTab[8 + l * 4 + v]);
                const TC *s1e = reinterpret_cast<const TC *>(&ropeTab[16 + l * 4 + v]), *s2e = reinterpret_cast<const TC *>(&ropeTab[24 + l * 4 + v]);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float o1[2], o2[2];
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
                    const int e = v * 8 + q * 2 + h;
                    const float a = toF32(fromF32<TC>(__uint_as_float(x1[e]))), b2 = toF32(fromF32<TC>(__uint_as_float(x2[e])));
                    o1[h] = __fadd_rn(__fmul_rn(a, toF32(c1e[q * 2 + h])), __fmul_rn(-b2, toF32(s1e[q * 2 + h])));
                    o2[h] = __fadd_rn(__fmul_rn(b2, toF32(c2e[q * 2 + h])), __fmul_rn(a, toF32(s2e[q * 2 + h])));
                  }
                  wA[q] = pack2<TC>(o1[0], o1[1]);
                  wB[q] = pack2<TC>(o2[0], o2[1]);
                }
                const uint32_t off = static_cast<uint32_t>((l * 4 + v) ^ (lane & 7)) << 4;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowA + off), "r"(wA[0]), "r"(wA[1]), "r"(wA[2]), "r"(wA[3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowB + off), "r"(wB[0]), "r"(wB[1]), "r"(wB[2]), "r"(wB[3]) : "memory");
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              // one group per store: the chunk loop below reuses a buffer once all groups but the latest have been read
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(reinterpret_cast<uint64_t>(mc)), "r"(stageOut), "r"(static_cast<int>(col0)), "r"(rowBase) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(reinterpret_cast<uint64_t>(mc)), "r"(stageOut + 4096u), "r"(static_cast<int>(col0 + CH)), "r"(rowBase) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            chunkIt += 2;
          }
        }
      }
#pragma unroll 1
      for (int cc = dualDone ? BN / CH : ((shared && helper) ? 1 : 0); cc < BN / CH; cc += shared ? 2 : 1) {
        const int64_t col0 = n0 + cc * CH;
        if (col0 >= segN) break; // warp-uniform
        const uint32_t buf = stageOut + (chunkIt & 1u) * 4096u;
        const uint32_t rowAddr = buf + static_cast<uint32_t>(lane) * 128u;
        // The second operand's 32 x 128 B block is brought into the staging buffer by TMA (the
        // layout the result will have), combined in place, and stored from there.
        bool useExtra = false;
        if constexpr (!PLAIN && sizeof(TC) == 2) {
          useExtra = p.extraOp != 0;
          if (useExtra) {
            if (lane == 0) {
              asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); // the store before the last has read this buffer
              mbarArriveExpectTx(extraBar(warp - 2), 4096);
              if (p.cTw) tmaLoad4d(buf, &mapE, extraBar(warp - 2), static_cast<int>(col0), pOx, pOy, pImg);
              else tmaLoad2d(buf, &mapE, extraBar(warp - 2), static_cast<int>(col0), static_cast<int>(m0 + quarter * 32));
            }
            __syncwarp();
          }
        }
        // The chunk is worked through in passes of 32 columns (64 or 128 bytes of the output row),
        // which keeps the registers of a pass small enough for two epilogue warps per scheduler.
#pragma unroll
        for (int l = 0; l < NLD; ++l) {
          constexpr int HW = 32;
          const int64_t colH = col0 + l * HW;
          // bias of this pass first, so that it is in flight while TMEM is read
          float biasReg = 0.0f;
          BiasRow<TC> biasRow;
          bool biasWide = false; // the whole pass lies inside the matrix and the bias can be fetched as vectors
          if constexpr (!PLAIN) {
            if constexpr (sizeof(TC) == 2) {
              biasWide = p.bias && p.biasVec && colH + HW <= p.N;
              if (biasWide) biasRow.load(p.bias, colH);
            }
            if (p.bias && !biasWide && colH + lane < p.N) biasReg = loadBias(p.bias, p.biasDt, colH + lane);
          }
          uint32_t r[HW];
          tcLoad32(taddrRow + static_cast<uint32_t>(cc * CH + l * HW), r);
          tcWaitLd();
          uint4 ev[sizeof(TC) == 2 && !PLAIN ? HW / 8 : 1] = {};
          if constexpr (!PLAIN && sizeof(TC) == 2) {
            if (useExtra) {
              if (l == 0) {
                if (!__all_sync(0xffffffffu, mbarWait(extraBar(warp - 2), extraPhase, abortFlag, 5))) { alive = false; break; }
              }
#pragma unroll
              for (int g = 0; g < HW / 8; ++g) {
                const uint32_t addr = rowAddr + (static_cast<uint32_t>((l * (HW / 8) + g) ^ (lane & 7)) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(ev[g].x), "=r"(ev[g].y), "=r"(ev[g].z), "=r"(ev[g].w) : "r"(addr) : "memory");
              }
            }
          }
          if constexpr (!PLAIN) {
            if constexpr (I8) {
              if (p.deq) {
                // quantized contraction followed by dequantize: float(accumulator) * scale, one rounding
                float sc = p.deqScalar;
                if (p.deq == 2) sc = colH + lane < p.N ? p.deqScale[colH + lane] : 0.0f;
#pragma unroll
                for (int e = 0; e < HW; ++e) {
                  const float se = p.deq == 2 ? __shfl_sync(0xffffffffu, sc, e) : sc;
                  r[e] = __float_as_uint(__fmul_rn(__int2float_rn(static_cast<int>(r[e])), se));
                }
              }
            }
            // One straight-line pass per case: runtime flags inside the unrolled loop would put
            // every variant's instructions on every element, and a per-element switch over the
            // activations would thrash the instruction cache.
            const bool hasBias = p.bias != nullptr, round1 = (p.roundSteps & 1) != 0, round2 = (p.roundSteps & 2) != 0;
            if (hasBias && !round1 && !round2 && biasWide) {
              if constexpr (sizeof(TC) == 2) {
#pragma unroll
                for (int e = 0; e < HW; ++e) r[e] = __float_as_uint(__fadd_rn(__uint_as_float(r[e]), biasRow.at(e)));
              }
            } else if (hasBias && !round1 && !round2) {
#pragma unroll
              for (int e = 0; e < HW; ++e) {
                const float bz = __shfl_sync(0xffffffffu, biasReg, e); // lane e holds column e's bias
                r[e] = __float_as_uint(__fadd_rn(__uint_as_float(r[e]), bz));
              }
            } else if (hasBias && biasWide) {
              if constexpr (sizeof(TC) == 2) {
#pragma unroll
                for (int e = 0; e < HW; ++e) {
                  float f = __uint_as_float(r[e]);
                  if (round1) f = toF32(fromF32<TC>(f));
                  f = __fadd_rn(f, biasRow.at(e));
                  if (round2) f = toF32(fromF32<TC>(f));
                  r[e] = __float_as_uint(f);
                }
              }
            } else if (hasBias) {
#pragma unroll
              for (int e = 0; e < HW; ++e) {
                float f = __uint_as_float(r[e]);
                const float bz = __shfl_sync(0xffffffffu, biasReg, e);
                if (round1) f = toF32(fromF32<TC>(f));
                f = __fadd_rn(f, bz);
                if (round2) f = toF32(fromF32<TC>(f));
                r[e] = __float_as_uint(f);
              }
            } else if (round1) {
#pragma unroll
              for (int e = 0; e < HW; ++e) r[e] = __float_as_uint(toF32(fromF32<TC>(__uint_as_float(r[e]))));
            }
            switch (reluPacked ? TTB_ACT_NONE : p.act) {
            case TTB_ACT_RELU:
#pragma unroll
              for (int e = 0; e < HW; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(f < 0.0f ? 0.0f : f); } // NaN stays NaN
              break;
            case TTB_ACT_SILU:
#pragma unroll
              for (int e = 0; e < HW; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(f / (1.0f + expf(-f))); }
              break;
            case TTB_ACT_GELU:
#pragma unroll
              for (int e = 0; e < HW; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(applyAct(TTB_ACT_GELU, f)); }
              break;
            case TTB_ACT_SIGMOID:
#pragma unroll
              for (int e = 0; e < HW; ++e) { float f = __uint_as_float(r[e]); r[e] = __float_as_uint(1.0f / (1.0f + expf(-f))); }
              break;
            default: break;
            }
            if constexpr (sizeof(TC) == 2) {
              // A separate op consumed the (rounded) result of the chain so far.
              if (p.extraOp == TTB_EXTRA_ADD || p.extraOp == TTB_EXTRA_ADD_RELU) {
                const bool relu = p.extraOp == TTB_EXTRA_ADD_RELU;
#pragma unroll
                for (int e = 0; e < HW; ++e) {
                  const TC *x = reinterpret_cast<const TC *>(&ev[e / 8]) + (e & 7);
                  float f = __fadd_rn(toF32(fromF32<TC>(__uint_as_float(r[e]))), toF32(*x));
                  if (relu) f = f < 0.0f ? 0.0f : f;
                  r[e] = __float_as_uint(f);
                }
              } else if (p.extraOp == TTB_EXTRA_SILU_MUL) {
#pragma unroll
                for (int e = 0; e < HW; ++e) {
                  const TC *x = reinterpret_cast<const TC *>(&ev[e / 8]) + (e & 7);
                  const float g = toF32(*x);
                  const float sg = toF32(fromF32<TC>(__fdividef(g, 1.0f + __expf(-g))));
                  r[e] = __float_as_uint(__fmul_rn(sg, toF32(fromF32<TC>(__uint_as_float(r[e])))));
                }
              }
            }
          }
          if (l == 0 && !useExtra) {
            // the staging buffer is free once the bulk store issued from it has read it
            if (lane == 0) {
              asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
            __syncwarp();
          }
          constexpr int PIECES = HW * static_cast<int>(sizeof(TC)) / 16; // 16-byte pieces of this pass
#pragma unroll
          for (int v = 0; v < PIECES; ++v) {
            uint32_t w[4];
            if constexpr (sizeof(TC) == 2) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int e = v * 8 + q * 2;
                w[q] = pack2<TC>(__uint_as_float(r[e]), __uint_as_float(r[e + 1])); // one cvt.rn for the pair
                if constexpr (!PLAIN) {
                  if (reluPacked) w[q] = relu2<TC>(w[q]);
                }
              }
            } else {
#pragma unroll
              for (int q = 0; q < 4; ++q) w[q] = r[v * 4 + q];
            }
            // 128-byte swizzle (what the tensor map of C expects): 16-byte piece i of row `lane`
            // lives at piece i ^ (lane % 8); this also spreads the lanes over the banks
            const int pieceIdx = l * PIECES + v;
            const uint32_t addr = rowAddr + (static_cast<uint32_t>(pieceIdx ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
          }
        }
        if (!alive) break;
        if (useExtra) extraPhase ^= 1u;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (p.cTw) {
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                         ::"l"(reinterpret_cast<uint64_t>(mc)), "r"(buf), "r"(static_cast<int>(col0)), "r"(pOx), "r"(pOy),
                           "r"(pImg) : "memory");
          } else {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(reinterpret_cast<uint64_t>(mc)), "r"(buf), "r"(static_cast<int>(col0)), "r"(rowBase)
                         : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        ++chunkIt;
      }
      if (!alive) break;
      if (helper) break; // the helper's visit was the last thing this group does
      tcFenceBefore();
      // all 128 epilogue threads arrive (of both CTAs of a pair, at rank 0's barrier): the accumulator may be overwritten
      if constexpr (PAIR) mbarArriveRemote(mapToCta(tmemEmptyBar(acc), 0));
      else mbarArrive(tmemEmptyBar(acc));
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
  // Pair: a CTA's shared memory (barriers, operand halves) is used by its partner until both are done.
  if constexpr (PAIR) clusterSync();
  if (warp == 1) {
    tcFenceAfter();
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(TC_TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(TC_TMEM_COLS) : "memory");
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
  if (dtype == kI8 || dtype == kU8) dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (dtype == kI32) dt = CU_TENSOR_MAP_DATA_TYPE_INT32;
  CUresult r = fn(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// NHWC tensor [n, h, w, c] of a 16-bit type as a 4-D map {c, w, h, n}; box = boxC channels (128
// bytes) x boxW x boxH pixels of one image, 128-byte swizzle, zero fill outside.
static bool makeMap4(CUtensorMap *map, const void *ptr, int dtype, int64_t c, int64_t w, int64_t h, int64_t n, int boxC,
                     int boxW, int boxH) {
  EncodeTiledFn fn = encodeTiled();
  if (!fn) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(c), static_cast<cuuint64_t>(w), static_cast<cuuint64_t>(h),
                        static_cast<cuuint64_t>(n)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(c) * 2, static_cast<cuuint64_t>(w) * c * 2,
                           static_cast<cuuint64_t>(h) * w * c * 2};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(boxC), static_cast<cuuint32_t>(boxW), static_cast<cuuint32_t>(boxH), 1};
  cuuint32_t elemStrides[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Two CTAs per 256-row tile (cta_group::2) unless switched off (TTB_DISABLE_PAIR_MMA=1), the problem has fewer than
// 256 rows, or the reduction is short: with a handful of k-blocks per tile the hand-overs between the two CTAs
// (operands landed, stage free, accumulator full / drained all cross the pair) are no longer hidden behind the main
// loop, and one CTA per tile is faster (pointwise convolutions with K = 64: 54 against 61 us per launch).
// Convolutions with a gathered operand keep one CTA per tile.
static bool pairMmaWanted(int64_t m, int64_t k) {
  static const bool off = [] {
    const char *e = std::getenv("TTB_DISABLE_PAIR_MMA");
    return e && e[0] == '1';
  }();
  static const int64_t minK = [] {
    const char *e = std::getenv("TTB_PAIR_MMA_MIN_K");
    return e ? static_cast<int64_t>(atoll(e)) : static_cast<int64_t>(512);
  }();
  return !off && m >= 2 * TC_BM && k >= minK && smCount() >= 2;
}

template <int BN, typename TC, bool PLAIN, bool PAIR = false, bool I8 = false, bool DUALA = false>
static int launchTc(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mc, const CUtensorMap &me, void *c, const TcParams &p,
                    cudaStream_t st, const CUtensorMap *more = nullptr /* mapB1, mapC1, mapB2, mapC2 of a grouped launch */,
                    const PushMaps *push = nullptr) {
  using Cfg = TcCfg<BN, PAIR, PLAIN>;
  // Function attributes belong to a device: set the shared-memory limit once on each.
  static bool attrSet[64] = {};
  int dev = 0;
  TTB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attrSet[dev]) {
    TTB_CUDA(cudaFuncSetAttribute(gemmTcgen05Kernel<BN, TC, PLAIN, PAIR, I8, DUALA>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
    attrSet[dev] = true;
  }
  const int64_t tileM = PAIR ? 2 * TC_BM : TC_BM;
  int64_t tiles = (p.cTw ? p.cTilesM : (p.M + tileM - 1) / tileM) * p.segCum[2];
  const int workers = PAIR ? smCount() / 2 : smCount();
  int grid = static_cast<int>(tiles < workers ? tiles : workers) * (PAIR ? 2 : 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(PLAIN ? TC_THREADS : TC_THREADS_EPI8);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdlEnabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (PAIR) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  TTB_CUDA(cudaLaunchKernelEx(&cfg, gemmTcgen05Kernel<BN, TC, PLAIN, PAIR, I8, DUALA>, ma, mb, mc, me, more ? more[0] : mb, more ? more[1] : mc,
                              more ? more[2] : mb, more ? more[3] : mc, push ? *push : PushMaps{{mc, mc, mc, mc, mc, mc, mc, mc}},
                              static_cast<TC *>(c), p));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// Tile width for an m x n problem on `workers` workers of `tileM` rows: fewest (waves x per-tile cost).  A tile's
// cost per k-block follows the operand bytes its CTA fetches -- 128 rows of A whatever the width, plus the CTA's
// rows of B (all of them, or half in a CTA pair) -- because narrow tiles are bound by the rate at which an SM takes
// operands in, not by the tensor pipe: measured per tile and k-block, pairs, 1.0 : 0.80 : 0.64 for widths 256 : 128 :
// 64 (the model gives 1.0 : 0.75 : 0.63).
static int forcedTileWidth() {
  static const int v = [] {
    const char *e = std::getenv("TTB_FORCE_BN");
    return e ? atoi(e) : 0;
  }();
  return v;
}

static int64_t tileCost(int w, bool pair) { return 128 + (pair ? w / 2 : w); }

static int pickTileWidth(int64_t m, int64_t n, int64_t tileM, int workers, bool pair) {
  if (forcedTileWidth() && n >= forcedTileWidth()) return forcedTileWidth();
  int bn = 64;
  int64_t best = -1;
  for (int w : {256, 128, 64}) {
    if (w > 64 && n < w) continue;
    int64_t tiles = ((m + tileM - 1) / tileM) * ((n + w - 1) / w);
    int64_t waves = (tiles + workers - 1) / workers;
    int64_t cost = waves * tileCost(w, pair);
    if (best < 0 || cost < best) {
      best = cost;
      bn = w;
    }
  }
  return bn;
}

int gemmTcgen05Try(const void *a, const void *b, const void *bias, void *c, int abDtype, int biasDtype, int cDtype,
                   int64_t batch, int64_t m, int64_t n, int64_t k, int transA, int transB, int64_t, int64_t, int act,
                   int roundSteps, const void *extra, int extraOp, cudaStream_t stream, void *const *pushTargets,
                   int pushRanks) {
  // Push mode: C's row blocks go to `pushRanks` [m / pushRanks, n] matrices (one per rank) instead of c.
  const bool pushing = pushRanks > 0;
  if (pushing) {
    if (!pushTargets || pushRanks > 8 || bias || act != TTB_ACT_NONE || roundSteps || extraOp || cDtype != abDtype) return -1;
    if (m % pushRanks != 0 || (m / pushRanks) % TC_BM != 0) return -1;
    for (int o = 0; o < pushRanks; ++o) {
      if (!pushTargets[o] || !aligned16(pushTargets[o])) return -1;
    }
    c = pushTargets[0]; // only checked for alignment below
  }
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
  const bool pair = pairMmaWanted(m, k);
  const int bn = pickTileWidth(m, n, pair ? 2 * TC_BM : TC_BM, pair ? smCount() / 2 : smCount(), pair);
  CUtensorMap ma, mb, mc, me;
  if (!makeMap(&ma, a, abDtype, m, k, TC_BM) || !makeMap(&mb, b, abDtype, n, k, pair ? bn / 2 : bn) ||
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
  p.biasVec = bias && biasDtype == cDtype && cDtype != kF32 && aligned16(bias) ? 1 : 0;
  p.extra = extraOp ? extra : nullptr;
  p.extraOp = extra ? extraOp : 0;
  p.convX = nullptr;
  p.cTw = 0;
  p.cTilesM = 0;
  p.pushRows = 0;
  p.dual = 0;
  PushMaps pm;
  if (pushing) {
    p.pushRows = static_cast<int>(m / pushRanks);
    for (int o = 0; o < 8; ++o) {
      if (!makeMap(&pm.m[o], pushTargets[o < pushRanks ? o : 0], cDtype, p.pushRows, n, 32)) return -1;
    }
  }
  p.segCum[0] = p.segCum[1] = p.segCum[2] = static_cast<int>((n + bn - 1) / bn);
  p.segN[0] = p.segN[1] = p.segN[2] = n;
  p.fmt = abDtype == kBF16 ? 1 : 0;
  p.kElems = TC_BK; p.aSigned = p.bSigned = 0; p.deq = 0; p.deqScalar = 0.0f; p.deqScale = nullptr;
  double flops = 2.0 * double(m) * double(n) * double(k);
  double bytes = (double(m) * k + double(n) * k) * 2 + double(m) * n * dtypeSize(cDtype) * (extraOp ? 2 : 1);
  ProfScope prof("gemm_tcgen05", flops, bytes, stream);
  const bool plain = !bias && act == TTB_ACT_NONE && roundSteps == 0 && !extraOp;
#define TTB_TC(BNv, TCv)                                                                 \
  if (pair)                                                                              \
    return plain ? launchTc<BNv, TCv, true, true>(ma, mb, mc, me, c, p, stream, nullptr, pushing ? &pm : nullptr)             \
                 : launchTc<BNv, TCv, false, true>(ma, mb, mc, me, c, p, stream);        \
  return plain ? launchTc<BNv, TCv, true>(ma, mb, mc, me, c, p, stream, nullptr, pushing ? &pm : nullptr)                     \
               : launchTc<BNv, TCv, false>(ma, mb, mc, me, c, p, stream)
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

// out[M, N] = silu(A Wg^T) * (A Wu^T) as ONE launch (SwiGLU mode of the kernel): A is read once, the
// gate projection never leaves the SM.  Wg, Wu: [N, K].  -1 = not taken.
int gemmTcgen05SwigluTry(const void *a, const void *wGate, const void *wUp, void *out, int dtype, int64_t m, int64_t n,
                         int64_t k, cudaStream_t stream) {
  if (dtype != kBF16 && dtype != kF16) return -1;
  if (k % 8 != 0 || n % 8 != 0 || m < 1 || n < 64 || k < 8) return -1;
  if (!aligned16(a) || !aligned16(wGate) || !aligned16(wUp) || !aligned16(out)) return -1;
  if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return -1;
  if (m * n * k < (1ll << 18)) return -1;
  constexpr int BN = 256;
  CUtensorMap ma, mg, mu, mc;
  if (!makeMap(&ma, a, dtype, m, k, TC_BM) || !makeMap(&mg, wGate, dtype, n, k, BN / 2) ||
      !makeMap(&mu, wUp, dtype, n, k, BN / 2) || !makeMap(&mc, out, dtype, m, n, 32))
    return -1;
  TcParams p;
  p.M = m; p.N = n; p.K = k;
  p.bias = nullptr; p.biasDt = 0; p.act = TTB_ACT_NONE; p.roundSteps = 0;
  p.extra = nullptr; p.extraOp = 0;
  p.convX = nullptr; p.cTw = 0; p.cTilesM = 0; p.pushRows = 0;
  p.dual = 1;
  p.segCum[0] = p.segCum[1] = p.segCum[2] = static_cast<int>((n + BN / 2 - 1) / (BN / 2));
  p.segN[0] = p.segN[1] = p.segN[2] = n;
  p.fmt = dtype == kBF16 ? 1 : 0;
  p.kElems = TC_BK; p.aSigned = p.bSigned = 0; p.deq = 0; p.deqScalar = 0.0f; p.deqScale = nullptr;
  // both projections' FLOPs; A and both weights once, the result once
  ProfScope prof("gemm_tcgen05", 4.0 * double(m) * double(n) * double(k), (double(m) * k + 2.0 * double(n) * k + double(m) * n) * 2, stream);
  const CUtensorMap more[4] = {mu, mc, mu, mc};
  if (pairMmaWanted(m, k)) {
    if (dtype == kBF16) return launchTc<BN, __nv_bfloat16, false, true>(ma, mg, mc, mc, out, p, stream, more);
    return launchTc<BN, __half, false, true>(ma, mg, mc, mc, out, p, stream, more);
  }
  if (dtype == kBF16) return launchTc<BN, __nv_bfloat16, false>(ma, mg, mc, mc, out, p, stream, more);
  return launchTc<BN, __half, false>(ma, mg, mc, mc, out, p, stream, more);
}

// out[M, N] = act(round(A1 B1^T + bias1) + round(A2 B2^T + bias2)) as ONE launch (two-product mode of the kernel):
// a pointwise convolution and the pointwise projection of its residual branch, summed and activated, without
// either product reaching memory.  B1: [N, K1], B2: [N, K2]; biases nullable; act none or relu.  -1 = not taken.
int gemmTcgen05DualTry(const void *a1, const void *b1, const void *bias1, const void *a2, const void *b2, const void *bias2,
                       void *out, int dtype, int biasDtype, int64_t m, int64_t n, int64_t k1, int64_t k2, int act,
                       cudaStream_t stream) {
  if (dtype != kBF16 && dtype != kF16) return -1;
  if (act != TTB_ACT_NONE && act != TTB_ACT_RELU) return -1;
  if (k1 % 8 != 0 || k2 % 8 != 0 || n % 8 != 0 || m < 1 || n < 8 || k1 < 8 || k2 < 8) return -1;
  if (!aligned16(a1) || !aligned16(b1) || !aligned16(a2) || !aligned16(b2) || !aligned16(out)) return -1;
  if (m > 0x7fffffff || n > 0x7fffffff || k1 > 0x7fffffff || k2 > 0x7fffffff) return -1;
  if (m * n * (k1 + k2) < (1ll << 18)) return -1;
  const bool pair = pairMmaWanted(m, k1 < k2 ? k1 : k2);
  const int bn = n >= 128 ? 128 : 64; // two accumulators of BN columns, double buffered, in 512 TMEM columns
  CUtensorMap ma1, mb1, ma2, mb2, mc;
  if (!makeMap(&ma1, a1, dtype, m, k1, TC_BM) || !makeMap(&mb1, b1, dtype, n, k1, pair ? bn / 2 : bn) ||
      !makeMap(&ma2, a2, dtype, m, k2, TC_BM) || !makeMap(&mb2, b2, dtype, n, k2, pair ? bn / 2 : bn) ||
      !makeMap(&mc, out, dtype, m, n, 32))
    return -1;
  TcParams p;
  p.M = m; p.N = n; p.K = k1;
  p.bias = bias1; p.biasDt = biasDtype; p.act = act; p.roundSteps = 0;
  p.extra = nullptr; p.extraOp = 0;
  p.convX = nullptr; p.cTw = 0; p.cTilesM = 0; p.pushRows = 0; p.dual = 0;
  p.segCum[0] = p.segCum[1] = p.segCum[2] = static_cast<int>((n + bn - 1) / bn);
  p.segN[0] = p.segN[1] = p.segN[2] = n;
  p.fmt = dtype == kBF16 ? 1 : 0;
  p.kElems = TC_BK; p.aSigned = p.bSigned = 0; p.deq = 0; p.deqScalar = 0.0f; p.deqScale = nullptr;
  p.dualA = 1;
  p.K2 = k2;
  p.bias2 = bias2;
  p.bias2Dt = biasDtype;
  p.biasVec = bias1 && bias2 && biasDtype == dtype && aligned16(bias1) && aligned16(bias2) ? 1 : 0;
  ProfScope prof("gemm_tcgen05", 2.0 * double(m) * double(n) * double(k1 + k2),
                 (double(m) * (k1 + k2) + double(n) * (k1 + k2) + double(m) * n) * 2, stream);
  const CUtensorMap more[4] = {mb2, mc, mb2, mc};
#define TTB_TCD(BNv, TCv)                                                                \
  if (pair) return launchTc<BNv, TCv, false, true, false, true>(ma1, mb1, mc, ma2, out, p, stream, more); \
  return launchTc<BNv, TCv, false, false, false, true>(ma1, mb1, mc, ma2, out, p, stream, more)
  if (bn == 128) {
    if (dtype == kBF16) { TTB_TCD(128, __nv_bfloat16); }
    TTB_TCD(128, __half);
  }
  if (dtype == kBF16) { TTB_TCD(64, __nv_bfloat16); }
  TTB_TCD(64, __half);
#undef TTB_TCD
}

// Quantized contraction: C[M, N] = A[M, K] B[N, K]^T with 8-bit integer operands and exact 32-bit
// integer accumulation (tcgen05.mma kind::i8).  cDtype Int32 stores the accumulators; Float32 / BFloat16 /
// Float16 store float(accumulator) * scale, scale being `deqScalar` (deqScale null) or deqScale[column]:
// the dequantize op that follows a quantized matmul or convolution, fused.  -1 = not taken.
int gemmTcgen05I8Try(const void *a, const void *b, void *c, int aDtype, int bDtype, int cDtype, int64_t m, int64_t n,
                     int64_t k, const float *deqScale, float deqScalar, const void *bias, int biasDtype, cudaStream_t stream) {
  if (bias && cDtype == kI32) return -1;
  if ((aDtype != kI8 && aDtype != kU8) || (bDtype != kI8 && bDtype != kU8)) return -1;
  if (cDtype != kI32 && cDtype != kF32 && cDtype != kBF16 && cDtype != kF16) return -1;
  if (k % 16 != 0 || m < 1 || n < 8 || k < 16) return -1; // rows of A and B are whole 16-byte units for TMA
  if ((n * static_cast<int64_t>(dtypeSize(cDtype))) % 16 != 0) return -1;
  if (!aligned16(a) || !aligned16(b) || !aligned16(c) || (deqScale && (reinterpret_cast<uintptr_t>(deqScale) & 3))) return -1;
  if (m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff) return -1;
  if (m * n * k < (1ll << 18)) return -1;
  const bool pair = pairMmaWanted(m, k);
  const int bn = pickTileWidth(m, n, pair ? 2 * TC_BM : TC_BM, pair ? smCount() / 2 : smCount(), pair);
  CUtensorMap ma, mb, mc;
  if (!makeMap(&ma, a, kU8, m, k, TC_BM) || !makeMap(&mb, b, kU8, n, k, pair ? bn / 2 : bn) || !makeMap(&mc, c, cDtype, m, n, 32)) return -1;
  TcParams p;
  p.M = m; p.N = n; p.K = k;
  // a bias follows the dequantize as a separate add: the dequantized value is rounded before it (round step 1)
  p.bias = bias; p.biasDt = biasDtype; p.act = TTB_ACT_NONE; p.roundSteps = bias ? 1 : 0;
  p.biasVec = bias && biasDtype == cDtype && (cDtype == kBF16 || cDtype == kF16) && aligned16(bias) ? 1 : 0;
  p.extra = nullptr; p.extraOp = 0;
  p.convX = nullptr; p.cTw = 0; p.cTilesM = 0; p.pushRows = 0; p.dual = 0;
  p.segCum[0] = p.segCum[1] = p.segCum[2] = static_cast<int>((n + bn - 1) / bn);
  p.segN[0] = p.segN[1] = p.segN[2] = n;
  p.fmt = 2;
  p.kElems = 128;
  p.aSigned = aDtype == kI8 ? 1 : 0;
  p.bSigned = bDtype == kI8 ? 1 : 0;
  p.deq = cDtype == kI32 ? 0 : (deqScale ? 2 : 1);
  p.deqScalar = deqScalar;
  p.deqScale = deqScale;
  ProfScope prof("gemm_tcgen05_i8", 2.0 * double(m) * double(n) * double(k),
                 double(m) * k + double(n) * k + double(m) * n * dtypeSize(cDtype), stream);
#define TTB_TCI(BNv, TCv, PLAINv)                                                        \
  if (pair) return launchTc<BNv, TCv, PLAINv, true, true>(ma, mb, mc, mc, c, p, stream); \
  return launchTc<BNv, TCv, PLAINv, false, true>(ma, mb, mc, mc, c, p, stream)
#define TTB_TCI_BN(TCv, PLAINv)                                                          \
  switch (bn) {                                                                          \
  case 256: TTB_TCI(256, TCv, PLAINv);                                                   \
  case 128: TTB_TCI(128, TCv, PLAINv);                                                   \
  default: TTB_TCI(64, TCv, PLAINv);                                                     \
  }
  // Int32 output: the plain kernel's 32-bit store path moves the accumulator bits unchanged.
  if (cDtype == kI32) { TTB_TCI_BN(float, true) }
  if (cDtype == kF32) { TTB_TCI_BN(float, false) }
  if (cDtype == kBF16) { TTB_TCI_BN(__nv_bfloat16, false) }
  TTB_TCI_BN(__half, false)
#undef TTB_TCI_BN
#undef TTB_TCI
}

// Up to three GEMMs C_i[M, N_i] = A[M, K] B_i[N_i, K]^T that share A (the q / k / v projections of
// one activation) as ONE launch: their tiles form one list, so the narrow problems fill the SMs
// the wide one leaves idle in its last wave.  Plain epilogue only.  -1 = not taken.
// ropeMask != 0: the results of the problems in the mask are rotated in the epilogue (see TcParams::ropeMask).
int gemmTcgen05GroupedTry(const void *a, const void *const *b, void *const *c, const int64_t *n, int count, int abDtype,
                          int cDtype, int64_t m, int64_t k, cudaStream_t stream, const void *ropeCos, const void *ropeSin,
                          int ropeMask, int64_t ropeSeq) {
  if (count < 2 || count > 3) return -1;
  if (ropeMask) {
    if (!ropeCos || !ropeSin || !aligned16(ropeCos) || !aligned16(ropeSin) || ropeSeq < 1 || ropeSeq > 0x7fffffff) return -1;
    if (cDtype != abDtype || (ropeMask >> count) != 0) return -1;
    for (int i = 0; i < count; ++i) {
      if (((ropeMask >> i) & 1) && n[i] % 128 != 0) return -1;
    }
  }
  if (abDtype != kBF16 && abDtype != kF16) return -1;
  if (cDtype != abDtype && cDtype != kF32) return -1;
  if (k % 8 != 0 || m < 1 || k < 8 || m > 0x7fffffff || k > 0x7fffffff || !aligned16(a)) return -1;
  int64_t nSum = 0;
  for (int i = 0; i < count; ++i) {
    if (n[i] < 8 || n[i] > 0x7fffffff || (n[i] * static_cast<int64_t>(dtypeSize(cDtype))) % 16 != 0) return -1;
    if (!aligned16(b[i]) || !aligned16(c[i])) return -1;
    nSum += n[i];
  }
  if (m * nSum * k < (1ll << 18)) return -1;
  const bool pair = pairMmaWanted(m, k);
  const int64_t tileM = pair ? 2 * TC_BM : TC_BM;
  const int workers = pair ? smCount() / 2 : smCount();
  int bn = 64;
  if (forcedTileWidth()) {
    bn = forcedTileWidth();
  } else {
    int64_t best = -1;
    for (int w : {256, 128, 64}) {
      if (ropeMask && w < 128) continue; // a head's two halves have to lie in one tile
      int64_t tiles = 0;
      bool fits = true;
      for (int i = 0; i < count; ++i) {
        if (w > 64 && n[i] < w) fits = false;
        tiles += ((m + tileM - 1) / tileM) * ((n[i] + w - 1) / w);
      }
      if (!fits) continue;
      int64_t waves = (tiles + workers - 1) / workers;
      int64_t cost = waves * tileCost(w, pair);
      if (best < 0 || cost < best) {
        best = cost;
        bn = w;
      }
    }
  }
  CUtensorMap ma, mb[3], mc[3];
  if (!makeMap(&ma, a, abDtype, m, k, TC_BM)) return -1;
  for (int i = 0; i < count; ++i) {
    if (!makeMap(&mb[i], b[i], abDtype, n[i], k, pair ? bn / 2 : bn) || !makeMap(&mc[i], c[i], cDtype, m, n[i], 32)) return -1;
  }
  for (int i = count; i < 3; ++i) {
    mb[i] = mb[0];
    mc[i] = mc[0];
  }
  TcParams p;
  p.M = m; p.N = n[0]; p.K = k;
  p.bias = nullptr; p.biasDt = 0; p.act = TTB_ACT_NONE; p.roundSteps = 0;
  p.extra = nullptr; p.extraOp = 0;
  p.convX = nullptr; p.cTw = 0; p.cTilesM = 0; p.pushRows = 0; p.dual = 0;
  int cum = 0;
  double flops = 0, bytes = double(m) * k * 2;
  for (int i = 0; i < 3; ++i) {
    if (i < count) cum += static_cast<int>((n[i] + bn - 1) / bn);
    p.segCum[i] = cum;
    p.segN[i] = n[i < count ? i : count - 1];
    if (i < count) {
      flops += 2.0 * double(m) * double(n[i]) * double(k);
      bytes += double(n[i]) * k * 2 + double(m) * n[i] * dtypeSize(cDtype);
    }
  }
  p.fmt = abDtype == kBF16 ? 1 : 0;
  p.kElems = TC_BK; p.aSigned = p.bSigned = 0; p.deq = 0; p.deqScalar = 0.0f; p.deqScale = nullptr;
  if (ropeMask) {
    if (bn < 128) return -1; // some problem is narrower than a head
    p.ropeMask = ropeMask;
    p.ropeSeq = static_cast<int>(ropeSeq);
    p.ropeCos = ropeCos;
    p.ropeSin = ropeSin;
    bytes += 2.0 * double(ropeSeq) * 128 * 2;
  }
  ProfScope prof("gemm_tcgen05", flops, bytes, stream);
  const CUtensorMap more[4] = {mb[1], mc[1], mb[2], mc[2]};
#define TTB_TCG(BNv, TCv)                                                                \
  if (pair) return launchTc<BNv, TCv, true, true>(ma, mb[0], mc[0], mc[0], c[0], p, stream, more); \
  return launchTc<BNv, TCv, true>(ma, mb[0], mc[0], mc[0], c[0], p, stream, more)
#define TTB_TCG_BN(TCv)                                                                  \
  switch (bn) {                                                                          \
  case 256: TTB_TCG(256, TCv);                                                           \
  case 128: TTB_TCG(128, TCv);                                                           \
  default: TTB_TCG(64, TCv);                                                             \
  }
  if (cDtype == kBF16) { TTB_TCG_BN(__nv_bfloat16) }
  if (cDtype == kF16) { TTB_TCG_BN(__half) }
  TTB_TCG_BN(float)
#undef TTB_TCG_BN
#undef TTB_TCG
}

// Convolution as an implicit GEMM on the same kernel: the producer warp gathers the receptive
// fields (see the kernel), `wre` is the weight reordered to [O, kH, kW, C].  Returns -1 when the
// problem is outside what this path takes (the caller then materialises the im2col operand).
int convTcgen05Try(const void *x, const void *wre, const void *bias, void *out, int dtype, int biasDtype, int64_t n,
                   int64_t h, int64_t w, int64_t c, int64_t o, int64_t ho, int64_t wo, int kh, int kw, int sh, int sw,
                   int pt, int pl, int dh, int dw, int act, const void *extra, int extraOp, cudaStream_t stream) {
  if (dtype != kBF16 && dtype != kF16) return -1;
  if (c % TC_BK != 0 || o < 8 || (o * 2) % 16 != 0) return -1;
  if (!aligned16(x) || !aligned16(wre) || !aligned16(out) || (extraOp && (!extra || !aligned16(extra)))) return -1;
  const int64_t m = n * ho * wo, k = static_cast<int64_t>(kh) * kw * c;
  if (m < 1 || m > 0x7fffffff || k > 0x7fffffff || h > 32767 || w > 32767 || pt > 8192 || pl > 8192 || pt < 0 || pl < 0) return -1;
  if (n * h * w * c > 0x7fffffff) return -1; // element offsets are kept in 32 bits
  int bn = 64;
  {
    int64_t best = -1;
    for (int wd : {256, 128, 64}) {
      if (wd > 64 && o < wd) continue;
      int64_t tiles = ((m + TC_BM - 1) / TC_BM) * ((o + wd - 1) / wd);
      int64_t waves = (tiles + smCount() - 1) / smCount();
      int64_t cost = waves * (wd + 64);
      if (best < 0 || cost < best) {
        best = cost;
        bn = wd;
      }
    }
  }
  // Stride-1 convolutions run in patch mode; the patch width is the divisor of 32 that wastes
  // the fewest rows on ragged image edges.
  int tw = 0;
  int64_t tilesX = 0, tilesY = 0;
  if (sh == 1 && sw == 1) {
    int64_t best = -1;
    for (int cand : {8, 16, 32, 4}) {
      int64_t tx = (wo + cand - 1) / cand, ty = (ho + (TC_BM / cand) - 1) / (TC_BM / cand);
      if (best < 0 || tx * ty < best) {
        best = tx * ty;
        tw = cand;
        tilesX = tx;
        tilesY = ty;
      }
    }
    if (n * tilesX * tilesY > 0x7fffffff) tw = 0;
  }
  CUtensorMap ma, mb, mc, me;
  if (!makeMap(&mb, wre, dtype, o, k, bn)) return -1;
  if (tw) {
    if (!makeMap4(&ma, x, dtype, c, w, h, n, TC_BK, tw, TC_BM / tw) || !makeMap4(&mc, out, dtype, o, wo, ho, n, 64, tw, 32 / tw))
      return -1;
  } else {
    ma = mb; // not used: the producer warp gathers A
    if (!makeMap(&mc, out, dtype, m, o, 32)) return -1;
  }
  if (extraOp) {
    if (tw ? !makeMap4(&me, extra, dtype, o, wo, ho, n, 64, tw, 32 / tw) : !makeMap(&me, extra, dtype, m, o, 32)) return -1;
  } else {
    me = mc;
  }
  TcParams p;
  p.M = m; p.N = o; p.K = k;
  p.bias = bias; p.biasDt = biasDtype; p.act = act; p.roundSteps = 0;
  p.biasVec = bias && biasDtype == dtype && aligned16(bias) ? 1 : 0;
  p.extra = extraOp ? extra : nullptr;
  p.extraOp = extra ? extraOp : 0;
  p.convX = x;
  p.pushRows = 0;
  p.dual = 0;
  p.cH = static_cast<int>(h); p.cW = static_cast<int>(w); p.cC = static_cast<int>(c);
  p.cHo = static_cast<int>(ho); p.cWo = static_cast<int>(wo);
  p.ckw = kw; p.csh = sh; p.csw = sw; p.cpt = pt; p.cpl = pl; p.cdh = dh; p.cdw = dw;
  p.cTw = tw; p.cTilesX = static_cast<int>(tilesX); p.cTilesY = static_cast<int>(tilesY);
  p.cTilesM = tw ? n * tilesX * tilesY : 0;
  p.segCum[0] = p.segCum[1] = p.segCum[2] = static_cast<int>((o + bn - 1) / bn);
  p.segN[0] = p.segN[1] = p.segN[2] = o;
  p.fmt = dtype == kBF16 ? 1 : 0;
  p.kElems = TC_BK; p.aSigned = p.bSigned = 0; p.deq = 0; p.deqScalar = 0.0f; p.deqScale = nullptr;
  // algorithmic bytes: the input and the output once each (plus the residual operand), the weights
  ProfScope prof("conv2d_tcgen05", 2.0 * double(m) * o * k,
                 (double(n) * h * w * c + double(o) * k + double(m) * o * (extraOp ? 2 : 1)) * 2, stream);
#define TTB_CONV(BNv, TCv) return launchTc<BNv, TCv, false>(ma, mb, mc, me, out, p, stream)
#define TTB_CONV_BN(TCv)                                                                 \
  switch (bn) {                                                                          \
  case 256: TTB_CONV(256, TCv);                                                          \
  case 128: TTB_CONV(128, TCv);                                                          \
  default: TTB_CONV(64, TCv);                                                            \
  }
  if (dtype == kBF16) { TTB_CONV_BN(__nv_bfloat16) }
  TTB_CONV_BN(__half)
#undef TTB_CONV_BN
#undef TTB_CONV
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

namespace ttb {
int sdpaTcgen05StatusAccess(int *status, const int *newValue, const long long *waitCycles);
}

// Both tensor-core kernels' status words of the current device in one call, without a device-wide
// synchronise (the caller has synchronised the streams it cares about).  clear != 0 resets a word
// that was set, so one timeout is reported once.
extern "C" int ttb_tcgen05_status(int *gemm_status, int *sdpa_status, int clear) {
  int g = 0, a = 0;
  TTB_CUDA(cudaMemcpyFromSymbol(&g, ttb::g_tcStatus, sizeof(int)));
  int rc = ttb::sdpaTcgen05StatusAccess(&a, nullptr, nullptr);
  if (rc) return rc;
  const int zero = 0;
  if (clear && g) TTB_CUDA(cudaMemcpyToSymbol(ttb::g_tcStatus, &zero, sizeof(int)));
  if (clear && a) {
    rc = ttb::sdpaTcgen05StatusAccess(nullptr, &zero, nullptr);
    if (rc) return rc;
  }
  if (gemm_status) *gemm_status = g;
  if (sdpa_status) *sdpa_status = a;
  return TTB_OK;
}

// Writes the status words as a timed-out launch would (or clears them with zeros).  Exists so that
// the reporting path above the kernels can be exercised without making a GPU wait run out.
extern "C" int ttb_tcgen05_set_status(int gemm_status, int sdpa_status) {
  TTB_CUDA(cudaMemcpyToSymbol(ttb::g_tcStatus, &gemm_status, sizeof(int)));
  return ttb::sdpaTcgen05StatusAccess(nullptr, &sdpa_status, nullptr);
}

// The limit of every bounded wait in the tensor-core kernels on the current device, in SM clock
// cycles; cycles <= 0 restores the default (2e9, about a second).
extern "C" int ttb_tcgen05_set_wait_limit(long long cycles) {
  if (cycles <= 0) cycles = 2000000000ll;
  TTB_CUDA(cudaMemcpyToSymbol(ttb::g_tcWaitCycles, &cycles, sizeof(cycles)));
  return ttb::sdpaTcgen05StatusAccess(nullptr, nullptr, &cycles);
}
