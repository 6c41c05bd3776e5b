// Flash attention on the 5th-generation tensor cores: out = softmax(q k^T * scale [+ causal]) v
// for 16-bit q/k/v with head_dim 128 and no explicit mask tensor (semantics:
// include/ttmlir/Dialect/TTNN/IR/TTNNOps.td ScaledDotProductAttentionOp, golden
// tools/golden/mapping.py:8398-8500).
//
// One CTA owns 128 query rows of one head and walks the key/value sequence in tiles of 128:
//   warp 0      TMA producer: Q once, then K and V tiles through two-stage rings
//   warp 1      issues tcgen05.mma: S = Q K^T into one of two TMEM buffers, then O += P V
//   warps 2..9  two threads per query row (one takes keys 0..63 of a tile, the other 64..127):
//               read S from TMEM, online softmax in f32, write the probabilities P (16-bit)
//               into shared memory in the operand layout of the second contraction; O stays in
//               TMEM and is rescaled there only when the row maximum has grown by more than a
//               factor 2^8 since the last rescale.  Two warps per scheduler hide each other's
//               instruction latencies, which is what bounds this kernel.
// S_{j+1} is issued before P_j V_j, so the tensor pipe computes the next scores while the
// softmax warps work on the current ones.  V tiles are used as loaded ([key][d] rows) through
// an MN-major operand descriptor; nothing is transposed.
//
// TMEM: columns 0..127 and 128..255 hold S (double buffer), 256..383 hold O.
// Shared memory (each tile 128 x 128 x 2 B = 32 KiB, stored as two 64-column swizzled halves):
//   Q | K0 | K1 | V0 | V1 | P | barriers.
// Every wait is bounded; a wait that runs out records its site in the status word, the CTA
// drains and returns, and ttb_sdpa_tcgen05_status reports it.
#include "common.cuh"
#include "tcgen05.cuh"

#include <algorithm>

#include <cstdlib>

namespace ttb {

constexpr int AT_BM = 128;
constexpr int AT_BN = 128;
constexpr int AT_D = 128;
constexpr int AT_THREADS = 320; // TMA warp, MMA warp, two softmax groups of four warps
constexpr int AT_TILE = AT_BM * AT_D * 2; // bytes
constexpr int AT_HALF = AT_TILE / 2;
constexpr int AT_TMEM_COLS = 512;
constexpr int AT_SMEM = 6 * AT_TILE + 1024 /* alignment slack */ + 256 /* barriers */;

struct AtParams {
  int64_t Hq, Hkv, Sq, Skv;
  int64_t ob, oh, os; // element strides of out over batch, head, query row
  int causal;
  int causalOff; // under a causal mask, query row r sees keys 0 .. r + causalOff (a prefill chunk that starts at causalOff)
  int fmt; // 1 bf16, 0 f16
  float scaleLog2;
  // Split mode (few heads: fewer query blocks than SMs, and a causal block's work grows with its
  // index): a query block's key tiles are cut into pieces of at most splitLen tiles, one CTA per
  // piece; pieceStart[qb] is the first piece of query block qb (pieceStart[nQ] = pieces per head).
  // A piece stores its unnormalised O (f32), row maxima and row sums; sdpaMergeKernel combines
  // them.  splitLen = 0: one CTA per query block, which writes the result itself.
  int splitLen;
  unsigned short pieceStart[66];
  float *partO, *partM, *partL;
};

__device__ __forceinline__ float fastExp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Blackwell's two-wide f32 arithmetic and three-input maximum: half the instructions for the softmax's scaling,
// summing and maximum, which matters because these warps are bound by instruction issue latency, not by a pipe
// (0.36 instructions issued per cycle and scheduler, 2.5 warps each).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack2(float x, float y) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
  return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t x, uint32_t y) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(x), "r"(y));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t r, float &x, float &y) { asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(r)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <typename T> __device__ __forceinline__ uint32_t packPair(float a, float b);
template <> __device__ __forceinline__ uint32_t packPair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t packPair<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&v);
}

template <typename T>
__global__ void __launch_bounds__(AT_THREADS, 1)
    sdpaTcgen05Kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapV, T *__restrict__ out, AtParams p) {
  extern __shared__ unsigned char smemRaw[];
  __shared__ uint32_t tmemBaseSlot;
  __shared__ int abortFlag;
  __shared__ float xchg[2][2][AT_BM]; // [exchange parity][group][row]: what the two threads of a query row tell each other

  const uint32_t base = (smemU32(smemRaw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = base + AT_TILE, sV = base + 3 * AT_TILE, sP = base + 5 * AT_TILE;
  const uint32_t bars = base + 6 * AT_TILE;
  const uint32_t qFull = bars, kFull = bars + 8, kEmpty = bars + 24, vFull = bars + 40, vEmpty = bars + 56,
                 sFull = bars + 72, sEmpty = bars + 88, pReady = bars + 104, pEmpty = bars + 112, xBar = bars + 120;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nQ = (p.Sq + AT_BM - 1) / AT_BM;
  const int64_t perHead = p.splitLen ? p.pieceStart[nQ] : nQ; // CTAs per (batch, head)
  const int64_t BH = static_cast<int64_t>(gridDim.x) / perHead;
  int qb, piece = 0;
  if (p.splitLen) {
    const int pi = static_cast<int>(blockIdx.x / BH);
    qb = 0;
    while (qb + 1 < nQ && p.pieceStart[qb + 1] <= pi) ++qb;
    piece = pi - p.pieceStart[qb];
  } else {
    // Heaviest (latest, under a causal mask) query blocks first.
    qb = static_cast<int>(nQ - 1 - blockIdx.x / BH);
  }
  const int bh = static_cast<int>(blockIdx.x % BH);
  const int b = static_cast<int>(bh / p.Hq), h = static_cast<int>(bh % p.Hq);
  const int hkv = static_cast<int>(h / (p.Hq / p.Hkv));
  const int q0 = qb * AT_BM;
  int nAll = static_cast<int>((p.Skv + AT_BN - 1) / AT_BN); // key tiles this query block sees
  if (p.causal) {
    int lim = (q0 + AT_BM - 1 + p.causalOff) / AT_BN + 1;
    nAll = nAll < lim ? nAll : lim;
  }
  // this CTA's tiles: [t0, t0 + nT)
  const int t0 = p.splitLen ? piece * p.splitLen : 0;
  const int nT = p.splitLen ? (nAll - t0 < p.splitLen ? nAll - t0 : p.splitLen) : nAll;

  if (threadIdx.x == 0) {
    abortFlag = 0;
    mbarInit(qFull, 1);
    for (int i = 0; i < 2; ++i) {
      mbarInit(kFull + 8 * i, 1);
      mbarInit(kEmpty + 8 * i, 1);
      mbarInit(vFull + 8 * i, 1);
      mbarInit(vEmpty + 8 * i, 1);
      mbarInit(sFull + 8 * i, 1);
      mbarInit(sEmpty + 8 * i, 256);
    }
    mbarInit(pReady, 256);
    mbarInit(pEmpty, 1);
    mbarInit(xBar, 256);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&tmemBaseSlot)), "r"(AT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = tmemBaseSlot;
  pdlLaunchDependents(); // the prologue above touched no global memory
  pdlWait();
  volatile int *abortP = &abortFlag;

  if (warp == 0) {
    if (lane == 0) {
      prefetchTensorMap(&mapQ);
      prefetchTensorMap(&mapK);
      prefetchTensorMap(&mapV);
      mbarArriveExpectTx(qFull, AT_TILE);
      tmaLoad4d(sQ, &mapQ, qFull, 0, q0, h, b);
      tmaLoad4d(sQ + AT_HALF, &mapQ, qFull, 64, q0, h, b);
      for (int j = 0; j < nT; ++j) {
        const int s = j & 1, ph = (j >> 1) & 1;
        if (!mbarWait(kEmpty + 8 * s, ph ^ 1, abortP, 1)) break;
        mbarArriveExpectTx(kFull + 8 * s, AT_TILE);
        tmaLoad4d(sK + s * AT_TILE, &mapK, kFull + 8 * s, 0, (t0 + j) * AT_BN, hkv, b);
        tmaLoad4d(sK + s * AT_TILE + AT_HALF, &mapK, kFull + 8 * s, 64, (t0 + j) * AT_BN, hkv, b);
        if (!mbarWait(vEmpty + 8 * s, ph ^ 1, abortP, 2)) break;
        mbarArriveExpectTx(vFull + 8 * s, AT_TILE);
        tmaLoad4d(sV + s * AT_TILE, &mapV, vFull + 8 * s, 0, (t0 + j) * AT_BN, hkv, b);
        tmaLoad4d(sV + s * AT_TILE + AT_HALF, &mapV, vFull + 8 * s, 64, (t0 + j) * AT_BN, hkv, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idS = instrDescF16(p.fmt, AT_BM, AT_BN, 0, 0);
      const uint32_t idPV = instrDescF16(p.fmt, AT_BM, AT_D, 0, 1);
      bool ok = mbarWait(qFull, 0, abortP, 3);
      // S_j = Q K_j^T: eight steps of 16 along d; both operands K-major.
      auto issueS = [&](int j) -> bool {
        const int s = j & 1, ph = (j >> 1) & 1;
        if (!mbarWait(kFull + 8 * s, ph, abortP, 4)) return false;
        if (!mbarWait(sEmpty + 8 * s, ph ^ 1, abortP, 5)) return false;
        tcFenceAfter();
        const uint32_t kb = sK + s * AT_TILE;
#pragma unroll
        for (int ks = 0; ks < AT_D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * AT_HALF + (ks & 3) * 32;
          tcMma(tmemBase + s * AT_BN, smemDescSw128(sQ + off, 0, 1024), smemDescSw128(kb + off, 0, 1024), idS, ks > 0);
        }
        tcCommit(kEmpty + 8 * s);
        tcCommit(sFull + 8 * s);
        return true;
      };
      if (ok && nT > 0) ok = issueS(0);
      for (int j = 0; ok && j < nT; ++j) {
        if (j + 1 < nT && !issueS(j + 1)) break;
        const int s = j & 1, ph = (j >> 1) & 1;
        if (!mbarWait(vFull + 8 * s, ph, abortP, 6)) break;
        if (!mbarWait(pReady, j & 1, abortP, 7)) break;
        tcFenceAfter();
        // O += P V_j: eight steps of 16 keys.  P is K-major (keys along its rows); V is
        // MN-major: 128-byte rows of 64 d values, one row per key, the second 64 d values one
        // half tile further on.
        const uint32_t vb = sV + s * AT_TILE;
#pragma unroll
        for (int ks = 0; ks < AT_BN / 16; ++ks) {
          const uint32_t offP = (ks >> 2) * AT_HALF + (ks & 3) * 32;
          tcMma(tmemBase + 2 * AT_BN, smemDescSw128(sP + offP, 0, 1024), smemDescSw128(vb + ks * 2048, AT_HALF, 1024),
                idPV, (j | ks) > 0);
        }
        tcCommit(vEmpty + 8 * s);
        tcCommit(pEmpty);
      }
    }
  } else {
    // Softmax / accumulation.  TMEM lanes are reachable per warp quarter (warp id mod 4), so the
    // two warps with the same quarter share 32 query rows: warp group `wg` takes keys
    // [64 wg, 64 wg + 64) of every score tile and columns [64 wg, 64 wg + 64) of O.  A row's two
    // threads agree on the reference maximum once per tile through shared memory.
    const int wg = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int64_t qrow = static_cast<int64_t>(q0) + row;
    const uint32_t laneAddr = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16);
    const float sl2 = p.scaleLog2;
    // `m` is the reference maximum the exponentials are taken against.  It follows the true row
    // maximum lazily: it moves (and O and the row sum are rescaled) only when the maximum grew
    // by more than 2^kLazy in the exponent, so most tiles skip the rescale and P stays <= 2^kLazy.
    constexpr float kLazy = 8.0f;
    constexpr int HALF = AT_BN / 2;
    float m = 0.0f, l = 0.0f;
    const uint32_t oAddr = laneAddr + 2 * AT_BN + wg * HALF;
    const uint32_t pRow = sP + wg * AT_HALF + row * 128; // this group's keys are one swizzled half of P
    const uint32_t swz = static_cast<uint32_t>(row & 7);
    uint32_t xPhase = 0;
    bool ok = true;
    // Both threads of a row have published their value for this step (bounded like every wait).
    auto exchange = [&](float mine) -> float {
      // Slots alternate with the exchange's parity: a slot is rewritten two exchanges later, by
      // which time its reader has gone through the barrier in between.
      xchg[xPhase][wg][row] = mine;
      mbarArrive(xBar); // release: the store above is visible to whoever observes the phase flip
      const bool fine = __all_sync(0xffffffffu, mbarWait(xBar, xPhase, abortP, 12));
      const float other = xchg[xPhase][wg ^ 1][row];
      xPhase ^= 1u;
      if (!fine) ok = false;
      return other;
    };
    // The TMEM loads are warp-wide: a warp leaves the loop together or not at all.
    for (int j = 0; j < nT && ok; ++j) {
      const int s = j & 1, ph = (j >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbarWait(sFull + 8 * s, ph, abortP, 9))) { ok = false; break; }
      tcFenceAfter();
      const uint32_t sAddr = laneAddr + s * AT_BN + wg * HALF;
      const int key0 = (t0 + j) * AT_BN + wg * HALF;
      const bool needMask = (p.causal && key0 + HALF - 1 > q0 + p.causalOff) || key0 + HALF > p.Skv;
      // Last visible key of this row inside this half tile (relative, may be negative or >= 64).
      int64_t lastKey = p.Skv - 1;
      if (p.causal && qrow + p.causalOff < lastKey) lastKey = qrow + p.causalOff;
      const int lastRel = static_cast<int>(lastKey - key0 < HALF ? lastKey - key0 : HALF);
      // This thread's 64 scores are read from TMEM once (both loads in flight together) and stay
      // in registers for the maximum and for the exponentials.
      uint32_t sc[2][32];
      tcLoad32(sAddr, sc[0]);
      tcLoad32(sAddr + 32, sc[1]);
      tcWaitLd();
      tcFenceBefore();
      mbarArrive(sEmpty + 8 * s); // the score buffer can take the tile after next
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (needMask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, c * 32 + i <= lastRel ? __uint_as_float(sc[c][i]) : -INFINITY);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sc[c][i]));
        }
      }
      mx = fmaxf(mx, exchange(mx)); // the whole row's maximum in this tile, the same in both threads
      if (!ok) break;
      float corr = 1.0f;
      if (j == 0) {
        m = mx == -INFINITY ? 0.0f : mx;
      } else if ((mx - m) * sl2 > kLazy) {
        corr = fastExp2((m - mx) * sl2);
        m = mx;
      }
      // P's buffer is free, and O holds every earlier tile, once P V_{j-1} has completed.
      if (!__all_sync(0xffffffffu, mbarWait(pEmpty, (j & 1) ^ 1, abortP, 10))) { ok = false; break; }
      if (__any_sync(0xffffffffu, corr != 1.0f)) {
        tcFenceAfter();
        l *= corr;
#pragma unroll
        for (int c = 0; c < HALF / 32; ++c) {
          uint32_t r[32];
          tcLoad32(oAddr + c * 32, r);
          tcWaitLd();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
          tcStore32(oAddr + c * 32, r);
        }
        tcWaitSt();
      }
      const float negM = -m * sl2;
      // Pass 2: probabilities, their sum, and P in the swizzled K-major operand layout.
      float sum = 0.0f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a = fastExp2(fmaf(__uint_as_float(sc[c][i]), sl2, negM));
          float bb = fastExp2(fmaf(__uint_as_float(sc[c][i + 1]), sl2, negM));
          if (needMask) {
            a = c * 32 + i <= lastRel ? a : 0.0f;
            bb = c * 32 + i + 1 <= lastRel ? bb : 0.0f;
          }
          sum += a + bb;
          w[i >> 1] = packPair<T>(a, bb);
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t chunk = static_cast<uint32_t>(c * 4 + q4);
          const uint32_t addr = pRow + ((chunk ^ swz) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[q4 * 4]), "r"(w[q4 * 4 + 1]),
                       "r"(w[q4 * 4 + 2]), "r"(w[q4 * 4 + 3]) : "memory");
        }
      }
      l += sum;
      fenceProxyAsyncShared();
      mbarArrive(pReady);
    }
    // The last P V has to land before O is read; the row sum is the two halves' sums.
    if (ok && nT > 0 && !__all_sync(0xffffffffu, mbarWait(pEmpty, (nT & 1) ^ 1, abortP, 11))) ok = false;
    if (ok) l += exchange(l);
    if (ok && p.splitLen) {
      // this piece's partial result: O as accumulated (f32), the reference maximum and the row sum
      tcFenceAfter();
      const size_t pieceIdx = static_cast<size_t>(bh) * p.pieceStart[nQ] + p.pieceStart[qb] + piece;
      float *po = p.partO + (pieceIdx * AT_BM + row) * AT_D + wg * HALF;
#pragma unroll
      for (int c = 0; c < HALF / 32; ++c) {
        uint32_t r[32];
        tcLoad32(oAddr + c * 32, r);
        tcWaitLd();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          *reinterpret_cast<uint4 *>(po + c * 32 + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
        }
      }
      if (wg == 0) {
        p.partM[pieceIdx * AT_BM + row] = m;
        p.partL[pieceIdx * AT_BM + row] = l;
      }
    } else if (ok) {
      tcFenceAfter();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      T *orow = out + b * p.ob + h * p.oh + qrow * p.os + wg * HALF;
#pragma unroll
      for (int c = 0; c < HALF / 32; ++c) {
        uint32_t r[32];
        tcLoad32(oAddr + c * 32, r);
        tcWaitLd();
        if (qrow < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = packPair<T>(__uint_as_float(r[g * 8]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
            v.y = packPair<T>(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
            v.z = packPair<T>(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
            v.w = packPair<T>(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4 *>(orow + c * 32 + g * 8) = v;
          }
        }
      }
    }
  }

  tcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcFenceAfter();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(AT_TMEM_COLS) : "memory");
  }
}

// ---- two query heads per CTA ---------------------------------------------------------------------
// With grouped-query attention the heads of a group read the same K and V.  The kernel above
// streams K/V once per (head, query block) and ends up limited by L2 -> SM bandwidth (4.5 TB/s
// at the decoder shape).  This one gives a CTA the same 128 query rows of TWO heads of a group:
// every K/V tile (64 keys, four-stage rings) is loaded once and used by both heads, which halves
// that traffic, and each head has its own softmax warp group, score buffers (two per head) and
// output accumulator in TMEM, so the two heads' softmax and contractions interleave.  The probabilities never touch
// shared memory: a softmax thread packs its row's 64 values to 16 bits and writes them over the first 32 columns of
// the score buffer they came from, and O += P V reads them from there as the tensor-memory A operand.
//   TMEM: S(head, buffer) at 64 * (2 head + buffer) (P over its first 32 columns), O(head) at 256 + 128 head.
//   Shared memory: Q_A | Q_B (32 KiB each) | K x4 | V x4 (16 KiB each) | barriers.
// Measured with parts of the kernel switched off (decoder shape, 58 us whole): without the exponentials 59 us,
// without the score loads 58 us, without P V 50 us, without Q K^T 48 us, without any contraction 44 us.  So
// neither the special-function unit nor the tensor pipe nor shared-memory bandwidth (P in shared memory cost
// 1 us more) is what the launch waits for: three quarters of it is the per-tile hand-over between the softmax
// warps, the issuing thread and the TMA ring, plus the tail of the 1.7 waves of unequal (causal) CTAs.
constexpr int AP_BN = 64;
constexpr int AP_STAGES = 4;
constexpr int AP_KV = AP_BN * AT_D * 2;  // bytes of a K or V tile
constexpr int AP_SMEM = 2 * AT_TILE + 2 * AP_STAGES * AP_KV + 1024 + 256;

template <typename T>
__global__ void __launch_bounds__(AT_THREADS, 1)
    sdpaTcgen05PairKernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                          const __grid_constant__ CUtensorMap mapV, T *__restrict__ out, AtParams p) {
  extern __shared__ unsigned char smemRaw[];
  __shared__ uint32_t tmemBaseSlot;
  __shared__ int abortFlag;

  const uint32_t base = (smemU32(smemRaw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = base + 2 * AT_TILE, sV = sK + AP_STAGES * AP_KV;
  const uint32_t bars = sV + AP_STAGES * AP_KV;
  const uint32_t qFull = bars, kFull = bars + 8, kEmpty = kFull + 8 * AP_STAGES, vFull = kEmpty + 8 * AP_STAGES,
                 vEmpty = vFull + 8 * AP_STAGES, sFull = vEmpty + 8 * AP_STAGES, sEmpty = sFull + 32, pReady = sEmpty + 32,
                 pEmpty = pReady + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = static_cast<int>(p.Hq / p.Hkv), pairs = G / 2;
  const int64_t nQ = (p.Sq + AT_BM - 1) / AT_BM;
  const int64_t perQ = static_cast<int64_t>(gridDim.x) / nQ; // batch * kv heads * pairs
  const int qb = static_cast<int>(nQ - 1 - blockIdx.x / perQ); // heaviest query blocks first
  const int rem = static_cast<int>(blockIdx.x % perQ);
  const int b = rem / static_cast<int>(p.Hkv * pairs), r2 = rem % static_cast<int>(p.Hkv * pairs);
  const int hk = r2 / pairs, hA = hk * G + 2 * (r2 % pairs);
  const int q0 = qb * AT_BM;
  int nT = static_cast<int>((p.Skv + AP_BN - 1) / AP_BN);
  if (p.causal) {
    int lim = (q0 + AT_BM - 1 + p.causalOff) / AP_BN + 1;
    nT = nT < lim ? nT : lim;
  }

  if (threadIdx.x == 0) {
    abortFlag = 0;
    mbarInit(qFull, 1);
    for (int i = 0; i < AP_STAGES; ++i) {
      mbarInit(kFull + 8 * i, 1);
      mbarInit(kEmpty + 8 * i, 1);
      mbarInit(vFull + 8 * i, 1);
      mbarInit(vEmpty + 8 * i, 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbarInit(sFull + 8 * i, 1);
      mbarInit(sEmpty + 8 * i, 4); // one arrival per softmax warp (its lane 0, after the warp has synchronised)
    }
    for (int i = 0; i < 2; ++i) {
      mbarInit(pReady + 8 * i, 4);
      mbarInit(pEmpty + 8 * i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemU32(&tmemBaseSlot)), "r"(AT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = tmemBaseSlot;
  pdlLaunchDependents(); // the prologue above touched no global memory
  pdlWait();
  volatile int *abortP = &abortFlag;

  if (warp == 0) {
    if (lane == 0) {
      prefetchTensorMap(&mapQ);
      prefetchTensorMap(&mapK);
      prefetchTensorMap(&mapV);
      mbarArriveExpectTx(qFull, 2 * AT_TILE);
      for (int hd = 0; hd < 2; ++hd) {
        tmaLoad4d(sQ + hd * AT_TILE, &mapQ, qFull, 0, q0, hA + hd, b);
        tmaLoad4d(sQ + hd * AT_TILE + AT_HALF, &mapQ, qFull, 64, q0, hA + hd, b);
      }
      for (int j = 0; j < nT; ++j) {
        const int st = j % AP_STAGES, ph = (j / AP_STAGES) & 1;
        if (!mbarWait(kEmpty + 8 * st, ph ^ 1, abortP, 1)) break;
        mbarArriveExpectTx(kFull + 8 * st, AP_KV);
        tmaLoad4d(sK + st * AP_KV, &mapK, kFull + 8 * st, 0, j * AP_BN, hk, b);
        tmaLoad4d(sK + st * AP_KV + AP_KV / 2, &mapK, kFull + 8 * st, 64, j * AP_BN, hk, b);
        if (!mbarWait(vEmpty + 8 * st, ph ^ 1, abortP, 2)) break;
        mbarArriveExpectTx(vFull + 8 * st, AP_KV);
        tmaLoad4d(sV + st * AP_KV, &mapV, vFull + 8 * st, 0, j * AP_BN, hk, b);
        tmaLoad4d(sV + st * AP_KV + AP_KV / 2, &mapV, vFull + 8 * st, 64, j * AP_BN, hk, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idS = instrDescF16(p.fmt, AT_BM, AP_BN, 0, 0);
      const uint32_t idPV = instrDescF16(p.fmt, AT_BM, AT_D, 0, 1);
      bool ok = mbarWait(qFull, 0, abortP, 3);
      // S_hd(j) = Q_hd K_j^T for both heads: eight steps of 16 along d, both operands K-major.
      auto issueS = [&](int j) -> bool {
        const int st = j % AP_STAGES, ph = (j / AP_STAGES) & 1, buf = j & 1, bph = (j >> 1) & 1;
        if (!mbarWait(kFull + 8 * st, ph, abortP, 4)) return false;
        const uint32_t kb = sK + st * AP_KV;
        for (int hd = 0; hd < 2; ++hd) {
          if (!mbarWait(sEmpty + 8 * (hd * 2 + buf), bph ^ 1, abortP, 5)) return false;
          tcFenceAfter();
#pragma unroll
          for (int ks = 0; ks < AT_D / 16; ++ks) {
            const uint32_t offQ = hd * AT_TILE + (ks >> 2) * AT_HALF + (ks & 3) * 32;
            const uint32_t offK = (ks >> 2) * (AP_KV / 2) + (ks & 3) * 32;
            tcMma(tmemBase + (hd * 2 + buf) * AP_BN, smemDescSw128(sQ + offQ, 0, 1024), smemDescSw128(kb + offK, 0, 1024), idS,
                  ks > 0);
          }
          tcCommit(sFull + 8 * (hd * 2 + buf));
        }
        tcCommit(kEmpty + 8 * st);
        return true;
      };
      if (ok && nT > 0) ok = issueS(0);
      for (int j = 0; ok && j < nT; ++j) {
        if (j + 1 < nT && !issueS(j + 1)) break;
        const int st = j % AP_STAGES, ph = (j / AP_STAGES) & 1;
        if (!mbarWait(vFull + 8 * st, ph, abortP, 6)) break;
        const uint32_t vb = sV + st * AP_KV;
        bool fine = true;
        for (int hd = 0; hd < 2 && fine; ++hd) {
          if (!mbarWait(pReady + 8 * hd, j & 1, abortP, 7)) { fine = false; break; }
          tcFenceAfter();
          // O_hd += P_hd V_j: four steps of 16 keys.  P is read from tensor memory, where the softmax warps wrote
          // it over the first 32 columns of the score buffer it came from (row i in lane i, keys 2c and 2c + 1 in
          // column c); V is MN-major: 128-byte rows of 64 d values, one row per key, the second 64 d values half a
          // tile further on.  The next scores for this buffer, S_{j+2}, are issued after these products and the
          // tensor pipe runs one thread's contractions in issue order, so P is consumed before it is overwritten.
#pragma unroll
          for (int ks = 0; ks < AP_BN / 16; ++ks) {
            tcMmaTmemA(tmemBase + 4 * AP_BN + hd * AT_D, tmemBase + (hd * 2 + (j & 1)) * AP_BN + ks * 8,
                       smemDescSw128(vb + ks * 2048, AP_KV / 2, 1024), idPV, (j | ks) > 0);
          }
          tcCommit(pEmpty + 8 * hd);
        }
        if (!fine) break;
        tcCommit(vEmpty + 8 * st);
      }
    }
  } else {
    // Softmax / accumulation: warp group `hd` owns head hA + hd, one query row per thread.
    const int hd = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int64_t qrow = static_cast<int64_t>(q0) + row;
    const uint32_t laneAddr = tmemBase + (static_cast<uint32_t>(quarter * 32) << 16);
    const float sl2 = p.scaleLog2;
    constexpr float kLazy = 8.0f; // see the single-head kernel
    float m = 0.0f, l = 0.0f;
    const uint32_t oAddr = laneAddr + 4 * AP_BN + hd * AT_D;
    bool ok = true;
    for (int j = 0; j < nT; ++j) {
      const int buf = j & 1, bph = (j >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbarWait(sFull + 8 * (hd * 2 + buf), bph, abortP, 9))) { ok = false; break; }
      tcFenceAfter();
      const uint32_t sAddr = laneAddr + (hd * 2 + buf) * AP_BN;
      const int key0 = j * AP_BN;
      const bool needMask = (p.causal && key0 + AP_BN - 1 > q0 + p.causalOff) || key0 + AP_BN > p.Skv;
      int64_t lastKey = p.Skv - 1;
      if (p.causal && qrow + p.causalOff < lastKey) lastKey = qrow + p.causalOff;
      const int lastRel = static_cast<int>(lastKey - key0 < AP_BN ? lastKey - key0 : AP_BN);
      // This thread's 64 scores are read from TMEM once (both loads in flight together) and stay
      // in registers for the maximum and for the exponentials.
      uint32_t sc[2][32];
      tcLoad32(sAddr, sc[0]);
      tcLoad32(sAddr + 32, sc[1]);
      tcWaitLd();
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(sEmpty + 8 * (hd * 2 + buf)); // the score buffer can take the tile after next
      // Four independent chains: a single running maximum is 64 dependent instructions.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (needMask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], c * 32 + i <= lastRel ? __uint_as_float(sc[c][i]) : -INFINITY);
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) mx4[q4] = max3(mx4[q4], __uint_as_float(sc[c][i + q4]), __uint_as_float(sc[c][i + 4 + q4]));
          }
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float corr = 1.0f;
      if (j == 0) {
        m = mx == -INFINITY ? 0.0f : mx;
      } else if ((mx - m) * sl2 > kLazy) {
        corr = fastExp2((m - mx) * sl2);
        m = mx;
      }
      // The probabilities are computed into registers first: P's buffer and O are only touched once P V_{j-1}
      // has completed, and that contraction runs while these exponentials do.
      const float negM = -m * sl2;
      const uint64_t sl2x2 = pack2(sl2, sl2), negMx2 = pack2(negM, negM);
      uint64_t sumx2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
      uint32_t w[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float ta, tb;
          unpack2(fma2(pack2u(sc[c][i], sc[c][i + 1]), sl2x2, negMx2), ta, tb);
          float a = fastExp2(ta), bb = fastExp2(tb);
          if (needMask) {
            a = c * 32 + i <= lastRel ? a : 0.0f;
            bb = c * 32 + i + 1 <= lastRel ? bb : 0.0f;
          }
          sumx2[(i >> 1) & 1] = add2(sumx2[(i >> 1) & 1], pack2(a, bb));
          w[c * 16 + (i >> 1)] = packPair<T>(a, bb);
        }
      }
      float s0, s1, s2, s3;
      unpack2(sumx2[0], s0, s1);
      unpack2(sumx2[1], s2, s3);
      const float sum = (s0 + s1) + (s2 + s3);
      // O may only be rescaled once P V_{j-1} has completed (P itself goes into this tile's own score buffer and
      // would not need the wait).  Every warp waits, rescale or not: a warp that ran ahead would arrive on pReady
      // for tile j + 1 while slower warps still owe their arrival for tile j, and the barrier would count it as theirs.
      if (!__all_sync(0xffffffffu, mbarWait(pEmpty + 8 * hd, (j & 1) ^ 1, abortP, 10))) { ok = false; break; }
      if (__any_sync(0xffffffffu, corr != 1.0f)) {
        tcFenceAfter();
        l *= corr;
#pragma unroll
        for (int c = 0; c < AT_D / 32; ++c) {
          uint32_t r[32];
          tcLoad32(oAddr + c * 32, r);
          tcWaitLd();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
          tcStore32(oAddr + c * 32, r);
        }
      }
      tcStore32(sAddr, w);
      tcWaitSt();
      tcFenceBefore();
      l += sum;
      __syncwarp();
      if (lane == 0) mbarArrive(pReady + 8 * hd);
    }
    if (ok && nT > 0 && !__all_sync(0xffffffffu, mbarWait(pEmpty + 8 * hd, (nT & 1) ^ 1, abortP, 11))) ok = false;
    if (ok) {
      tcFenceAfter();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      T *orow = out + b * p.ob + (hA + hd) * p.oh + qrow * p.os;
#pragma unroll
      for (int c = 0; c < AT_D / 32; ++c) {
        uint32_t r[32];
        tcLoad32(oAddr + c * 32, r);
        tcWaitLd();
        if (qrow < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = packPair<T>(__uint_as_float(r[g * 8]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
            v.y = packPair<T>(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
            v.z = packPair<T>(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
            v.w = packPair<T>(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4 *>(orow + c * 32 + g * 8) = v;
          }
        }
      }
    }
  }

  tcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcFenceAfter();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(AT_TMEM_COLS) : "memory");
  }
}

// [batch, heads, seq, 128] 16-bit tensor addressed through element strides, box = 64 columns x
// `boxRows` rows of one head, 128-byte swizzle; rows past the end of a head read as zero.
static bool makeHeadMap(CUtensorMap *map, const void *ptr, int dtype, int64_t batch, int64_t heads, int64_t seq,
                        const int64_t *strides3, int boxRows = AT_BM) {
  EncodeTiledFn fn = encodeTiled();
  if (!fn) return false;
  cuuint64_t dims[4] = {AT_D, static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  // A dimension of extent 1 never advances; give it a stride the encoder accepts.
  auto bytes = [&](int64_t s, cuuint64_t fallback) { return s > 0 ? static_cast<cuuint64_t>(s) * 2 : fallback; };
  cuuint64_t sSeq = bytes(strides3[2], AT_D * 2);
  cuuint64_t sHead = bytes(strides3[1], sSeq * static_cast<cuuint64_t>(seq));
  cuuint64_t sBatch = bytes(strides3[0], sHead * static_cast<cuuint64_t>(heads));
  cuuint64_t strides[3] = {sSeq, sHead, sBatch};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(boxRows), 1, 1};
  cuuint32_t elemStrides[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <typename T>
static int launchPair(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, void *out, const AtParams &p,
                      unsigned grid, cudaStream_t st) {
  static bool attrSet[64] = {}; // function attributes belong to a device
  int dev = 0;
  TTB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attrSet[dev]) {
    TTB_CUDA(cudaFuncSetAttribute(sdpaTcgen05PairKernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, AP_SMEM));
    attrSet[dev] = true;
  }
  TTB_CUDA(launchPdl(sdpaTcgen05PairKernel<T>, dim3(grid), dim3(AT_THREADS), AP_SMEM, st, mq, mk, mv, static_cast<T *>(out), p));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// Combines the pieces of a query block (split mode): one warp per query row, lane = 4 head dims.
template <typename T>
__global__ void __launch_bounds__(256) sdpaMergeKernel(T *__restrict__ out, AtParams p, int rows) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int64_t nQ = (p.Sq + AT_BM - 1) / AT_BM;
  const int bh = static_cast<int>(r / (nQ * AT_BM)), rem = static_cast<int>(r % (nQ * AT_BM));
  const int qb = rem / AT_BM, row = rem % AT_BM;
  const int64_t qrow = static_cast<int64_t>(qb) * AT_BM + row;
  if (qrow >= p.Sq) return;
  const int first = p.pieceStart[qb], count = p.pieceStart[qb + 1] - first;
  const size_t base = static_cast<size_t>(bh) * p.pieceStart[nQ] + first;
  // pieces with an empty row sum saw no visible key and carry no maximum
  float mx = -INFINITY;
  for (int k = 0; k < count; ++k) {
    if (p.partL[(base + k) * AT_BM + row] > 0.0f) mx = fmaxf(mx, p.partM[(base + k) * AT_BM + row]);
  }
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, den = 0.0f;
  for (int k = 0; k < count; ++k) {
    const float lk = p.partL[(base + k) * AT_BM + row];
    if (!(lk > 0.0f)) continue;
    const float w = fastExp2((p.partM[(base + k) * AT_BM + row] - mx) * p.scaleLog2);
    den += lk * w;
    const float4 o = *reinterpret_cast<const float4 *>(p.partO + ((base + k) * AT_BM + row) * AT_D + lane * 4);
    acc[0] = fmaf(o.x, w, acc[0]);
    acc[1] = fmaf(o.y, w, acc[1]);
    acc[2] = fmaf(o.z, w, acc[2]);
    acc[3] = fmaf(o.w, w, acc[3]);
  }
  const float inv = den > 0.0f ? 1.0f / den : 0.0f;
  const int b = static_cast<int>(bh / p.Hq), h = static_cast<int>(bh % p.Hq);
  T *orow = out + b * p.ob + h * p.oh + qrow * p.os + lane * 4;
  uint2 v;
  v.x = packPair<T>(acc[0] * inv, acc[1] * inv);
  v.y = packPair<T>(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2 *>(orow) = v;
}

template <typename T>
static int launchAt(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, void *out, const AtParams &p,
                    unsigned grid, cudaStream_t st) {
  static bool attrSet[64] = {}; // function attributes belong to a device
  int dev = 0;
  TTB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attrSet[dev]) {
    TTB_CUDA(cudaFuncSetAttribute(sdpaTcgen05Kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM));
    attrSet[dev] = true;
  }
  TTB_CUDA(launchPdl(sdpaTcgen05Kernel<T>, dim3(grid), dim3(AT_THREADS), AT_SMEM, st, mq, mk, mv, static_cast<T *>(out), p));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// Returns -1 when the problem is outside what this kernel takes (the caller then uses another
// kernel), otherwise a TTB status.
int sdpaTcgen05Try(const void *q, const void *k, const void *v, void *out, int dtype, int64_t batch, int64_t hq,
                   int64_t hkv, int64_t sq, int64_t skv, int64_t headDim, const int64_t *qs, const int64_t *ks,
                   const int64_t *vs, const int64_t *os, int causal, float scale, cudaStream_t st, int64_t causalOff) {
  if (headDim != AT_D || (dtype != kBF16 && dtype != kF16)) return -1;
  if (causalOff < 0 || causalOff > 0x3fffffff) return -1;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return -1;
  if (sq > 0x7fffff00 || skv > 0x7fffff00) return -1;
  for (int i = 0; i < 3; ++i) {
    if (qs[i] < 0 || ks[i] < 0 || vs[i] < 0 || os[i] < 0) return -1;
    if (qs[i] % 8 || ks[i] % 8 || vs[i] % 8 || os[i] % 8) return -1; // 16-byte units for TMA and the vector stores
  }
  const int64_t nQ = (sq + AT_BM - 1) / AT_BM;
  const int64_t ctas = nQ * batch * hq;
  if (ctas > 0x7fffffff) return -1;
  // Two heads of a grouped-query group per CTA when the group size is even (TTB_SDPA_ONE_HEAD=1: never).
  static const bool oneHead = [] {
    const char *e = std::getenv("TTB_SDPA_ONE_HEAD");
    return e && e[0] == '1';
  }();
  // ... and when the halved grid still fills the machine.
  const bool pair = !oneHead && (hq / hkv) % 2 == 0 && nQ * batch * hq / 2 >= smCount();
  CUtensorMap mq, mk, mv;
  if (!makeHeadMap(&mq, q, dtype, batch, hq, sq, qs) || !makeHeadMap(&mk, k, dtype, batch, hkv, skv, ks, pair ? AP_BN : AT_BM) ||
      !makeHeadMap(&mv, v, dtype, batch, hkv, skv, vs, pair ? AP_BN : AT_BM))
    return -1;
  AtParams p;
  p.Hq = hq; p.Hkv = hkv; p.Sq = sq; p.Skv = skv;
  p.ob = os[0]; p.oh = os[1]; p.os = os[2];
  p.causal = causal ? 1 : 0;
  p.causalOff = causal ? static_cast<int>(causalOff) : 0;
  p.fmt = dtype == kBF16 ? 1 : 0;
  p.scaleLog2 = scale * 1.4426950408889634f;
  p.splitLen = 0;
  p.partO = p.partM = p.partL = nullptr;
  double work = 4.0 * double(batch) * hq * sq * skv * headDim * (causal ? 0.5 : 1.0);
  ProfScope prof("sdpa_tcgen05", work, 2.0 * batch * (2.0 * hq * sq + 2.0 * hkv * skv) * headDim, st);
  if (pair) {
    const unsigned grid = static_cast<unsigned>(ctas / 2);
    if (dtype == kBF16) return launchPair<__nv_bfloat16>(mq, mk, mv, out, p, grid, st);
    return launchPair<__half>(mq, mk, mv, out, p, grid, st);
  }
  // Few heads and long sequences: fewer query blocks than SMs, and under a causal mask the launch
  // lasts as long as its last query block.  Cut the key ranges into pieces of L tiles, L chosen to
  // minimise waves x (L + 6) + 3, in units of one key tile's steady-state time: 6 for a CTA's fixed
  // cost (allocation, Q tile, first trip through the load / contraction / softmax pipeline,
  // epilogue), 3 for the merge launch.  Measured: 2 heads x 4096 tokens 49.5 -> 33.6 us; at 4 heads x
  // 2048 tokens (a 1/8 tensor-parallel shard of the decoder block) only 29.1 -> 27.4 us, because all
  // pieces then stream the same few heads' K and V at once and the launch becomes bound by L2
  // bandwidth (each key tile is still read once per query block), and at 8 heads the second wave of
  // pieces made it slower; so the split is taken only when the model promises at least 40 %.
  // TTB_SDPA_NO_SPLIT=1 switches it off.
  static const bool noSplit = [] {
    const char *e = std::getenv("TTB_SDPA_NO_SPLIT");
    return e && e[0] == '1';
  }();
  void *scratch = nullptr;
  unsigned grid = static_cast<unsigned>(ctas);
  const int64_t tilesAll = (skv + AT_BN - 1) / AT_BN;
  if (!noSplit && causal && nQ <= 64 && ctas < smCount() && tilesAll >= 4) {
    auto tilesOf = [&](int64_t qb) { return std::min<int64_t>(tilesAll, (qb * AT_BM + AT_BM - 1 + causalOff) / AT_BN + 1); };
    const int64_t unsplit = (tilesOf(nQ - 1) + 6) * ((ctas + smCount() - 1) / smCount());
    int64_t bestCost = unsplit * 6 / 10;
    int bestL = 0;
    for (int L = static_cast<int>(tilesOf(nQ - 1)) - 1; L >= 2; --L) {
      int64_t pieces = 0;
      for (int64_t qb = 0; qb < nQ; ++qb) pieces += (tilesOf(qb) + L - 1) / L;
      pieces *= batch * hq;
      const int64_t cost = ((pieces + smCount() - 1) / smCount()) * (L + 6) + 3;
      if (cost < bestCost) {
        bestCost = cost;
        bestL = L;
      }
    }
    if (bestL) {
      int64_t perHead = 0;
      for (int64_t qb = 0; qb < nQ; ++qb) {
        p.pieceStart[qb] = static_cast<unsigned short>(perHead);
        perHead += (tilesOf(qb) + bestL - 1) / bestL;
      }
      p.pieceStart[nQ] = static_cast<unsigned short>(perHead);
      const size_t pieces = static_cast<size_t>(perHead) * batch * hq;
      const size_t bytes = pieces * AT_BM * (AT_D + 2) * sizeof(float);
      int rc = ttb_malloc(&scratch, bytes, st);
      if (rc) return rc;
      p.splitLen = bestL;
      p.partO = static_cast<float *>(scratch);
      p.partM = p.partO + pieces * AT_BM * AT_D;
      p.partL = p.partM + pieces * AT_BM;
      grid = static_cast<unsigned>(pieces);
    }
  }
  int rc = dtype == kBF16 ? launchAt<__nv_bfloat16>(mq, mk, mv, out, p, grid, st) : launchAt<__half>(mq, mk, mv, out, p, grid, st);
  if (p.splitLen) {
    if (rc == TTB_OK) {
      const int rows = static_cast<int>(batch * hq * nQ * AT_BM);
      if (dtype == kBF16) sdpaMergeKernel<__nv_bfloat16><<<(rows + 7) / 8, 256, 0, st>>>(static_cast<__nv_bfloat16 *>(out), p, rows);
      else sdpaMergeKernel<__half><<<(rows + 7) / 8, 256, 0, st>>>(static_cast<__half *>(out), p, rows);
      countLaunch();
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) rc = cudaFail(e, "sdpaMergeKernel", __FILE__, __LINE__);
    }
    int rc2 = ttb_free(scratch, st);
    if (rc == TTB_OK) rc = rc2;
  }
  return rc;
}

} // namespace ttb

namespace ttb {
// Reads and / or writes this file's copies of the status word and the wait limit (current device).
int sdpaTcgen05StatusAccess(int *status, const int *newValue, const long long *waitCycles) {
  if (status) TTB_CUDA(cudaMemcpyFromSymbol(status, g_tcStatus, sizeof(int)));
  if (newValue) TTB_CUDA(cudaMemcpyToSymbol(g_tcStatus, newValue, sizeof(int)));
  if (waitCycles) TTB_CUDA(cudaMemcpyToSymbol(g_tcWaitCycles, waitCycles, sizeof(long long)));
  return TTB_OK;
}
} // namespace ttb

extern "C" int ttb_sdpa_tcgen05_status(int *status) {
  TTB_CHECK(status != nullptr, "null argument");
  TTB_CUDA(cudaMemcpyFromSymbol(status, ttb::g_tcStatus, sizeof(int)));
  return TTB_OK;
}
