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
  int fmt; // 1 bf16, 0 f16
  float scaleLog2;
};

__device__ __forceinline__ float fastExp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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
  const int64_t BH = static_cast<int64_t>(gridDim.x) / nQ;
  // Heaviest (latest, under a causal mask) query blocks first.
  const int qb = static_cast<int>(nQ - 1 - blockIdx.x / BH);
  const int bh = static_cast<int>(blockIdx.x % BH);
  const int b = static_cast<int>(bh / p.Hq), h = static_cast<int>(bh % p.Hq);
  const int hkv = static_cast<int>(h / (p.Hq / p.Hkv));
  const int q0 = qb * AT_BM;
  int nT = static_cast<int>((p.Skv + AT_BN - 1) / AT_BN);
  if (p.causal) {
    int lim = q0 / AT_BN + 1;
    nT = nT < lim ? nT : lim;
  }

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
        tmaLoad4d(sK + s * AT_TILE, &mapK, kFull + 8 * s, 0, j * AT_BN, hkv, b);
        tmaLoad4d(sK + s * AT_TILE + AT_HALF, &mapK, kFull + 8 * s, 64, j * AT_BN, hkv, b);
        if (!mbarWait(vEmpty + 8 * s, ph ^ 1, abortP, 2)) break;
        mbarArriveExpectTx(vFull + 8 * s, AT_TILE);
        tmaLoad4d(sV + s * AT_TILE, &mapV, vFull + 8 * s, 0, j * AT_BN, hkv, b);
        tmaLoad4d(sV + s * AT_TILE + AT_HALF, &mapV, vFull + 8 * s, 64, j * AT_BN, hkv, b);
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
      const int key0 = j * AT_BN + wg * HALF;
      const bool needMask = (p.causal && key0 + HALF - 1 > q0) || key0 + HALF > p.Skv;
      // Last visible key of this row inside this half tile (relative, may be negative or >= 64).
      int64_t lastKey = p.Skv - 1;
      if (p.causal && qrow < lastKey) lastKey = qrow;
      const int lastRel = static_cast<int>(lastKey - key0 < HALF ? lastKey - key0 : HALF);
      // Pass 1: the maximum of this half of the row.
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < HALF / 32; ++c) {
        uint32_t r[32];
        tcLoad32(sAddr + c * 32, r);
        tcWaitLd();
        if (needMask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, c * 32 + i <= lastRel ? __uint_as_float(r[i]) : -INFINITY);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
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
      for (int c = 0; c < HALF / 32; ++c) {
        uint32_t r[32];
        tcLoad32(sAddr + c * 32, r);
        tcWaitLd();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a = fastExp2(fmaf(__uint_as_float(r[i]), sl2, negM));
          float bb = fastExp2(fmaf(__uint_as_float(r[i + 1]), sl2, negM));
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
      tcFenceBefore();
      mbarArrive(sEmpty + 8 * s);
      fenceProxyAsyncShared();
      mbarArrive(pReady);
    }
    // The last P V has to land before O is read; the row sum is the two halves' sums.
    if (ok && nT > 0 && !__all_sync(0xffffffffu, mbarWait(pEmpty, (nT & 1) ^ 1, abortP, 11))) ok = false;
    if (ok) l += exchange(l);
    if (ok) {
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

// [batch, heads, seq, 128] 16-bit tensor addressed through element strides, box = 64 columns x 128
// rows of one head, 128-byte swizzle; rows past the end of a head read as zero.
static bool makeHeadMap(CUtensorMap *map, const void *ptr, int dtype, int64_t batch, int64_t heads, int64_t seq,
                        const int64_t *strides3) {
  EncodeTiledFn fn = encodeTiled();
  if (!fn) return false;
  cuuint64_t dims[4] = {AT_D, static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  // A dimension of extent 1 never advances; give it a stride the encoder accepts.
  auto bytes = [&](int64_t s, cuuint64_t fallback) { return s > 0 ? static_cast<cuuint64_t>(s) * 2 : fallback; };
  cuuint64_t sSeq = bytes(strides3[2], AT_D * 2);
  cuuint64_t sHead = bytes(strides3[1], sSeq * static_cast<cuuint64_t>(seq));
  cuuint64_t sBatch = bytes(strides3[0], sHead * static_cast<cuuint64_t>(heads));
  cuuint64_t strides[3] = {sSeq, sHead, sBatch};
  cuuint32_t box[4] = {64, AT_BM, 1, 1};
  cuuint32_t elemStrides[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 4, const_cast<void *>(ptr), dims, strides, box, elemStrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
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
  sdpaTcgen05Kernel<T><<<grid, AT_THREADS, AT_SMEM, st>>>(mq, mk, mv, static_cast<T *>(out), p);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// Returns -1 when the problem is outside what this kernel takes (the caller then uses another
// kernel), otherwise a TTB status.
int sdpaTcgen05Try(const void *q, const void *k, const void *v, void *out, int dtype, int64_t batch, int64_t hq,
                   int64_t hkv, int64_t sq, int64_t skv, int64_t headDim, const int64_t *qs, const int64_t *ks,
                   const int64_t *vs, const int64_t *os, int causal, float scale, cudaStream_t st) {
  if (headDim != AT_D || (dtype != kBF16 && dtype != kF16)) return -1;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return -1;
  if (sq > 0x7fffff00 || skv > 0x7fffff00) return -1;
  for (int i = 0; i < 3; ++i) {
    if (qs[i] < 0 || ks[i] < 0 || vs[i] < 0 || os[i] < 0) return -1;
    if (qs[i] % 8 || ks[i] % 8 || vs[i] % 8 || os[i] % 8) return -1; // 16-byte units for TMA and the vector stores
  }
  const int64_t nQ = (sq + AT_BM - 1) / AT_BM;
  const int64_t ctas = nQ * batch * hq;
  if (ctas > 0x7fffffff) return -1;
  CUtensorMap mq, mk, mv;
  if (!makeHeadMap(&mq, q, dtype, batch, hq, sq, qs) || !makeHeadMap(&mk, k, dtype, batch, hkv, skv, ks) ||
      !makeHeadMap(&mv, v, dtype, batch, hkv, skv, vs))
    return -1;
  AtParams p;
  p.Hq = hq; p.Hkv = hkv; p.Sq = sq; p.Skv = skv;
  p.ob = os[0]; p.oh = os[1]; p.os = os[2];
  p.causal = causal ? 1 : 0;
  p.fmt = dtype == kBF16 ? 1 : 0;
  p.scaleLog2 = scale * 1.4426950408889634f;
  double work = 4.0 * double(batch) * hq * sq * skv * headDim * (causal ? 0.5 : 1.0);
  ProfScope prof("sdpa_tcgen05", work, 2.0 * batch * (2.0 * hq * sq + 2.0 * hkv * skv) * headDim, st);
  if (dtype == kBF16) return launchAt<__nv_bfloat16>(mq, mk, mv, out, p, static_cast<unsigned>(ctas), st);
  return launchAt<__half>(mq, mk, mv, out, p, static_cast<unsigned>(ctas), st);
}

} // namespace ttb

extern "C" int ttb_sdpa_tcgen05_status(int *status) {
  TTB_CHECK(status != nullptr, "null argument");
  TTB_CUDA(cudaMemcpyFromSymbol(status, ttb::g_tcStatus, sizeof(int)));
  return TTB_OK;
}
