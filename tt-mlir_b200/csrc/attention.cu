// scaled_dot_product_attention: out = softmax(q k^T * scale + mask) v, f32 softmax
// (reference op: runtime/lib/ttnn/operations/transformer/scaled_dot_product_attention.cpp:41-45;
// golden tools/golden/mapping.py:8398-8500: GQA by repeating k/v heads, causal mask = -inf for
// key index > query index, softmax over keys, f32 math, one rounding of the result).
//
// Two kernels:
//  * flashKernel: bf16 / f16, head_dim 128, no explicit mask tensor.  One CTA = 64 query rows
//    of one head, 4 warps x 16 rows; keys and values stream through a double-buffered
//    cp.async pipeline in 64-row tiles; S = QK^T and O += P V run on mma.sync m16n8k16 with
//    f32 accumulators held in registers; online softmax (running max / sum) per row.  The score
//    matrix never leaves the SM, so HBM traffic is q + k + v + out.
//  * genericKernel: any float dtype, any head_dim, optional additive mask; one CTA per query
//    row with the scores in shared memory.  Used for shapes the fast kernel does not take.
#include "common.cuh"

#include <cstdlib>

#include <cfloat>

namespace ttb {

// ---- small PTX wrappers ------------------------------------------------------------------
__device__ __forceinline__ uint32_t smemAddr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cpAsync16(uint32_t dst, const void *src, bool pred) {
  int sz = pred ? 16 : 0; // size 0 zero-fills the destination
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cpAsyncWait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrixX4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrixX4T(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <typename T> __device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// ---- fast kernel ---------------------------------------------------------------------------
constexpr int FA_D = 128;          // head dim
constexpr int FA_BM = 64;          // query rows per CTA
constexpr int FA_BN = 64;          // keys per tile
constexpr int FA_THREADS = 128;
constexpr int FA_ROW_BYTES = FA_D * 2;               // 256 B per tile row
constexpr int FA_TILE_BYTES = FA_BM * FA_ROW_BYTES;  // 16 KB
constexpr int FA_SMEM = FA_TILE_BYTES * 5;           // q + 2 x (k, v)

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` in a [64][128] 16-bit tile; the XOR
// spreads the 8 rows an ldmatrix touches over all banks.
__device__ __forceinline__ uint32_t tileOff(int row, int chunk) {
  return static_cast<uint32_t>(row * FA_ROW_BYTES + ((chunk ^ (row & 7)) << 4));
}

// Copies rows [row0, row0+64) x 128 of a [rows, 128] matrix into a swizzled tile; rows past
// `rows` are zero-filled.
template <typename T>
__device__ __forceinline__ void loadTile(uint32_t smemBase, const T *g, int64_t row0, int64_t rows) {
#pragma unroll
  for (int i = 0; i < (FA_BM * 16) / FA_THREADS; ++i) {
    int idx = threadIdx.x + i * FA_THREADS;
    int r = idx >> 4, c = idx & 15;
    int64_t gr = row0 + r;
    bool ok = gr < rows;
    cpAsync16(smemBase + tileOff(r, c), g + (ok ? gr : 0) * FA_D + c * 8, ok);
  }
}

template <typename T>
__global__ void __launch_bounds__(FA_THREADS)
    flashKernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ out,
                int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int causal, float scaleLog2) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smemAddr(smem);
  const uint32_t sK = sQ + FA_TILE_BYTES;      // 2 stages
  const uint32_t sV = sK + 2 * FA_TILE_BYTES;  // 2 stages
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  // Heavy (late) query blocks of a causal problem are scheduled first.
  const int64_t nQBlocks = (Sq + FA_BM - 1) / FA_BM;
  const int64_t qb = causal ? (nQBlocks - 1 - blockIdx.x) : blockIdx.x;
  const int64_t head = blockIdx.y, batch = blockIdx.z;
  const int64_t kvHead = head / (Hq / Hkv);
  const T *qg = q + ((batch * Hq + head) * Sq) * FA_D;
  const T *kg = k + ((batch * Hkv + kvHead) * Skv) * FA_D;
  const T *vg = v + ((batch * Hkv + kvHead) * Skv) * FA_D;
  T *og = out + ((batch * Hq + head) * Sq) * FA_D;
  const int64_t q0 = qb * FA_BM;

  int64_t nKv = (Skv + FA_BN - 1) / FA_BN;
  if (causal) {
    int64_t last = (q0 + FA_BM - 1) / FA_BN + 1; // tiles that contain a key index <= the last query index
    nKv = last < nKv ? last : nKv;
  }

  loadTile(sQ, qg, q0, Sq);
  loadTile(sK, kg, 0, Skv);
  loadTile(sV, vg, 0, Skv);
  cpAsyncCommit();

  uint32_t qf[8][4];
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float mRow[2] = {-INFINITY, -INFINITY}, lRow[2] = {0.0f, 0.0f};

  for (int64_t j = 0; j < nKv; ++j) {
    const int stage = static_cast<int>(j & 1);
    if (j + 1 < nKv) {
      loadTile(sK + (stage ^ 1) * FA_TILE_BYTES, kg, (j + 1) * FA_BN, Skv);
      loadTile(sV + (stage ^ 1) * FA_TILE_BYTES, vg, (j + 1) * FA_BN, Skv);
      cpAsyncCommit();
      cpAsyncWait<1>();
    } else {
      cpAsyncWait<0>();
    }
    __syncthreads();
    if (j == 0) {
      // Q fragments stay in registers for the whole kernel.
      const int mi = lane >> 3;
      const int row = warp * 16 + (lane & 7) + ((mi & 1) << 3);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) ldmatrixX4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], sQ + tileOff(row, kk * 2 + (mi >> 1)));
    }
    const uint32_t kBase = sK + stage * FA_TILE_BYTES, vBase = sV + stage * FA_TILE_BYTES;

    // S = Q K^T for this warp's 16 rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
      for (int np = 0; np < 4; ++np) { // pairs of 8-key tiles
        const int mi = lane >> 3;
        const int nrow = np * 16 + (lane & 7) + ((mi >> 1) << 3);
        uint32_t b0, b1, b2, b3;
        ldmatrixX4(b0, b1, b2, b3, kBase + tileOff(nrow, kk * 2 + (mi & 1)));
        mma16816<T>(s[np * 2], qf[kk], b0, b1);
        mma16816<T>(s[np * 2 + 1], qf[kk], b2, b3);
      }
    }

    // mask: keys past the end, and (causal) keys after the query
    const int64_t key0 = j * FA_BN;
    const bool needMask = (key0 + FA_BN > Skv) || (causal && key0 + FA_BN - 1 > q0 + warp * 16);
    if (needMask) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int64_t key = key0 + i * 8 + t * 2 + (e & 1);
          int64_t qi = q0 + warp * 16 + g + ((e >> 1) << 3);
          if (key >= Skv || (causal && key > qi)) s[i][e] = -INFINITY;
        }
      }
    }

    // online softmax
    float mNew[2] = {mRow[0], mRow[1]};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mNew[0] = fmaxf(mNew[0], fmaxf(s[i][0], s[i][1]));
      mNew[1] = fmaxf(mNew[1], fmaxf(s[i][2], s[i][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mNew[r] = fmaxf(mNew[r], __shfl_xor_sync(0xffffffffu, mNew[r], 1));
      mNew[r] = fmaxf(mNew[r], __shfl_xor_sync(0xffffffffu, mNew[r], 2));
    }
    float corr[2], mScaled[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      // A fully masked row keeps m = -inf; use 0 as the reference so exp2 yields 0, not NaN.
      mScaled[r] = mNew[r] == -INFINITY ? 0.0f : mNew[r] * scaleLog2;
      corr[r] = mRow[r] == -INFINITY ? 0.0f : exp2f(mRow[r] * scaleLog2 - mScaled[r]);
      mRow[r] = mNew[r];
    }
    float rowSum[2] = {0.0f, 0.0f};
    uint32_t pf[4][4]; // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p0 = exp2f(s[i][0] * scaleLog2 - mScaled[0]);
      float p1 = exp2f(s[i][1] * scaleLog2 - mScaled[0]);
      float p2 = exp2f(s[i][2] * scaleLog2 - mScaled[1]);
      float p3 = exp2f(s[i][3] * scaleLog2 - mScaled[1]);
      rowSum[0] += p0 + p1;
      rowSum[1] += p2 + p3;
      pf[i >> 1][(i & 1) * 2] = pack2<T>(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack2<T>(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) lRow[r] = lRow[r] * corr[r] + rowSum[r];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int np = 0; np < 8; ++np) { // pairs of 8-wide d tiles
        const int mi = lane >> 3;
        const int krow = kk * 16 + (lane & 7) + ((mi & 1) << 3);
        uint32_t b0, b1, b2, b3;
        ldmatrixX4T(b0, b1, b2, b3, vBase + tileOff(krow, np * 2 + (mi >> 1)));
        mma16816<T>(o[np * 2], pf[kk], b0, b1);
        mma16816<T>(o[np * 2 + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads(); // everyone is done with this stage before the next prefetch overwrites it
  }

  // finish: divide by the row sums (summed over the 4 lanes of a quad) and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lRow[r] += __shfl_xor_sync(0xffffffffu, lRow[r], 1);
    lRow[r] += __shfl_xor_sync(0xffffffffu, lRow[r], 2);
  }
  const float inv0 = lRow[0] > 0.0f ? 1.0f / lRow[0] : 0.0f, inv1 = lRow[1] > 0.0f ? 1.0f / lRow[1] : 0.0f;
  const int64_t r0 = q0 + warp * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    int col = i * 8 + t * 2;
    if (r0 < Sq) *reinterpret_cast<uint32_t *>(og + r0 * FA_D + col) = pack2<T>(o[i][0] * inv0, o[i][1] * inv0);
    if (r1 < Sq) *reinterpret_cast<uint32_t *>(og + r1 * FA_D + col) = pack2<T>(o[i][2] * inv1, o[i][3] * inv1);
  }
}

// ---- general kernel ------------------------------------------------------------------------
// One CTA per (batch, head, query row); scores for the row live in shared memory.
template <typename T>
__global__ void __launch_bounds__(128)
    genericKernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ mask,
                  T *__restrict__ out, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, int64_t maskB,
                  int64_t maskH, int causal, float scale) {
  extern __shared__ float sc[]; // Skv scores + 33 scratch
  float *scratch = sc + Skv;
  const int64_t row = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int64_t kvHead = head / (Hq / Hkv);
  const T *qr = q + (((batch * Hq + head) * Sq) + row) * D;
  const T *kg = k + ((batch * Hkv + kvHead) * Skv) * D;
  const T *vg = v + ((batch * Hkv + kvHead) * Skv) * D;
  const T *mr = mask ? mask + ((((maskB > 1 ? batch : 0) * maskH + (maskH > 1 ? head : 0)) * Sq) + row) * Skv : nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  // scores: one warp per key, lanes over D
  float mx = -INFINITY;
  for (int64_t j = warp; j < Skv; j += nwarp) {
    float acc = 0.0f;
    for (int64_t d = lane; d < D; d += 32) acc = fmaf(toF32(qr[d]), toF32(kg[j * D + d]), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    float s = acc * scale;
    if (causal && j > row) s = -INFINITY;
    if (mr) s += toF32(mr[j]);
    if (lane == 0) sc[j] = s;
    mx = fmaxf(mx, s);
  }
  if (lane == 0) scratch[warp] = mx;
  __syncthreads();
  mx = -INFINITY;
  for (int w = 0; w < nwarp; ++w) mx = fmaxf(mx, scratch[w]);
  __syncthreads();
  float sum = 0.0f;
  for (int64_t j = threadIdx.x; j < Skv; j += blockDim.x) {
    float p = mx == -INFINITY ? 0.0f : expf(sc[j] - mx);
    sc[j] = p;
    sum += p;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) scratch[warp] = sum;
  __syncthreads();
  sum = 0.0f;
  for (int w = 0; w < nwarp; ++w) sum += scratch[w];
  float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
  T *orow = out + (((batch * Hq + head) * Sq) + row) * D;
  for (int64_t d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.0f;
    for (int64_t j = 0; j < Skv; ++j) acc = fmaf(sc[j], toF32(vg[j * D + d]), acc);
    orow[d] = fromF32<T>(acc * inv);
  }
}

} // namespace ttb

namespace ttb {
int sdpaTcgen05Try(const void *q, const void *k, const void *v, void *out, int dtype, int64_t batch, int64_t hq,
                   int64_t hkv, int64_t sq, int64_t skv, int64_t headDim, const int64_t *qs, const int64_t *ks,
                   const int64_t *vs, const int64_t *os, int causal, float scale, cudaStream_t st, int64_t causalOff = 0);
static bool sdpaLegacy() {
  static const bool legacy = [] {
    const char *e = std::getenv("TTB_SDPA_MMA_SYNC");
    return e && e[0] == '1';
  }();
  return legacy;
}
}

using namespace ttb;

// Multi-latent attention prefill (::ttnn::transformer::flash_mla_prefill, operations/transformer/flash_mla_prefill.cpp;
// golden tools/golden/mapping.py:8662-8692): queries and keys have Dqk columns, values the first Dv columns of the keys
// (or their own tensor), the result has Dv columns.  One CTA per (batch, head, query row), the row's scores in shared
// memory, f32 throughout, one rounding: the general kernel above with its own value width and row stride.  A CUDA-core
// path: the tensor-core attention kernels take head_dim 128 on both sides only.
template <typename T>
__global__ void __launch_bounds__(128)
    mlaPrefillKernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ mask,
                     T *__restrict__ out, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t Dqk, int64_t Dv, int64_t vRow,
                     int64_t maskB, int64_t maskH, int causal, float scale) {
  extern __shared__ float sc[]; // Skv scores + 33 scratch
  float *scratch = sc + Skv;
  const int64_t row = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int64_t kvHead = head / (Hq / Hkv);
  const T *qr = q + (((batch * Hq + head) * Sq) + row) * Dqk;
  const T *kg = k + ((batch * Hkv + kvHead) * Skv) * Dqk;
  const T *vg = v + ((batch * Hkv + kvHead) * Skv) * vRow;
  const T *mr = mask ? mask + ((((maskB > 1 ? batch : 0) * maskH + (maskH > 1 ? head : 0)) * Sq) + row) * Skv : nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float mx = -INFINITY;
  for (int64_t j = warp; j < Skv; j += nwarp) {
    float acc = 0.0f;
    for (int64_t d = lane; d < Dqk; d += 32) acc = fmaf(toF32(qr[d]), toF32(kg[j * Dqk + d]), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    float s = acc * scale;
    if (causal && j > row) s = -INFINITY;
    if (mr) s += toF32(mr[j]);
    if (lane == 0) sc[j] = s;
    mx = fmaxf(mx, s);
  }
  if (lane == 0) scratch[warp] = mx;
  __syncthreads();
  mx = -INFINITY;
  for (int w = 0; w < nwarp; ++w) mx = fmaxf(mx, scratch[w]);
  __syncthreads();
  float sum = 0.0f;
  for (int64_t j = threadIdx.x; j < Skv; j += blockDim.x) {
    const float p = mx == -INFINITY ? 0.0f : expf(sc[j] - mx);
    sc[j] = p;
    sum += p;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) scratch[warp] = sum;
  __syncthreads();
  sum = 0.0f;
  for (int w = 0; w < nwarp; ++w) sum += scratch[w];
  const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
  T *orow = out + (((batch * Hq + head) * Sq) + row) * Dv;
  for (int64_t d = threadIdx.x; d < Dv; d += blockDim.x) {
    float acc = 0.0f;
    for (int64_t j = 0; j < Skv; ++j) acc = fmaf(sc[j], toF32(vg[j * vRow + d]), acc);
    orow[d] = fromF32<T>(acc * inv);
  }
}

extern "C" int ttb_flash_mla_prefill(const void *q, const void *k, const void *v, const void *mask, void *out, int dtype, int64_t batch,
                                     int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int64_t head_dim_qk,
                                     int64_t head_dim_v, int64_t mask_batch, int64_t mask_heads, int is_causal, float scale,
                                     void *stream) {
  TTB_CHECK(q && k && out, "null tensor");
  TTB_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0, "bad head configuration");
  TTB_CHECK(seq_q > 0 && seq_kv > 0 && head_dim_qk > 0 && head_dim_v > 0, "empty attention problem");
  TTB_CHECK(v != nullptr || head_dim_v <= head_dim_qk, "values taken from the keys cannot be wider than the keys");
  TTB_CHECK(batch <= 65535 && heads_q <= 65535 && seq_q <= 2147483647, "grid too large");
  const size_t smem = (static_cast<size_t>(seq_kv) + 40) * sizeof(float);
  TTB_CHECK(smem <= 200 * 1024, "sequence too long for the multi-latent attention kernel");
  cudaStream_t st = asStream(stream);
  ProfScope prof("flash_mla_prefill", 2.0 * double(batch) * heads_q * seq_q * seq_kv * (head_dim_qk + head_dim_v), 0, st);
  dim3 grid(static_cast<unsigned>(seq_q), static_cast<unsigned>(heads_q), static_cast<unsigned>(batch));
  const void *vals = v ? v : k;
  const int64_t vRow = v ? head_dim_v : head_dim_qk;
  TTB_DISPATCH_FLOAT(dtype, T, {
    if (smem > 48 * 1024) {
      TTB_CUDA(cudaFuncSetAttribute(mlaPrefillKernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    mlaPrefillKernel<T><<<grid, 128, smem, st>>>(static_cast<const T *>(q), static_cast<const T *>(k), static_cast<const T *>(vals),
                                                 static_cast<const T *>(mask), static_cast<T *>(out), heads_q, heads_kv, seq_q, seq_kv,
                                                 head_dim_qk, head_dim_v, vRow, mask_batch, mask_heads, is_causal, scale);
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// Additive mask of a decode step: user u sees keys 0 .. cur_pos[u] ([users, 1, 1, seq_kv], 0 or -inf).
template <typename T>
__global__ void __launch_bounds__(256) curPosMaskKernel(T *__restrict__ mask, const int32_t *__restrict__ curPos, int64_t users, int64_t seqKv) {
  const size_t total = static_cast<size_t>(users) * seqKv, stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t u = static_cast<int64_t>(i / seqKv), c = static_cast<int64_t>(i % seqKv);
    mask[i] = fromF32<T>(c <= static_cast<int64_t>(curPos[u]) ? 0.0f : -INFINITY);
  }
}

extern "C" int ttb_cur_pos_mask(void *mask, const int32_t *cur_pos, int dtype, int64_t users, int64_t seq_kv, void *stream) {
  TTB_CHECK(mask && cur_pos, "null tensor");
  TTB_CHECK(users > 0 && seq_kv > 0, "empty mask");
  cudaStream_t st = asStream(stream);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (curPosMaskKernel<T><<<gridFor(static_cast<size_t>(users) * seq_kv, 256), 256, 0, st>>>(static_cast<T *>(mask), cur_pos,
                                                                                                          users, seq_kv)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

// Additive mask of a prefill chunk: row r sees keys 0 .. r + offset.  Only for problems the tensor-core kernel,
// which applies the offset itself, does not take.
template <typename T>
__global__ void __launch_bounds__(256) causalOffsetMaskKernel(T *__restrict__ mask, int64_t seqQ, int64_t seqKv, int64_t offset) {
  const size_t total = static_cast<size_t>(seqQ) * seqKv, stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = static_cast<int64_t>(i / seqKv), c = static_cast<int64_t>(i % seqKv);
    mask[i] = fromF32<T>(c <= r + offset ? 0.0f : -INFINITY);
  }
}

// out[u, h, t, :] = cache[table[u, t / block], h, t % block, :]: a user's paged keys or values as one sequence.
template <typename I>
__global__ void __launch_bounds__(256) pagedGatherKernel(const uint4 *__restrict__ cache, const I *__restrict__ table, uint4 *__restrict__ out,
                                                         int64_t users, int64_t heads, int64_t blockSize, int64_t maxBlocks,
                                                         int64_t vecPerRow, int64_t numBlocks) {
  const int64_t seq = maxBlocks * blockSize;
  const size_t total = static_cast<size_t>(users) * heads * seq * vecPerRow, stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t v = static_cast<int64_t>(i % vecPerRow);
    size_t q = i / vecPerRow;
    const int64_t t = static_cast<int64_t>(q % seq);
    q /= seq;
    const int64_t h = static_cast<int64_t>(q % heads), u = static_cast<int64_t>(q / heads);
    int64_t blk = static_cast<int64_t>(table[u * maxBlocks + t / blockSize]);
    blk = blk < 0 ? 0 : (blk >= numBlocks ? numBlocks - 1 : blk); // a table entry outside the cache reads a valid block
    out[i] = cache[((blk * heads + h) * blockSize + t % blockSize) * vecPerRow + v];
  }
}

extern "C" int ttb_paged_gather(const void *cache, const void *page_table, void *out, int dtype, int table_dtype, int64_t users,
                                int64_t heads, int64_t block_size, int64_t max_blocks, int64_t head_dim, int64_t num_blocks,
                                void *stream) {
  TTB_CHECK(cache && page_table && out, "null tensor");
  TTB_CHECK(users > 0 && heads > 0 && block_size > 0 && max_blocks > 0 && head_dim > 0 && num_blocks > 0, "empty paged cache");
  const int64_t rowBytes = head_dim * static_cast<int64_t>(dtypeSize(dtype));
  TTB_CHECK(rowBytes % 16 == 0 && aligned16(cache) && aligned16(out), "cache rows must be multiples of 16 bytes");
  cudaStream_t st = asStream(stream);
  const size_t total = static_cast<size_t>(users) * heads * max_blocks * block_size * (rowBytes / 16);
  ProfScope prof("paged_gather", 0, double(total) * 32, st);
  const int grid = gridFor(total, 256);
  switch (table_dtype) {
  case kI32:
    pagedGatherKernel<int32_t><<<grid, 256, 0, st>>>(static_cast<const uint4 *>(cache), static_cast<const int32_t *>(page_table),
                                                     static_cast<uint4 *>(out), users, heads, block_size, max_blocks, rowBytes / 16, num_blocks);
    break;
  case kU32:
    pagedGatherKernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint4 *>(cache), static_cast<const uint32_t *>(page_table),
                                                      static_cast<uint4 *>(out), users, heads, block_size, max_blocks, rowBytes / 16, num_blocks);
    break;
  default: setLastError("paged_gather: the page table must be Int32 or UInt32"); return TTB_ERR_UNSUPPORTED;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

extern "C" int ttb_sdpa(const void *q, const void *k, const void *v, const void *mask, void *out, int dtype, int64_t batch,
                        int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int64_t head_dim, int64_t mask_batch,
                        int64_t mask_heads, int is_causal, float scale, void *stream);

extern "C" size_t ttb_sdpa_causal_offset_workspace_bytes(int dtype, int64_t seq_q, int64_t seq_kv) {
  return static_cast<size_t>(seq_q) * static_cast<size_t>(seq_kv) * dtypeSize(dtype);
}

extern "C" int ttb_sdpa_causal_offset(const void *q, const void *k, const void *v, void *out, int dtype, int64_t batch, int64_t heads_q,
                                      int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int64_t head_dim, int64_t offset, float scale,
                                      void *workspace, void *stream) {
  TTB_CHECK(q && k && v && out, "null tensor");
  TTB_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0, "bad head configuration");
  TTB_CHECK(seq_q > 0 && seq_kv > 0 && head_dim > 0 && offset >= 0, "empty attention problem");
  cudaStream_t st = asStream(stream);
  if (!sdpaLegacy()) {
    int64_t qs[3] = {heads_q * seq_q * head_dim, seq_q * head_dim, head_dim};
    int64_t ks[3] = {heads_kv * seq_kv * head_dim, seq_kv * head_dim, head_dim};
    int rc = sdpaTcgen05Try(q, k, v, out, dtype, batch, heads_q, heads_kv, seq_q, seq_kv, head_dim, qs, ks, ks, qs, 1, scale, st, offset);
    if (rc >= 0) return rc;
  }
  TTB_CHECK(workspace != nullptr, "this problem needs the mask workspace");
  TTB_DISPATCH_FLOAT(dtype, T,
                     (causalOffsetMaskKernel<T><<<gridFor(static_cast<size_t>(seq_q) * seq_kv, 256), 256, 0, st>>>(
                         static_cast<T *>(workspace), seq_q, seq_kv, offset)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return ttb_sdpa(q, k, v, workspace, out, dtype, batch, heads_q, heads_kv, seq_q, seq_kv, head_dim, 1, 1, 0, scale, stream);
}

extern "C" int ttb_sdpa(const void *q, const void *k, const void *v, const void *mask, void *out, int dtype,
                        int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv,
                        int64_t head_dim, int64_t mask_batch, int64_t mask_heads, int is_causal, float scale,
                        void *stream) {
  TTB_CHECK(q && k && v && out, "null tensor");
  TTB_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0, "bad head configuration");
  TTB_CHECK(seq_q > 0 && seq_kv > 0 && head_dim > 0, "empty attention problem");
  TTB_CHECK(batch <= 65535 && heads_q <= 65535, "grid too large");
  cudaStream_t st = asStream(stream);
  bool fast = !mask && head_dim == FA_D && (dtype == kBF16 || dtype == kF16) && aligned16(q) && aligned16(k) &&
              aligned16(v) && aligned16(out);
  if (fast) {
    // The tcgen05 kernel first; TTB_SDPA_MMA_SYNC=1 keeps the warp-level tensor-core kernel.
    if (!sdpaLegacy()) {
      int64_t qs[3] = {heads_q * seq_q * head_dim, seq_q * head_dim, head_dim};
      int64_t ks[3] = {heads_kv * seq_kv * head_dim, seq_kv * head_dim, head_dim};
      int rc = sdpaTcgen05Try(q, k, v, out, dtype, batch, heads_q, heads_kv, seq_q, seq_kv, head_dim, qs, ks, ks, qs,
                              is_causal, scale, st);
      if (rc >= 0) return rc;
    }
    dim3 grid(static_cast<unsigned>((seq_q + FA_BM - 1) / FA_BM), static_cast<unsigned>(heads_q),
              static_cast<unsigned>(batch));
    float scaleLog2 = scale * 1.4426950408889634f;
    int dev = 0;
    TTB_CUDA(cudaGetDevice(&dev));
    TTB_CHECK(dev >= 0 && dev < 64, "device ordinal out of range");
    double work = 4.0 * double(batch) * heads_q * seq_q * seq_kv * head_dim * (is_causal ? 0.5 : 1.0);
    ProfScope prof("sdpa_flash", work, 2.0 * batch * (2.0 * heads_q * seq_q + 2.0 * heads_kv * seq_kv) * head_dim, st);
    if (dtype == kBF16) {
      static bool attrSet[64] = {}; // function attributes belong to a device
      if (!attrSet[dev]) {
        TTB_CUDA(cudaFuncSetAttribute(flashKernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
        attrSet[dev] = true;
      }
      flashKernel<__nv_bfloat16><<<grid, FA_THREADS, FA_SMEM, st>>>(
          static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
          static_cast<const __nv_bfloat16 *>(v), static_cast<__nv_bfloat16 *>(out), heads_q, heads_kv, seq_q, seq_kv,
          is_causal, scaleLog2);
    } else {
      static bool attrSet[64] = {};
      if (!attrSet[dev]) {
        TTB_CUDA(cudaFuncSetAttribute(flashKernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM));
        attrSet[dev] = true;
      }
      flashKernel<__half><<<grid, FA_THREADS, FA_SMEM, st>>>(
          static_cast<const __half *>(q), static_cast<const __half *>(k), static_cast<const __half *>(v),
          static_cast<__half *>(out), heads_q, heads_kv, seq_q, seq_kv, is_causal, scaleLog2);
    }
    countLaunch();
    TTB_LAUNCH_CHECK();
    return TTB_OK;
  }
  size_t smem = (static_cast<size_t>(seq_kv) + 40) * sizeof(float);
  TTB_CHECK(smem <= 200 * 1024, "sequence too long for the general attention kernel");
  TTB_CHECK(seq_q <= 2147483647, "sequence too long");
  dim3 grid(static_cast<unsigned>(seq_q), static_cast<unsigned>(heads_q), static_cast<unsigned>(batch));
  ProfScope prof("sdpa_generic", 4.0 * double(batch) * heads_q * seq_q * seq_kv * head_dim, 0, st);
  TTB_DISPATCH_FLOAT(dtype, T, {
    if (smem > 48 * 1024) {
      TTB_CUDA(cudaFuncSetAttribute(genericKernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    genericKernel<T><<<grid, 128, smem, st>>>(static_cast<const T *>(q), static_cast<const T *>(k),
                                              static_cast<const T *>(v), static_cast<const T *>(mask),
                                              static_cast<T *>(out), heads_q, heads_kv, seq_q, seq_kv, head_dim,
                                              mask_batch, mask_heads, is_causal, scale);
  });
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

extern "C" int ttb_sdpa_strided(const void *q, const void *k, const void *v, void *out, int dtype, int64_t batch,
                                int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int64_t head_dim,
                                const int64_t *q_strides3, const int64_t *k_strides3, const int64_t *v_strides3,
                                const int64_t *out_strides3, int is_causal, float scale, void *stream) {
  TTB_CHECK(q && k && v && out && q_strides3 && k_strides3 && v_strides3 && out_strides3, "null argument");
  TTB_CHECK(batch > 0 && heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0, "bad head configuration");
  TTB_CHECK(seq_q > 0 && seq_kv > 0 && head_dim > 0, "empty attention problem");
  if (!sdpaLegacy()) {
    int rc = sdpaTcgen05Try(q, k, v, out, dtype, batch, heads_q, heads_kv, seq_q, seq_kv, head_dim, q_strides3, k_strides3,
                            v_strides3, out_strides3, is_causal, scale, asStream(stream));
    if (rc >= 0) return rc;
  }
  const int64_t dq[3] = {heads_q * seq_q * head_dim, seq_q * head_dim, head_dim};
  const int64_t dk[3] = {heads_kv * seq_kv * head_dim, seq_kv * head_dim, head_dim};
  bool dense = true;
  for (int i = 0; i < 3; ++i) {
    // a stride is irrelevant along a dimension of extent 1
    const int64_t extQ = i == 0 ? batch : (i == 1 ? heads_q : seq_q), extK = i == 0 ? batch : (i == 1 ? heads_kv : seq_kv);
    if (extQ > 1 && (q_strides3[i] != dq[i] || out_strides3[i] != dq[i])) dense = false;
    if (extK > 1 && (k_strides3[i] != dk[i] || v_strides3[i] != dk[i])) dense = false;
  }
  if (!dense) {
    setLastError("sdpa_strided: no kernel takes this problem with non-dense strides");
    return TTB_ERR_UNSUPPORTED;
  }
  return ttb_sdpa(q, k, v, nullptr, out, dtype, batch, heads_q, heads_kv, seq_q, seq_kv, head_dim, 0, 0, is_causal, scale,
                  stream);
}
