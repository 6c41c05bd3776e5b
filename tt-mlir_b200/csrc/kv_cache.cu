// KV-cache maintenance and single-token ("decode") attention over the cache.
//
// Reference semantics (goldens in tools/golden/mapping.py; runtime call sites in
// runtime/lib/ttnn/operations/kv_cache/{fill_cache,update_cache}.cpp and
// operations/transformer/scaled_dot_product_attention_decode.cpp):
//  fill_cache    cache[batch_offset + b, h, :S, :] = input[b, h, :, :]; rows S .. roundup(S, 32) of
//                those users are zeroed when they exist (mapping.py:3582-3611, the tile padding)
//  update_cache  cache[batch_offset + b, h, index, :] = input[0, h, b, :], `index` = element 0 of a
//                tensor (mapping.py:3614-3670).  The kernel reads the index on the device: no
//                host round trip (the reference reads it on the host, update_cache.cpp:17-37)
//  sdpa_decode   q [1, B, H, D] against k, v [B, Hkv, S, D]: scores = q k^T (+ mask [B|1, 1, H|1, S]),
//                keys after cur_pos[b] masked when causal, then * scale, softmax, P v; f32 math,
//                one rounding (mapping.py:2417-2482)
//
// Decode attention is HBM-bound: every byte of the live part of K and V is read exactly once.
// One CTA takes (chunk of keys, kv head, user) and serves all G = H / Hkv query heads of that kv
// head, so GQA does not multiply the traffic; the key range is split into chunks so that small
// batches still fill the GPU; a second small kernel merges the chunks' partial results with the
// usual running-max rescaling.
#include "common.cuh"

#include <cfloat>

namespace ttb {

// ---- cache writes --------------------------------------------------------------------------
template <typename U>
__global__ void __launch_bounds__(256)
    fillCacheKernel(U *__restrict__ cache, const U *__restrict__ in, size_t users, size_t heads, size_t seq, size_t padSeq,
                    size_t maxSeq, size_t rowUnits, size_t batchOffset) {
  const size_t total = users * heads * padSeq * rowUnits;
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const size_t u = i % rowUnits;
    size_t r = i / rowUnits;
    const size_t s = r % padSeq;
    r /= padSeq;
    const size_t h = r % heads, b = r / heads;
    U v = {};
    if (s < seq) v = in[((b * heads + h) * seq + s) * rowUnits + u];
    cache[(((batchOffset + b) * heads + h) * maxSeq + s) * rowUnits + u] = v;
  }
}

template <typename U, typename I>
__global__ void __launch_bounds__(256)
    updateCacheKernel(U *__restrict__ cache, const U *__restrict__ in, const I *__restrict__ index, size_t users, size_t heads,
                      size_t maxSeq, size_t rowUnits, size_t batchOffset, int *__restrict__ bad) {
  const long long at = static_cast<long long>(index[0]);
  if (at < 0 || static_cast<size_t>(at) >= maxSeq) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *bad = 1;
    return;
  }
  const size_t total = users * heads * rowUnits;
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const size_t u = i % rowUnits;
    size_t r = i / rowUnits;
    const size_t b = r % users, h = r / users; // input is [1, heads, users, D]
    cache[(((batchOffset + b) * heads + h) * maxSeq + static_cast<size_t>(at)) * rowUnits + u] = in[i];
  }
}

// Paged caches (mapping.py:8926-9007): the cache is [blocks, heads, block_size, D]; a page table
// [users, pages] names the physical block of each logical block of a user.
//  paged_update_cache  token s of user b (input [users, seq, heads, D]) goes to position update_index[b] + s
//  paged_fill_cache    position s of input [users, heads, seq, D] of user b, whose page-table row is
//                      batch_idx[b] (or b), goes to position s
// Page-table entries and rows are clamped into range, as the goldens clamp them.
template <typename U, typename I, typename P>
__global__ void __launch_bounds__(256)
    pagedUpdateCacheKernel(U *__restrict__ cache, const U *__restrict__ in, const I *__restrict__ index, const P *__restrict__ pageTable,
                           size_t users, size_t seq, size_t heads, size_t blocks, size_t blockSize, size_t pages, size_t rowUnits) {
  const size_t total = users * seq * heads * rowUnits;
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const size_t u = i % rowUnits;
    size_t r = i / rowUnits;
    const size_t h = r % heads;
    r /= heads;
    const size_t s = r % seq, b = r / seq; // input is [users, seq, heads, D]
    const long long pos = static_cast<long long>(index[b]) + static_cast<long long>(s);
    if (pos < 0) continue;
    size_t blk = static_cast<size_t>(pos) / blockSize;
    const size_t off = static_cast<size_t>(pos) % blockSize;
    if (pageTable) {
      const size_t col = blk < pages ? blk : pages - 1;
      const long long phys = static_cast<long long>(pageTable[b * pages + col]);
      blk = phys < 0 ? 0 : static_cast<size_t>(phys);
    }
    if (blk >= blocks) blk = blocks - 1;
    cache[((blk * heads + h) * blockSize + off) * rowUnits + u] = in[i];
  }
}

template <typename U, typename P, typename I>
__global__ void __launch_bounds__(256)
    pagedFillCacheKernel(U *__restrict__ cache, const U *__restrict__ in, const P *__restrict__ pageTable, const I *__restrict__ batchIdx,
                         size_t users, size_t heads, size_t seq, size_t blocks, size_t blockSize, size_t tableRows, size_t pages,
                         size_t rowUnits) {
  const size_t total = users * heads * seq * rowUnits;
  const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const size_t u = i % rowUnits;
    size_t r = i / rowUnits;
    const size_t s = r % seq;
    r /= seq;
    const size_t h = r % heads, b = r / heads; // input is [users, heads, seq, D]
    long long row = batchIdx ? static_cast<long long>(batchIdx[b]) : static_cast<long long>(b);
    row = row < 0 ? 0 : (row >= static_cast<long long>(tableRows) ? static_cast<long long>(tableRows) - 1 : row);
    size_t col = s / blockSize;
    if (col >= pages) col = pages - 1;
    long long phys = static_cast<long long>(pageTable[static_cast<size_t>(row) * pages + col]);
    size_t blk = phys < 0 ? 0 : static_cast<size_t>(phys);
    if (blk >= blocks) blk = blocks - 1;
    cache[((blk * heads + h) * blockSize + s % blockSize) * rowUnits + u] = in[i];
  }
}

__device__ int g_cacheBadIndex; // an update index outside the cache was seen (nothing was written); cleared when read

// ---- decode attention ------------------------------------------------------------------------
// D += A(16x16, row) * B(16x8, col), 16-bit operands, f32 accumulators.
template <typename T> __device__ __forceinline__ void decMma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void decMma<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void decMma<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ uint32_t decPack(float lo, float hi);
template <> __device__ __forceinline__ uint32_t decPack<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t decPack<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
// Transposes the 8 x 8 matrix of 16-bit elements that the warp holds one register per lane
// (lane 4r + c: row r, columns 2c and 2c + 1).
__device__ __forceinline__ uint32_t decTranspose(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
  return r;
}

constexpr int DEC_THREADS = 128; // four CTAs per SM in different phases fill each other's bubbles
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int DEC_CHUNK = 512; // keys per CTA

struct DecodeParams {
  int B, H, Hkv, S, chunks;
  // Paged cache: k / v are [blocks, Hkv, blockSize, D] and pageTable [B, pages] (Int32) names the block of
  // each run of blockSize positions; S = pages * blockSize.  pageTable null: k / v are [B, Hkv, S, D].
  const int32_t *pageTable;
  int blockSize, pages, blocks;
  int maskB, maskH; // extents of the mask's user and head dimensions (1 = broadcast), 0 = no mask
  float scale;
  int causal;
};

// Partial attention of G query heads over one chunk of keys.  Writes, per (user, head, chunk):
// m (running max), l (sum of exp(s - m)) and the unnormalised o[D] = sum exp(s - m) v.
template <typename T, int G, int D>
__global__ void __launch_bounds__(DEC_THREADS, D <= 128 ? 4 : 2)
    sdpaDecodeChunkKernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                          const int32_t *__restrict__ curPos, const T *__restrict__ mask, float *__restrict__ pm,
                          float *__restrict__ pl, float *__restrict__ po, DecodeParams p) {
  __shared__ float sc[G][DEC_CHUNK];
  __shared__ float so[2][G][D]; // exchange slots of the cross-warp sum
  __shared__ float sm[G], sl[G];
  pdlLaunchDependents();
  pdlWait();
  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int last = p.S - 1; // last key a query of this user may see
  if (p.causal && curPos) last = min(last, curPos[b]);
  const int k0 = chunk * DEC_CHUNK, k1 = min(k0 + DEC_CHUNK, last + 1);
  const int h0 = kvh * G;
  const size_t part = (static_cast<size_t>(b) * p.H + h0) * p.chunks + chunk; // + g * chunks per head
  if (k1 <= k0) {
    // nothing of this chunk is visible: an empty partial
    if (threadIdx.x < G) {
      pm[part + static_cast<size_t>(threadIdx.x) * p.chunks] = -INFINITY;
      pl[part + static_cast<size_t>(threadIdx.x) * p.chunks] = 0.0f;
    }
    for (int i = threadIdx.x; i < G * D; i += DEC_THREADS) {
      po[(part + static_cast<size_t>(i / D) * p.chunks) * D + (i % D)] = 0.0f;
    }
    return;
  }
  // Row (in units of D elements) of position j of this user's kv head.
  auto rowOf = [&](int j) -> size_t {
    if (!p.pageTable) return (static_cast<size_t>(b) * p.Hkv + kvh) * p.S + j;
    int blk = p.pageTable[static_cast<size_t>(b) * p.pages + j / p.blockSize];
    blk = blk < 0 ? 0 : (blk >= p.blocks ? p.blocks - 1 : blk);
    return (static_cast<size_t>(blk) * p.Hkv + kvh) * p.blockSize + j % p.blockSize;
  };

  // Scores on the tensor pipe: S[16 x 8] = Q[16 x D] K^T for 8 keys per mma tile, the G query heads
  // being rows 0..G-1 of the 16-row operand (the other rows are zero).  A dot product does not care
  // in which order its terms are summed, so the k index of the mma is mapped to head dims in a way
  // that lets one 16-byte load per lane feed two k-steps: in every block of 32 dims, lane t of a
  // quad holds dims 8t .. 8t+7 of its key; pairs (8t, 8t+1) and (8t+2, 8t+3) are the b0 / b1 of the
  // first k-step, (8t+4, 8t+5) and (8t+6, 8t+7) of the second, and Q's fragments use the same map.
  {
    constexpr int NB = D / 32; // 32-dim blocks
    const int quad = lane >> 2, t = lane & 3;
    uint32_t qa[NB][2][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
      if (quad < G) lo = *reinterpret_cast<const uint4 *>(q + (static_cast<size_t>(b) * p.H + h0 + quad) * D + nb * 32 + 8 * t);
      if (quad + 8 < G) hi = *reinterpret_cast<const uint4 *>(q + (static_cast<size_t>(b) * p.H + h0 + quad + 8) * D + nb * 32 + 8 * t);
      qa[nb][0][0] = lo.x; qa[nb][0][1] = hi.x; qa[nb][0][2] = lo.y; qa[nb][0][3] = hi.y;
      qa[nb][1][0] = lo.z; qa[nb][1][1] = hi.z; qa[nb][1][2] = lo.w; qa[nb][1][3] = hi.w;
    }
    // UK tiles of 8 keys per iteration with all their loads issued first (NB * UK * 16 bytes in flight per lane)
    constexpr int UK = 2;
    for (int j0 = k0 + warp * 8; j0 < k1; j0 += DEC_WARPS * 8 * UK) {
      uint4 raw[UK][NB];
#pragma unroll
      for (int u = 0; u < UK; ++u) {
        const int j = j0 + u * DEC_WARPS * 8 + quad;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          raw[u][nb] = j < k1 ? __ldcs(reinterpret_cast<const uint4 *>(k + rowOf(j) * D + nb * 32 + 8 * t))
                              : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < UK; ++u) {
        const int jt = j0 + u * DEC_WARPS * 8; // first key of the tile
        if (jt >= k1) break;                    // warp-uniform
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          decMma<T>(c, qa[nb][0], raw[u][nb].x, raw[u][nb].y);
          decMma<T>(c, qa[nb][1], raw[u][nb].z, raw[u][nb].w);
        }
        // c[0], c[1]: head `quad`, keys jt + 2t, jt + 2t + 1; c[2], c[3]: head quad + 8, same keys
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int g = quad + 8 * half;
          if (g < G) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int j = jt + 2 * t + e;
              if (j < k1) {
                float sv = c[2 * half + e];
                if (mask) {
                  const size_t mb = p.maskB == 1 ? 0 : b, mh = p.maskH == 1 ? 0 : h0 + g;
                  sv += toF32(mask[(mb * p.maskH + mh) * p.S + j]);
                }
                sc[g][j - k0] = sv * p.scale;
              }
            }
          }
        }
      }
    }
  }
  __syncthreads();
  // softmax statistics of the chunk: one warp per head
  for (int g = warp; g < G; g += DEC_WARPS) {
    float m = -INFINITY;
    for (int i = lane; i < k1 - k0; i += 32) m = fmaxf(m, sc[g][i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.0f;
    for (int i = lane; i < k1 - k0; i += 32) {
      const float e = m == -INFINITY ? 0.0f : __expf(sc[g][i] - m);
      sc[g][i] = e;
      l += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) {
      sm[g] = m;
      sl[g] = l;
    }
  }
  __syncthreads();
  // Values on the tensor pipe too: O[16 x D] += P[16 x 16] V[16 x D], 16 keys per step.  The B
  // operand wants pairs of consecutive KEYS of one dim in a register, while a row-major V gives
  // pairs of consecutive DIMS of one key: each of the four registers of a lane's 16-byte load is an
  // 8 x 8 matrix (key x dim pair) over the warp, and movmatrix transposes it in registers.  Which
  // head dim an accumulator column then stands for follows from the load map (lane t of a quad
  // holds dims 8t .. 8t+7 of a 32-dim block): register i, column 2t+e  <->  dim 32 nb + 8t + 2i + e.
  {
    constexpr int NB = D / 32;
    const int quad = lane >> 2, t = lane & 3;
    float acc[NB][4][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nb][i][c] = 0.0f;
    auto prob = [&](int g, int j) -> float { return (g < G && j < k1) ? sc[g][j - k0] : 0.0f; };
    for (int j0 = k0 + warp * 16; j0 < k1; j0 += DEC_WARPS * 16) {
      uint4 raw[2][NB];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = j0 + 8 * h + quad;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          raw[h][nb] = j < k1 ? __ldcs(reinterpret_cast<const uint4 *>(v + rowOf(j) * D + nb * 32 + 8 * t))
                              : make_uint4(0, 0, 0, 0);
        }
      }
      uint32_t pa[4];
      pa[0] = decPack<T>(prob(quad, j0 + 2 * t), prob(quad, j0 + 2 * t + 1));
      pa[1] = decPack<T>(prob(quad + 8, j0 + 2 * t), prob(quad + 8, j0 + 2 * t + 1));
      pa[2] = decPack<T>(prob(quad, j0 + 2 * t + 8), prob(quad, j0 + 2 * t + 9));
      pa[3] = decPack<T>(prob(quad + 8, j0 + 2 * t + 8), prob(quad + 8, j0 + 2 * t + 9));
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const uint32_t lo[4] = {raw[0][nb].x, raw[0][nb].y, raw[0][nb].z, raw[0][nb].w};
        const uint32_t hi[4] = {raw[1][nb].x, raw[1][nb].y, raw[1][nb].z, raw[1][nb].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) decMma<T>(acc[nb][i], pa, decTranspose(lo[i]), decTranspose(hi[i]));
      }
    }
    // Sum over the warps in a fixed order (the same bits every run): warps (2,3) hand their sums to
    // (0,1), and warp 1 to warp 0, through two exchange slots.
    auto each = [&](auto &&f) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int g = quad + 8 * half;
        if (g < G) {
#pragma unroll
          for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int e = 0; e < 2; ++e) f(g, nb * 32 + 8 * t + 2 * i + e, acc[nb][i][2 * half + e]);
        }
      }
    };
    auto give = [&](int slot) { each([&](int g, int d, float &v) { so[slot][g][d] = v; }); };
    auto take = [&](int slot) { each([&](int g, int d, float &v) { v += so[slot][g][d]; }); };
#pragma unroll
    for (int base = DEC_WARPS - 2; base >= 2; base -= 2) {
      if (warp == base || warp == base + 1) give(warp - base);
      __syncthreads();
      if (warp == base - 2 || warp == base - 1) take(warp - (base - 2));
      __syncthreads();
    }
    if (warp == 1) give(0);
    __syncthreads();
    if (warp == 0) {
      take(0);
      each([&](int g, int d, float &v) { po[(part + static_cast<size_t>(g) * p.chunks) * D + d] = v; });
    }
  }
  if (threadIdx.x < G) {
    pm[part + static_cast<size_t>(threadIdx.x) * p.chunks] = sm[threadIdx.x];
    pl[part + static_cast<size_t>(threadIdx.x) * p.chunks] = sl[threadIdx.x];
  }
}

// Merges the chunks of one (user, head): one warp per pair.
template <typename T, int D>
__global__ void __launch_bounds__(256) sdpaDecodeMergeKernel(const float *__restrict__ pm, const float *__restrict__ pl,
                                                             const float *__restrict__ po, T *__restrict__ out, int pairs,
                                                             int chunks) {
  constexpr int DPL = D / 32;
  pdlLaunchDependents();
  pdlWait();
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (pair >= pairs) return;
  const float *m = pm + static_cast<size_t>(pair) * chunks, *l = pl + static_cast<size_t>(pair) * chunks;
  float mx = -INFINITY;
  for (int c = 0; c < chunks; ++c) mx = fmaxf(mx, m[c]);
  float acc[DPL], den = 0.0f;
#pragma unroll
  for (int d = 0; d < DPL; ++d) acc[d] = 0.0f;
  for (int c = 0; c < chunks; ++c) {
    if (m[c] == -INFINITY) continue;
    const float w = __expf(m[c] - mx);
    den += l[c] * w;
    const float *o = po + (static_cast<size_t>(pair) * chunks + c) * D + lane * DPL;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[d] = fmaf(o[d], w, acc[d]);
  }
  const float inv = den > 0.0f ? 1.0f / den : 0.0f;
#pragma unroll
  for (int d = 0; d < DPL; ++d) out[static_cast<size_t>(pair) * D + lane * DPL + d] = fromF32<T>(acc[d] * inv);
}

template <typename T, int G, int D>
static int launchDecode(const void *q, const void *k, const void *v, const void *curPos, const void *mask, void *out,
                        float *pm, float *pl, float *po, const DecodeParams &p, cudaStream_t st) {
  dim3 grid(static_cast<unsigned>(p.chunks), static_cast<unsigned>(p.Hkv), static_cast<unsigned>(p.B));
  TTB_CUDA(launchPdl(sdpaDecodeChunkKernel<T, G, D>, grid, dim3(DEC_THREADS), 0, st, static_cast<const T *>(q),
                     static_cast<const T *>(k), static_cast<const T *>(v), static_cast<const int32_t *>(curPos),
                     static_cast<const T *>(mask), pm, pl, po, p));
  const int pairs = p.B * p.H;
  TTB_CUDA(launchPdl(sdpaDecodeMergeKernel<T, D>, dim3((pairs + 7) / 8), dim3(256), 0, st, static_cast<const float *>(pm),
                     static_cast<const float *>(pl), static_cast<const float *>(po), static_cast<T *>(out), pairs, p.chunks));
  countLaunch(2);
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

template <typename T, int D>
static int dispatchDecodeG(int g, const void *q, const void *k, const void *v, const void *curPos, const void *mask, void *out,
                           float *pm, float *pl, float *po, const DecodeParams &p, cudaStream_t st) {
  switch (g) {
  case 1: return launchDecode<T, 1, D>(q, k, v, curPos, mask, out, pm, pl, po, p, st);
  case 2: return launchDecode<T, 2, D>(q, k, v, curPos, mask, out, pm, pl, po, p, st);
  case 4: return launchDecode<T, 4, D>(q, k, v, curPos, mask, out, pm, pl, po, p, st);
  case 8: return launchDecode<T, 8, D>(q, k, v, curPos, mask, out, pm, pl, po, p, st);
  default: setLastError("sdpa_decode: query heads per kv head must be 1, 2, 4 or 8"); return TTB_ERR_UNSUPPORTED;
  }
}

} // namespace ttb

using namespace ttb;

// Set by ttb_sdpa_decode_paged around its call of ttb_sdpa_decode (same thread).
static thread_local const void *g_pagedTable = nullptr;
static thread_local int g_pagedBlockSize = 0, g_pagedPages = 0, g_pagedBlocks = 0;

extern "C" {

int ttb_fill_cache(void *cache, const void *input, int dtype, size_t users, size_t heads, size_t seq, size_t max_seq,
                   size_t head_dim, size_t batch_offset, size_t cache_users, void *stream) {
  TTB_CHECK(cache && input, "null tensor");
  TTB_CHECK(seq <= max_seq, "input is longer than the cache");
  TTB_CHECK(batch_offset + users <= cache_users, "input users do not fit the cache at this offset");
  const size_t rowBytes = head_dim * dtypeSize(dtype);
  TTB_CHECK(rowBytes > 0, "unsupported dtype");
  if (users * heads * seq == 0) return TTB_OK;
  size_t padSeq = (seq + 31) / 32 * 32; // the tile rows the reference's device op overwrites
  if (padSeq > max_seq) padSeq = seq;
  cudaStream_t st = asStream(stream);
  ProfScope prof("fill_cache", 0, double(users) * heads * seq * rowBytes * 2, st);
  const bool wide = rowBytes % 16 == 0 && aligned16(cache) && aligned16(input);
  const size_t items = users * heads * padSeq * (wide ? rowBytes / 16 : rowBytes / dtypeSize(dtype));
  const int grid = gridFor(items, 256);
  if (wide) {
    fillCacheKernel<uint4><<<grid, 256, 0, st>>>(static_cast<uint4 *>(cache), static_cast<const uint4 *>(input), users, heads,
                                                 seq, padSeq, max_seq, rowBytes / 16, batch_offset);
  } else if (dtypeSize(dtype) == 2) {
    fillCacheKernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<uint16_t *>(cache), static_cast<const uint16_t *>(input), users,
                                                    heads, seq, padSeq, max_seq, head_dim, batch_offset);
  } else if (dtypeSize(dtype) == 4) {
    fillCacheKernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<uint32_t *>(cache), static_cast<const uint32_t *>(input), users,
                                                    heads, seq, padSeq, max_seq, head_dim, batch_offset);
  } else {
    setLastError("fill_cache: unsupported element size");
    return TTB_ERR_UNSUPPORTED;
  }
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_update_cache(void *cache, const void *input, const void *index, int dtype, int index_dtype, size_t users,
                     size_t heads, size_t max_seq, size_t head_dim, size_t batch_offset, size_t cache_users, void *stream) {
  TTB_CHECK(cache && input && index, "null tensor");
  TTB_CHECK(batch_offset + users <= cache_users, "input users do not fit the cache at this offset");
  TTB_CHECK(index_dtype == kI32 || index_dtype == kU32, "update index must be Int32 or UInt32");
  const size_t es = dtypeSize(dtype);
  TTB_CHECK(es == 2 || es == 4, "unsupported element size");
  if (users * heads * head_dim == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  int *bad = nullptr;
  TTB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&bad), g_cacheBadIndex));
  ProfScope prof("update_cache", 0, double(users) * heads * head_dim * es * 2, st);
  const size_t items = users * heads * head_dim;
  const int grid = gridFor(items, 256);
#define TTB_UPD(U)                                                                                                    \
  if (index_dtype == kI32)                                                                                            \
    updateCacheKernel<U, int32_t><<<grid, 256, 0, st>>>(static_cast<U *>(cache), static_cast<const U *>(input),       \
                                                        static_cast<const int32_t *>(index), users, heads, max_seq,   \
                                                        head_dim, batch_offset, bad);                                 \
  else                                                                                                                \
    updateCacheKernel<U, uint32_t><<<grid, 256, 0, st>>>(static_cast<U *>(cache), static_cast<const U *>(input),      \
                                                         static_cast<const uint32_t *>(index), users, heads, max_seq, \
                                                         head_dim, batch_offset, bad);
  if (es == 2) { TTB_UPD(uint16_t) } else { TTB_UPD(uint32_t) }
#undef TTB_UPD
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_update_cache_status(int *bad_index_seen) {
  TTB_CHECK(bad_index_seen != nullptr, "null result");
  TTB_CUDA(cudaDeviceSynchronize());
  TTB_CUDA(cudaMemcpyFromSymbol(bad_index_seen, g_cacheBadIndex, sizeof(int)));
  if (*bad_index_seen) { // reported once
    const int zero = 0;
    TTB_CUDA(cudaMemcpyToSymbol(g_cacheBadIndex, &zero, sizeof(int)));
  }
  return TTB_OK;
}

size_t ttb_sdpa_decode_workspace_bytes(int batch, int heads, int seq, int head_dim) {
  const size_t chunks = static_cast<size_t>((seq + DEC_CHUNK - 1) / DEC_CHUNK);
  return static_cast<size_t>(batch) * heads * chunks * (static_cast<size_t>(head_dim) + 2) * sizeof(float);
}

int ttb_sdpa_decode(const void *q, const void *k, const void *v, const void *cur_pos, const void *mask, void *out, int dtype,
                    int batch, int heads, int kv_heads, int seq, int head_dim, int mask_users, int mask_heads, float scale,
                    int is_causal, void *workspace, size_t workspace_bytes, void *stream) {
  TTB_CHECK(q && k && v && out, "null tensor");
  TTB_CHECK(batch > 0 && heads > 0 && kv_heads > 0 && seq > 0, "empty problem");
  TTB_CHECK(heads % kv_heads == 0, "query heads must be a multiple of kv heads");
  TTB_CHECK(!mask || ((mask_users == 1 || mask_users == batch) && (mask_heads == 1 || mask_heads == heads)),
            "mask must be [B or 1, 1, H or 1, S]");
  if (dtype != kBF16 && dtype != kF16) {
    setLastError("sdpa_decode: bf16 or f16 only");
    return TTB_ERR_UNSUPPORTED;
  }
  if (!aligned16(k) || !aligned16(v)) {
    setLastError("sdpa_decode: the cache must be 16-byte aligned");
    return TTB_ERR_UNSUPPORTED;
  }
  DecodeParams p;
  p.B = batch; p.H = heads; p.Hkv = kv_heads; p.S = seq;
  p.pageTable = static_cast<const int32_t *>(g_pagedTable);
  p.blockSize = g_pagedBlockSize; p.pages = g_pagedPages; p.blocks = g_pagedBlocks;
  p.chunks = (seq + DEC_CHUNK - 1) / DEC_CHUNK;
  p.maskB = mask ? mask_users : 0;
  p.maskH = mask ? mask_heads : 0;
  p.scale = scale;
  p.causal = is_causal;
  const size_t need = ttb_sdpa_decode_workspace_bytes(batch, heads, seq, head_dim);
  TTB_CHECK(workspace && workspace_bytes >= need, "workspace too small (see ttb_sdpa_decode_workspace_bytes)");
  const size_t pairs = static_cast<size_t>(batch) * heads * p.chunks;
  float *pm = static_cast<float *>(workspace), *pl = pm + pairs, *po = pl + pairs;
  cudaStream_t st = asStream(stream);
  const int g = heads / kv_heads;
  // algorithmic bytes: the whole cache once (an upper bound when cur_pos cuts it short), q and out
  ProfScope prof("sdpa_decode", 4.0 * batch * heads * double(seq) * head_dim,
                 2.0 * batch * kv_heads * double(seq) * head_dim * 2 + 2.0 * batch * heads * head_dim * 2, st);
#define TTB_DEC(T)                                                                                                     \
  switch (head_dim) {                                                                                                  \
  case 32: return dispatchDecodeG<T, 32>(g, q, k, v, cur_pos, mask, out, pm, pl, po, p, st);                          \
  case 64: return dispatchDecodeG<T, 64>(g, q, k, v, cur_pos, mask, out, pm, pl, po, p, st);                          \
  case 128: return dispatchDecodeG<T, 128>(g, q, k, v, cur_pos, mask, out, pm, pl, po, p, st);                        \
  case 256: return dispatchDecodeG<T, 256>(g, q, k, v, cur_pos, mask, out, pm, pl, po, p, st);                        \
  default: setLastError("sdpa_decode: head_dim must be 32, 64, 128 or 256"); return TTB_ERR_UNSUPPORTED;                  \
  }
  if (dtype == kBF16) { TTB_DEC(__nv_bfloat16) }
  TTB_DEC(__half)
#undef TTB_DEC
}

int ttb_sdpa_decode_paged(const void *q, const void *k, const void *v, const void *page_table, const void *cur_pos,
                          const void *mask, void *out, int dtype, int batch, int heads, int kv_heads, int blocks, int block_size,
                          int pages_per_user, int head_dim, int mask_users, int mask_heads, float scale, int is_causal,
                          void *workspace, size_t workspace_bytes, void *stream) {
  TTB_CHECK(page_table != nullptr, "null page table");
  TTB_CHECK(blocks > 0 && block_size > 0 && pages_per_user > 0, "empty paged cache");
  g_pagedTable = page_table;
  g_pagedBlockSize = block_size;
  g_pagedPages = pages_per_user;
  g_pagedBlocks = blocks;
  const int rc = ttb_sdpa_decode(q, k, v, cur_pos, mask, out, dtype, batch, heads, kv_heads, pages_per_user * block_size, head_dim,
                                 mask_users, mask_heads, scale, is_causal, workspace, workspace_bytes, stream);
  g_pagedTable = nullptr;
  g_pagedBlockSize = g_pagedPages = g_pagedBlocks = 0;
  return rc;
}

int ttb_paged_update_cache(void *cache, const void *input, const void *update_index, const void *page_table, int dtype,
                           int index_dtype, int table_dtype, size_t users, size_t seq, size_t heads, size_t blocks,
                           size_t block_size, size_t pages, size_t head_dim, void *stream) {
  TTB_CHECK(cache && input && update_index, "null tensor");
  TTB_CHECK(index_dtype == kI32 || index_dtype == kU32, "update index must be Int32 or UInt32");
  TTB_CHECK(!page_table || table_dtype == kI32 || table_dtype == kU32, "page table must be Int32 or UInt32");
  TTB_CHECK(blocks > 0 && block_size > 0 && (!page_table || pages > 0), "empty paged cache");
  const size_t es = dtypeSize(dtype);
  TTB_CHECK(es == 2 || es == 4, "unsupported element size");
  if (users * seq * heads * head_dim == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("paged_update_cache", 0, double(users) * seq * heads * head_dim * es * 2, st);
  const int grid = gridFor(users * seq * heads * head_dim, 256);
#define TTB_PU(U, I, P)                                                                                                        pagedUpdateCacheKernel<U, I, P><<<grid, 256, 0, st>>>(static_cast<U *>(cache), static_cast<const U *>(input),                                                                      static_cast<const I *>(update_index), static_cast<const P *>(page_table),                                                         users, seq, heads, blocks, block_size, pages, head_dim)
#define TTB_PU_P(U, I)                                                                     if (table_dtype == kU32) TTB_PU(U, I, uint32_t);                                         else TTB_PU(U, I, int32_t);
#define TTB_PU_I(U)                                                                        if (index_dtype == kU32) { TTB_PU_P(U, uint32_t) } else { TTB_PU_P(U, int32_t) }
  if (es == 2) { TTB_PU_I(uint16_t) } else { TTB_PU_I(uint32_t) }
#undef TTB_PU_I
#undef TTB_PU_P
#undef TTB_PU
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_paged_fill_cache(void *cache, const void *input, const void *page_table, const void *batch_idx, int dtype,
                         int table_dtype, int batch_idx_dtype, size_t users, size_t heads, size_t seq, size_t blocks,
                         size_t block_size, size_t table_rows, size_t pages, size_t head_dim, void *stream) {
  TTB_CHECK(cache && input && page_table, "null tensor");
  TTB_CHECK(table_dtype == kI32 || table_dtype == kU32, "page table must be Int32 or UInt32");
  TTB_CHECK(!batch_idx || batch_idx_dtype == kI32 || batch_idx_dtype == kU32, "batch index must be Int32 or UInt32");
  TTB_CHECK(blocks > 0 && block_size > 0 && table_rows > 0 && pages > 0, "empty paged cache");
  const size_t es = dtypeSize(dtype);
  TTB_CHECK(es == 2 || es == 4, "unsupported element size");
  if (users * heads * seq * head_dim == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("paged_fill_cache", 0, double(users) * heads * seq * head_dim * es * 2, st);
  const int grid = gridFor(users * heads * seq * head_dim, 256);
#define TTB_PF(U, P, I)                                                                                                        pagedFillCacheKernel<U, P, I><<<grid, 256, 0, st>>>(static_cast<U *>(cache), static_cast<const U *>(input),                                                                      static_cast<const P *>(page_table), static_cast<const I *>(batch_idx), users,                                                       heads, seq, blocks, block_size, table_rows, pages, head_dim)
#define TTB_PF_I(U, P)                                                                     if (batch_idx_dtype == kU32) TTB_PF(U, P, uint32_t);                                     else TTB_PF(U, P, int32_t);
#define TTB_PF_P(U)                                                                        if (table_dtype == kU32) { TTB_PF_I(U, uint32_t) } else { TTB_PF_I(U, int32_t) }
  if (es == 2) { TTB_PF_P(uint16_t) } else { TTB_PF_P(uint32_t) }
#undef TTB_PF_P
#undef TTB_PF_I
#undef TTB_PF
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
