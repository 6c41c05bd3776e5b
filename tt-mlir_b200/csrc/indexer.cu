// Lightning-indexer scores of DeepSeek sparse attention (::ttnn::experimental::indexer_score_dsa,
// operations/transformer/indexer_score_dsa.cpp; golden tools/golden/mapping.py:8695-8742):
//
//   score[b, 0, s, t] = sum over heads h of relu(q[b, h, s, :] . k[b, 0, t, :]) * w[b, h, s, 0]   for t <= offset + s,
//                       -inf for later keys.
//
// A contraction with a reduction behind it: the rows of the left operand are the (query, head) pairs of a group of
// eight queries (heads fastest), the right operand is a strip of 64 keys, both read as they are stored (keys are
// [t][d], which is the column-major operand of mma.sync).  One CTA of four warps walks its group's rows 64 at a
// time: products of a 64 x 64 tile on mma.sync m16n8k16 with f32 accumulators, relu and the per-row gate applied to
// the accumulators, the tile laid down in shared memory, and every (query, key) sum taken by ONE thread over the heads
// in ascending order, so the result does not depend on the schedule.  Strips that lie wholly in the future of all
// eight queries are written as -inf without loading anything.  Bound by the tensor pipe (2 * Hi * D flops per output
// element against 2 bytes written); the operands of a group come from L2.
#include "common.cuh"

#include <cmath>

namespace ttb {

constexpr int IX_BM = 64, IX_BN = 64, IX_BK = 32, IX_QG = 8;
constexpr int IX_P = IX_BK + 8; // padded row length (elements): conflict-free ldmatrix rows

template <typename T> __device__ __forceinline__ void ixMma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void ixMma<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void ixMma<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Eight consecutive elements of a row of `dim` elements starting at column d (zeros beyond the row's end).
template <typename T> __device__ __forceinline__ uint4 ixLoad8(const T *row, int d, int dim, bool vec) {
  if (vec && d + 8 <= dim) return *reinterpret_cast<const uint4 *>(row + d);
  __align__(16) T tmp[8];
  for (int j = 0; j < 8; ++j) tmp[j] = d + j < dim ? row[d + j] : fromF32<T>(0.0f);
  return *reinterpret_cast<uint4 *>(tmp);
}

template <typename T>
__global__ void __launch_bounds__(128) indexerScoreKernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ w,
                                                          T *__restrict__ out, int heads, int seqQ, int seqK, int dim, long long offset) {
  __shared__ __align__(16) T Qs[IX_BM * IX_P];
  __shared__ __align__(16) T Ks[IX_BN * IX_P];
  __shared__ float Ws[IX_BM][IX_BN + 1];
  __shared__ float sums[IX_QG][IX_BN];
  __shared__ float gate[IX_BM];
  const int b = blockIdx.z, s0 = blockIdx.y * IX_QG, t0 = blockIdx.x * IX_BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int queries = seqQ - s0 < IX_QG ? seqQ - s0 : IX_QG;
  T *outB = out + static_cast<size_t>(b) * seqQ * seqK;
  const T minusInf = fromF32<T>(-INFINITY);

  if (static_cast<long long>(t0) > offset + s0 + queries - 1) { // the whole strip lies in the future of every query here
    for (int i = tid; i < queries * IX_BN; i += blockDim.x) {
      const int t = t0 + i % IX_BN;
      if (t < seqK) outB[static_cast<size_t>(s0 + i / IX_BN) * seqK + t] = minusInf;
    }
    return;
  }

  const int rowsTotal = queries * heads; // row r = (query r / heads, head r % heads)
  const T *kB = k + static_cast<size_t>(b) * seqK * dim;
  const bool vec = (dim % 8) == 0;
  for (int i = tid; i < IX_QG * IX_BN; i += blockDim.x) (&sums[0][0])[i] = 0.0f;

  for (int chunk = 0; chunk < rowsTotal; chunk += IX_BM) {
    if (tid < IX_BM) {
      const int r = chunk + tid;
      gate[tid] = r < rowsTotal ? toF32(w[(static_cast<size_t>(b) * heads + r % heads) * seqQ + s0 + r / heads]) : 0.0f;
    }
    float acc[4][2][4] = {};
    for (int d0 = 0; d0 < dim; d0 += IX_BK) {
      // 64 rows x 32 columns of each operand = 256 vectors of 8: two per thread and operand.
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int idx = tid + h * 128, rr = idx >> 2, dv = d0 + (idx & 3) * 8;
        const int r = chunk + rr, t = t0 + rr;
        uint4 qv = make_uint4(0, 0, 0, 0), kv = make_uint4(0, 0, 0, 0);
        if (r < rowsTotal) qv = ixLoad8(q + ((static_cast<size_t>(b) * heads + r % heads) * seqQ + s0 + r / heads) * dim, dv, dim, vec);
        if (t < seqK) kv = ixLoad8(kB + static_cast<size_t>(t) * dim, dv, dim, vec);
        *reinterpret_cast<uint4 *>(&Qs[rr * IX_P + (idx & 3) * 8]) = qv;
        *reinterpret_cast<uint4 *>(&Ks[rr * IX_P + (idx & 3) * 8]) = kv;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < IX_BK; kk += 16) {
        uint32_t bf[4];
        {
          // keys are stored [t][d]: four 8 x 8 blocks (keys 0-7 / 8-15 of this warp's 16) x (d 0-7 / 8-15)
          const uint32_t addr = static_cast<uint32_t>(
              __cvta_generic_to_shared(&Ks[(warp * 16 + (lane & 7) + (lane >> 4) * 8) * IX_P + kk + ((lane >> 3) & 1) * 8]));
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(bf[0]), "=r"(bf[1]), "=r"(bf[2]), "=r"(bf[3]) : "r"(addr));
        }
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          uint32_t af[4];
          const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(&Qs[(mt * 16 + (lane & 15)) * IX_P + kk + (lane >> 4) * 8]));
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3]) : "r"(addr));
          ixMma<T>(acc[mt][0], af, bf[0], bf[1]);
          ixMma<T>(acc[mt][1], af, bf[2], bf[3]);
        }
      }
      __syncthreads();
    }
    // relu and the gate of the row, then the tile goes to shared memory
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int rr = mt * 16 + (lane >> 2) + h * 8, col = warp * 16 + nt * 8 + (lane & 3) * 2;
          const float g = gate[rr], x0 = acc[mt][nt][h * 2], x1 = acc[mt][nt][h * 2 + 1];
          Ws[rr][col] = (x0 > 0.0f ? x0 : (x0 != x0 ? x0 : 0.0f)) * g;
          Ws[rr][col + 1] = (x1 > 0.0f ? x1 : (x1 != x1 ? x1 : 0.0f)) * g;
        }
      }
    }
    __syncthreads();
    {
      // thread (col, part) owns the sums of the queries whose number has parity `part`: heads in ascending order
      const int col = tid & (IX_BN - 1), part = tid >> 6;
      for (int rr = 0; rr < IX_BM && chunk + rr < rowsTotal; ++rr) {
        const int ql = (chunk + rr) / heads;
        if ((ql & 1) == part) sums[ql][col] += Ws[rr][col];
      }
    }
    __syncthreads();
  }

  for (int i = tid; i < queries * IX_BN; i += blockDim.x) {
    const int ql = i / IX_BN, col = i % IX_BN, t = t0 + col, s = s0 + ql;
    if (t < seqK) outB[static_cast<size_t>(s) * seqK + t] = static_cast<long long>(t) <= offset + s ? fromF32<T>(sums[ql][col]) : minusInf;
  }
}

} // namespace ttb

using namespace ttb;

extern "C" int ttb_indexer_score_dsa(const void *q, const void *k, const void *weights, void *out, int dtype, int64_t batch, int64_t heads,
                                     int64_t seq_q, int64_t seq_kv, int64_t head_dim, int64_t offset, void *stream) {
  TTB_CHECK(q && k && weights && out, "null tensor");
  TTB_CHECK(batch >= 0 && heads > 0 && seq_q >= 0 && seq_kv >= 0 && head_dim > 0, "bad indexer geometry");
  TTB_CHECK(batch <= 65535 && (seq_q + IX_QG - 1) / IX_QG <= 65535 && heads <= (1 << 20) && seq_q < (int64_t(1) << 31) &&
                seq_kv < (int64_t(1) << 31) - IX_BN && head_dim < (int64_t(1) << 31) - IX_BK,
            "indexer problem too large for one launch");
  if (batch == 0 || seq_q == 0 || seq_kv == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("indexer_score_dsa", 2.0 * double(batch) * heads * seq_q * seq_kv * head_dim, double(batch) * seq_q * seq_kv * dtypeSize(dtype), st);
  dim3 grid(static_cast<unsigned>((seq_kv + IX_BN - 1) / IX_BN), static_cast<unsigned>((seq_q + IX_QG - 1) / IX_QG), static_cast<unsigned>(batch));
#define TTB_IX(T)                                                                                                            \
  indexerScoreKernel<T><<<grid, 128, 0, st>>>(static_cast<const T *>(q), static_cast<const T *>(k), static_cast<const T *>(weights), \
                                              static_cast<T *>(out), static_cast<int>(heads), static_cast<int>(seq_q),      \
                                              static_cast<int>(seq_kv), static_cast<int>(head_dim), static_cast<long long>(offset))
  switch (dtype) {
  case kBF16: TTB_IX(__nv_bfloat16); break;
  case kF16: TTB_IX(__half); break;
  default: setLastError("indexer_score_dsa takes bf16 or f16 tensors"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_IX
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}
