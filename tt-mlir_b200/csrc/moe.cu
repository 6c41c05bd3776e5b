// Mixture-of-experts routing and expert contractions, the generic (unfused) flow of the reference:
//   all_to_all_dispatch      operations/ccl/all_to_all_dispatch.cpp (::ttnn::all_to_all_dispatch)
//   moe_expert_token_remap   operations/ccl/moe_expert_token_remap.cpp (::ttnn::moe_expert_token_remap)
//   sparse_matmul            operations/matmul/matmul.cpp (::ttnn::sparse_matmul)
//   all_to_all_combine       operations/ccl/all_to_all_combine.cpp (::ttnn::all_to_all_combine)
// Goldens: tools/golden/mapping.py:1596-1760 (sparse_matmul, dispatch), 2030-2186 (combine, remap).
//
// Conventions shared by the kernels: T = D * B * S global tokens (device-major: tokens of mesh coordinate p come p-th,
// along the batch or the sequence dimension), K selected experts per token, E experts in all, `mapping` is the
// [E, D] one-hot ownership table, and a device numbers its own experts 0 .. E_local - 1 in ascending global order
// (`localIdx[e]`, -1 for experts that live elsewhere).
//
// Everything but the contraction is index work bound by HBM: one pass over the rows that move.  The contraction
// (`sparseMatmulKernel`) runs 32-row token blocks against one expert's [K, N] weights on mma.sync with the weights
// read as they are stored (ldmatrix.trans): per active (block, expert) pair it is bound by reading that expert's
// weights once from L2 / HBM, which is why pairs whose sparsity entry is zero are skipped before anything is loaded.
#include "common.cuh"

#include <type_traits>

namespace ttb {

// localIdx[e] = number of experts below e that this device owns when it owns e, else -1.  One block.
__global__ void moeLocalIndexKernel(const int32_t *__restrict__ mapping, int32_t *__restrict__ localIdx, int experts, int devices, int me) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int next = 0;
    for (int e = 0; e < experts; ++e) localIdx[e] = mapping[e * devices + me] != 0 ? next++ : -1;
  }
}

// The same from a table of owners (owner[e] = mesh coordinate of expert e), the format all_to_all_dispatch_metadata takes.
__global__ void moeLocalIndexOwnerKernel(const int32_t *__restrict__ owner, int32_t *__restrict__ localIdx, int experts, int me) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int next = 0;
    for (int e = 0; e < experts; ++e) localIdx[e] = owner[e] == me ? next++ : -1;
  }
}

// Rows of the gathered token buffer [T, H] that none of whose K experts lives here are cleared.
template <typename T>
__global__ void __launch_bounds__(256) moeDispatchMaskKernel(T *__restrict__ tokens, const int32_t *__restrict__ indices,
                                                             const int32_t *__restrict__ localIdx, size_t rows, size_t hidden, int k,
                                                             int experts) {
  for (size_t t = blockIdx.x; t < rows; t += gridDim.x) {
    bool routed = false;
    for (int j = 0; j < k; ++j) {
      const int32_t e = indices[t * k + j];
      routed = routed || (e >= 0 && e < experts && localIdx[e] >= 0);
    }
    if (routed) continue;
    for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) tokens[t * hidden + i] = fromF32<T>(0.0f);
  }
}

// partial[p, k, b, s, :] = expertOut[localIdx[e], token(p, b, s), :] when e = metadata[token, k] lives here, else 0.
// Summed over devices (exactly one owner per selected expert) this is the combine result of destination p.
template <typename T>
__global__ void __launch_bounds__(256) moeCombinePartialKernel(const T *__restrict__ expertOut, const int32_t *__restrict__ metadata,
                                                               const int32_t *__restrict__ localIdx, T *__restrict__ partial, int devices,
                                                               int k, int batch, int seq, size_t hidden, int experts, int localExperts,
                                                               int seqSharded) {
  const size_t rows = static_cast<size_t>(devices) * k * batch * seq;
  const int gBatch = seqSharded ? batch : batch * devices, gSeq = seqSharded ? seq * devices : seq;
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
    size_t q = r;
    const int s = static_cast<int>(q % seq);
    q /= seq;
    const int b = static_cast<int>(q % batch);
    q /= batch;
    const int slot = static_cast<int>(q % k);
    const int p = static_cast<int>(q / k);
    const int gb = seqSharded ? b : p * batch + b, gs = seqSharded ? p * seq + s : s;
    const size_t token = static_cast<size_t>(gb) * gSeq + gs;
    const int32_t e = metadata[token * k + slot];
    const int le = (e >= 0 && e < experts) ? localIdx[e] : -1;
    T *dst = partial + r * hidden;
    if (le >= 0 && le < localExperts) {
      const T *src = expertOut + ((static_cast<size_t>(le) * gBatch + gb) * gSeq + gs) * hidden;
      for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
    } else {
      for (size_t i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = fromF32<T>(0.0f);
    }
  }
}

// One block per `reduction` consecutive tokens: mapping[t, le] = topk[t, e] for the selected experts that live here,
// reduced[block, le] = 1 when any token of the block selected local expert le.
template <typename T, typename R>
__global__ void __launch_bounds__(256) moeRemapKernel(const T *__restrict__ topk, const int32_t *__restrict__ metadata,
                                                      const int32_t *__restrict__ localIdx, T *__restrict__ mapping, R *__restrict__ reduced,
                                                      size_t tokens, int k, int experts, int localExperts, int reduction) {
  extern __shared__ int used[]; // localExperts flags
  const size_t first = static_cast<size_t>(blockIdx.x) * reduction;
  const size_t last = first + reduction < tokens ? first + reduction : tokens;
  for (int i = threadIdx.x; i < localExperts; i += blockDim.x) used[i] = 0;
  for (size_t i = first * localExperts + threadIdx.x; i < last * localExperts; i += blockDim.x) mapping[i] = fromF32<T>(0.0f);
  __syncthreads();
  const size_t pairs = (last - first) * k;
  for (size_t i = threadIdx.x; i < pairs; i += blockDim.x) {
    const size_t t = first + i / k;
    const int32_t e = metadata[t * k + i % k];
    const int le = (e >= 0 && e < experts) ? localIdx[e] : -1;
    if (le >= 0 && le < localExperts) {
      mapping[t * localExperts + le] = topk[t * experts + e];
      used[le] = 1;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < localExperts; i += blockDim.x) {
    if constexpr (std::is_integral<R>::value) {
      reduced[static_cast<size_t>(blockIdx.x) * localExperts + i] = static_cast<R>(used[i]);
    } else {
      reduced[static_cast<size_t>(blockIdx.x) * localExperts + i] = fromF32<R>(used[i] ? 1.0f : 0.0f);
    }
  }
}

// ---- masked batched contraction -------------------------------------------------------------------
// C[i] = A[aIdx(i)] (M x K, row-major) * B[i % E] (K x N, row-major) for every entry i whose mask is non-zero; other
// entries are cleared.  One CTA (4 warps) per (64-column strip, 32-row block, entry); each warp owns 16 columns and
// both 16-row halves: four m16n8k16 products per 16-deep step.  A and B tiles go through padded shared memory;
// ldmatrix gives A's fragments, ldmatrix.trans turns B's [k][n] rows into the [n][k] fragments the instruction takes.
constexpr int SM_BM = 32, SM_BN = 64, SM_BK = 32;
constexpr int SM_AP = SM_BK + 8;  // padded row lengths (elements): conflict-free ldmatrix rows
constexpr int SM_BP = SM_BN + 8;

template <typename T> __device__ __forceinline__ void mmaM16N8K16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mmaM16N8K16<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mmaM16N8K16<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T, typename S>
__global__ void __launch_bounds__(128) sparseMatmulKernel(const T *__restrict__ a, const T *__restrict__ b, const S *__restrict__ mask,
                                                          T *__restrict__ c, int M, int N, int K, int experts, int aPerEntry) {
  __shared__ __align__(16) T As[SM_BM * SM_AP];
  __shared__ __align__(16) T Bs[SM_BK * SM_BP];
  const int entry = blockIdx.z, n0 = blockIdx.x * SM_BN, m0 = blockIdx.y * SM_BM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T *C = c + static_cast<size_t>(entry) * M * N;
  bool active;
  if constexpr (std::is_integral<S>::value) active = mask[entry] != 0;
  else active = toF32(mask[entry]) != 0.0f;
  if (!active) {
    for (int i = threadIdx.x; i < SM_BM * SM_BN; i += blockDim.x) {
      const int r = m0 + i / SM_BN, col = n0 + i % SM_BN;
      if (r < M && col < N) C[static_cast<size_t>(r) * N + col] = fromF32<T>(0.0f);
    }
    return;
  }
  const T *A = a + static_cast<size_t>(aPerEntry ? entry : entry / experts) * M * K;
  const T *B = b + static_cast<size_t>(entry % experts) * K * N;
  const bool vecA = (K % 8) == 0, vecB = (N % 8) == 0;
  float acc[2][2][4] = {};
  for (int k0 = 0; k0 < K; k0 += SM_BK) {
    // A tile: 32 rows x 32 k = 128 vectors of 8; B tile: 32 k x 64 columns = 256 vectors of 8.
    {
      const int r = threadIdx.x >> 2, kv = (threadIdx.x & 3) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int gr = m0 + r, gk = k0 + kv;
      if (gr < M && vecA && gk + 8 <= K) {
        v = *reinterpret_cast<const uint4 *>(A + static_cast<size_t>(gr) * K + gk);
      } else if (gr < M) {
        T tmp[8];
        for (int j = 0; j < 8; ++j) tmp[j] = gk + j < K ? A[static_cast<size_t>(gr) * K + gk + j] : fromF32<T>(0.0f);
        v = *reinterpret_cast<uint4 *>(tmp);
      }
      *reinterpret_cast<uint4 *>(&As[r * SM_AP + kv]) = v;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int idx = threadIdx.x + h * 128, r = idx >> 3, nv = (idx & 7) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int gk = k0 + r, gn = n0 + nv;
      if (gk < K && vecB && gn + 8 <= N) {
        v = *reinterpret_cast<const uint4 *>(B + static_cast<size_t>(gk) * N + gn);
      } else if (gk < K) {
        T tmp[8];
        for (int j = 0; j < 8; ++j) tmp[j] = gn + j < N ? B[static_cast<size_t>(gk) * N + gn + j] : fromF32<T>(0.0f);
        v = *reinterpret_cast<uint4 *>(tmp);
      }
      *reinterpret_cast<uint4 *>(&Bs[r * SM_BP + nv]) = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SM_BK; kk += 16) {
      uint32_t af[2][4], bf[4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(&As[(mt * 16 + (lane & 15)) * SM_AP + kk + (lane >> 4) * 8]));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(af[mt][0]), "=r"(af[mt][1]), "=r"(af[mt][2]), "=r"(af[mt][3]) : "r"(addr));
      }
      {
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(&Bs[(kk + (lane & 15)) * SM_BP + warp * 16 + (lane >> 4) * 8]));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(bf[0]), "=r"(bf[1]), "=r"(bf[2]), "=r"(bf[3]) : "r"(addr));
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        mmaM16N8K16<T>(acc[mt][0], af[mt], bf[0], bf[1]);
        mmaM16N8K16<T>(acc[mt][1], af[mt], bf[2], bf[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = m0 + mt * 16 + (lane >> 2) + h * 8, col = n0 + warp * 16 + nt * 8 + (lane & 3) * 2;
        if (r >= M) continue;
        if (col < N) C[static_cast<size_t>(r) * N + col] = fromF32<T>(acc[mt][nt][h * 2]);
        if (col + 1 < N) C[static_cast<size_t>(r) * N + col + 1] = fromF32<T>(acc[mt][nt][h * 2 + 1]);
      }
    }
  }
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_moe_local_index(const int32_t *mapping, int32_t *local_idx, int experts, int devices, int device, void *stream) {
  TTB_CHECK(mapping && local_idx, "null tensor");
  TTB_CHECK(experts > 0 && devices > 0 && device >= 0 && device < devices, "bad expert mapping geometry");
  moeLocalIndexKernel<<<1, 32, 0, asStream(stream)>>>(mapping, local_idx, experts, devices, device);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_moe_local_index_owner(const int32_t *owner, int32_t *local_idx, int experts, int device, void *stream) {
  TTB_CHECK(owner && local_idx, "null tensor");
  TTB_CHECK(experts > 0 && device >= 0, "bad expert mapping geometry");
  moeLocalIndexOwnerKernel<<<1, 32, 0, asStream(stream)>>>(owner, local_idx, experts, device);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_moe_dispatch_mask(void *tokens, const int32_t *indices, const int32_t *local_idx, int dtype, size_t rows, size_t hidden, int k,
                          int experts, void *stream) {
  TTB_CHECK(tokens && indices && local_idx, "null tensor");
  if (rows == 0 || hidden == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("moe_dispatch_mask", 0, double(rows) * k * 4, st);
  const int grid = static_cast<int>(rows < static_cast<size_t>(smCount()) * 8 ? rows : static_cast<size_t>(smCount()) * 8);
  TTB_DISPATCH_FLOAT(dtype, T, (moeDispatchMaskKernel<T><<<grid, 256, 0, st>>>(static_cast<T *>(tokens), indices, local_idx, rows, hidden, k, experts)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_moe_combine_partial(const void *expert_out, const int32_t *metadata, const int32_t *local_idx, void *partial, int dtype,
                            int devices, int k, int batch, int seq, size_t hidden, int experts, int local_experts, int seq_sharded,
                            void *stream) {
  TTB_CHECK(expert_out && metadata && local_idx && partial, "null tensor");
  const size_t rows = static_cast<size_t>(devices) * k * batch * seq;
  if (rows == 0 || hidden == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("moe_combine_partial", 0, double(rows) * hidden * dtypeSize(dtype) * 2, st);
  const int grid = static_cast<int>(rows < static_cast<size_t>(smCount()) * 8 ? rows : static_cast<size_t>(smCount()) * 8);
  TTB_DISPATCH_FLOAT(dtype, T,
                     (moeCombinePartialKernel<T><<<grid, 256, 0, st>>>(static_cast<const T *>(expert_out), metadata, local_idx,
                                                                      static_cast<T *>(partial), devices, k, batch, seq, hidden, experts,
                                                                      local_experts, seq_sharded)));
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_moe_expert_token_remap(const void *topk, const int32_t *metadata, const int32_t *local_idx, void *mapping, void *reduced,
                               int dtype, int reduced_dtype, size_t tokens, int k, int experts, int local_experts, int reduction,
                               void *stream) {
  TTB_CHECK(topk && metadata && local_idx && mapping && reduced, "null tensor");
  TTB_CHECK(reduction > 0 && local_experts > 0 && local_experts <= 4096, "bad reduction size or expert count");
  if (tokens == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  const unsigned blocks = static_cast<unsigned>((tokens + reduction - 1) / reduction);
  ProfScope prof("moe_expert_token_remap", 0, double(tokens) * (k * 4 + local_experts * dtypeSize(dtype)), st);
  const size_t smem = static_cast<size_t>(local_experts) * sizeof(int);
#define TTB_REMAP(R)                                                                                                        \
  TTB_DISPATCH_FLOAT(dtype, T,                                                                                              \
                     (moeRemapKernel<T, R><<<blocks, 256, smem, st>>>(static_cast<const T *>(topk), metadata, local_idx,     \
                                                                      static_cast<T *>(mapping), static_cast<R *>(reduced), tokens, k,      \
                                                                      experts, local_experts, reduction)))
  switch (reduced_dtype) {
  case kF32: TTB_REMAP(float); break;
  case kBF16: TTB_REMAP(__nv_bfloat16); break;
  case kF16: TTB_REMAP(__half); break;
  case kU16: TTB_REMAP(uint16_t); break;
  case kI32: TTB_REMAP(int32_t); break;
  case kU32: TTB_REMAP(uint32_t); break;
  default: setLastError("moe_expert_token_remap: unsupported type of the reduced tensor"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_REMAP
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

int ttb_sparse_matmul(const void *a, const void *b, const void *sparsity, void *c, int dtype, int sparsity_dtype, int64_t entries,
                      int64_t experts, int a_per_entry, int64_t m, int64_t n, int64_t k, void *stream) {
  TTB_CHECK(a && b && sparsity && c, "null tensor");
  TTB_CHECK(entries >= 0 && experts > 0 && m >= 0 && n >= 0 && k >= 0, "negative dimension");
  TTB_CHECK(entries <= 65535 && (m + SM_BM - 1) / SM_BM <= 65535, "grid too large");
  if (entries * m * n == 0) return TTB_OK;
  cudaStream_t st = asStream(stream);
  ProfScope prof("sparse_matmul", 2.0 * double(entries) * m * n * k, double(experts) * k * n * dtypeSize(dtype), st);
  dim3 grid(static_cast<unsigned>((n + SM_BN - 1) / SM_BN), static_cast<unsigned>((m + SM_BM - 1) / SM_BM), static_cast<unsigned>(entries));
#define TTB_SPMM(T, S)                                                                                                       \
  sparseMatmulKernel<T, S><<<grid, 128, 0, st>>>(static_cast<const T *>(a), static_cast<const T *>(b), static_cast<const S *>(sparsity), \
                                                 static_cast<T *>(c), static_cast<int>(m), static_cast<int>(n), static_cast<int>(k),   \
                                                 static_cast<int>(experts), a_per_entry)
#define TTB_SPMM_MASK(T)                                                                                                     \
  switch (sparsity_dtype) {                                                                                                  \
  case kF32: TTB_SPMM(T, float); break;                                                                                      \
  case kBF16: TTB_SPMM(T, __nv_bfloat16); break;                                                                             \
  case kF16: TTB_SPMM(T, __half); break;                                                                                     \
  case kU16: TTB_SPMM(T, uint16_t); break;                                                                                   \
  case kI32: TTB_SPMM(T, int32_t); break;                                                                                    \
  case kU32: TTB_SPMM(T, uint32_t); break;                                                                                   \
  default: setLastError("sparse_matmul: unsupported sparsity type"); return TTB_ERR_UNSUPPORTED;                             \
  }
  switch (dtype) {
  case kBF16: TTB_SPMM_MASK(__nv_bfloat16) break;
  case kF16: TTB_SPMM_MASK(__half) break;
  default: setLastError("sparse_matmul takes bf16 or f16 operands"); return TTB_ERR_UNSUPPORTED;
  }
#undef TTB_SPMM_MASK
#undef TTB_SPMM
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

} // extern "C"
