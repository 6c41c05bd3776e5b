// ttb_gemm: picks the kernel for a matmul / linear.  bf16 and f16 problems whose shapes fit
// the tile constraints run on the tcgen05 tensor-core kernel (gemm_tcgen05.cu); f32 problems
// and everything else run on the CUDA-core kernel (gemm_simt.cu).
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace ttb {
// Returns -1 when the problem is not one the tensor-core kernel takes.
int gemmTcgen05Try(const void *a, const void *b, const void *bias, void *c, int abDtype, int biasDtype, int cDtype,
                   int64_t batch, int64_t m, int64_t n, int64_t k, int transA, int transB, int64_t aBatchStride,
                   int64_t bBatchStride, int act, int roundSteps, const void *extra, int extraOp, cudaStream_t stream,
                   void *const *pushTargets = nullptr, int pushRanks = 0);
int gemmTcgen05SwigluTry(const void *a, const void *wGate, const void *wUp, void *out, int dtype, int64_t m, int64_t n,
                         int64_t k, cudaStream_t stream);
int gemmTcgen05DualTry(const void *a1, const void *b1, const void *bias1, const void *a2, const void *b2, const void *bias2,
                       void *out, int dtype, int biasDtype, int64_t m, int64_t n, int64_t k1, int64_t k2, int act,
                       cudaStream_t stream);
int gemmTcgen05GroupedTry(const void *a, const void *const *b, void *const *c, const int64_t *n, int count, int abDtype,
                          int cDtype, int64_t m, int64_t k, cudaStream_t stream, const void *ropeCos = nullptr,
                          const void *ropeSin = nullptr, int ropeMask = 0, int64_t ropeSeq = 1);
} // namespace ttb

static bool tcgen05Disabled() {
  static const bool disabled = [] {
    const char *e = std::getenv("TTB_DISABLE_TCGEN05");
    return e && e[0] && std::strcmp(e, "0") != 0;
  }();
  return disabled;
}

extern "C" int ttb_gemm(const void *a, const void *b, const void *bias, void *c, int ab_dtype, int bias_dtype,
                        int c_dtype, int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                        int64_t a_batch_stride, int64_t b_batch_stride, int act, int round_steps, void *stream) {
  return ttb_gemm_fused(a, b, bias, c, ab_dtype, bias_dtype, c_dtype, batch, m, n, k, trans_a, trans_b, a_batch_stride,
                        b_batch_stride, act, round_steps, nullptr, TTB_EXTRA_NONE, stream);
}

extern "C" int ttb_gemm_fused(const void *a, const void *b, const void *bias, void *c, int ab_dtype, int bias_dtype,
                              int c_dtype, int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                              int64_t a_batch_stride, int64_t b_batch_stride, int act, int round_steps,
                              const void *extra, int extra_op, void *stream) {
  TTB_CHECK(extra_op >= TTB_EXTRA_NONE && extra_op <= TTB_EXTRA_ADD_RELU, "unknown extra_op");
  TTB_CHECK(extra_op == TTB_EXTRA_NONE || extra != nullptr, "extra_op without its operand");
  if (!tcgen05Disabled()) {
    int rc = ttb::gemmTcgen05Try(a, b, bias, c, ab_dtype, bias_dtype, c_dtype, batch, m, n, k, trans_a, trans_b,
                                 a_batch_stride, b_batch_stride, act, round_steps, extra, extra_op, ttb::asStream(stream));
    if (rc != -1) return rc;
  }
  int rc = ttb_gemm_simt(a, b, bias, c, ab_dtype, bias_dtype, c_dtype, batch, m, n, k, trans_a, trans_b, a_batch_stride,
                         b_batch_stride, act, round_steps, stream);
  if (rc || extra_op == TTB_EXTRA_NONE) return rc;
  // The CUDA-core kernel has no second epilogue operand: apply it in place with the elementwise kernels.
  const size_t count = static_cast<size_t>(batch * m * n);
  if (extra_op == TTB_EXTRA_SILU_MUL) return ttb_silu_mul(extra, c, c, c_dtype, count, stream);
  int64_t shape[1] = {static_cast<int64_t>(count)}, ones[1] = {1};
  rc = ttb_eltwise_binary(0 /* EltwiseBinaryOpType::Add */, c, c_dtype, extra, c_dtype, c, c_dtype, 1, shape, ones, ones, stream);
  if (rc || extra_op == TTB_EXTRA_ADD) return rc;
  return ttb_eltwise_unary(8 /* EltwiseUnaryOpType::Relu */, c, c_dtype, c, c_dtype, count, 0.0f, stream);
}

extern "C" int ttb_gemm_grouped(const void *a, const void *const *b, void *const *c, const int64_t *n, int count,
                                int ab_dtype, int c_dtype, int64_t m, int64_t k, void *stream) {
  TTB_CHECK(a && b && c && n && count >= 1 && count <= 3, "bad argument");
  for (int i = 0; i < count; ++i) TTB_CHECK(b[i] && c[i] && n[i] >= 0, "bad argument");
  if (!tcgen05Disabled()) {
    int rc = ttb::gemmTcgen05GroupedTry(a, b, c, n, count, ab_dtype, c_dtype, m, k, ttb::asStream(stream));
    if (rc != -1) return rc;
  }
  for (int i = 0; i < count; ++i) {
    int rc = ttb_gemm(a, b[i], nullptr, c[i], ab_dtype, 0, c_dtype, 1, m, n[i], k, 0, 1, 0, 0, TTB_ACT_NONE, 0, stream);
    if (rc) return rc;
  }
  return TTB_OK;
}

// ttb_gemm_grouped whose results, for the problems in `rope_mask`, leave the kernel already rotated: C_i's columns
// are heads of 128 values, row r has position r mod seq, and every head is replaced by
// x cos[pos] + rotate_half(x) sin[pos] computed from the rounded product, exactly what rotary_embedding makes of the
// stored result of the linear op.  Only the tensor-core kernel has this mode: TTB_ERR_UNSUPPORTED tells the caller to
// run the grouped product and the rotary embeddings separately.
extern "C" int ttb_gemm_grouped_rope(const void *a, const void *const *b, void *const *c, const int64_t *n, int count,
                                     int dtype, int64_t m, int64_t k, const void *cos, const void *sin, int rope_mask,
                                     int64_t seq, int64_t head_dim, void *stream) {
  TTB_CHECK(a && b && c && n && count >= 2 && count <= 3 && cos && sin, "bad argument");
  for (int i = 0; i < count; ++i) TTB_CHECK(b[i] && c[i] && n[i] >= 0, "bad argument");
  TTB_CHECK(rope_mask > 0 && (rope_mask >> count) == 0 && seq >= 1, "bad rope mask or sequence length");
  if (head_dim == 128 && !tcgen05Disabled()) {
    int rc = ttb::gemmTcgen05GroupedTry(a, b, c, n, count, dtype, dtype, m, k, ttb::asStream(stream), cos, sin, rope_mask, seq);
    if (rc != -1) return rc;
  }
  ttb::setLastError("gemm_grouped_rope: shape, type or alignment not taken by the tensor-core kernel");
  return TTB_ERR_UNSUPPORTED;
}

// out[M, N] = act(round(A1 B1^T + bias1) + round(A2 B2^T + bias2)): two linear ops (or pointwise convolutions) with
// their biases, the add of their results and an optional relu, every intermediate rounded to `dtype` as the chain of
// separate ops rounds it, in one launch in which neither product reaches memory.  Only the tensor-core kernel has
// this mode: TTB_ERR_UNSUPPORTED tells the caller to run the ops one by one.
extern "C" int ttb_gemm_dual_add(const void *a1, const void *b1, const void *bias1, const void *a2, const void *b2,
                                 const void *bias2, void *out, int dtype, int bias_dtype, int64_t m, int64_t n, int64_t k1,
                                 int64_t k2, int act, void *stream) {
  TTB_CHECK(a1 && b1 && a2 && b2 && out, "null tensor");
  TTB_CHECK(m >= 0 && n >= 0 && k1 >= 0 && k2 >= 0, "negative dimension");
  if (m * n == 0) return TTB_OK;
  if (!tcgen05Disabled()) {
    int rc = ttb::gemmTcgen05DualTry(a1, b1, bias1, a2, b2, bias2, out, dtype, bias_dtype, m, n, k1, k2, act, ttb::asStream(stream));
    if (rc != -1) return rc;
  }
  ttb::setLastError("gemm_dual_add: shape, type or alignment not taken by the tensor-core kernel");
  return TTB_ERR_UNSUPPORTED;
}

// C = A[M, K] B[N, K]^T whose row block o (M / nranks rows) is stored into targets[o] instead of
// one matrix: the producer half of an all-reduce over peer memory (ttb_symm_push_targets gives the
// targets, ttb_symm_all_reduce_pushed finishes the sum).  Only the tensor-core kernel has this
// mode; TTB_ERR_UNSUPPORTED tells the caller to produce C normally and use ttb_symm_all_reduce.
extern "C" int ttb_gemm_push(const void *a, const void *b, void *const *targets, int nranks, int ab_dtype, int64_t m,
                             int64_t n, int64_t k, void *stream) {
  TTB_CHECK(a && b && targets, "null tensor");
  TTB_CHECK(nranks >= 2 && nranks <= 8, "nranks must be between 2 and 8");
  if (!tcgen05Disabled()) {
    int rc = ttb::gemmTcgen05Try(a, b, nullptr, nullptr, ab_dtype, 0, ab_dtype, 1, m, n, k, 0, 1, 0, 0, TTB_ACT_NONE, 0, nullptr,
                                 TTB_EXTRA_NONE, ttb::asStream(stream), targets, nranks);
    if (rc != -1) return rc;
  }
  ttb::setLastError("gemm_push: shape, type or alignment not taken by the tensor-core kernel");
  return TTB_ERR_UNSUPPORTED;
}

// out[M, N] = silu(A Wg^T) * (A Wu^T), every intermediate rounded to the element type as the chain
// linear, linear, silu, multiply rounds it.  One launch of the tensor-core kernel when it takes the
// shape; otherwise the gate projection goes to a temporary and the up projection's epilogue gates it.
extern "C" int ttb_gemm_swiglu(const void *a, const void *w_gate, const void *w_up, void *out, int dtype, int64_t m,
                               int64_t n, int64_t k, void *stream) {
  TTB_CHECK(a && w_gate && w_up && out, "null tensor");
  TTB_CHECK(m >= 0 && n >= 0 && k >= 0, "negative dimension");
  if (m * n == 0) return TTB_OK;
  if (!tcgen05Disabled()) {
    int rc = ttb::gemmTcgen05SwigluTry(a, w_gate, w_up, out, dtype, m, n, k, ttb::asStream(stream));
    if (rc != -1) return rc;
  }
  void *gate = nullptr;
  int rc = ttb_malloc(&gate, static_cast<size_t>(m) * n * ttb::dtypeSize(dtype), stream);
  if (rc) return rc;
  rc = ttb_gemm(a, w_gate, nullptr, gate, dtype, 0, dtype, 1, m, n, k, 0, 1, 0, 0, TTB_ACT_NONE, 0, stream);
  if (!rc) {
    rc = ttb_gemm_fused(a, w_up, nullptr, out, dtype, 0, dtype, 1, m, n, k, 0, 1, 0, 0, TTB_ACT_NONE, 0, gate, TTB_EXTRA_SILU_MUL,
                        stream);
  }
  int rc2 = ttb_free(gate, stream);
  return rc ? rc : rc2;
}
