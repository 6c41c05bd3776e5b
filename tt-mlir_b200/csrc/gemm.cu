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
                   int64_t bBatchStride, int act, int roundSteps, cudaStream_t stream);
} // namespace ttb

extern "C" int ttb_gemm(const void *a, const void *b, const void *bias, void *c, int ab_dtype, int bias_dtype,
                        int c_dtype, int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                        int64_t a_batch_stride, int64_t b_batch_stride, int act, int round_steps, void *stream) {
  static const bool disabled = [] {
    const char *e = std::getenv("TTB_DISABLE_TCGEN05");
    return e && e[0] && std::strcmp(e, "0") != 0;
  }();
  if (!disabled) {
    int rc = ttb::gemmTcgen05Try(a, b, bias, c, ab_dtype, bias_dtype, c_dtype, batch, m, n, k, trans_a, trans_b,
                                 a_batch_stride, b_batch_stride, act, round_steps, ttb::asStream(stream));
    if (rc != -1) return rc;
  }
  return ttb_gemm_simt(a, b, bias, c, ab_dtype, bias_dtype, c_dtype, batch, m, n, k, trans_a, trans_b, a_batch_stride,
                       b_batch_stride, act, round_steps, stream);
}
