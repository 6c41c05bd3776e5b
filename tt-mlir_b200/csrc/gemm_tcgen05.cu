#include "common.cuh"
namespace ttb {
int gemmTcgen05Try(const void *, const void *, const void *, void *, int, int, int, int64_t, int64_t, int64_t, int64_t,
                   int, int, int64_t, int64_t, int, int, cudaStream_t) {
  return -1;
}
} // namespace ttb
