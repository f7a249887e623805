// W4A16 prefill GEMM on the 5th-generation tensor cores (placeholder until the tcgen05 kernel lands).
#include "common.cuh"

using namespace ab200;

extern "C" int ab200_w4a16_gemm(const void *x, const int32_t *qweight, const void *scales, void *out, int M, int K,
                                int N, int group, int dtype, void *stream) {
  clear_error();
  (void)x; (void)qweight; (void)scales; (void)out; (void)M; (void)K; (void)N; (void)group; (void)dtype; (void)stream;
  return fail(AB200_EUNSUPPORTED, "w4a16_gemm: prefill kernel not built into this library");
}
