// Prefill LUT GEMM (placeholder until the tcgen05 kernel lands in this file).
#include "common.cuh"
using namespace b200lut;
extern "C" int b200lut_gemm(const void*, int64_t, int, int, int, const b200lut_segment*, int, int,
                            void*) {
  return fail(B200LUT_ERR_UNSUPPORTED, "b200lut_gemm is not built yet");
}
