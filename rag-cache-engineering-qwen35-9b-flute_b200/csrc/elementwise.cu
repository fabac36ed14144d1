// SiLU(gate) * up over [M, N] 16-bit matrices, in place on the gate buffer: the pass between the
// gate/up projections and the down projection of an MLP at prefill width, where the two
// projections run as separate full-width tensor-core GEMMs (the reference's MLP does the same
// at M > 1: gate, up, act_fn(gate) * up; src/scripts/palettized_modules.py:1643-1723).
// Folding the multiply into the second GEMM's epilogue was measured slower (857 vs 894
// TFLOP/s on the stack with three torch kernels, because that epilogue is not hidden);
// this is one streaming pass: 16-byte loads and stores, fp32 silu, one rounding.
#include "common.cuh"

namespace b200lut {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(uint16_t* __restrict__ gate,
                                                       const uint16_t* __restrict__ up,
                                                       long long ldg, long long ldu, int M, int N8) {
  const long long total = (long long)M * N8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / N8;
    const int c = int(i - m * N8) * 8;
    uint4* gp = reinterpret_cast<uint4*>(gate + m * ldg + c);
    const uint4 g = *gp;
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(up + m * ldu + c));
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g0 = DType<T>::to_float(uint16_t(gw[e] & 0xFFFFu));
      const float g1 = DType<T>::to_float(uint16_t(gw[e] >> 16));
      const float u0 = DType<T>::to_float(uint16_t(uw[e] & 0xFFFFu));
      const float u1 = DType<T>::to_float(uint16_t(uw[e] >> 16));
      r[e] = uint32_t(DType<T>::from_float(g0 / (1.f + __expf(-g0)) * u0)) |
             (uint32_t(DType<T>::from_float(g1 / (1.f + __expf(-g1)) * u1)) << 16);
    }
    *gp = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

}  // namespace
}  // namespace b200lut

using namespace b200lut;

extern "C" int b200lut_silu_mul(void* gate, const void* up, int M, int N, int64_t ld_gate,
                                int64_t ld_up, int dtype, void* stream) {
  B200LUT_REQUIRE(gate && up, B200LUT_ERR_INVALID, "null gate or up");
  B200LUT_REQUIRE(M >= 0 && N >= 8 && N % 8 == 0, B200LUT_ERR_INVALID,
                  "N must be a positive multiple of 8 (got M=%d, N=%d)", M, N);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(gate) && aligned16(up) && ld_gate % 8 == 0 && ld_up % 8 == 0 &&
                      ld_gate >= N && ld_up >= N,
                  B200LUT_ERR_ALIGN, "rows must be 16-byte aligned (pointers and strides) and >= N");
  if (M == 0) return B200LUT_OK;
  const long long total = (long long)M * (N / 8);
  long long grid = (total + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  uint16_t* g = static_cast<uint16_t*>(gate);
  const uint16_t* u = static_cast<const uint16_t*>(up);
  if (dtype == B200LUT_BF16)
    silu_mul_kernel<__nv_bfloat16><<<unsigned(grid), 256, 0, cudaStream_t(stream)>>>(g, u, ld_gate, ld_up, M, N / 8);
  else
    silu_mul_kernel<__half><<<unsigned(grid), 256, 0, cudaStream_t(stream)>>>(g, u, ld_gate, ld_up, M, N / 8);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}
