// Low-rank residual of the decode path, first factor: t[m, r] = sum_k x[m, k] * resB[r, k]
// (fp32), for M <= 16 activation rows and any number of stacked residual rows (the rB factors
// of the projections that share an input — Q/K/V, or gate and up — are stacked along r, so
// one launch serves a whole merged GEMV). The second factor is folded into the GEMV epilogue
// (out[m, n] += sum_r t[m, r] * resA[n, r] before bias and the single rounding), which is
// what the reference's split-K kernel does inside one launch
// (src/flute_extended/src/kernel_gemv_splitk.cu:260-292, 340-349); there every block of a
// tile recomputes its slice of t, here t is computed once per launch chain and read back
// from L2.
//
// One block per residual row r: 256 threads stride over K with 16-byte loads of the row, the
// activation rows come from L2 (ld.global.cg — they were just written by the previous
// kernel), partial sums meet in a fixed order (lane tree, then warps in index order), so the
// result does not depend on the schedule. Written for programmatic dependent launch: the
// residual row is requested before griddepcontrol.wait, only x depends on the predecessor.
#include "common.cuh"

namespace b200lut {
namespace {

constexpr int kProjThreads = 256;
constexpr int kProjMaxM = 16;

template <typename T>
__device__ __forceinline__ float elem(uint32_t packed, int hi) {
  return DType<T>::to_float(uint16_t(hi ? packed >> 16 : packed & 0xFFFFu));
}

template <typename T>
__global__ void __launch_bounds__(kProjThreads) residual_project_kernel(
    const uint16_t* __restrict__ x, long long ldx, int M, int K, const uint16_t* __restrict__ resB,
    float* __restrict__ t, long long ldt) {
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint16_t* row = resB + size_t(r) * K;
  asm volatile("griddepcontrol.launch_dependents;");

  float acc[kProjMaxM];
#pragma unroll
  for (int m = 0; m < kProjMaxM; ++m) acc[m] = 0.f;
  // 8 elements (16 bytes) per thread and step (K is a multiple of 64); the row's next piece is
  // requested one step ahead, the first one before the dependency wait
  int k0 = threadIdx.x * 8;
  uint4 b = make_uint4(0u, 0u, 0u, 0u);
  if (k0 < K) b = __ldg(reinterpret_cast<const uint4*>(row + k0));
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (; k0 < K; k0 += kProjThreads * 8) {
    const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
    const int kn = k0 + kProjThreads * 8;
    if (kn < K) b = __ldg(reinterpret_cast<const uint4*>(row + kn));
#pragma unroll
    for (int m = 0; m < kProjMaxM; ++m) {
      if (m < M) {   // block-uniform
        const uint4 a = __ldcg(reinterpret_cast<const uint4*>(x + size_t(m) * ldx + k0));
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s = fmaf(elem<T>(aw[i], 0), elem<T>(bw[i], 0), s);
          s = fmaf(elem<T>(aw[i], 1), elem<T>(bw[i], 1), s);
        }
        acc[m] += s;
      }
    }
  }

  __shared__ float red[kProjThreads / 32][kProjMaxM];
#pragma unroll
  for (int m = 0; m < kProjMaxM; ++m) {
    if (m < M) {
      float v = acc[m];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
      if (lane == 0) red[warp][m] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < M) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kProjThreads / 32; ++w) v += red[w][threadIdx.x];
    t[size_t(threadIdx.x) * ldt + r] = v;
  }
}

}  // namespace
}  // namespace b200lut

using namespace b200lut;

extern "C" int b200lut_residual_project(const void* x, int64_t ldx, int M, int K, int dtype,
                                        const void* resB, int R, float* t, int64_t ldt, int flags,
                                        void* stream) {
  B200LUT_REQUIRE(x && resB && t, B200LUT_ERR_INVALID, "null x, resB or t");
  B200LUT_REQUIRE(M >= 1 && M <= kProjMaxM, B200LUT_ERR_UNSUPPORTED,
                  "the fused residual serves 1 <= M <= 16 rows, got M=%d", M);
  B200LUT_REQUIRE(K > 0 && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a positive multiple of 64, got %d", K);
  B200LUT_REQUIRE(R >= 1 && R <= 4096 && ldt >= R, B200LUT_ERR_INVALID,
                  "1 <= R <= 4096 stacked residual rows and ldt >= R (got R=%d, ldt=%lld)", R,
                  (long long)ldt);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(x) && aligned16(resB) && ldx % 8 == 0 && ldx >= K, B200LUT_ERR_ALIGN,
                  "x and resB must be 16-byte aligned, the x row stride a multiple of 8 and >= K");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(R), 1, 1);
  cfg.blockDim = dim3(kProjThreads, 1, 1);
  cfg.stream = cudaStream_t(stream);
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (flags & 1) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(na);
  const uint16_t* xp = static_cast<const uint16_t*>(x);
  const uint16_t* bp = static_cast<const uint16_t*>(resB);
  const long long ldx_ = ldx, ldt_ = ldt;
  if (dtype == B200LUT_BF16)
    B200LUT_CUDA_OK(cudaLaunchKernelEx(&cfg, residual_project_kernel<__nv_bfloat16>, xp, ldx_, M, K, bp, t, ldt_));
  else
    B200LUT_CUDA_OK(cudaLaunchKernelEx(&cfg, residual_project_kernel<__half>, xp, ldx_, M, K, bp, t, ldt_));
  return B200LUT_OK;
}
