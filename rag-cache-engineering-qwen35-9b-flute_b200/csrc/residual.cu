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


// Prefill form of the same first factor, for any number of activation rows: t[m, c] rounded
// once to the compute dtype (the reference route rounds x @ resB^T to the factors' dtype before
// the second product, src/scripts/palettized_modules.py:1363-1364), written as a [M, ldt]
// matrix whose columns [R, cols) are zero so that the prefill GEMM can take 64-column blocks
// of it as extra k-blocks of its accumulator.
//
// One block per (16 activation rows, 64 columns of t): eight warps take the 32-wide k steps
// round-robin and run mma.sync m16n8k16 (bf16 / f16, fp32 sums) with the SAME permutation of
// k inside a step on both operands — lane (g, c) reads 16 contiguous bytes of its rows at
// k0 + 8 c and feeds elements (0,1) / (2,3) to the first instruction and (4,5) / (6,7) to the
// second — so every global load is a full 16-byte one and no shuffle is needed. The warps'
// partial sums meet in shared memory in warp order (the result does not depend on the
// schedule), then one rounding and the store.
constexpr int kRowsProjWarps = 8;
constexpr int kRowsProjCols = 64;
constexpr int kRowsProjPitch = kRowsProjCols + 4;   // floats per staged row

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (DType<T>::id == B200LUT_BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// TILES: 8-wide column tiles a block computes (4 when R <= 32 — the deployed rank — else 8).
// The kernel is a chain of memory round trips (activations from DRAM, residual rows from L2), so
// a warp fetches UNROLL k steps at a time with cp.async into its own two-stage staging area — no
// registers held while the loads fly — and multiplies one batch while the next one lands.
__device__ __forceinline__ void rp_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 rp_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

template <int TILES> struct RowsProj {
  static constexpr int kUnroll = TILES <= 4 ? 4 : 2;
  static constexpr int kRows = 16 + 8 * TILES;                 // staged rows of one k step
  static constexpr uint32_t kStepBytes = kRows * 64u;          // 32 k = 64 bytes per row
  static constexpr uint32_t kStageBytes = kUnroll * kStepBytes;
  static constexpr uint32_t kWarpBytes = 2u * kStageBytes;
  static constexpr uint32_t kRedBytes = kRowsProjWarps * 16 * kRowsProjPitch * 4;
  static constexpr uint32_t kSmem = kRowsProjWarps * kWarpBytes > kRedBytes ? kRowsProjWarps * kWarpBytes : kRedBytes;
};

template <typename T, int TILES>
__global__ void __launch_bounds__(kRowsProjWarps * 32) residual_rows_kernel(
    const uint16_t* __restrict__ x, long long ldx, int M, int K, const uint16_t* __restrict__ resB,
    int R, uint16_t* __restrict__ t, long long ldt, int cols) {
  using P = RowsProj<TILES>;
  extern __shared__ __align__(16) uint8_t rp_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int m0 = blockIdx.x * 16, c0 = blockIdx.y * kRowsProjCols;
  asm volatile("griddepcontrol.launch_dependents;");

  float acc[TILES][4];
#pragma unroll
  for (int j = 0; j < TILES; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
  const uint32_t mine = uint32_t(__cvta_generic_to_shared(rp_smem)) + uint32_t(warp) * P::kWarpBytes;
  const int steps = K / 32;
  const int nb = (steps > warp ? (steps - warp + kRowsProjWarps - 1) / kRowsProjWarps : 0);   // this warp's steps
  const int batches = (nb + P::kUnroll - 1) / P::kUnroll;
  // Rows beyond M and residual rows beyond R are read from the last valid row instead (their
  // products land in outputs that are never stored, or are stored as zero).
  auto fetch = [&](int batch) {
    const uint32_t st = mine + uint32_t(batch & 1) * P::kStageBytes;
#pragma unroll
    for (int u = 0; u < P::kUnroll; ++u) {
      const int i = batch * P::kUnroll + u;
      if (i < nb) {      // warp-uniform
        const int k0 = 32 * (warp + i * kRowsProjWarps);
#pragma unroll
        for (int pc = lane; pc < P::kRows * 4; pc += 32) {
          const int row = pc >> 2, part = pc & 3;
          const uint16_t* src;
          if (row < 16) {
            int m = m0 + row;
            m = m < M ? m : M - 1;
            src = x + size_t(m) * ldx + k0 + 8 * part;
          } else {
            int r = c0 + row - 16;
            r = r < R ? r : R - 1;
            src = resB + size_t(r) * K + k0 + 8 * part;
          }
          rp_cp_async16(st + uint32_t(u) * P::kStepBytes + uint32_t(row) * 64u + uint32_t(part) * 16u, src);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (batches > 0) fetch(0);
  for (int bt = 0; bt < batches; ++bt) {
    if (bt + 1 < batches) {
      fetch(bt + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncwarp();
    const uint32_t st = mine + uint32_t(bt & 1) * P::kStageBytes;
#pragma unroll
    for (int u = 0; u < P::kUnroll; ++u) {
      if (bt * P::kUnroll + u < nb) {      // warp-uniform
        const uint32_t sb = st + uint32_t(u) * P::kStepBytes + uint32_t(c) * 16u;
        const uint4 a = rp_lds128(sb + uint32_t(g) * 64u), b = rp_lds128(sb + uint32_t(g + 8) * 64u);
#pragma unroll
        for (int j = 0; j < TILES; ++j) {
          const uint4 w = rp_lds128(sb + uint32_t(16 + 8 * j + g) * 64u);
          mma16816<T>(acc[j], a.x, b.x, a.y, b.y, w.x, w.y);
          mma16816<T>(acc[j], a.z, b.z, a.w, b.w, w.z, w.w);
        }
      }
    }
    __syncwarp();      // the stage is refilled two batches on
  }
  __syncthreads();     // the staging areas are done with: the fold buffer takes their place
  float (*red)[16][kRowsProjPitch] = reinterpret_cast<float (*)[16][kRowsProjPitch]>(rp_smem);
#pragma unroll
  for (int j = 0; j < TILES; ++j) {
    red[warp][g][8 * j + 2 * c] = acc[j][0];
    red[warp][g][8 * j + 2 * c + 1] = acc[j][1];
    red[warp][g + 8][8 * j + 2 * c] = acc[j][2];
    red[warp][g + 8][8 * j + 2 * c + 1] = acc[j][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * kRowsProjCols; idx += kRowsProjWarps * 32) {
    const int r = idx / kRowsProjCols, col = idx % kRowsProjCols;
    if (m0 + r < M && c0 + col < cols) {
      float v = 0.f;
      if (col < 8 * TILES && c0 + col < R) {
#pragma unroll
        for (int w2 = 0; w2 < kRowsProjWarps; ++w2) v += red[w2][r][col];
      }
      t[size_t(m0 + r) * ldt + c0 + col] = DType<T>::from_float(v);
    }
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

extern "C" int b200lut_residual_project_rows(const void* x, int64_t ldx, int M, int K, int dtype,
                                             const void* resB, int R, void* t, int64_t ldt,
                                             int cols, int flags, void* stream) {
  B200LUT_REQUIRE(x && resB && t, B200LUT_ERR_INVALID, "null x, resB or t");
  B200LUT_REQUIRE(M >= 1, B200LUT_ERR_INVALID, "M must be >= 1, got %d", M);
  B200LUT_REQUIRE(K > 0 && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a positive multiple of 64, got %d", K);
  B200LUT_REQUIRE(R >= 1 && cols >= R && cols % kRowsProjCols == 0 && ldt >= cols && ldt % 8 == 0,
                  B200LUT_ERR_INVALID,
                  "need 1 <= R <= cols, cols a multiple of 64 and ldt >= cols, a multiple of 8 "
                  "(got R=%d, cols=%d, ldt=%lld)", R, cols, (long long)ldt);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(x) && aligned16(resB) && aligned16(t) && ldx % 8 == 0 && ldx >= K,
                  B200LUT_ERR_ALIGN,
                  "x, resB and t must be 16-byte aligned, the x row stride a multiple of 8 and >= K");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned((M + 15) / 16), unsigned(cols / kRowsProjCols), 1);
  cfg.blockDim = dim3(kRowsProjWarps * 32, 1, 1);
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
  uint16_t* tp = static_cast<uint16_t*>(t);
  const long long ldx_ = ldx, ldt_ = ldt;
  const bool narrow = R <= 32;     // four 8-wide column tiles hold every residual row
  cfg.dynamicSmemBytes = narrow ? RowsProj<4>::kSmem : RowsProj<8>::kSmem;
  auto go = [&](auto kern, int which) -> int {
    static bool configured[4][64] = {};     // the four instantiations share this lambda's type
    int dev = 0;
    B200LUT_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 64 || !configured[which][dev]) {
      B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           int(cfg.dynamicSmemBytes)));
      if (dev < 64) configured[which][dev] = true;
    }
    B200LUT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, xp, ldx_, M, K, bp, R, tp, ldt_, cols));
    return B200LUT_OK;
  };
  if (dtype == B200LUT_BF16)
    return narrow ? go(residual_rows_kernel<__nv_bfloat16, 4>, 0) : go(residual_rows_kernel<__nv_bfloat16, 8>, 1);
  return narrow ? go(residual_rows_kernel<__half, 4>, 2) : go(residual_rows_kernel<__half, 8>, 3);
}
