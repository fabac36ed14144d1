// Row-wise fast Hadamard transform of the activations (the rotation in front of
// the palettized GEMV / GEMM). Replaces the reference's FHT kernels
// (src/flute_extended/src/kernel_fht.cu:70-255, include/flute/fht.cuh:84-178) and
// follows the arithmetic of its torch twin (src/flute_extended/fht.py:174-238):
// fp32 butterfly with stage length doubling from 1, each stage writing (a + b)
// to the low and (a - b) to the high element of a pair; forward applies
// * signs then * (1/sqrt(b)); adjoint applies * signs on load; the AWQ form
// multiplies by the scale on load and truly divides by it on store. Every output
// element is a fixed expression tree of fp32 adds, so results do not depend on
// the thread schedule and match the torch twin bit for bit.
//
// One block per (row, segment). In block mode (independent `block`-point
// transforms) the same butterfly simply stops after log2(block) stages.
#include "common.cuh"

namespace b200lut {
namespace {

constexpr int kMaxSegments = 16;
constexpr int kMaxPoints = 16384;   // 64 KB of fp32 per block

struct FhtParams {
  const void* x;
  void* out;
  const float* signs;
  const float* scale;
  long long ldx, ldo;
  int dtype, mode, nseg;
  int seg_off[kMaxSegments];
  int seg_len[kMaxSegments];     // points held by the block
  int seg_stages[kMaxSegments];  // butterfly stages to run (log2 of the transform size)
  float seg_inv[kMaxSegments];   // 1 / sqrt(transform size)
};

__device__ __forceinline__ float load_elem(const void* p, long long i, int dtype) {
  if (dtype == B200LUT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (dtype == B200LUT_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return static_cast<const float*>(p)[i];
}

__device__ __forceinline__ void store_elem(void* p, long long i, int dtype, float v) {
  if (dtype == B200LUT_BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else if (dtype == B200LUT_F16) static_cast<__half*>(p)[i] = __float2half_rn(v);
  else static_cast<float*>(p)[i] = v;
}

__global__ void __launch_bounds__(1024) fht_kernel(const FhtParams p) {
  extern __shared__ float buf[];
  const int row = blockIdx.x, sg = blockIdx.y;
  const int off = p.seg_off[sg], n = p.seg_len[sg], stages = p.seg_stages[sg];
  const float inv = p.seg_inv[sg];
  const long long xin = (long long)row * p.ldx + off;
  const long long xout = (long long)row * p.ldo + off;

  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = load_elem(p.x, xin + i, p.dtype);
    if (p.mode == B200LUT_FHT_AWQ) v = v * p.scale[off + i];
    else if (p.mode == B200LUT_FHT_ADJOINT && p.signs) v = v * p.signs[off + i];
    buf[i] = v;
  }
  __syncthreads();
  for (int st = 0; st < stages; ++st) {
    const int len = 1 << st;
    for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
      const int lo = ((i >> st) << (st + 1)) + (i & (len - 1));
      const float a = buf[lo], b = buf[lo + len];
      buf[lo] = a + b;
      buf[lo + len] = a - b;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = buf[i];
    if (p.mode == B200LUT_FHT_ADJOINT) {
      v = v * inv;
    } else {
      if (p.signs) v = v * p.signs[off + i];
      v = v * inv;
      if (p.mode == B200LUT_FHT_AWQ) v = __fdiv_rn(v, p.scale[off + i]);
    }
    store_elem(p.out, xout + i, p.dtype, v);
  }
}

// 128-point block transform, one block of 128 elements per warp, entirely in registers:
// lane L holds elements 4L .. 4L+3; stages of length 1 and 2 pair elements inside the lane,
// stages 4 .. 64 pair lanes L and L ^ (len / 4) through shuffles. Each output is the same
// expression tree of fp32 adds as in the shared-memory kernel (low element a + b, high
// element a - b), so the bits are identical; the kernel is a pure stream (HBM bound).
__global__ void __launch_bounds__(256) fht_block128_kernel(const FhtParams p, long long nblocks,
                                                          int blocks_per_row) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv = p.seg_inv[0];
  for (long long blk = warp0; blk < nblocks; blk += stride) {
    const long long row = blk / blocks_per_row;
    const int off = int(blk - row * blocks_per_row) * 128 + 4 * lane;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = load_elem(p.x, row * p.ldx + off + j, p.dtype);
      if (p.mode == B200LUT_FHT_AWQ) v[j] = v[j] * p.scale[off + j];
      else if (p.mode == B200LUT_FHT_ADJOINT && p.signs) v[j] = v[j] * p.signs[off + j];
    }
    {   // len 1, then len 2
      const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
      v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {   // len = 4 * m
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], m);
        v[j] = (lane & m) ? other - v[j] : v[j] + other;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float r = v[j];
      if (p.mode == B200LUT_FHT_ADJOINT) {
        r = r * inv;
      } else {
        if (p.signs) r = r * p.signs[off + j];
        r = r * inv;
        if (p.mode == B200LUT_FHT_AWQ) r = __fdiv_rn(r, p.scale[off + j]);
      }
      store_elem(p.out, row * p.ldo + off + j, p.dtype, r);
    }
  }
}

// The same transform for 16-bit data with 16-byte accesses: a lane holds 8 consecutive elements,
// 16 lanes hold one 128-point block, a warp two of them. Stages of length 1, 2, 4 stay inside
// the lane, stages 8 .. 64 pair lanes L and L ^ (len / 8). Same expression tree per output as
// above, so the bits are identical; half the memory instructions per byte.
template <typename T>
__global__ void __launch_bounds__(256) fht_block128_vec_kernel(const FhtParams p, long long npairs,
                                                              int pairs_per_row) {
  const int lane = threadIdx.x & 31, l16 = lane & 15, half = lane >> 4;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv = p.seg_inv[0];
  const uint16_t* xin = static_cast<const uint16_t*>(p.x);
  uint16_t* xout = static_cast<uint16_t*>(p.out);
  for (long long pr = warp0; pr < npairs; pr += stride) {
    const long long row = pr / pairs_per_row;
    const int off = int(pr - row * pairs_per_row) * 256 + 128 * half + 8 * l16;
    const uint4 raw = *reinterpret_cast<const uint4*>(xin + row * p.ldx + off);
    const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = DType<T>::to_float(uint16_t((j & 1) ? rw[j >> 1] >> 16 : rw[j >> 1] & 0xFFFFu));
      if (p.mode == B200LUT_FHT_AWQ) v[j] = v[j] * p.scale[off + j];
      else if (p.mode == B200LUT_FHT_ADJOINT && p.signs) v[j] = v[j] * p.signs[off + j];
    }
#pragma unroll
    for (int len = 1; len < 8; len <<= 1) {   // inside the lane
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if ((j & len) == 0) {
          const float a = v[j], b = v[j + len];
          v[j] = a + b;
          v[j + len] = a - b;
        }
      }
    }
#pragma unroll
    for (int m = 1; m < 16; m <<= 1) {        // len = 8 * m, partner lane inside the 16-lane half
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], m);
        v[j] = (l16 & m) ? other - v[j] : v[j] + other;
      }
    }
    uint32_t ow[4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float r = v[j];
      if (p.mode == B200LUT_FHT_ADJOINT) {
        r = r * inv;
      } else {
        if (p.signs) r = r * p.signs[off + j];
        r = r * inv;
        if (p.mode == B200LUT_FHT_AWQ) r = __fdiv_rn(r, p.scale[off + j]);
      }
      const uint32_t h = DType<T>::from_float(r);
      ow[j >> 1] = (j & 1) ? (ow[j >> 1] | (h << 16)) : h;
    }
    *reinterpret_cast<uint4*>(xout + row * p.ldo + off) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

}  // namespace
}  // namespace b200lut

using namespace b200lut;

extern "C" int b200lut_fht(const void* x, void* out, const float* signs, const float* scale,
                           int M, int K, int64_t ldx, int64_t ldo, int dtype, int mode, int block,
                           void* stream) {
  B200LUT_REQUIRE(x && out, B200LUT_ERR_INVALID, "null x or out");
  B200LUT_REQUIRE(M >= 0 && K >= 1, B200LUT_ERR_INVALID, "bad shape M=%d K=%d", M, K);
  B200LUT_REQUIRE(dtype >= 0 && dtype <= 2, B200LUT_ERR_INVALID, "dtype must be 0 (bf16), 1 (f16) or 2 (f32)");
  B200LUT_REQUIRE(mode >= B200LUT_FHT_FORWARD && mode <= B200LUT_FHT_AWQ, B200LUT_ERR_INVALID,
                  "unknown mode %d", mode);
  B200LUT_REQUIRE(mode != B200LUT_FHT_AWQ || scale, B200LUT_ERR_INVALID,
                  "the AWQ form needs a scale vector");
  B200LUT_REQUIRE(ldx >= K && ldo >= K, B200LUT_ERR_INVALID, "row strides must be >= K");
  if (M == 0) return B200LUT_OK;

  FhtParams p = {};
  p.x = x; p.out = out; p.signs = signs; p.scale = scale;
  p.ldx = ldx; p.ldo = ldo; p.dtype = dtype; p.mode = mode;
  int max_len = 0;
  if (block > 0) {
    B200LUT_REQUIRE((block & (block - 1)) == 0 && K % block == 0, B200LUT_ERR_INVALID,
                    "block must be a power of two dividing K (block=%d, K=%d)", block, K);
    int stages = 0;
    while ((1 << stages) < block) ++stages;
    // a block of threads takes as many whole transforms as fit 8192 points
    int span = block;
    while (span * 2 <= 8192 && K % (span * 2) == 0) span *= 2;
    B200LUT_REQUIRE(block == 128 || (span <= kMaxPoints && K / span <= kMaxSegments),
                    B200LUT_ERR_UNSUPPORTED, "K=%d with block=%d needs more than %d row pieces", K,
                    block, kMaxSegments);
    if (block == 128) span = K;
    p.nseg = K / span;
    for (int i = 0; i < p.nseg; ++i) {
      p.seg_off[i] = i * span;
      p.seg_len[i] = span;
      p.seg_stages[i] = stages;
      p.seg_inv[i] = float(1.0 / sqrt(double(block)));
    }
    max_len = span;
  } else {
    int off = 0;
    while (off < K) {
      int b = 1;
      while (b * 2 <= K - off) b *= 2;
      B200LUT_REQUIRE(p.nseg < kMaxSegments && b <= kMaxPoints, B200LUT_ERR_UNSUPPORTED,
                      "K=%d: segment of %d points or more than %d segments is not served", K, b,
                      kMaxSegments);
      int stages = 0;
      while ((1 << stages) < b) ++stages;
      p.seg_off[p.nseg] = off;
      p.seg_len[p.nseg] = b;
      p.seg_stages[p.nseg] = stages;
      p.seg_inv[p.nseg] = float(1.0 / sqrt(double(b)));
      ++p.nseg;
      if (b > max_len) max_len = b;
      off += b;
    }
  }
  if (block == 128 && dtype != 2 && K % 256 == 0 && ldx % 8 == 0 && ldo % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const long long npairs = (long long)M * (K / 256);
    long long grid = (npairs + 7) / 8;
    if (grid > 148 * 16) grid = 148 * 16;
    if (dtype == B200LUT_BF16)
      fht_block128_vec_kernel<__nv_bfloat16><<<unsigned(grid), 256, 0, cudaStream_t(stream)>>>(p, npairs, K / 256);
    else
      fht_block128_vec_kernel<__half><<<unsigned(grid), 256, 0, cudaStream_t(stream)>>>(p, npairs, K / 256);
    B200LUT_CUDA_OK(cudaGetLastError());
    return B200LUT_OK;
  }
  if (block == 128) {
    const long long nblocks = (long long)M * (K / 128);
    long long grid = (nblocks + 7) / 8;
    if (grid > 148 * 8) grid = 148 * 8;
    fht_block128_kernel<<<unsigned(grid), 256, 0, cudaStream_t(stream)>>>(p, nblocks, K / 128);
    B200LUT_CUDA_OK(cudaGetLastError());
    return B200LUT_OK;
  }
  const size_t smem = size_t(max_len) * sizeof(float);
  static bool configured[64] = {false};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(fht_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kMaxPoints * int(sizeof(float))));
    configured[dev] = true;
  }
  int threads = max_len / 2;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  fht_kernel<<<dim3(unsigned(M), unsigned(p.nseg)), threads, smem, cudaStream_t(stream)>>>(p);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}
