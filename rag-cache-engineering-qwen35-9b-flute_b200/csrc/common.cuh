// Shared host/device helpers of the B200 LUT-linear library: status plumbing,
// the slab weight layout, and small PTX wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/b200_lut.h"

namespace b200lut {

// ---- per-thread error text -------------------------------------------------
char* error_buffer();            // 512-byte thread-local buffer (api.cu)
int fail(int code, const char* fmt, ...);

#define B200LUT_CUDA_OK(expr)                                                        \
  do {                                                                               \
    cudaError_t e__ = (expr);                                                        \
    if (e__ != cudaSuccess)                                                          \
      return ::b200lut::fail(B200LUT_ERR_CUDA, "%s failed: %s", #expr,               \
                             cudaGetErrorString(e__));                               \
  } while (0)

#define B200LUT_REQUIRE(cond, code, ...)                                             \
  do {                                                                               \
    if (!(cond)) return ::b200lut::fail(code, __VA_ARGS__);                          \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- the slab layout ---------------------------------------------------------
//
// The [N, K] code matrix is cut into chunks of 128 rows x 64 k, stored
// tile-major like the idxN blob: chunk (t, g) starts at byte
// ((t * K/64) + g) * 1024 * bits. Inside a chunk every lane L of a warp owns a
// private string of 256*bits bits, kept as 8*bits 32-bit words w[0 .. 8*bits):
//   word w[m] lives at chunk byte (m / 8) * 1024 + 32 * L + 4 * (m % 8)
// so a warp reads the chunk with `bits` fully coalesced 32-byte (256-bit) loads per
// lane, 1 KB per warp instruction.
// The string holds, for slab s = 0..7 (rows 16s .. 16s+15 of the tile) and field
// i = 4*kt + f (kt = 0..3, f = 0..3), a 2*bits-bit pair at bit
//   32*bits*s + 2*bits*i:   code(row, k0) | code(row, k0 + 1) << bits
// with  row = 16*s + (L >> 2) + 8*(f & 1)
//       k0  = 16*kt + 4*(L & 3) + 2*(f >> 1).
// This is exactly the A-operand register order of mma.m16n8k16 (and the
// 16x256b TMEM store shape) once each pair is replaced by its two palette
// entries: for step kt, registers f = 0..3 are (row g, k 0-1), (row g+8, k 0-1),
// (row g, k 2-3), (row g+8, k 2-3) of the lane's four k.
constexpr int kTileRows = 128;
constexpr int kChunkK = 64;

struct SlabPos {
  int lane;   // owning lane
  int bit;    // bit offset of the code inside the lane's string
};

__host__ __device__ inline SlabPos slab_pos(int r /*0..127*/, int kk /*0..63*/, int bits) {
  const int s = r >> 4, rr = r & 15, gid = rr & 7, half = rr >> 3;
  const int kt = kk >> 4, tig = (kk >> 2) & 3, h = (kk >> 1) & 1, e = kk & 1;
  const int f = half + 2 * h;
  SlabPos p;
  p.lane = gid * 4 + tig;
  p.bit = 32 * bits * s + 2 * bits * (4 * kt + f) + bits * e;
  return p;
}

// byte offset inside the chunk of 32-bit word m of lane L
__host__ __device__ inline int slab_word_offset(int lane, int m) {
  return (m >> 3) * 1024 + lane * 32 + (m & 7) * 4;
}

// ---- dtype helpers -------------------------------------------------------------
template <typename T> struct DType;
template <> struct DType<__nv_bfloat16> {
  static constexpr int id = B200LUT_BF16;
  __device__ static float to_float(uint16_t raw) { return __uint_as_float(uint32_t(raw) << 16); }
  __device__ static uint16_t from_float(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  }
};
template <> struct DType<__half> {
  static constexpr int id = B200LUT_F16;
  __device__ static float to_float(uint16_t raw) { return __half2float(__ushort_as_half(raw)); }
  __device__ static uint16_t from_float(float v) { return __half_as_ushort(__float2half_rn(v)); }
};

// Status word of the decode kernels' exchange waits (defined with the GEMV): value and clear.
int exchange_status_take();
// Status word of the embedding gather (an id outside the table): value and clear.
int embed_status_take();

}  // namespace b200lut
