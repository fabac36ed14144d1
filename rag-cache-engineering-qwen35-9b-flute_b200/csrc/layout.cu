// Weight-layout kernels: idxN blob <-> slab layout, logical code export and the
// dequantised-weight export used as the bit-exactness probe.
//
// The idxN addressing implemented here is the normative text of the reference
// format (src/flute_extended/flute_extended/idxN.py:37-55): a 128-row x 64-k tile
// of 1024*bits bytes at ((t * K/64) + g) * 1024*bits; thread chunk th = wx*32+lane
// of 16*bits bytes at th*16*bits; element e = 2*p + j of the chunk is a bits-wide
// LSB-first field at bit bits*e with p = kt*16 + v*4 + d*2 + s2 covering
// row = wx*64 + v*16 + d*8 + (lane >> 2), k = kt*16 + 2*(lane & 3) + 8*s2 + j.
#include "common.cuh"

namespace b200lut {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t bits_at(const uint8_t* bytes, int bit, int nbits) {
  // little-endian bit string; fields are at most 8 bits wide here
  const int byte = bit >> 3, sh = bit & 7;
  uint32_t v = bytes[byte];
  if (sh + nbits > 8) v |= uint32_t(bytes[byte + 1]) << 8;
  return (v >> sh) & ((1u << nbits) - 1u);
}

// code of tile-local (r, kk) read from a slab chunk staged in shared memory
__device__ __forceinline__ uint32_t slab_code(const uint8_t* chunk, int r, int kk, int bits) {
  const SlabPos p = slab_pos(r, kk, bits);
  const int m = p.bit >> 5, sh = p.bit & 31;
  const uint32_t lo = *reinterpret_cast<const uint32_t*>(chunk + slab_word_offset(p.lane, m));
  uint64_t v = lo;
  if (sh + bits > 32)
    v |= uint64_t(*reinterpret_cast<const uint32_t*>(chunk + slab_word_offset(p.lane, m + 1))) << 32;
  return uint32_t(v >> sh) & ((1u << bits) - 1u);
}

__device__ __forceinline__ void idxn_coord(int th, int e, int& row, int& col) {
  const int wx = th >> 5, lane = th & 31;
  const int j = e & 1, p = e >> 1;
  const int s2 = p & 1, d = (p >> 1) & 1, v = (p >> 2) & 3, kt = p >> 4;
  row = wx * 64 + v * 16 + d * 8 + (lane >> 2);
  col = kt * 16 + 2 * (lane & 3) + 8 * s2 + j;
}

__device__ __forceinline__ void load_chunk(uint8_t* dst, const uint8_t* src, int bytes) {
  const int4* s4 = reinterpret_cast<const int4*>(src);
  int4* d4 = reinterpret_cast<int4*>(dst);
  for (int i = threadIdx.x; i < bytes / 16; i += kThreads) d4[i] = s4[i];
}

__global__ void __launch_bounds__(kThreads) idxn_to_slab_kernel(const uint8_t* __restrict__ blob,
                                                                uint8_t* __restrict__ packed,
                                                                int bits) {
  __shared__ __align__(16) uint8_t raw[4096 + 16];
  __shared__ uint8_t codes[kTileRows][kChunkK + 4];
  const size_t chunk_bytes = size_t(1024) * bits;
  const size_t base = size_t(blockIdx.x) * chunk_bytes;
  load_chunk(raw, blob + base, int(chunk_bytes));
  if (threadIdx.x < 16) raw[chunk_bytes + threadIdx.x] = 0;
  __syncthreads();
  for (int c = threadIdx.x; c < kTileRows * kChunkK; c += kThreads) {
    const int th = c >> 7, e = c & 127;
    int row, col;
    idxn_coord(th, e, row, col);
    codes[row][col] = uint8_t(bits_at(raw + th * 16 * bits, bits * e, bits));
  }
  __syncthreads();
  // one thread per (lane, slab): assemble the slab's 32*bits-bit string
  const int lane = threadIdx.x & 31, s = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  for (int i = 0; i < 16; ++i) {
    const int kt = i >> 2, f = i & 3;
    const int row = 16 * s + gid + 8 * (f & 1);
    const int k0 = 16 * kt + 4 * tig + 2 * (f >> 1);
    const uint32_t field = uint32_t(codes[row][k0]) | (uint32_t(codes[row][k0 + 1]) << bits);
    const int pos = 2 * bits * i, m = pos >> 5, sh = pos & 31;
    w[m] |= field << sh;
    if (sh + 2 * bits > 32) w[m + 1] |= field >> (32 - sh);
  }
  for (int j = 0; j < bits; ++j)
    *reinterpret_cast<uint32_t*>(packed + base + slab_word_offset(lane, s * bits + j)) = w[j];
}

__global__ void __launch_bounds__(kThreads) slab_to_idxn_kernel(const uint8_t* __restrict__ packed,
                                                                uint8_t* __restrict__ blob,
                                                                int bits) {
  __shared__ __align__(16) uint8_t raw[4096];
  __shared__ uint8_t codes[kTileRows][kChunkK + 4];
  const size_t chunk_bytes = size_t(1024) * bits;
  const size_t base = size_t(blockIdx.x) * chunk_bytes;
  load_chunk(raw, packed + base, int(chunk_bytes));
  __syncthreads();
  for (int c = threadIdx.x; c < kTileRows * kChunkK; c += kThreads)
    codes[c >> 6][c & 63] = uint8_t(slab_code(raw, c >> 6, c & 63, bits));
  __syncthreads();
  for (int ob = threadIdx.x; ob < int(chunk_bytes); ob += kThreads) {
    const int th = ob / (16 * bits), byte_in = ob % (16 * bits);
    uint32_t v = 0;
    for (int bit = 0; bit < 8; ++bit) {
      const int pos = byte_in * 8 + bit, e = pos / bits, cb = pos % bits;
      int row, col;
      idxn_coord(th, e, row, col);
      v |= ((uint32_t(codes[row][col]) >> cb) & 1u) << bit;
    }
    blob[base + ob] = uint8_t(v);
  }
}

__global__ void __launch_bounds__(kThreads) slab_codes_kernel(const uint8_t* __restrict__ packed,
                                                              uint8_t* __restrict__ out, int K,
                                                              int bits) {
  __shared__ __align__(16) uint8_t raw[4096];
  const int G = K / kChunkK;
  const int t = blockIdx.x / G, g = blockIdx.x % G;
  const size_t chunk_bytes = size_t(1024) * bits;
  load_chunk(raw, packed + size_t(blockIdx.x) * chunk_bytes, int(chunk_bytes));
  __syncthreads();
  for (int c = threadIdx.x; c < kTileRows * kChunkK; c += kThreads) {
    const int r = c >> 6, kk = c & 63;
    out[size_t(t * kTileRows + r) * K + g * kChunkK + kk] = uint8_t(slab_code(raw, r, kk, bits));
  }
}

__global__ void __launch_bounds__(kThreads) slab_dequant_kernel(const uint8_t* __restrict__ packed,
                                                                const uint16_t* __restrict__ lut,
                                                                int n_groups,
                                                                uint16_t* __restrict__ out, int K,
                                                                int bits, int group_size) {
  __shared__ __align__(16) uint8_t raw[4096];
  const int G = K / kChunkK;
  const int t = blockIdx.x / G, g = blockIdx.x % G;
  const size_t chunk_bytes = size_t(1024) * bits;
  load_chunk(raw, packed + size_t(blockIdx.x) * chunk_bytes, int(chunk_bytes));
  __syncthreads();
  for (int c = threadIdx.x; c < kTileRows * kChunkK; c += kThreads) {
    const int r = c >> 6, kk = c & 63;
    const int n = t * kTileRows + r;
    int grp = n / group_size;
    if (grp > n_groups - 1) grp = n_groups - 1;
    const uint32_t code = slab_code(raw, r, kk, bits);
    out[size_t(n) * K + g * kChunkK + kk] = lut[(size_t(grp) << bits) + code];
  }
}

int check_shape(int N, int K, int bits) {
  B200LUT_REQUIRE(bits >= 1 && bits <= 4, B200LUT_ERR_INVALID,
                  "bit width must be 1..4, got %d", bits);
  B200LUT_REQUIRE(N > 0 && N % kTileRows == 0, B200LUT_ERR_INVALID,
                  "N must be a positive multiple of 128, got %d", N);
  B200LUT_REQUIRE(K > 0 && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a positive multiple of 64, got %d", K);
  return B200LUT_OK;
}

}  // namespace
}  // namespace b200lut

using namespace b200lut;

extern "C" size_t b200lut_packed_bytes(int N, int K, int bits) {
  if (bits < 1 || bits > 4 || N <= 0 || K <= 0 || N % kTileRows || K % kChunkK) return 0;
  return size_t(N) * size_t(K) * size_t(bits) / 8;
}

extern "C" int b200lut_repack_from_idxn(const void* idxn_blob, void* packed, int N, int K,
                                        int bits, void* stream) {
  if (int rc = check_shape(N, K, bits)) return rc;
  B200LUT_REQUIRE(idxn_blob && packed, B200LUT_ERR_INVALID, "null buffer");
  B200LUT_REQUIRE(aligned16(idxn_blob) && aligned16(packed), B200LUT_ERR_ALIGN,
                  "blob and packed buffers must be 16-byte aligned");
  const int chunks = (N / kTileRows) * (K / kChunkK);
  idxn_to_slab_kernel<<<chunks, kThreads, 0, cudaStream_t(stream)>>>(
      static_cast<const uint8_t*>(idxn_blob), static_cast<uint8_t*>(packed), bits);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}

extern "C" int b200lut_repack_to_idxn(const void* packed, void* idxn_blob, int N, int K, int bits,
                                      void* stream) {
  if (int rc = check_shape(N, K, bits)) return rc;
  B200LUT_REQUIRE(idxn_blob && packed, B200LUT_ERR_INVALID, "null buffer");
  B200LUT_REQUIRE(aligned16(idxn_blob) && aligned16(packed), B200LUT_ERR_ALIGN,
                  "blob and packed buffers must be 16-byte aligned");
  const int chunks = (N / kTileRows) * (K / kChunkK);
  slab_to_idxn_kernel<<<chunks, kThreads, 0, cudaStream_t(stream)>>>(
      static_cast<const uint8_t*>(packed), static_cast<uint8_t*>(idxn_blob), bits);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}

extern "C" int b200lut_unpack_codes(const void* packed, uint8_t* codes, int N, int K, int bits,
                                    void* stream) {
  if (int rc = check_shape(N, K, bits)) return rc;
  B200LUT_REQUIRE(packed && codes, B200LUT_ERR_INVALID, "null buffer");
  B200LUT_REQUIRE(aligned16(packed), B200LUT_ERR_ALIGN, "packed buffer must be 16-byte aligned");
  const int chunks = (N / kTileRows) * (K / kChunkK);
  slab_codes_kernel<<<chunks, kThreads, 0, cudaStream_t(stream)>>>(
      static_cast<const uint8_t*>(packed), codes, K, bits);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}

extern "C" int b200lut_dequant(const void* packed, const void* lut, int n_groups, void* out, int N,
                               int K, int bits, int group_size, void* stream) {
  if (int rc = check_shape(N, K, bits)) return rc;
  B200LUT_REQUIRE(packed && lut && out, B200LUT_ERR_INVALID, "null buffer");
  B200LUT_REQUIRE(group_size >= 1 && n_groups >= 1, B200LUT_ERR_INVALID,
                  "group_size and n_groups must be >= 1 (got %d, %d)", group_size, n_groups);
  B200LUT_REQUIRE(aligned16(packed), B200LUT_ERR_ALIGN, "packed buffer must be 16-byte aligned");
  const int chunks = (N / kTileRows) * (K / kChunkK);
  slab_dequant_kernel<<<chunks, kThreads, 0, cudaStream_t(stream)>>>(
      static_cast<const uint8_t*>(packed), static_cast<const uint16_t*>(lut), n_groups,
      static_cast<uint16_t*>(out), K, bits, group_size);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}
