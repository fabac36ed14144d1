// Decode GEMV for the K-GROUPED palette variant: one 2^bits-entry palette per (block of 128
// input columns, output row),
//     out[m, n] = sum_k x[m, k] * lut_k[k / 128][n][code(n, k)]        (M <= 16)
// The reference groups palettes along the OUTPUT rows and has no kernel (and no module) of
// this form; its reference route expresses it as K/128 modules with group_size = 1 over 128
// columns each, summed in fp32 before the one rounding
// (src/scripts/palettized_modules.py:125-162 with rg = arange(N) // 1). The palettes are half
// as large again as the 4-bit codes (N*K/4 bytes), so they are streamed like the codes; a pair
// table per palette (what the row-grouped GEMV builds once per 128 rows) cannot pay off for
// 128 weights, and the lookups go straight to a staged copy of the palettes.
//
// One block (256 threads) per (128-row tile, K range). Warp w owns slab w of the tile (rows
// 16w .. 16w+15, see the slab layout): a lane's fields are rows (gid, gid + 8) x 16 k per
// chunk, so it keeps 2 x M fp32 sums, the four lanes of a row meet by two shuffles at the
// end, and no cross-warp reduction exists. Per 128-column group the block stages the
// tile's palettes (128 rows x 2^bits entries) and the activation slice (fp32) in shared
// memory through a four-deep ring of asynchronous 16-byte copies (cp.async), so three groups
// are in flight behind the one being computed. K ranges are folded through an fp32 workspace by
// the last block to arrive, in range order (deterministic; the ticket resets itself).
// Bound: HBM (codes N*K*bits/8 + palettes N*K*2^bits/64 bytes per launch).
#include <cstdlib>

#include "common.cuh"
#include "pairtable.cuh"
#include "gemv_kgrouped_rows.cuh"

namespace b200lut {
namespace {

constexpr int kKgThreads = 256;
constexpr int kKgGroup = 128;          // input columns per palette
constexpr int kKgMaxM = 16;

struct KgParams {
  const uint16_t* x;
  long long ldx;
  const uint8_t* packed;
  const uint16_t* lut;     // [K / 128][N][2^bits]
  const uint16_t* bias;
  uint16_t* out;
  long long ldo;
  float* ws;               // [split][M][N] fp32
  int* tickets;            // [N / 128]
  int M, N, K, bits, split;
};

// field `i` (0..15, a compile-time constant after unrolling) of a slab string of BITS words
template <int BITS>
__device__ __forceinline__ uint32_t slab_field(const uint32_t (&w)[4], int i) {
  const int pos = 2 * BITS * i, m = pos >> 5, sh = pos & 31;
  uint32_t v = w[m] >> sh;
  if (sh + 2 * BITS > 32) v |= w[(m + 1) & 3] << (32 - sh);   // only a 3-bit field straddles words
  return v;
}

constexpr int kKgStages = 4;           // groups in flight per block (cp.async ring)

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  const uint32_t d = uint32_t(__cvta_generic_to_shared(dst_smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// bytes of one ring stage: palettes of the tile, the two code chunks, the activation slice
__host__ __device__ inline int kg_stage_bytes(int bits, int M) {
  return kTileRows * (1 << bits) * 2 + 2 * 1024 * bits + ((M * kKgGroup * 2 + 15) & ~15);
}

template <typename T, int MT, int BITS>
__global__ void __launch_bounds__(kKgThreads) gemv_kgrouped_kernel(const KgParams p) {
  extern __shared__ __align__(16) uint8_t ring[];
  __shared__ int last_flag;
  const int tile = blockIdx.x, sp = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  constexpr int bits = BITS, E = 1 << BITS;
  const int NG = p.K / kKgGroup, G = p.K / kChunkK;
  const int j0 = (NG * sp) / p.split, j1 = (NG * (sp + 1)) / p.split;
  const int n0 = tile * kTileRows;
  constexpr uint32_t mask = (1u << BITS) - 1u;
  const int lut_bytes = kTileRows * E * 2, code_bytes = 2 * 1024 * bits;
  const int stage_bytes = kg_stage_bytes(bits, p.M);

  float acc[2][MT];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[h][m] = 0.f;

  // group j -> ring slot (j - j0) % kKgStages: palettes, the group's two chunks (contiguous in
  // the slab layout), the activation slice; 16-byte asynchronous copies, one commit per group
  auto request = [&](int j) {
    if (j < j1) {
      uint8_t* st = ring + ((j - j0) % kKgStages) * stage_bytes;
      const uint8_t* lut_g = reinterpret_cast<const uint8_t*>(p.lut + (size_t(j) * p.N + n0) * E);
      for (int i = threadIdx.x; i < lut_bytes / 16; i += kKgThreads) cp_async16(st + 16 * i, lut_g + 16 * i);
      const uint8_t* codes_g = p.packed + (size_t(tile) * G + 2 * j) * 1024 * bits;
      for (int i = threadIdx.x; i < code_bytes / 16; i += kKgThreads)
        cp_async16(st + lut_bytes + 16 * i, codes_g + 16 * i);
      for (int i = threadIdx.x; i < p.M * (kKgGroup / 8); i += kKgThreads) {
        const int m = i / (kKgGroup / 8), c8 = i % (kKgGroup / 8);
        cp_async16(st + lut_bytes + code_bytes + 16 * i, p.x + size_t(m) * p.ldx + j * kKgGroup + 8 * c8);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int d = 0; d < kKgStages - 1; ++d) request(j0 + d);
  for (int j = j0; j < j1; ++j) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kKgStages - 2) : "memory");
    __syncthreads();            // group j has landed for everyone; group j - 1 has been read
    request(j + kKgStages - 1);
    const uint8_t* st = ring + ((j - j0) % kKgStages) * stage_bytes;
    const uint16_t* lut_s = reinterpret_cast<const uint16_t*>(st);
    const uint16_t* x_s = reinterpret_cast<const uint16_t*>(st + lut_bytes + code_bytes);
    uint32_t cw[2][4];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint8_t* chunk = st + lut_bytes + c * 1024 * bits;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        cw[c][i] = i < bits ? *reinterpret_cast<const uint32_t*>(chunk + slab_word_offset(lane, warp * bits + i))
                            : 0u;
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int k = c * kChunkK + 16 * kt + 4 * tig + 2 * hh;
          float w0[2], w1[2];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t f = slab_field<BITS>(cw[c], 4 * kt + half + 2 * hh);
            const uint16_t* pal = lut_s + (16 * warp + gid + 8 * half) * E;
            w0[half] = DType<T>::to_float(pal[f & mask]);
            w1[half] = DType<T>::to_float(pal[(f >> bits) & mask]);
          }
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            if (m < p.M) {
              const uint32_t xp = *reinterpret_cast<const uint32_t*>(x_s + m * kKgGroup + k);
              const float x0 = DType<T>::to_float(uint16_t(xp & 0xFFFFu));
              const float x1 = DType<T>::to_float(uint16_t(xp >> 16));
              acc[0][m] = fmaf(w1[0], x1, fmaf(w0[0], x0, acc[0][m]));
              acc[1][m] = fmaf(w1[1], x1, fmaf(w0[1], x0, acc[1][m]));
            }
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // the four lanes of a row hold its four k residues
#pragma unroll
  for (int half = 0; half < 2; ++half)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float v = acc[half][m];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      acc[half][m] = v;
    }
  auto finish = [&](int m, int n, float v) {
    if (p.bias) v += DType<T>::to_float(p.bias[n]);
    p.out[size_t(m) * p.ldo + n] = DType<T>::from_float(v);
  };
  if (p.split == 1) {
    if (tig == 0)
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int m = 0; m < MT; ++m)
          if (m < p.M) finish(m, n0 + 16 * warp + gid + 8 * half, acc[half][m]);
    return;
  }
  if (tig == 0)
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (m < p.M)
          __stcg(p.ws + (size_t(sp) * p.M + m) * p.N + n0 + 16 * warp + gid + 8 * half, acc[half][m]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(p.tickets + tile, 1);
    last_flag = old == p.split - 1;
    if (last_flag) p.tickets[tile] = 0;            // ready for the next launch
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < p.M * kTileRows; idx += kKgThreads) {
    const int m = idx >> 7, n = n0 + (idx & 127);
    float v = 0.f;
    for (int s0 = 0; s0 < p.split; s0 += 8) {      // eight partial sums in flight, added in range order
      float t[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        t[i] = s0 + i < p.split ? __ldcg(p.ws + (size_t(s0 + i) * p.M + m) * p.N + n) : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (s0 + i < p.split) v += t[i];
    }
    finish(m, n, v);
  }
}

template <typename T, int MT, int BITS>
int launch_kg_bits(const KgParams& p, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = gemv_kgrouped_kernel<T, MT, BITS>;
  static bool configured[64] = {false};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
    configured[dev] = true;
  }
  kern<<<grid, kKgThreads, smem, st>>>(p);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}

template <typename T, int MT>
int launch_kg(const KgParams& p, dim3 grid, size_t smem, cudaStream_t st) {
  switch (p.bits) {
    case 4: return launch_kg_bits<T, MT, 4>(p, grid, smem, st);
    case 3: return launch_kg_bits<T, MT, 3>(p, grid, smem, st);
    case 2: return launch_kg_bits<T, MT, 2>(p, grid, smem, st);
    default: return launch_kg_bits<T, MT, 1>(p, grid, smem, st);
  }
}

int sm_count() {
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

int pick_kg_split(int tiles, int NG) {
  // about four resident blocks per SM, at least two groups per block
  int s = (4 * sm_count() + tiles - 1) / tiles;
  if (s > NG / 2) s = NG / 2;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

}  // namespace
}  // namespace b200lut

using namespace b200lut;

extern "C" int b200lut_gemv_kgrouped_split(int N, int K) {
  if (N < kTileRows || K < kKgGroup) return 1;
  return pick_kg_split(N / kTileRows, K / kKgGroup);
}

extern "C" size_t b200lut_gemv_kgrouped_workspace_bytes(int N, int M, int split) {
  if (split <= 1 || N <= 0 || M <= 0) return 0;
  return size_t(N / kTileRows) * sizeof(int) + 256 + size_t(split) * M * N * sizeof(float);
}

extern "C" int b200lut_gemv_kgrouped(const void* x, int64_t ldx, int M, int K, int dtype,
                                     const void* packed, const void* lut_k, const void* bias,
                                     int N, int bits, void* out, int64_t ldo, int split,
                                     void* workspace, size_t workspace_bytes, void* stream) {
  B200LUT_REQUIRE(x && packed && lut_k && out, B200LUT_ERR_INVALID, "null x, codes, palettes or output");
  B200LUT_REQUIRE(M >= 1 && M <= kKgMaxM, B200LUT_ERR_UNSUPPORTED,
                  "the K-grouped GEMV serves 1 <= M <= 16 rows, got M=%d", M);
  B200LUT_REQUIRE(K > 0 && K % kKgGroup == 0 && N > 0 && N % kTileRows == 0, B200LUT_ERR_INVALID,
                  "K and N must be positive multiples of 128 (got K=%d, N=%d)", K, N);
  B200LUT_REQUIRE(bits >= 1 && bits <= 4, B200LUT_ERR_INVALID, "bit width must be 1..4, got %d", bits);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(x) && aligned16(packed) && aligned16(lut_k) && ldx % 8 == 0 && ldx >= K &&
                      ldo >= N,
                  B200LUT_ERR_ALIGN,
                  "x, codes and palettes must be 16-byte aligned, the x row stride a multiple of 8 "
                  "and >= K, ldo >= N");
  const int tiles = N / kTileRows, NG = K / kKgGroup;
  // Library policy (split == 0): the row-range form for 4-bit codes at M <= 8 where its rows and
  // fold buffer fit in shared memory (B200LUT_KG_KERNEL=simt keeps the SIMT kernel, for A/B runs).
  if (split <= 0 && bits == 4 && M <= 8) {
    static const bool simt_only = [] {
      const char* e = getenv("B200LUT_KG_KERNEL");
      return e != nullptr && e[0] == 's';
    }();
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    KgRowsGeom g;
    if (!simt_only && kg_rows_plan(M, N, K, sms, &g)) {
      KgRowsParams rp = {};
      rp.x = static_cast<const uint16_t*>(x);
      rp.ldx = ldx;
      rp.packed = static_cast<const uint8_t*>(packed);
      rp.lut = static_cast<const uint16_t*>(lut_k);
      rp.bias = static_cast<const uint16_t*>(bias);
      rp.out = static_cast<uint16_t*>(out);
      rp.ldo = ldo;
      rp.M = M; rp.Mp = g.Mp; rp.N = N; rp.K = K; rp.G = K / kChunkK;
      rp.units_total = g.units_total; rp.row_blocks = g.row_blocks; rp.red_planes = g.red_planes;
      rp.xs_off = g.xs_off; rp.red_off = g.red_off;
      auto go = [&](auto kern, int which) -> int {
        static bool configured[2][64] = {};
        if (dev >= 64 || !configured[which][dev]) {
          B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
          if (dev < 64) configured[which][dev] = true;
        }
        kern<<<unsigned(g.row_blocks), kKrThreads, g.bytes, cudaStream_t(stream)>>>(rp);
        B200LUT_CUDA_OK(cudaGetLastError());
        return B200LUT_OK;
      };
      return dtype == B200LUT_BF16 ? go(gemv_kgrouped_rows_kernel<__nv_bfloat16>, 0)
                                   : go(gemv_kgrouped_rows_kernel<__half>, 1);
    }
  }
  if (split <= 0) split = pick_kg_split(tiles, NG);
  B200LUT_REQUIRE(split <= NG && split <= 65535, B200LUT_ERR_INVALID,
                  "split %d exceeds the %d column groups", split, NG);
  KgParams p = {};
  p.x = static_cast<const uint16_t*>(x);
  p.ldx = ldx;
  p.packed = static_cast<const uint8_t*>(packed);
  p.lut = static_cast<const uint16_t*>(lut_k);
  p.bias = static_cast<const uint16_t*>(bias);
  p.out = static_cast<uint16_t*>(out);
  p.ldo = ldo;
  p.M = M; p.N = N; p.K = K; p.bits = bits; p.split = split;
  if (split > 1) {
    const size_t need = b200lut_gemv_kgrouped_workspace_bytes(N, M, split);
    B200LUT_REQUIRE(workspace && workspace_bytes >= need && aligned16(workspace), B200LUT_ERR_WORKSPACE,
                    "split %d needs a zero-initialised, 16-byte aligned workspace of %zu bytes", split,
                    need);
    p.tickets = static_cast<int*>(workspace);
    p.ws = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                    ((size_t(tiles) * sizeof(int) + 255) / 256) * 256);
  }
  const dim3 grid(unsigned(tiles), unsigned(split), 1);
  const size_t smem = size_t(kKgStages) * kg_stage_bytes(bits, M);   // <= 64 KB
  cudaStream_t st = cudaStream_t(stream);
  if (dtype == B200LUT_BF16) {
    if (M == 1) return launch_kg<__nv_bfloat16, 1>(p, grid, smem, st);
    if (M <= 2) return launch_kg<__nv_bfloat16, 2>(p, grid, smem, st);
    if (M <= 4) return launch_kg<__nv_bfloat16, 4>(p, grid, smem, st);
    if (M <= 8) return launch_kg<__nv_bfloat16, 8>(p, grid, smem, st);
    return launch_kg<__nv_bfloat16, 16>(p, grid, smem, st);
  }
  if (M == 1) return launch_kg<__half, 1>(p, grid, smem, st);
  if (M <= 2) return launch_kg<__half, 2>(p, grid, smem, st);
  if (M <= 4) return launch_kg<__half, 4>(p, grid, smem, st);
  if (M <= 8) return launch_kg<__half, 8>(p, grid, smem, st);
  return launch_kg<__half, 16>(p, grid, smem, st);
}
