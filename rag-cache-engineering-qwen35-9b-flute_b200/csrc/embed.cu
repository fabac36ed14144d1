// Embedding gather over palettized rows: out[t, :] = W[ids[t], :] with
//   W[n, k] = lut1[min(n / gs, G-1)][code1(n, k)]  (+ lut2[...][code2(n, k)], one 16-bit add,
//             stream 1 first)  (+ sum_r resA[n, r] * resB[r, k] in fp32),  one final rounding.
// The reference's PalettizedEmbedding (src/scripts/palettized_modules.py:1979-2335) has no
// kernel for this: it keeps an unpacked [N, K] uint8 copy of the codes (0.95 GiB per stream at
// the 248320 x 4096 head geometry) and gathers through torch indexing. Here the rows are read
// straight out of the packed slab layout the GEMV uses, so a tied lm_head / embedding pair
// shares ONE copy of the codes and nothing is unpacked.
//
// A row's codes are scattered through its tile: in chunk (t, g) row r owns, in each of the four
// lanes 4*(r & 7) + tig, the fields f = ((r >> 3) & 1) + 2h of k-step kt inside slab r >> 4 (see
// the layout notes next to slab_pos). A thread produces 8 consecutive k of one token: two
// lanes' slab strings (`bits` words each), 16-byte output store. Bound: HBM/L2 latency of
// short scattered reads; per token 4 sectors per chunk are touched for 8*bits useful bytes.
//
// An id outside [0, N) never indexes memory: its row is written as zeros and a status word is
// raised that b200lut_device_status() reports (the reference aborts the CUDA context through a
// device-side assertion, :1957-1976; a library must not).
#include "common.cuh"

namespace b200lut {

__device__ int g_embed_status = 0;

int embed_status_take() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_embed_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_embed_status, &zero, sizeof(int));
  return v;
}

namespace {

constexpr int kEmbedThreads = 256;
constexpr int kBadId = 0x6000;

struct EmbedParams {
  const long long* ids;
  const uint8_t* packed[2];
  const uint16_t* lut[2];
  int bits[2];
  const uint16_t* resA;   // [N, R]
  const uint16_t* resB;   // [R, K]
  int R;
  void* out;
  long long ldo;
  int out_f32;
  int vec_ok;             // 16-byte stores allowed
  int N, K, group_size, n_groups;
};

// the 8 codes k0 .. k0+7 (k0 % 8 == 0) of tile row r in the chunk at `chunk`
__device__ __forceinline__ void row_codes8(const uint8_t* chunk, int r, int kk0, int bits,
                                           uint32_t (&code)[8]) {
  const int s = r >> 4, gid = r & 7, half = (r >> 3) & 1;
  const int kt = kk0 >> 4, tig0 = (kk0 >> 2) & 3;          // tig0 is 0 or 2
  const uint32_t mask = (1u << bits) - 1u;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int lane = gid * 4 + tig0 + q;
    // the slab's string of this lane: `bits` words, 32 * bits bits, as up to 128 bits
    uint64_t lo = 0, hi = 0;
    for (int j = 0; j < bits; ++j) {
      const uint64_t w = __ldg(reinterpret_cast<const uint32_t*>(
          chunk + slab_word_offset(lane, s * bits + j)));
      if (j < 2) lo |= w << (32 * j); else hi |= w << (32 * (j - 2));
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int pos = 2 * bits * (4 * kt + half + 2 * h);   // < 128; 3-bit fields may straddle bit 64
      const uint64_t src = pos >= 64 ? hi >> (pos - 64)
                                     : (lo >> pos) | (pos ? hi << (64 - pos) : 0ull);
      const uint32_t field = uint32_t(src);
      code[4 * q + 2 * h] = field & mask;
      code[4 * q + 2 * h + 1] = (field >> bits) & mask;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kEmbedThreads) embed_gather_kernel(const EmbedParams p) {
  const long long tok = blockIdx.x;
  const int k0 = (blockIdx.y * kEmbedThreads + threadIdx.x) * 8;
  if (k0 >= p.K) return;
  const long long id = p.ids[tok];
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.f;
  if (id < 0 || id >= p.N) {
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicExch(&g_embed_status, kBadId);
  } else {
    const int n = int(id), t = n >> 7, r = n & 127;
    int grp = n / p.group_size;
    if (grp > p.n_groups - 1) grp = p.n_groups - 1;
    const int G = p.K / kChunkK, g = k0 >> 6, kk0 = k0 & 63;
    uint32_t code[8];
    row_codes8(p.packed[0] + (size_t(t) * G + g) * 1024 * p.bits[0], r, kk0, p.bits[0], code);
    const uint16_t* l1 = p.lut[0] + (size_t(grp) << p.bits[0]);
    uint16_t w[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = __ldg(l1 + code[e]);
    if (p.packed[1]) {
      row_codes8(p.packed[1] + (size_t(t) * G + g) * 1024 * p.bits[1], r, kk0, p.bits[1], code);
      const uint16_t* l2 = p.lut[1] + (size_t(grp) << p.bits[1]);
#pragma unroll
      for (int e = 0; e < 8; ++e)   // one add in the palette's own precision, stream 1 first
        w[e] = DType<T>::from_float(DType<T>::to_float(w[e]) + DType<T>::to_float(__ldg(l2 + code[e])));
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = DType<T>::to_float(w[e]);
    if (p.R > 0) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      const uint16_t* a = p.resA + size_t(n) * p.R;
      for (int j = 0; j < p.R; ++j) {   // ascending r, fp32
        const float aj = DType<T>::to_float(__ldg(a + j));
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.resB + size_t(j) * p.K + k0));
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] = fmaf(aj, DType<T>::to_float(uint16_t(bw[i] & 0xFFFFu)), acc[2 * i]);
          acc[2 * i + 1] = fmaf(aj, DType<T>::to_float(uint16_t(bw[i] >> 16)), acc[2 * i + 1]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += acc[e];
    }
  }
  if (p.out_f32) {
    float* o = static_cast<float*>(p.out) + tok * p.ldo + k0;
    if (p.vec_ok) {
      reinterpret_cast<float4*>(o)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4*>(o)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[e];
    }
  } else {
    uint16_t* o = static_cast<uint16_t*>(p.out) + tok * p.ldo + k0;
    uint16_t h[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) h[e] = DType<T>::from_float(v[e]);
    if (p.vec_ok) {
      *reinterpret_cast<uint4*>(o) =
          make_uint4(h[0] | uint32_t(h[1]) << 16, h[2] | uint32_t(h[3]) << 16,
                     h[4] | uint32_t(h[5]) << 16, h[6] | uint32_t(h[7]) << 16);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = h[e];
    }
  }
}

// The common case on its own path: 4-bit codes, one stream, no residual, 16-bit output rows that
// take 8-byte stores. One block per token. The row's palette becomes a 256-entry pair table in
// shared memory (entry e = palette[e & 15] | palette[e >> 4] << 16: two consecutive k in one
// word; 1 KB, eight words per bank, so a warp's lookups take a few wavefronts each). A thread
// owns (chunk g, tig): ONE 16-byte load fetches the four words of the row's slab in lane
// 4 * (r & 7) + tig — 16 codes of this row, interleaved with 16 of row r ^ 8 —, eight table
// lookups turn them into four 8-byte pieces (k = 64 g + 16 kt + 4 tig .. + 3), and the four
// threads of a chunk's k-step fill whole 32-byte sectors. Against the generic kernel above: an
// eighth of the load instructions and half of the lookups per output.
template <typename T>
__global__ void __launch_bounds__(kEmbedThreads) embed_gather4_kernel(const EmbedParams p) {
  __shared__ uint32_t pair[256];
  const long long tok = blockIdx.x;
  const long long id = p.ids[tok];
  uint16_t* orow = static_cast<uint16_t*>(p.out) + tok * p.ldo;
  const int G = p.K / kChunkK;
  if (id < 0 || id >= p.N) {
    if (threadIdx.x == 0) atomicExch(&g_embed_status, kBadId);
    for (int item = threadIdx.x; item < G * 16; item += kEmbedThreads)
      *reinterpret_cast<uint2*>(orow + item * 4) = make_uint2(0u, 0u);
    return;
  }
  const int n = int(id), t = n >> 7, r = n & 127;
  int grp = n / p.group_size;
  if (grp > p.n_groups - 1) grp = p.n_groups - 1;
  {
    const uint16_t* l1 = p.lut[0] + size_t(grp) * 16;
    const int e = threadIdx.x;
    pair[e] = uint32_t(__ldg(l1 + (e & 15))) | (uint32_t(__ldg(l1 + (e >> 4))) << 16);
  }
  __syncthreads();
  const int s = r >> 4, gid = r & 7, half = (r >> 3) & 1;
  // chunk g of the tile, plane s >> 1, lane 4 gid + tig, the slab's four words
  const uint8_t* base = p.packed[0] + size_t(t) * G * 4096 + (s >> 1) * 1024 + gid * 128 + (s & 1) * 16;
  const int sh0 = 8 * half, sh1 = 8 * (half + 2);
  for (int item = threadIdx.x; item < G * 4; item += kEmbedThreads) {
    const int g = item >> 2, tig = item & 3;
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(base + size_t(g) * 4096 + tig * 32));
    const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
    uint16_t* o = orow + g * kChunkK + 4 * tig;
#pragma unroll
    for (int kt = 0; kt < 4; ++kt)
      *reinterpret_cast<uint2*>(o + 16 * kt) =
          make_uint2(pair[(w[kt] >> sh0) & 0xFFu], pair[(w[kt] >> sh1) & 0xFFu]);
  }
}

// fp32 rows -> 16-bit rows, one rounding (the cast after the un-rotation of tied rows)
template <typename T>
__global__ void __launch_bounds__(256) round_rows_kernel(const float* __restrict__ in,
                                                         long long ldi, uint16_t* __restrict__ out,
                                                         long long ldo, long long M, int K) {
  const long long total = M * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / K;
    const int k = int(i - m * K);
    out[m * ldo + k] = DType<T>::from_float(in[m * ldi + k]);
  }
}

}  // namespace
}  // namespace b200lut

using namespace b200lut;

extern "C" int b200lut_embed_gather(const int64_t* ids, int64_t n_ids, int K, int dtype,
                                    const b200lut_segment* table, const void* resB, int out_fp32,
                                    void* stream) {
  B200LUT_REQUIRE(table, B200LUT_ERR_INVALID, "null table descriptor");
  const b200lut_segment& s = *table;
  B200LUT_REQUIRE(n_ids >= 0 && n_ids <= 0x7fffffffLL, B200LUT_ERR_INVALID,
                  "0 <= n_ids < 2^31 required, got %lld", (long long)n_ids);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(K > 0 && K % kChunkK == 0 && s.N > 0 && s.N % kTileRows == 0,
                  B200LUT_ERR_INVALID,
                  "the idxN layout requires N %% 128 == 0 and K %% 64 == 0, got N=%d, K=%d", s.N, K);
  B200LUT_REQUIRE(s.bits >= 1 && s.bits <= 4 && (!s.packed2 || (s.lut2 && s.bits2 >= 1 && s.bits2 <= 4)),
                  B200LUT_ERR_INVALID, "bit widths must be 1..4 (got %d / %d)", s.bits, s.bits2);
  B200LUT_REQUIRE(s.group_size >= 1 && s.n_groups >= 1, B200LUT_ERR_INVALID,
                  "group_size and n_groups must be positive");
  B200LUT_REQUIRE(s.res_rank >= 0 && (s.res_rank == 0 || (s.resA && resB)), B200LUT_ERR_INVALID,
                  "a residual of rank %d needs both resA and resB", s.res_rank);
  if (n_ids == 0) return B200LUT_OK;
  B200LUT_REQUIRE(ids && s.packed && s.lut && s.out, B200LUT_ERR_INVALID,
                  "null ids, codes, palette or output");
  B200LUT_REQUIRE(s.ldo >= K, B200LUT_ERR_INVALID, "ldo must be >= K");
  B200LUT_REQUIRE((reinterpret_cast<uintptr_t>(s.packed) & 3u) == 0 &&
                      (!s.packed2 || (reinterpret_cast<uintptr_t>(s.packed2) & 3u) == 0) &&
                      (s.res_rank == 0 || aligned16(resB)),
                  B200LUT_ERR_ALIGN, "codes must be 4-byte aligned and resB 16-byte aligned");
  EmbedParams p = {};
  p.ids = reinterpret_cast<const long long*>(ids);
  p.packed[0] = static_cast<const uint8_t*>(s.packed);
  p.packed[1] = static_cast<const uint8_t*>(s.packed2);
  p.lut[0] = static_cast<const uint16_t*>(s.lut);
  p.lut[1] = static_cast<const uint16_t*>(s.lut2);
  p.bits[0] = s.bits;
  p.bits[1] = s.packed2 ? s.bits2 : 0;
  p.resA = static_cast<const uint16_t*>(s.resA);
  p.resB = static_cast<const uint16_t*>(resB);
  p.R = s.res_rank;
  p.out = s.out;
  p.ldo = s.ldo;
  p.out_f32 = out_fp32 ? 1 : 0;
  const int esz = out_fp32 ? 4 : 2;
  p.vec_ok = aligned16(s.out) && (s.ldo * esz) % 16 == 0;
  p.N = s.N; p.K = K; p.group_size = s.group_size; p.n_groups = s.n_groups;
  if (p.bits[0] == 4 && !p.packed[1] && p.R == 0 && !p.out_f32 && p.vec_ok && aligned16(p.packed[0])) {
    if (dtype == B200LUT_BF16)
      embed_gather4_kernel<__nv_bfloat16><<<unsigned(n_ids), kEmbedThreads, 0, cudaStream_t(stream)>>>(p);
    else
      embed_gather4_kernel<__half><<<unsigned(n_ids), kEmbedThreads, 0, cudaStream_t(stream)>>>(p);
    B200LUT_CUDA_OK(cudaGetLastError());
    return B200LUT_OK;
  }
  const dim3 grid(unsigned(n_ids), unsigned((K / 8 + kEmbedThreads - 1) / kEmbedThreads), 1);
  if (dtype == B200LUT_BF16)
    embed_gather_kernel<__nv_bfloat16><<<grid, kEmbedThreads, 0, cudaStream_t(stream)>>>(p);
  else
    embed_gather_kernel<__half><<<grid, kEmbedThreads, 0, cudaStream_t(stream)>>>(p);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}

extern "C" int b200lut_round_rows(const float* in, int64_t ldi, void* out, int64_t ldo,
                                  int64_t M, int K, int dtype, void* stream) {
  B200LUT_REQUIRE(M >= 0 && K >= 0 && ldi >= K && ldo >= K, B200LUT_ERR_INVALID,
                  "M, K >= 0 and row strides >= K required");
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  if (M == 0 || K == 0) return B200LUT_OK;
  B200LUT_REQUIRE(in && out, B200LUT_ERR_INVALID, "null buffer");
  long long grid = (M * K + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  uint16_t* o = static_cast<uint16_t*>(out);
  const long long ldi_ = ldi, ldo_ = ldo, M_ = M;
  if (dtype == B200LUT_BF16)
    round_rows_kernel<__nv_bfloat16><<<unsigned(grid), 256, 0, cudaStream_t(stream)>>>(in, ldi_, o, ldo_, M_, K);
  else
    round_rows_kernel<__half><<<unsigned(grid), 256, 0, cudaStream_t(stream)>>>(in, ldi_, o, ldo_, M_, K);
  B200LUT_CUDA_OK(cudaGetLastError());
  return B200LUT_OK;
}
