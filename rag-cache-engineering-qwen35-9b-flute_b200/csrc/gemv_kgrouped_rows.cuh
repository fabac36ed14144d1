// Row-range form of the K-grouped decode GEMV (4-bit codes, M <= 8) for sm_100a.
// Included by gemv_kgrouped.cu.
//
// The SIMT kernel of that file spends two shared-memory reads and M FMAs per weight in scalar
// code and is bound by instruction issue (ncu: 10.4 warp instructions per 32 weights). This form
// takes the structure of the row-grouped row-range kernel instead: a block owns a contiguous
// range of 32-row units over ALL of K (no fold across blocks), 16 warps take the k-chunks of a
// unit round-robin, a 1 KB piece of codes (32 rows x 64 k) sits in registers as one 256-bit load
// per lane, and the looked-up pairs are the A fragments of mma.sync.m16n8k16 with the activation
// rows as B fragments (every n8 column carries batch row column mod M'). What differs is the
// lookup: a palette belongs to one (row, 128-column group), so there is no pair table — the 1 KB
// palette block of the piece's 32 rows x 16 entries travels with the codes (cp.async into a
// four-slot ring per warp, requested four pieces ahead) and every weight is one 16-bit
// ld.shared at row * 32 + code * 2. The warps' sums meet in shared memory in warp order
// (deterministic), then bias and ONE rounding.
#pragma once

namespace b200lut {
namespace {

constexpr int kKrWarps = 16;
constexpr int kKrThreads = kKrWarps * 32;
constexpr int kKrRing = 4;                 // pieces in flight per warp
constexpr int kKrUnitRows = 32;            // output rows of one 1 KB plane at 4 bits
constexpr int kKrMaxPlanes = 16;           // units per block
constexpr uint32_t kKrSlotBytes = 1024;    // palettes of 32 rows x 16 entries
constexpr uint32_t kKrPalBytes = kKrWarps * kKrRing * kKrSlotBytes;   // 64 KB

struct KgRowsParams {
  const uint16_t* x;
  long long ldx;
  const uint8_t* packed;
  const uint16_t* lut;     // [K / 128][N][16]
  const uint16_t* bias;
  uint16_t* out;
  long long ldo;
  int M, Mp, N, K, G;      // G = K / 64 chunks
  int units_total, row_blocks, red_planes;
  uint32_t xs_off, red_off;   // byte offsets of the staged rows and the fold buffer in dynamic smem
};

__device__ __forceinline__ uint32_t kr_lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t kr_bfe(uint32_t v, int pos, int len) {
  uint32_t r;
  asm("bfe.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(v), "r"(pos), "r"(len));
  return r;
}
__device__ __forceinline__ void kr_lds128(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void kr_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
template <typename T>
__device__ __forceinline__ void kr_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (DType<T>::id == B200LUT_BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <typename T>
__global__ void __launch_bounds__(kKrThreads, 1) gemv_kgrouped_rows_kernel(const __grid_constant__ KgRowsParams p) {
  extern __shared__ __align__(16) uint8_t kr_smem[];
  constexpr int NW = kKrWarps, R = kKrRing;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int G = p.G, M = p.M, Mp = p.Mp;
  const int rb = blockIdx.x;
  const int u0 = int((long long)p.units_total * rb / p.row_blocks);
  const int u1 = int((long long)p.units_total * (rb + 1) / p.row_blocks);
  const int nplanes = u1 - u0;
  const uint32_t smem_base = smem_u32(kr_smem);
  const uint32_t my_ring = smem_base + uint32_t(warp) * (R * kKrSlotBytes);

  asm volatile("griddepcontrol.launch_dependents;");

  // this warp's pieces: chunk warp + 16 j of plane pl, plane after plane
  const int cnt = G > warp ? (G - warp + NW - 1) / NW : 0;
  const int total = nplanes * cnt;
  struct Cursor { int pl, j; };
  auto code_ptr = [&](const Cursor& cu) -> const uint8_t* {
    const int u = u0 + cu.pl, c = warp + NW * cu.j;
    return p.packed + (size_t(u >> 2) * G + c) * 4096 + size_t(u & 3) * 1024 + lane * 32;
  };
  auto fetch_palette = [&](int slot, const Cursor& cu, bool on) {
    if (on) {
      const int u = u0 + cu.pl, c = warp + NW * cu.j;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.lut) +
                           (size_t(c >> 1) * p.N + size_t(u) * kKrUnitRows) * 32;
      kr_cp_async16(my_ring + uint32_t(slot) * kKrSlotBytes + uint32_t(lane) * 16u, src + lane * 16);
      kr_cp_async16(my_ring + uint32_t(slot) * kKrSlotBytes + uint32_t(lane + 32) * 16u, src + (lane + 32) * 16);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto advance = [&](Cursor& cu) {
    if (++cu.j == cnt) { cu.j = 0; ++cu.pl; }
  };

  // ---- the first R pieces (codes to registers, palettes to the ring) before anything else -------
  Cursor ld = {0, 0};
  uint32_t w[R][8];
#pragma unroll
  for (int s = 0; s < R; ++s) {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[s][i] = 0u;
    const bool on = s < total;
    ldg_stream256_if(w[s], on ? code_ptr(ld) : p.packed, on ? 1u : 0u);
    fetch_palette(s, ld, on);
    if (on) advance(ld);
  }

  // ---- activation rows into shared memory, B-fragment order:
  //      element (chunk g, tig, kt, j) at g*128 + tig*32 + kt*8 + 2j bytes = x[64g + 16kt + 4tig + j]
  asm volatile("griddepcontrol.wait;" ::: "memory");
  {
    uint8_t* xs = kr_smem + p.xs_off;
    const int per_row = G * 8;   // 16-byte pieces of one row
    const int all = Mp * per_row;
    for (int idx = threadIdx.x; idx < all; idx += kKrThreads) {
      const int m = idx / per_row, pc = idx - m * per_row;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m < M) v = __ldcg(reinterpret_cast<const uint4*>(p.x + size_t(m) * p.ldx + size_t(pc) * 8));
      const int g = pc >> 3, o = pc & 7, kt = o >> 1, tg = (o & 1) * 2;
      uint8_t* dst = xs + (size_t(m) * G + g) * 128 + tg * 32 + kt * 8;
      *reinterpret_cast<uint2*>(dst) = make_uint2(v.x, v.y);
      *reinterpret_cast<uint2*>(dst + 32) = make_uint2(v.z, v.w);
    }
  }
  __syncthreads();

  // ---- main loop ------------------------------------------------------------------------------
  float acc[2][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[s][r] = 0.f;
  float* red = reinterpret_cast<float*>(kr_smem + p.red_off);
  const uint32_t xs_lane = smem_base + p.xs_off + uint32_t(gid & (Mp - 1)) * uint32_t(G) * 128u +
                           uint32_t(tig) * 32u + uint32_t(warp) * 128u;
  Cursor use = {0, 0};
  for (int i0 = 0; i0 < total; i0 += R) {
#pragma unroll
    for (int s = 0; s < R; ++s) {
      if (i0 + s < total) {      // warp-uniform
        // the group of this slot (and every older one) has landed
        asm volatile("cp.async.wait_group %0;" ::"n"(R - 1) : "memory");
        __syncwarp();
        const uint32_t slot = my_ring + uint32_t(s) * kKrSlotBytes;
        uint32_t xb[2][4];
        const uint32_t xa = xs_lane + uint32_t(use.j) * uint32_t(NW * 128);
        kr_lds128(xb[0], xa);
        kr_lds128(xb[1], xa + 16);
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          const uint32_t row_lo = slot + uint32_t(16 * sl + gid) * 32u, row_hi = row_lo + 8u * 32u;
          uint32_t a[4][4];
#pragma unroll
          for (int kt = 0; kt < 4; ++kt)
#pragma unroll
            for (int f = 0; f < 4; ++f) {   // fields (g, k 0-1), (g+8, k 0-1), (g, k 2-3), (g+8, k 2-3)
              // one bit-field extract and one scaled add per code, one byte permute per pair
              const uint32_t word = w[s][4 * sl + kt];
              const uint32_t rowb = (f & 1) ? row_hi : row_lo;
              const uint32_t lo = kr_lds16(rowb + 2u * kr_bfe(word, 8 * f, 4));
              const uint32_t hi = kr_lds16(rowb + 2u * kr_bfe(word, 8 * f + 4, 4));
              a[kt][f] = __byte_perm(lo, hi, 0x5410u);
            }
#pragma unroll
          for (int kt = 0; kt < 4; ++kt)
            kr_mma<T>(acc[sl], a[kt], xb[kt >> 1][2 * (kt & 1)], xb[kt >> 1][2 * (kt & 1) + 1]);
        }
        // refill the slot: the piece R pieces on (the mma above were warp-collective, so every
        // lane is done with the slot's palettes)
        {
          const bool on = ld.pl < nplanes;
          ldg_stream256_if(w[s], on ? code_ptr(ld) : p.packed, on ? 1u : 0u);
          fetch_palette(s, ld, on);
          if (on) advance(ld);
        }
        if (use.j == cnt - 1) {   // this warp's share of the plane is done
#pragma unroll
          for (int sl = 0; sl < 2; ++sl)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int col = 2 * tig + (r & 1);
              if (col < Mp)
                red[((warp * p.red_planes + use.pl) * Mp + col) * kKrUnitRows + 16 * sl + gid + 8 * (r >> 1)] =
                    acc[sl][r];
              acc[sl][r] = 0.f;
            }
        }
        advance(use);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // ---- fold the warps' sums (warp order), bias, one rounding -----------------------------------
  const int nwa = G < NW ? G : NW;   // warps that held chunks
  const int stride = p.red_planes * Mp * kKrUnitRows;
  for (int idx = threadIdx.x; idx < nplanes * M * kKrUnitRows; idx += kKrThreads) {
    const int row = idx & 31, m = (idx >> 5) % M, pl = (idx >> 5) / M;
    const float* r0 = red + (pl * Mp + m) * kKrUnitRows + row;
    float v = 0.f;
    for (int wi = 0; wi < nwa; ++wi) v += r0[wi * stride];
    const int n = (u0 + pl) * kKrUnitRows + row;
    if (p.bias) v += DType<T>::to_float(p.bias[n]);
    p.out[size_t(m) * p.ldo + n] = DType<T>::from_float(v);
  }
}

// Geometry of a launch, or false when the shapes do not fit (the SIMT kernel serves them).
struct KgRowsGeom { int units_total, row_blocks, red_planes, Mp; uint32_t xs_off, red_off, bytes; };

inline bool kg_rows_plan(int M, int N, int K, int sms, KgRowsGeom* g) {
  if (M < 1 || M > 8 || N % kKrUnitRows || K % 128) return false;
  const int Mp = M == 1 ? 1 : (M == 2 ? 2 : (M <= 4 ? 4 : 8));
  const int G = K / kChunkK, U = N / kKrUnitRows;
  const uint32_t xs_bytes = uint32_t(Mp) * uint32_t(G) * 128u;
  const uint32_t limit = 227u * 1024u;
  if (kKrPalBytes + xs_bytes >= limit) return false;
  int cap = int((limit - kKrPalBytes - xs_bytes) / (uint32_t(kKrWarps) * uint32_t(Mp) * 128u));
  if (cap > kKrMaxPlanes) cap = kKrMaxPlanes;
  if (cap < 1) return false;
  int row_blocks = U;
  if (U > sms) {
    row_blocks = 0;
    for (int k = 1; k * sms <= U && !row_blocks; ++k)
      if ((U + k * sms - 1) / (k * sms) <= cap) row_blocks = k * sms;
    if (!row_blocks) row_blocks = U;
  }
  g->units_total = U;
  g->row_blocks = row_blocks;
  g->red_planes = (U + row_blocks - 1) / row_blocks;
  g->Mp = Mp;
  g->xs_off = kKrPalBytes;
  g->red_off = kKrPalBytes + xs_bytes;
  g->bytes = g->red_off + uint32_t(kKrWarps) * uint32_t(g->red_planes) * uint32_t(Mp) * 128u;
  return g->bytes <= limit;
}

}  // namespace
}  // namespace b200lut
