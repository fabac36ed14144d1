// Pair-table machinery shared by the decode GEMV and the prefill GEMM: streaming code
// loads, the bank-replicated pair table in shared memory and its one-instruction lookup.
//
// A pair of codes (2*bits bits) becomes a packed pair of 16-bit palette entries with ONE
// shared-memory load. The table is replicated 32 times so that lane L only touches bank
// L: entry e of slot s lives at table + e*256 + s*128 + 4*L. A table is 64 KB aligned in
// the shared window, so at 4 bits the address is a single byte permute of (code word,
// lane base): no shift, mask or add per lookup.
#pragma once

#include "common.cuh"

namespace b200lut {
namespace {

constexpr uint32_t kTableBytes = 65536;   // one pair table: 256 entries x 256 B (two slots)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 256-bit streaming load: read-only path, no L1 allocation, first in line for L2 eviction
__device__ __forceinline__ void ldg_stream256(uint32_t* r, const uint8_t* p) {
  asm volatile(
      "ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "l"(p));
}

// Same load, executed only when `on` is non-zero; the registers keep their old value
// otherwise (read-write operands: no select or copy after the load, so nothing waits
// on it until the data is actually used).
__device__ __forceinline__ void ldg_stream256_if(uint32_t* r, const uint8_t* p, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %9, 0;\n\t"
      "@q ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n\t}"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
        "+r"(r[7])
      : "l"(p), "r"(on));
}

// Pair-table lookup. Deliberately NOT volatile, so the scheduler may issue lookups of
// later fragments ahead of the current mma. Ordering against the barriers around the
// table's lifetime is carried by data: every address includes a token defined after
// the build barrier, and the accumulators are pinned before the barrier that ends it.
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// Fill the pair table(s) of one pass: entry v -> LUT[v & mask] | LUT[v >> bits] << 16,
// one table slot per distinct palette of the tile (nl = 1, 2 or 4 palettes per tile).
__device__ void build_tables(uint8_t* tbl_ptr, const uint16_t* __restrict__ lut, int bits,
                             int n_groups, int row0, int gs, int nl, int nthreads) {
  const int entries = 1 << (2 * bits);
  const uint32_t mask = (1u << bits) - 1u;
  const int rows_per_lut = kTileRows / nl;
  for (int idx = threadIdx.x; idx < nl * entries * 8; idx += nthreads) {
    const int q = idx & 7, e = (idx >> 3) & (entries - 1), sl = idx >> (3 + 2 * bits);
    int grp = (row0 + sl * rows_per_lut) / gs;
    if (grp > n_groups - 1) grp = n_groups - 1;
    const uint16_t* row = lut + (size_t(grp) << bits);
    const uint32_t v = uint32_t(__ldg(row + (e & mask))) | (uint32_t(__ldg(row + (e >> bits))) << 16);
    uint4* dst = reinterpret_cast<uint4*>(tbl_ptr + size_t(sl >> 1) * kTableBytes + e * 256 +
                                          (sl & 1) * 128 + q * 16);
    *dst = make_uint4(v, v, v, v);
  }
}

// The same fill in two halves with ONE register in between, for tiles with at most two
// palettes (one table): lane L of every warp fetches entry L % 16 of palette L / 16
// (palette_fetch, a single 2-byte load), and the pair entries are later assembled from
// warp shuffles (table_store_shfl). All threads of the block must call both.
__device__ __forceinline__ uint32_t palette_fetch(const uint16_t* __restrict__ lut, int bits,
                                                  int n_groups, int row0, int gs, int nl) {
  const int lane = threadIdx.x & 31;
  const int sl = (lane >> 4) < nl ? (lane >> 4) : 0;
  int grp = (row0 + sl * (kTileRows / nl)) / gs;
  if (grp > n_groups - 1) grp = n_groups - 1;
  const int e = lane & 15;
  return e < (1 << bits) ? uint32_t(__ldg(lut + (size_t(grp) << bits) + e)) : 0u;
}

template <int NT>
__device__ __forceinline__ void table_store_shfl(uint8_t* tbl_ptr, uint32_t lv, int bits, int nl) {
  const int entries = 1 << (2 * bits);
  const int mask = (1 << bits) - 1;
  constexpr int kIters = (4096 + NT - 1) / NT;
#pragma unroll
  for (int k = 0; k < kIters; ++k) {
    const int idx = threadIdx.x + k * NT;
    if (idx < nl * entries * 8) {   // warp-uniform: the bound is a multiple of 32
      const int q = idx & 7, e = (idx >> 3) & (entries - 1), sl = idx >> (3 + 2 * bits);
      const uint32_t lo = __shfl_sync(0xffffffffu, lv, 16 * sl + (e & mask));
      const uint32_t hi = __shfl_sync(0xffffffffu, lv, 16 * sl + (e >> bits));
      const uint32_t v = lo | (hi << 16);
      *reinterpret_cast<uint4*>(tbl_ptr + e * 256 + (sl & 1) * 128 + q * 16) = make_uint4(v, v, v, v);
    }
  }
}

// The same fill in two halves, for tiles with at most two palettes (one table):
// Palette entries this thread will write into the pair table of a pass: fetched early (one
// pass ahead), stored late (table_store), so the palette's DRAM round trip is off the path.
// registers per thread: nl (<= 2) * 256 entries * 8 sixteen-byte copies / threads
template <int NT> struct LutRegs { static constexpr int n = (4096 + NT - 1) / NT; };

template <int NT>
__device__ __forceinline__ void table_fetch(uint32_t (&v)[LutRegs<NT>::n], const uint16_t* __restrict__ lut,
                                            int bits, int n_groups, int row0, int gs, int nl) {
  const int entries = 1 << (2 * bits);
  const uint32_t mask = (1u << bits) - 1u;
  const int rows_per_lut = kTileRows / nl;
#pragma unroll
  for (int k = 0; k < LutRegs<NT>::n; ++k) {
    const int idx = threadIdx.x + k * NT;
    v[k] = 0u;
    if (idx < nl * entries * 8) {
      const int e = (idx >> 3) & (entries - 1), sl = idx >> (3 + 2 * bits);
      int grp = (row0 + sl * rows_per_lut) / gs;
      if (grp > n_groups - 1) grp = n_groups - 1;
      const uint16_t* row = lut + (size_t(grp) << bits);
      v[k] = uint32_t(__ldg(row + (e & mask))) | (uint32_t(__ldg(row + (e >> bits))) << 16);
    }
  }
}

template <int NT>
__device__ __forceinline__ void table_store(uint8_t* tbl_ptr, const uint32_t (&v)[LutRegs<NT>::n], int bits,
                                            int nl) {
  const int entries = 1 << (2 * bits);
#pragma unroll
  for (int k = 0; k < LutRegs<NT>::n; ++k) {
    const int idx = threadIdx.x + k * NT;
    if (idx < nl * entries * 8) {
      const int q = idx & 7, e = (idx >> 3) & (entries - 1), sl = idx >> (3 + 2 * bits);
      *reinterpret_cast<uint4*>(tbl_ptr + e * 256 + (sl & 1) * 128 + q * 16) =
          make_uint4(v[k], v[k], v[k], v[k]);
    }
  }
}

}  // namespace
}  // namespace b200lut
