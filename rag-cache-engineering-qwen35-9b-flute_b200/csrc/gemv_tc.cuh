// Decode GEMV on the Blackwell tensor-core path (tcgen05 + TMEM), 4-bit codes.
// Included by gemv.cu (shares its parameter structs, pair tables and fold).
//
// Same streaming and lookup as the mma.sync kernel, different back end: the looked-up
// palette pairs are written straight into tensor memory with tcgen05.st (the slab
// layout's register order is the 16x256b store shape), where they are the A operand
// (128 weight rows x 64 k per stage) of tcgen05.mma; the activation rows sit in shared
// memory as the B operand (16 token columns, zero beyond M), the fp32 sums live in
// TMEM. One thread issues the MMAs; the sixteen lookup warps never wait on tensor-core
// results, carry no accumulators and no activation fragments, so their registers hold
// codes in flight (6 KB per warp, 96 KB per SM).
//
//   warp w < 16 : lookup warp of TMEM lane quarter q = w % 4 and stage group w / 4;
//                 k-block i of the block's range belongs to group i % 4, stage i % 8
//   warp 16     : lane 0 issues 4 MMAs (K = 16 each) per k-block, then commits the
//                 stage's "empty" barrier; commits "done" after the last one
//   epilogue    : warps 0-3 read D (128 rows x 16 columns per plane) with tcgen05.ld
//                 into part[plane][m][row]; the split fold and store are shared code.
#pragma once

#include "tc05.cuh"

namespace b200lut {
namespace {

constexpr int kTcLookupWarps = 16;
constexpr int kTcThreads = (kTcLookupWarps + 1) * 32;
constexpr int kTcStages = 8;          // operand stages in TMEM (32 columns each)
constexpr int kTcRing = 6;            // k-blocks of codes in flight per warp (8 registers each)
constexpr uint32_t kTcCtrlBytes = 256;
constexpr uint32_t kTcTmemCols = 512;
constexpr uint32_t kTcDCol = 0;       // D: plane p at columns [16p, 16p + 16)
constexpr uint32_t kTcACol = 32;      // operand stage s at columns [32 + 32s, 64 + 32s)
constexpr int kTcTokens = 16;

__device__ int g_tc_status = 0;

// x rows of the block's K range as the B operand: [k/8][16 tokens][8 elements], no swizzle
__device__ __forceinline__ void tc_stage_x(uint8_t* xs, const uint16_t* __restrict__ x,
                                           long long ldx, int M, int k_begin, int k_count) {
  const int units = k_count / 8;
  for (int idx = threadIdx.x; idx < units * kTcTokens; idx += kTcThreads) {
    const int u = idx >> 4, t = idx & 15;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (t < M) v = *reinterpret_cast<const uint4*>(x + size_t(t) * ldx + k_begin + 8 * u);
    *reinterpret_cast<uint4*>(xs + size_t(idx) * 16) = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(kTcThreads, 1) gemv_tc_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  float* part = reinterpret_cast<float*>(smem);
  const uint32_t part_addr = smem_u32(smem);
  uint8_t* ctrl = smem + kPartBytes;
  const uint32_t ctrl_addr = part_addr + kPartBytes;
  const uint32_t bar_full = ctrl_addr, bar_empty = ctrl_addr + 64, bar_done = ctrl_addr + 128;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 136);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 140);
  const uint32_t tbl_addr = (ctrl_addr + kTcCtrlBytes + 0xFFFFu) & ~0xFFFFu;
  uint8_t* tbl_ptr = smem + (tbl_addr - part_addr);

  const int split = p.split;
  const int tile_g = blockIdx.x / split, sp = blockIdx.x % split;
  const int c0 = (p.G * sp) / split, c1 = (p.G * (sp + 1)) / split;
  const int nblk = c1 - c0;
  const bool silu = p.epilogue == B200LUT_EPI_SILU_MUL;
  int si = 0;
  {
    const int step = silu ? 2 : 1;
    for (int s = 0; s < p.nseg; s += step)
      if (tile_g >= p.seg[s].tile_begin) si = s;
  }
  const int tile = tile_g - p.seg[si].tile_begin;
  const int nplanes = silu ? 2 : 1;
  const int total = nblk * nplanes;       // k-blocks streamed by this block, plane-major
  const SegDev& sg0 = p.seg[si];
  int nl = kTileRows / sg0.gs;
  if (nl < 1) nl = 1;
  const int tables = (nplanes * nl + 1) / 2;
  uint8_t* xs = tbl_ptr + size_t(tables) * kTableBytes;
  const uint32_t xs_addr = tbl_addr + uint32_t(tables) * kTableBytes;

  asm volatile("griddepcontrol.launch_dependents;");

  // ---- code prefetch (independent of everything else) --------------------------------
  const int q = warp & 3, grp = warp >> 2;
  uint32_t w[kTcRing][8];
  auto block_ptr = [&](int i) -> const uint8_t* {       // i: index in the plane-major sequence
    const int plane = i >= nblk ? 1 : 0, c = c0 + (plane ? i - nblk : i);
    const uint8_t* base = p.seg[si + plane].packed;
    return base + (size_t(tile) * p.G + c) * 4096 + q * 1024 + lane * 32;
  };
  if (warp < kTcLookupWarps) {
#pragma unroll
    for (int u = 0; u < kTcRing; ++u) {
#pragma unroll
      for (int i = 0; i < 8; ++i) w[u][i] = 0u;
      const int i = grp + 4 * u;
      ldg_stream256_if(w[u], block_ptr(i < total ? i : 0), i < total ? 1u : 0u);
    }
  }

  // ---- setup ----------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      tc::mbar_init(bar_full + 8 * s, 4);     // the four lookup warps of the stage's group
      tc::mbar_init(bar_empty + 8 * s, 1);    // tcgen05.commit
    }
    tc::mbar_init(bar_done, 1);
    *abort_flag = 0;
    tc::mbar_init_fence();
  }
  if (warp == kTcLookupWarps) tc::tmem_alloc(ctrl_addr + 136, kTcTmemCols);
  for (int plane = 0; plane < nplanes; ++plane) {
    const SegDev& sg = p.seg[si + plane];
    // plane p occupies table slots [p * nl, (p + 1) * nl)
    build_tables(tbl_ptr + size_t((plane * nl) >> 1) * kTableBytes + ((plane * nl) & 1) * 128,
                 sg.lut, 4, sg.n_groups, tile * kTileRows, sg.gs, nl, kTcThreads);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");   // x is the predecessor's output
  tc_stage_x(xs, p.x, p.ldx, p.M, c0 * kChunkK, nblk * kChunkK);
  tc::fence_proxy_async();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp < kTcLookupWarps) {
    // ---- lookup warps ---------------------------------------------------------------------
    uint32_t token;   // defined after the build barrier; part of every lookup address
    asm volatile("mov.u32 %0, 0;" : "=r"(token));
    const uint32_t lane_base = tbl_addr + lane * 4 + token;
    for (int i0 = grp; i0 < total; i0 += 4 * kTcRing) {
#pragma unroll
      for (int u = 0; u < kTcRing; ++u) {
        const int i = i0 + 4 * u;
        if (i < total) {     // warp-uniform
          const int stage = i % kTcStages, use = i / kTcStages;
          const int plane = i >= nblk ? 1 : 0;
          if (use > 0)
            tc::mbar_wait(bar_empty + 8 * stage, uint32_t(use - 1) & 1u, abort_flag, &g_tc_status,
                          tc::kStatusWaitEmpty);
          tc::fence_after_sync();
#pragma unroll
          for (int sl = 0; sl < 2; ++sl) {
            // palette slot of this slab: rows 32q + 16sl of the tile
            const int rowslab = 2 * q + sl;                 // slab index 0..7 in the tile
            const int pal = plane * nl + (nl == 1 ? 0 : (nl == 2 ? rowslab >> 2 : rowslab >> 1));
            const uint32_t base = lane_base + uint32_t(pal >> 1) * kTableBytes + uint32_t(pal & 1) * 128u;
            uint32_t r[16];
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              const uint32_t word = w[u][4 * sl + kt];
              // fields f0..f3 = (row g, k 0-1), (row g+8, k 0-1), (row g, k 2-3), (row g+8, k 2-3);
              // the store shape wants (g, c), (g, c+1), (g+8, c), (g+8, c+1) -> f0, f2, f1, f3
              r[4 * kt + 0] = lds32(__byte_perm(word, base, 0x7604u));
              r[4 * kt + 1] = lds32(__byte_perm(word, base, 0x7624u));
              r[4 * kt + 2] = lds32(__byte_perm(word, base, 0x7614u));
              r[4 * kt + 3] = lds32(__byte_perm(word, base, 0x7634u));
            }
            tc::tmem_st_16x256b_x4(tmem + (uint32_t(32 * q + 16 * sl) << 16) + kTcACol + 32u * stage, r);
          }
          // refill this ring slot with the group's block kTcRing steps ahead
          const int in = i + 4 * kTcRing;
          ldg_stream256_if(w[u], block_ptr(in < total ? in : 0), in < total ? 1u : 0u);
          tc::wait_st();
          tc::fence_before_sync();
          if (lane == 0) tc::mbar_arrive(bar_full + 8 * stage);
        }
      }
    }
  } else {
    // ---- MMA issuer (the whole warp walks the loop, lane 0 issues) ---------------------------
    constexpr uint32_t kFmt = DType<T>::id == B200LUT_BF16 ? 1u : 0u;
    constexpr uint32_t idesc = tc::instr_desc(kFmt, 128, kTcTokens);
    for (int i = 0; i < total; ++i) {
      const int stage = i % kTcStages, use = i / kTcStages;
      const int plane = i >= nblk ? 1 : 0, blk = plane ? i - nblk : i;
      tc::mbar_wait(bar_full + 8 * stage, uint32_t(use) & 1u, abort_flag, &g_tc_status,
                    tc::kStatusWaitFull);
      tc::fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // k-step ks of k-block blk: K units 8*blk + 2*ks and + 1, 256 bytes per unit
          const uint64_t bdesc =
              tc::smem_desc(xs_addr + uint32_t(8 * blk + 2 * ks) * 256u, 256u, 128u, 0u);
          tc::mma_ts(tmem + kTcDCol + 16u * plane, tmem + kTcACol + 32u * stage + 8u * ks, bdesc,
                     idesc, (blk > 0 || ks > 0) ? 1u : 0u);
        }
        tc::mma_commit(bar_empty + 8 * stage);
        if (i == total - 1) tc::mma_commit(bar_done);
      }
      __syncwarp();
    }
  }

  // ---- epilogue: D -> part[plane][m][row] ---------------------------------------------------
  if (warp < 4) {
    tc::mbar_wait(bar_done, 0u, abort_flag, &g_tc_status, tc::kStatusWaitDone);
    tc::fence_after_sync();
    for (int plane = 0; plane < nplanes; ++plane) {
      uint32_t r[16];
      tc::tmem_ld_32x32b_x16(tmem + (uint32_t(32 * warp) << 16) + kTcDCol + 16u * plane, r);
      tc::wait_ld();
#pragma unroll
      for (int m = 0; m < kTcTokens; ++m)
        if (m < p.M) part[(plane * kMaxM + m) * kTileRows + 32 * warp + lane] = __uint_as_float(r[m]);
    }
    tc::fence_before_sync();
  }
  __syncthreads();
  if (warp == kTcLookupWarps) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTcTmemCols);
  }
  fold_and_store<T, kTcThreads>(p, part, si, tile, tile_g, sp);
}

}  // namespace
}  // namespace b200lut
