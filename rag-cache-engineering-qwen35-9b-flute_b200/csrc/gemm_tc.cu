// Prefill LUT GEMM (M > 16 tokens) on the Blackwell tensor-core path.
//
// out[m, n] = sum_k x[m, k] * LUT[n / gs][code(n, k)]: replaces the reference's streaming
// tensor-core GEMM family (src/flute_extended/src/kernel_streaming.cu:987-1108, K7/K8).
//
// One block computes a 128 (weight rows) x NT (tokens, up to 256) output tile over all
// of K with tcgen05.mma, weights on the M side:
//   * A operand = dequantised weights, 128 rows x 64 k per stage, living in TENSOR MEMORY.
//     Lookup warps stream the 4-bit codes from global memory into registers (256-bit
//     loads), turn each code pair into two palette entries with one shared-memory
//     lookup (pairtable.cuh) and write the result straight into TMEM with tcgen05.st —
//     the slab layout's register order is the 16x256b store shape. The dequantised tile
//     never passes through shared memory, which the B operand needs for itself.
//   * B operand = activations, NT tokens x 64 k per stage, brought by TMA
//     (cp.async.bulk.tensor, 128-byte swizzle, zero fill beyond M) into shared memory.
//   * D = fp32 accumulators in TMEM (128 lanes x NT columns, a second plane for the
//     fused gate/up form); the epilogue reads them with tcgen05.ld, adds bias, applies
//     SiLU*mul when asked, rounds once and stores.
// Warp roles: 0-7 lookup (TMEM lane quarter = warp % 4, two groups alternate k-blocks),
// 8 = TMA producer, 9 = MMA issuer; warps 0-7 run the epilogue. All mbarrier waits are
// bounded (tc05.cuh).
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "pairtable.cuh"
#include "tc05.cuh"

namespace b200lut {
namespace {

constexpr int kLookupWarps = 8;
constexpr int kThreads = (kLookupWarps + 2) * 32;
constexpr int kAStages = 4;            // operand stages in TMEM, 32 columns each
constexpr int kRing = 4;               // k-blocks of codes in flight per lookup warp
constexpr int kMaxXStages = kAStages;   // activation stage s pairs with operand stage s
constexpr uint32_t kCtrlBytes = 1024;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kACol = 256;        // operand stage s at columns [256 + 32 s, 288 + 32 s)
constexpr size_t kMaxDynSmem = 232448 - 1024;

__device__ int g_gemm_status = 0;

struct GemmParams {
  const uint8_t* packed[2];
  const uint16_t* lut[2];
  const uint16_t* bias[2];
  uint16_t* out;
  long long ldo;
  int M, N, K, G, gs, n_groups;
  int npass;        // 1, or 2 (second stream / up projection)
  int plane[2];     // accumulator plane of each pass (0, or 1 for the up projection)
  int silu;         // epilogue: out = silu(plane 0) * plane 1
  int NT;           // token tile (multiple of 16, <= 256; <= 128 with two planes)
  int m_tiles;
  uint32_t smem_bytes;
  int out_aligned;   // out rows are 16-byte aligned: staged, vectorised epilogue
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// The same for a CTA of a pair (cta_group::2): the tile lands in this CTA's shared memory, its
// bytes are reported to `bar`, which may be the other CTA's barrier. Not a multicast load.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const GemmParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = smem_u32(smem);
  // control block: barriers, the TMEM base and the abort flag
  const uint32_t bar_xfull = base, bar_afull = base + 128, bar_empty = base + 192,
                 bar_done = base + 256;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 264);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 268);

  int nl = kTileRows / p.gs;
  if (nl < 1) nl = 1;
  const int tables = (p.npass * nl + 1) / 2;
  const uint32_t tbl_addr = (base + kCtrlBytes + 0xFFFFu) & ~0xFFFFu;
  uint8_t* tbl_ptr = smem + (tbl_addr - base);
  // activation stages fill the space below and above the 64 KB-aligned tables
  const uint32_t stage_bytes = uint32_t(p.NT) * 128u;
  volatile uint32_t* xaddr = reinterpret_cast<volatile uint32_t*>(smem + 512);   // [kMaxXStages]
  volatile int* nxs_slot = reinterpret_cast<volatile int*>(smem + 544);
  if (threadIdx.x == 0) {
    int n = 0;
    uint32_t a = (base + kCtrlBytes + 1023u) & ~1023u;
    while (n < kMaxXStages && a + stage_bytes <= tbl_addr) { xaddr[n++] = a; a += stage_bytes; }
    a = tbl_addr + uint32_t(tables) * kTableBytes;
    while (n < kMaxXStages && a + stage_bytes <= base + p.smem_bytes) { xaddr[n++] = a; a += stage_bytes; }
    *nxs_slot = n;
  }

  const int n_tile = blockIdx.x / p.m_tiles, m_tile = blockIdx.x % p.m_tiles;
  const int m0 = m_tile * p.NT, n0 = n_tile * kTileRows;
  const int total = p.G * p.npass;     // k-blocks streamed, pass-major

  asm volatile("griddepcontrol.launch_dependents;");

  // ---- code prefetch ---------------------------------------------------------------------
  const int q = warp & 3, grp = warp >> 2;
  uint32_t w[kRing][8];
  auto block_ptr = [&](int i) -> const uint8_t* {
    const int pass = i >= p.G ? 1 : 0, c = pass ? i - p.G : i;
    return p.packed[pass] + (size_t(n_tile) * p.G + c) * 4096 + q * 1024 + lane * 32;
  };
  if (warp < kLookupWarps) {
#pragma unroll
    for (int u = 0; u < kRing; ++u) {
#pragma unroll
      for (int i = 0; i < 8; ++i) w[u][i] = 0u;
      const int i = grp + 2 * u;
      ldg_stream256_if(w[u], block_ptr(i < total ? i : 0), i < total ? 1u : 0u);
    }
  }

  // ---- setup ----------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) {
      tc::mbar_init(bar_xfull + 8 * s, 1);    // TMA transaction bytes
      tc::mbar_init(bar_afull + 8 * s, 4);    // the four lookup warps that filled the stage
      tc::mbar_init(bar_empty + 8 * s, 1);    // tcgen05.commit: both operands of the stage consumed
    }
    tc::mbar_init(bar_done, 1);
    *abort_flag = (*nxs_slot < 2) ? 1 : 0;   // cannot pipeline: drain at once (host prevents this)
    tc::mbar_init_fence();
  }
  if (warp == kLookupWarps) tc::tmem_alloc(base + 264, kTmemCols);
  for (int pass = 0; pass < p.npass; ++pass)
    build_tables(tbl_ptr + size_t((pass * nl) >> 1) * kTableBytes + ((pass * nl) & 1) * 128,
                 p.lut[pass], 4, p.n_groups, n0, p.gs, nl, kThreads);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const int nst = *nxs_slot > 0 ? *nxs_slot : 1;   // pipeline depth: 2..4 stages of both operands

  if (warp < kLookupWarps) {
    // ---- lookup warps: codes -> palette pairs -> TMEM -------------------------------------------
    uint32_t token;
    asm volatile("mov.u32 %0, 0;" : "=r"(token));
    const uint32_t lane_base = tbl_addr + lane * 4 + token;
    for (int i0 = grp; i0 < total; i0 += 2 * kRing) {
#pragma unroll
      for (int u = 0; u < kRing; ++u) {
        const int i = i0 + 2 * u;
        if (i < total) {
          const int stage = i % nst, use = i / nst;
          const int pass = i >= p.G ? 1 : 0;
          if (use > 0)
            tc::mbar_wait(bar_empty + 8 * stage, uint32_t(use - 1) & 1u, abort_flag,
                          &g_gemm_status, tc::kStatusWaitEmpty);
          tc::fence_after_sync();
#pragma unroll
          for (int sl = 0; sl < 2; ++sl) {
            const int rowslab = 2 * q + sl;
            const int pal = pass * nl + (nl == 1 ? 0 : (nl == 2 ? rowslab >> 2 : rowslab >> 1));
            const uint32_t tb = lane_base + uint32_t(pal >> 1) * kTableBytes + uint32_t(pal & 1) * 128u;
            uint32_t r[16];
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              const uint32_t word = w[u][4 * sl + kt];
              // slab fields (row g, k 0-1), (g+8, k 0-1), (g, k 2-3), (g+8, k 2-3); the store
              // shape wants (g, c), (g, c+1), (g+8, c), (g+8, c+1): fields 0, 2, 1, 3
              r[4 * kt + 0] = lds32(__byte_perm(word, tb, 0x7604u));
              r[4 * kt + 1] = lds32(__byte_perm(word, tb, 0x7624u));
              r[4 * kt + 2] = lds32(__byte_perm(word, tb, 0x7614u));
              r[4 * kt + 3] = lds32(__byte_perm(word, tb, 0x7634u));
            }
            tc::tmem_st_16x256b_x4(tmem + (uint32_t(32 * q + 16 * sl) << 16) + kACol + 32u * stage, r);
          }
          const int in = i + 2 * kRing;
          ldg_stream256_if(w[u], block_ptr(in < total ? in : 0), in < total ? 1u : 0u);
          tc::wait_st();
          tc::fence_before_sync();
          if (lane == 0) tc::mbar_arrive(bar_afull + 8 * stage);
        }
      }
    }
  } else if (warp == kLookupWarps) {
    // ---- TMA producer: activations of k-block c, tokens m0 .. m0 + NT ---------------------------
    for (int i = 0; i < total; ++i) {
      const int xs = i % nst, use = i / nst;
      const int c = i >= p.G ? i - p.G : i;
      if (use > 0)
        tc::mbar_wait(bar_empty + 8 * xs, uint32_t(use - 1) & 1u, abort_flag, &g_gemm_status,
                      tc::kStatusWaitEmpty);
      if (lane == 0 && !*abort_flag) {
        tc::mbar_expect_tx(bar_xfull + 8 * xs, stage_bytes);
        tma_load_2d(xaddr[xs], &xmap, bar_xfull + 8 * xs, c * kChunkK, m0);
      }
      __syncwarp();
    }
  } else {
    // ---- MMA issuer ---------------------------------------------------------------------------
    constexpr uint32_t kFmt = DType<T>::id == B200LUT_BF16 ? 1u : 0u;
    const uint32_t idesc = tc::instr_desc(kFmt, 128, uint32_t(p.NT));
    // One thread issues; its instruction stream is the limit (an MMA must leave every 128
    // cycles), so nothing is computed per MMA: stage descriptors sit in registers, stage
    // and phase advance by increment, a K step is a 64-bit add, one commit per k-block.
    const uint64_t dtemplate = tc::smem_desc(0u, 16u, 1024u, 2u);
    uint64_t xd[kAStages];
#pragma unroll
    for (int s = 0; s < kAStages; ++s) xd[s] = dtemplate + uint64_t(xaddr[s < nst ? s : 0] >> 4);
    const uint32_t dcol[2] = {tmem + uint32_t(p.plane[0] * p.NT), tmem + uint32_t(p.plane[1] * p.NT)};
    const bool two_planes = p.plane[1] != p.plane[0];
    const int G = p.G;
    auto block = [&](int i, int stage, uint32_t phase, uint64_t bdesc0) {
      const int pass = i >= G ? 1 : 0;
      const bool first = (i == 0) || (two_planes && i == G);
      tc::mbar_wait(bar_xfull + 8 * stage, phase, abort_flag, &g_gemm_status, tc::kStatusWaitLoad);
      tc::mbar_wait(bar_afull + 8 * stage, phase, abort_flag, &g_gemm_status, tc::kStatusWaitFull);
      tc::fence_after_sync();
      if (lane == 0) {
        const uint32_t a0 = tmem + kACol + 32u * uint32_t(stage), d0 = pass ? dcol[1] : dcol[0];
        tc::mma_ts(d0, a0, bdesc0, idesc, first ? 0u : 1u);   // first k-block of a plane overwrites
        tc::mma_ts(d0, a0 + 8u, bdesc0 + 2u, idesc, 1u);      // +32 bytes of K per step
        tc::mma_ts(d0, a0 + 16u, bdesc0 + 4u, idesc, 1u);
        tc::mma_ts(d0, a0 + 24u, bdesc0 + 6u, idesc, 1u);
        tc::mma_commit(bar_empty + 8 * stage);
        if (i == total - 1) tc::mma_commit(bar_done);
      }
      __syncwarp();
    };
    if (nst == kAStages) {
      uint32_t phase = 0;
      for (int i0 = 0; i0 < total; i0 += kAStages, phase ^= 1u) {
#pragma unroll
        for (int s = 0; s < kAStages; ++s)
          if (i0 + s < total) block(i0 + s, s, phase, xd[s]);
      }
    } else {
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < total; ++i) {
        block(i, stage, phase, dtemplate + uint64_t(xaddr[stage] >> 4));
        if (++stage == nst) { stage = 0; phase ^= 1u; }
      }
    }
  }

  // ---- epilogue: TMEM -> bias / SiLU*mul -> one rounding -> global -----------------------------
  if (warp < kLookupWarps) {
    tc::mbar_wait(bar_done, 0u, abort_flag, &g_gemm_status, tc::kStatusWaitDone);
    tc::fence_after_sync();
    const int n = n0 + 32 * q + lane;
    const float b0 = p.bias[0] ? DType<T>::to_float(p.bias[0][n]) : 0.f;
    const float b1 = (p.npass > 1 && p.bias[1]) ? DType<T>::to_float(p.bias[1][n]) : 0.f;
    const int half_cols = p.NT / 2;
    // The output tile is staged in the (now idle) pair-table region as [token][128 rows] and
    // then written with 16-byte stores, 256 contiguous bytes per token row; a thread-per-
    // element store would issue 2-byte writes at a stride of ldo.
    uint16_t* stage_out = reinterpret_cast<uint16_t*>(tbl_ptr);
    const bool staged = p.out_aligned != 0;
    for (int cb = grp * half_cols; cb < (grp + 1) * half_cols; cb += 16) {
      uint32_t r0[16], r1[16];
      tc::tmem_ld_32x32b_x16(tmem + (uint32_t(32 * q) << 16) + uint32_t(cb), r0);
      if (p.silu) tc::tmem_ld_32x32b_x16(tmem + (uint32_t(32 * q) << 16) + uint32_t(p.NT + cb), r1);
      tc::wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int tok = m0 + cb + j;
        float v = __uint_as_float(r0[j]) + b0;
        if (p.silu) {
          const float u = __uint_as_float(r1[j]) + b1;
          v = v / (1.f + __expf(-v)) * u;
        } else if (p.npass > 1) {
          v += b1;     // second stream: both biases belong to the one output
        }
        if (staged) stage_out[(cb + j) * kTileRows + 32 * q + lane] = DType<T>::from_float(v);
        else if (tok < p.M) p.out[size_t(tok) * p.ldo + n] = DType<T>::from_float(v);
      }
    }
    if (staged) {
      asm volatile("bar.sync 1, %0;" ::"r"(kLookupWarps * 32) : "memory");   // the eight epilogue warps
      const uint4* src = reinterpret_cast<const uint4*>(stage_out);
      for (int idx = threadIdx.x; idx < p.NT * 16; idx += kLookupWarps * 32) {
        const int r = idx >> 4, c = idx & 15;
        if (m0 + r < p.M)
          *reinterpret_cast<uint4*>(p.out + size_t(m0 + r) * p.ldo + n0 + 8 * c) = src[idx];
      }
    }
    tc::fence_before_sync();
  }
  __syncthreads();
  if (warp == kLookupWarps) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Persistent form for one code stream (no second plane): a block walks a contiguous range of
// (row tile, token tile) output tiles of 128 x 256 and never tears its pipeline down.
// Measured on B200: a tcgen05.mma with the A operand in tensor memory costs the issuing
// thread about 70 cycles whatever N is, and 128 cycles of tensor pipe at N = 256, so N = 256
// is the only efficient tile width; the accumulator then fills 256 of the 512 TMEM columns and
// cannot be double-buffered next to the operand stages. What the persistent form removes is
// everything around the main loop: no block launch, TMEM allocation or barrier set-up per
// tile, the pair table is rebuilt only when the row tile changes, and while eight dedicated
// epilogue warps drain tile i (tcgen05.ld -> bias -> one rounding -> staged, 16-byte global
// stores) the lookup warps and the TMA producer already refill all operand stages of tile
// i + 1, so its MMAs start the moment the accumulator is free.
// Per k-block the lookup warps (codes -> pair lookups -> tcgen05.st) and the TMA producer
// arrive on ONE "full" barrier; the MMA issuer — a single thread, its loop flat over the
// block's k-blocks and unrolled by the ring size: one barrier test, one fence, one four-MMA
// instruction group, one commit — commits to one "done" barrier that frees the stage.
// Warps 0-7 lookup, 8 TMA producer, 9 MMA issuer, 10-17 epilogue.
constexpr int kPEpiWarps = 8;
constexpr int kPThreads = (kLookupWarps + 2 + kPEpiWarps) * 32;
constexpr int kPMaxNT = 256;
constexpr int kPStages = 4;             // ring depth of both operands
constexpr uint32_t kPACol = 256;        // operand stage s at columns [256 + 32 s, 288 + 32 s)
constexpr int kPStageTokens = 48;       // tokens per staged epilogue slice (12 KB per column half)

constexpr int kPMaxSeg = 4;             // projections that share x in one launch (Q/K/V/z, gate/up)

// One projection of a launch: its row tiles are the global row tiles [row0, next row0).
struct PersistSeg {
  const uint8_t* packed;
  const uint16_t* lut;
  const uint16_t* bias;
  uint16_t* out;
  long long ldo;
  int row0, n_groups, out_aligned;
  int res_rank;            // rank of the low-rank residual, 0 if the projection has none
  const uint16_t* resA;    // [N, res_rank], row-major
  int t_col0, pad;         // first column of this projection's block of the t matrix
};

struct PersistParams {
  PersistSeg seg[kPMaxSeg];
  int nsegs;
  int M, K, G, gs;
  int NT;            // token tile (multiple of 32, <= 256)
  int m_tiles;       // token tiles per row tile
  int n_tiles;       // row tiles
  int W;             // token columns of a row of tiles (the last tile rounded up to 32)
  uint32_t smem_bytes;
  long long wait_cycles;   // bound of every in-kernel wait, in SM clock cycles
  // Split mode (a workspace was given and the tile count leaves a partly filled last round):
  // every block takes `full` whole tiles; each of the `left` tiles behind them is cut along K
  // into `split` equal k-block ranges, one per block (blocks 0 .. left * split - 1 take one
  // each, before their whole tiles). The `split` blocks of a cut tile exchange fp32 partial
  // tiles through the workspace and each finishes its share of the tile's 16-column chunks,
  // adding the partial sums in ascending-k order.
  int split, full, left;
  // Low-rank residual: E extra k-blocks close every tile. Their weight operand is 64 columns of
  // the projection's resA rows (zero beyond the rank), written to the operand stage as they
  // are; their activation operand is the matching 64-column block of t = x @ resB^T, fetched
  // through the second tensor map. The sums, the bias and the single rounding are the tile's.
  int E;
  int kg_N;                // K-grouped palettes: output rows of the projection (rows of lut_k per k-group)
  // Two code streams of different widths: the first launch leaves its fp32 sums in acc_out
  // ([token][row], ld_acc floats per token) instead of rounding them, the second adds acc_in to
  // its own sums before bias and the single rounding.
  float* acc_out;
  const float* acc_in;
  long long ld_acc;
  float* ws;               // [left tile][part < split][column 256][row 128] fp32
  int* tickets;            // [left tile][2]: partial tiles stored, shares finished; zero between launches
};

// 64-bit code load (two consecutive words of a lane's string), executed only when `on`.
__device__ __forceinline__ void ldg64_if(uint32_t* r, const uint8_t* ptr, uint32_t on) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %3, 0;\n\t"
      "@q ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];\n\t}"
      : "+r"(r[0]), "+r"(r[1])
      : "l"(ptr), "r"(on));
}

// The 2 * BITS words of lane-string that hold row slabs 2q and 2q + 1 of one chunk
// (`chunk_lane` = chunk base + 32 * lane). At 4 bits they are one whole 256-bit plane; at
// other widths they straddle planes and come as BITS 64-bit loads.
template <int BITS>
__device__ __forceinline__ void load_slab_pair(uint32_t (&w)[2 * BITS], const uint8_t* chunk_lane,
                                               int q, uint32_t on) {
  if constexpr (BITS == 4) {
    ldg_stream256_if(w, chunk_lane + q * 1024, on);
  } else {
#pragma unroll
    for (int j = 0; j < BITS; ++j) {
      const int m = 2 * BITS * q + 2 * j;
      ldg64_if(&w[2 * j], chunk_lane + (m >> 3) * 1024 + 4 * (m & 7), on);
    }
  }
}

// Pair-table address of field i (0..15) of local slab sl (0, 1): the field's 2 * BITS bits
// moved to address bits 8.., joined with the lane base.
template <int BITS>
__device__ __forceinline__ uint32_t slab_field_addr(const uint32_t (&w)[2 * BITS], int sl, int i,
                                                    uint32_t base) {
  if constexpr (BITS == 4) {
    return __byte_perm(w[4 * sl + (i >> 2)], base, 0x7604u | (uint32_t(i & 3) << 4));
  } else {
    constexpr uint32_t kMask = ((1u << (2 * BITS)) - 1u) << 8;
    const int pos = 32 * BITS * sl + 2 * BITS * i, m = pos >> 5, sh = pos & 31;
    uint32_t v;
    if (sh + 2 * BITS > 32) v = __funnelshift_r(w[m], w[(m + 1) % (2 * BITS)], sh - 8);
    else if (sh >= 8) v = w[m] >> (sh - 8);
    else v = w[m] << (8 - sh);
    return (v & kMask) | base;
  }
}

// The projection that owns global row tile `row` (static indexing of the parameter block: a
// chain of selects, no local copy).
__device__ __forceinline__ PersistSeg segment_of_row(const PersistParams& p, int row) {
  PersistSeg sd = p.seg[0];
#pragma unroll
  for (int i = 1; i < kPMaxSeg; ++i)
    if (i < p.nsegs && row >= p.seg[i].row0) sd = p.seg[i];
  return sd;
}

// First tile of block b when the tile list is cut into gridDim.x ranges of equal cost
// (cost of a tile = its token columns).
__device__ __forceinline__ int persist_first_tile(const PersistParams& p, long long b, long long nb) {
  const long long total = (long long)p.n_tiles * p.W;
  const long long target = b * total / nb;
  long long r = target / p.W;
  const long long rem = target - r * p.W;
  long long j = (rem + p.NT - 1) / p.NT;
  if (j >= p.m_tiles) { ++r; j = 0; }
  return int(r * p.m_tiles + j);
}

// MODE (separate instantiations, so that a plain launch runs exactly the loop it always ran):
//   kModePlain     palettes shared by groups of output rows, looked up through the pair table;
//   kModeResidual  the same, and every tile ends with low-rank residual k-blocks;
//   kModeKGrouped  one palette per (128 input columns, output row): `lut` of the one segment is
//                  lut_k [K / 128][N][2^BITS]. A pair table per palette cannot pay off for 128
//                  weights, so a lookup warp keeps the palettes of its 32 rows for the k-blocks
//                  it has in flight in a private shared-memory ring (cp.async, requested together
//                  with the codes) and reads every weight with one 16-bit load; the rest of the
//                  pipeline does not know the difference.
constexpr int kModePlain = 0, kModeResidual = 1, kModeKGrouped = 2;

// The 2 * BITS bits of field i (0..15) of local slab sl (0, 1): two codes, the lower one first.
template <int BITS>
__device__ __forceinline__ uint32_t slab_field(const uint32_t (&w)[2 * BITS], int sl, int i) {
  constexpr uint32_t kMask = (1u << (2 * BITS)) - 1u;
  const int pos = 32 * BITS * sl + 2 * BITS * i, m = pos >> 5, sh = pos & 31;
  if (sh + 2 * BITS > 32) return __funnelshift_r(w[m], w[(m + 1) % (2 * BITS)], sh) & kMask;
  return (w[m] >> sh) & kMask;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

// PAIR: the grid is launched as clusters of two CTAs that work as one MMA unit (cta_group::2) on
// two row tiles of one token tile: the pair's leader issues MMAs of 256 weight rows (half the
// issue cost per row — the issuing thread, not the tensor pipe, bounds the one-CTA form) and each
// CTA fetches only HALF of the activation tile (half the L2 -> shared-memory traffic). Everything
// a CTA does for its own row tile — codes, lookups, its tensor memory, its epilogue — is as
// before. The schedule is computed on a virtual grid of pairs over pairs of row tiles; CTA r of
// a pair serves row tile 2 j + r. No multicast load: each CTA's bulk load lands in its own
// shared memory and reports its bytes to the leader's barrier.
template <typename T, int BITS, int MODE, bool PAIR>
__global__ void __launch_bounds__(kPThreads, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap xmap,
                          const __grid_constant__ CUtensorMap tmap, const PersistParams p) {
  constexpr bool RES = MODE == kModeResidual, KG = MODE == kModeKGrouped;
  // Ring depth of both operands. A pair's stages hold half an activation tile each, and its
  // stage round trip crosses to the other CTA and back, so it runs twice as many: eight operand
  // stages of 32 columns fill the tensor memory next to the 256-column accumulator.
  constexpr int NS = PAIR ? 2 * kPStages : kPStages;
  static_assert(kPACol + 32 * NS <= kTmemCols, "operand stages must fit beside the accumulator");
  const uint32_t crank = PAIR ? tc::cluster_ctarank() : 0u;      // 0: the pair's leader
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = smem_u32(smem);
  const uint32_t bar_full = base, bar_done = base + 64, bar_dfull = base + 128,
                 bar_dempty = base + 144;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 264);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 268);

  int nl = kTileRows / p.gs;
  if (nl < 1) nl = 1;
  const uint32_t tbl_addr = (base + kCtrlBytes + 0xFFFFu) & ~0xFFFFu;
  uint8_t* tbl_ptr = smem + (tbl_addr - base);
  // bytes of one activation stage in THIS CTA (a pair splits the tile's tokens between its CTAs)
  const uint32_t stage_bytes = uint32_t(PAIR ? p.NT / 2 : p.NT) * 128u;
  // below the table: control block, the epilogue's two staging slices, one activation stage;
  // above it: three more
  uint16_t* stage_out = reinterpret_cast<uint16_t*>(smem + kCtrlBytes);   // 2 x [token][128 rows]
  const uint32_t xlow = (base + kCtrlBytes + 2u * kPStageTokens * 256u + 1023u) & ~1023u;
  const uint32_t xhigh = tbl_addr + kTableBytes;
  constexpr int kLow = PAIR ? 2 : 1;       // stages that fit below the table
  auto xstage = [&](int s) {
    return s < kLow ? xlow + uint32_t(s) * stage_bytes : xhigh + uint32_t(s - kLow) * stage_bytes;
  };
  const bool fits = xhigh + (NS - kLow) * stage_bytes <= base + p.smem_bytes &&
                    xlow + kLow * stage_bytes <= tbl_addr;

  // The block's work is a list of segments (tile, k-blocks [c0, c1)). Plain mode: the whole
  // tiles of a cost-balanced contiguous range. Split mode: first the block's k-range of a cut
  // tile (if it has one), then `full` whole tiles.
  const int G = p.G;           // k-blocks of codes
  const int Gx = RES ? p.G + p.E : p.G;    // k-blocks of a tile, the residual's included
  const int bid = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);        // block (or pair) of the schedule
  const int nblk = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
  int t0, ntile, has_cut = 0, cut_tile = 0, cut_c0 = 0, cut_c1 = 0, cut_part = 0;
  if (p.split) {
    t0 = bid * p.full;
    ntile = p.full;
    if (bid < p.left * p.split) {
      has_cut = 1;
      cut_part = bid % p.split;
      cut_tile = nblk * p.full + bid / p.split;
      cut_c0 = (Gx * cut_part) / p.split;
      cut_c1 = (Gx * (cut_part + 1)) / p.split;
    }
  } else {
    t0 = persist_first_tile(p, bid, nblk);
    ntile = persist_first_tile(p, bid + 1, nblk) - t0;
  }
  const int nseg = ntile + has_cut;
  const int iters = ntile * Gx + (cut_c1 - cut_c0);
  // segment s of this block
  auto seg_tile = [&](int sg) { return (has_cut && sg == 0) ? cut_tile : t0 + sg - has_cut; };
  auto seg_c0 = [&](int sg) { return (has_cut && sg == 0) ? cut_c0 : 0; };
  auto seg_c1 = [&](int sg) { return (has_cut && sg == 0) ? cut_c1 : Gx; };
  // row tile of a scheduled tile (a pair schedules pairs of row tiles), and the slot of a cut
  // tile in the workspace and the ticket array
  auto tile_row = [&](int tile) { return PAIR ? 2 * (tile / p.m_tiles) + int(crank) : tile / p.m_tiles; };
  auto cut_slot = [&](int tile) { return PAIR ? 2 * (tile - nblk * p.full) + int(crank) : tile - nblk * p.full; };

  asm volatile("griddepcontrol.launch_dependents;");

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      // four lookup warps (of each CTA of a pair) + the TMA producer's expect_tx (and the bytes)
      tc::mbar_init(bar_full + 8 * s, PAIR ? 9 : 5);
      tc::mbar_init(bar_done + 8 * s, 1);    // tcgen05.commit of the k-block that used the stage
    }
    tc::mbar_init(bar_dfull, 1);              // tcgen05.commit: the tile's last MMA
    tc::mbar_init(bar_dempty, PAIR ? 2 * kPEpiWarps : kPEpiWarps);    // the epilogue warps have read the accumulator
    *abort_flag = fits ? 0 : 1;
    if (!fits) atomicCAS(&g_gemm_status, tc::kStatusOk, tc::kStatusWaitLoad);
    tc::mbar_init_fence();
  }
  if (warp == kLookupWarps) {
    if constexpr (PAIR) tc::tmem_alloc_pair(base + 264, kTmemCols);
    else tc::tmem_alloc(base + 264, kTmemCols);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  tc::fence_before_sync();
  if constexpr (PAIR) tc::cluster_sync();      // both CTAs' barriers exist before anyone signals across
  else __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp < kLookupWarps) {
    // ---- lookup warps ---------------------------------------------------------------------------
    const int q = warp & 3, grp = warp >> 2;
    // this warp's k-blocks are the iterations grp, grp + 2, ... of the block's flat sequence of
    // k-blocks (segment after segment; every segment has at least two k-blocks, so both groups
    // work in every segment); `load` runs kRing of them ahead of `use`
    struct Cursor { int s, c, c1, row; const uint8_t* base; };
    auto enter = [&](Cursor& cu, int over) {
      if (cu.s < nseg) {
        cu.c = seg_c0(cu.s) + over;
        cu.c1 = seg_c1(cu.s);
        cu.row = tile_row(seg_tile(cu.s));
        const PersistSeg sd = segment_of_row(p, cu.row);
        cu.base = sd.packed + size_t(cu.row - sd.row0) * G * (1024 * BITS);
      }
    };
    auto advance = [&](Cursor& cu) {
      cu.c += 2;
      while (cu.s < nseg && cu.c >= cu.c1) {
        const int over = cu.c - cu.c1;
        ++cu.s;
        enter(cu, over);
      }
    };
    auto code_ptr = [&](const Cursor& cu) -> const uint8_t* {
      return cu.base + size_t(cu.c) * (1024 * BITS) + lane * 32;
    };
    Cursor ld = {0, 0, 0, 0, p.seg[0].packed}, use = {0, 0, 0, 0, p.seg[0].packed};
    enter(ld, grp - 2);
    advance(ld);
    enter(use, grp - 2);
    advance(use);
    // K-grouped: the palettes of this warp's 32 rows for k-block `cu` go to slot u of the warp's
    // ring (where the pair tables of the other modes live); one commit group per slot and
    // iteration, issued or not, so that the group count tells which slot has landed.
    constexpr int kPal = 1 << BITS;
    constexpr uint32_t kPalSlot = 1024;          // 32 rows x 16 entries x 2 bytes at 4 bits
    const uint32_t pal_ring = tbl_addr + uint32_t(warp) * (kRing * kPalSlot);
    auto load_palette = [&](int u, const Cursor& cu, bool on) {
      if (on) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.seg[0].lut) +
                             ((size_t(cu.c >> 1) * p.kg_N + size_t(cu.row) * kTileRows + 32 * q) * kPal) * 2;
        for (int i = lane; i < 4 * kPal; i += 32)      // 64 * kPal bytes in 16-byte pieces
          cp_async16(pal_ring + uint32_t(u) * kPalSlot + uint32_t(i) * 16u, src + size_t(i) * 16);
      }
      cp_async_commit();
    };
    uint32_t w[kRing][2 * BITS];
#pragma unroll
    for (int u = 0; u < kRing; ++u) {
#pragma unroll
      for (int i = 0; i < 2 * BITS; ++i) w[u][i] = 0u;
      const bool on = ld.s < nseg;
      const bool codes = on && (!RES || ld.c < G);      // a residual k-block has no codes to fetch
      load_slab_pair<BITS>(w[u], codes ? code_ptr(ld) : p.seg[0].packed, q, codes ? 1u : 0u);
      if (KG) load_palette(u, ld, on);
      if (on) advance(ld);
    }
    int table_row = -1, table_seg = -1;
    uint32_t lane_base = 0;
    for (int it = grp; it < iters; it += 2 * kRing) {
#pragma unroll
      for (int u = 0; u < kRing; ++u) {
        if (it + 2 * u < iters) {     // warp-uniform
          if (!KG && use.s != table_seg) {
            // a new segment: all eight lookup warps pass here once per segment (block-uniform),
            // and rebuild the pair table together when the row tile has changed
            const int row = use.row;
            if (row != table_row) {
              asm volatile("bar.sync 1, %0;" ::"r"(kLookupWarps * 32) : "memory");
              const PersistSeg sd = segment_of_row(p, row);
              build_tables(tbl_ptr, sd.lut, BITS, sd.n_groups, (row - sd.row0) * kTileRows, p.gs, nl,
                           kLookupWarps * 32);
              asm volatile("bar.sync 1, %0;" ::"r"(kLookupWarps * 32) : "memory");
              uint32_t token;
              asm volatile("mov.u32 %0, 0;" : "=r"(token));
              lane_base = tbl_addr + lane * 4 + token;
              table_row = row;
            }
            table_seg = use.s;
          }
          const int i = it + 2 * u;
          const int stage = i % NS;
          if (i >= NS)        // the k-block that last used this operand stage has been consumed
            tc::mbar_wait(bar_done + 8 * stage, uint32_t(i / NS - 1) & 1u, abort_flag,
                          &g_gemm_status, tc::kStatusWaitEmpty, p.wait_cycles);
          tc::fence_after_sync();
          const bool residual = RES && use.c >= G;
          if (RES && residual) {
            // 64 columns of the tile's resA rows as they are. Register 4 kt + i of the store is
            // 32-bit column 8 kt + 2 (lane & 3) + (i & 1) of row (lane >> 2) + 8 (i >> 1): four
            // consecutive 16-bit values of each of the lane's two rows per 16-column block.
            const PersistSeg sd = segment_of_row(p, use.row);
            const int kk = (use.c - G) * kChunkK + 4 * (lane & 3);
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
              const int n = (use.row - sd.row0) * kTileRows + 32 * q + 16 * sl + (lane >> 2);
              const uint16_t* ra = sd.resA + size_t(n) * sd.res_rank + kk;
              const uint16_t* rb = ra + size_t(8) * sd.res_rank;
              uint32_t r[16];
#pragma unroll
              for (int kt = 0; kt < 4; ++kt) {
                uint2 lo = make_uint2(0u, 0u), hi = make_uint2(0u, 0u);
                if (sd.resA != nullptr && kk + 16 * kt < sd.res_rank) {   // the rank is a multiple of 8
                  lo = __ldg(reinterpret_cast<const uint2*>(ra + 16 * kt));
                  hi = __ldg(reinterpret_cast<const uint2*>(rb + 16 * kt));
                }
                r[4 * kt + 0] = lo.x; r[4 * kt + 1] = lo.y;
                r[4 * kt + 2] = hi.x; r[4 * kt + 3] = hi.y;
              }
              tc::tmem_st_16x256b_x4(tmem + (uint32_t(32 * q + 16 * sl) << 16) + kPACol + 32u * stage, r);
            }
          }
          if (KG) {
            cp_async_wait<kRing - 1>();      // the group of this slot (and every older one) has landed
            __syncwarp();
            const uint32_t slot = pal_ring + uint32_t(u) * kPalSlot;
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
              const uint32_t row_lo = slot + uint32_t(16 * sl + (lane >> 2)) * (2 * kPal);
              const uint32_t row_hi = row_lo + 8u * (2 * kPal);
              uint32_t r[16];
#pragma unroll
              for (int kt = 0; kt < 4; ++kt) {
                uint32_t v[4];
#pragma unroll
                for (int f = 0; f < 4; ++f) {   // fields (g, k 0-1), (g+8, k 0-1), (g, k 2-3), (g+8, k 2-3)
                  const uint32_t pair = slab_field<BITS>(w[u], sl, 4 * kt + f);
                  const uint32_t rowb = (f & 1) ? row_hi : row_lo;
                  v[f] = lds16(rowb + 2u * (pair & (kPal - 1))) | (lds16(rowb + 2u * (pair >> BITS)) << 16);
                }
                r[4 * kt + 0] = v[0]; r[4 * kt + 1] = v[2]; r[4 * kt + 2] = v[1]; r[4 * kt + 3] = v[3];
              }
              tc::tmem_st_16x256b_x4(tmem + (uint32_t(32 * q + 16 * sl) << 16) + kPACol + 32u * stage, r);
            }
          }
#pragma unroll
          for (int sl = 0; sl < 2; ++sl) {
            if (residual || KG) continue;
            const int rowslab = 2 * q + sl;
            const int pal = nl == 1 ? 0 : (nl == 2 ? rowslab >> 2 : rowslab >> 1);
            const uint32_t tb = lane_base + uint32_t(pal >> 1) * kTableBytes + uint32_t(pal & 1) * 128u;
            uint32_t r[16];
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              // slab fields (row g, k 0-1), (g+8, k 0-1), (g, k 2-3), (g+8, k 2-3); the store
              // shape wants (g, c), (g, c+1), (g+8, c), (g+8, c+1): fields 0, 2, 1, 3
              r[4 * kt + 0] = lds32(slab_field_addr<BITS>(w[u], sl, 4 * kt + 0, tb));
              r[4 * kt + 1] = lds32(slab_field_addr<BITS>(w[u], sl, 4 * kt + 2, tb));
              r[4 * kt + 2] = lds32(slab_field_addr<BITS>(w[u], sl, 4 * kt + 1, tb));
              r[4 * kt + 3] = lds32(slab_field_addr<BITS>(w[u], sl, 4 * kt + 3, tb));
            }
            tc::tmem_st_16x256b_x4(tmem + (uint32_t(32 * q + 16 * sl) << 16) + kPACol + 32u * stage, r);
          }
          {
            const bool on = ld.s < nseg;
            const bool codes = on && (!RES || ld.c < G);
            load_slab_pair<BITS>(w[u], codes ? code_ptr(ld) : p.seg[0].packed, q, codes ? 1u : 0u);
            if (KG) load_palette(u, ld, on);
            if (RES && on && !codes) {
              // a residual k-block four iterations ahead: pull this lane's resA rows into L1 now
              const PersistSeg sd = segment_of_row(p, ld.row);
              if (sd.resA != nullptr) {
                const int kk = (ld.c - G) * kChunkK;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int n = (ld.row - sd.row0) * kTileRows + 32 * q + 8 * j + (lane >> 2);
                  if (kk < sd.res_rank)
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(sd.resA + size_t(n) * sd.res_rank + kk));
                }
              }
            }
            if (on) advance(ld);
          }
          tc::wait_st();
          tc::fence_before_sync();
          if (lane == 0) {
            if constexpr (PAIR) tc::mbar_arrive_cluster((bar_full + 8 * stage) & tc::kPeerBitMask);
            else tc::mbar_arrive(bar_full + 8 * stage);
          }
          advance(use);
        }
      }
    }
  } else if (warp == kLookupWarps) {
    // ---- TMA producer ---------------------------------------------------------------------------
    int i = 0;
    for (int sg = 0; sg < nseg; ++sg) {
      int m0 = (seg_tile(sg) % p.m_tiles) * p.NT;
      if constexpr (PAIR) {
        // the pair's second CTA holds the upper half of the tile's tokens: nt / 2 rows on, where
        // nt is the width the MMA will run this tile at
        int nt = p.M - m0;
        nt = nt >= p.NT ? p.NT : ((nt + 31) & ~31);
        m0 += int(crank) * (nt >> 1);
      }
      const int c_hi = seg_c1(sg);
      const int tcol = RES ? segment_of_row(p, tile_row(seg_tile(sg))).t_col0 - G * kChunkK : 0;
      for (int c = seg_c0(sg); c < c_hi; ++c, ++i) {
        const int xs = i % NS;
        if (i >= NS)
          tc::mbar_wait(bar_done + 8 * xs, uint32_t(i / NS - 1) & 1u, abort_flag,
                        &g_gemm_status, tc::kStatusWaitEmpty, p.wait_cycles);
        if (lane == 0 && !*abort_flag) {
          if constexpr (PAIR) {
            // both halves report their bytes to the leader's barrier; the leader expects them
            if (crank == 0) tc::mbar_expect_tx(bar_full + 8 * xs, 2u * stage_bytes);
            const uint32_t lead = (bar_full + 8 * xs) & tc::kPeerBitMask;
            if (!RES || c < G) tma_load_2d_pair(xstage(xs), &xmap, lead, c * kChunkK, m0);
            else tma_load_2d_pair(xstage(xs), &tmap, lead, tcol + c * kChunkK, m0);
          } else {
            tc::mbar_expect_tx(bar_full + 8 * xs, stage_bytes);
            if (!RES || c < G) tma_load_2d(xstage(xs), &xmap, bar_full + 8 * xs, c * kChunkK, m0);
            else tma_load_2d(xstage(xs), &tmap, bar_full + 8 * xs, tcol + c * kChunkK, m0);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == kLookupWarps + 1) {
    // ---- MMA issuer -----------------------------------------------------------------------------
    constexpr uint32_t kFmt = DType<T>::id == B200LUT_BF16 ? 1u : 0u;
    const uint64_t dtemplate = tc::smem_desc(0u, 16u, 1024u, 2u);
    uint32_t xlo[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) xlo[s] = uint32_t(dtemplate) + (xstage(s) >> 4);
    const uint32_t xhi = uint32_t(dtemplate >> 32);
    if (lane == 0 && crank == 0) {               // of a pair only the leader issues
      int t = -1, c = 0, c_first = 0, c_end = 0;   // segment, k-block, the segment's k range
      uint32_t idesc = 0;
      const uint32_t d0 = tmem;
      uint32_t phase = 0;            // (i / ring size) & 1
      for (int i0 = 0; i0 < iters; i0 += NS, phase ^= 1u) {
#pragma unroll
        for (int u = 0; u < NS; ++u) {
          if (i0 + u < iters) {
            if (c == c_end) {        // a new segment: the accumulator must have been drained
              ++t;
              c = c_first = seg_c0(t);
              c_end = seg_c1(t);
              const int m0 = (seg_tile(t) % p.m_tiles) * p.NT;
              int nt = p.M - m0;                          // the row's last tile may be narrower
              nt = nt >= p.NT ? p.NT : ((nt + 31) & ~31);
              idesc = tc::instr_desc(kFmt, PAIR ? 256 : 128, uint32_t(nt));
              if (t >= 1)
                tc::mbar_wait(bar_dempty, uint32_t(t - 1) & 1u, abort_flag, &g_gemm_status,
                              tc::kStatusWaitDone, p.wait_cycles);
            }
            tc::mbar_wait(bar_full + 8 * u, phase, abort_flag, &g_gemm_status, tc::kStatusWaitFull, p.wait_cycles);
            tc::fence_after_sync();
            if constexpr (PAIR) {
              tc::mma_ts_kblock_pair(d0, tmem + kPACol + 32u * uint32_t(u), xlo[u], xhi, idesc,
                                     c == c_first ? 0u : 1u);
              tc::mma_commit_pair(bar_done + 8 * u);          // frees the stage in both CTAs
              if (++c == c_end) tc::mma_commit_pair(bar_dfull);
            } else {
              tc::mma_ts_kblock(d0, tmem + kPACol + 32u * uint32_t(u), xlo[u], xhi, idesc,
                                c == c_first ? 0u : 1u);   // a segment's first k-block overwrites
              tc::mma_commit(bar_done + 8 * u);
              if (++c == c_end) tc::mma_commit(bar_dfull);
            }
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue warps: TMEM -> bias -> one rounding -> staged slice -> global -----------------
    const int q = warp & 3;                              // TMEM lane quarter this warp may read
    const int h = (warp - (kLookupWarps + 2)) >> 2;      // column half of the tile it drains
    const int et = threadIdx.x - (kLookupWarps + 2 + 4 * h) * 32;   // 0..127 inside the half
    uint16_t* stg = stage_out + h * (kPStageTokens * kTileRows);
    volatile int* cut_flag = reinterpret_cast<volatile int*>(smem + 272);
    for (int t = 0; t < nseg; ++t) {
      const int tile = seg_tile(t);
      const bool cut = has_cut && t == 0;
      const PersistSeg sd = segment_of_row(p, tile_row(tile));
      const int n0 = (tile_row(tile) - sd.row0) * kTileRows, m0 = (tile % p.m_tiles) * p.NT;
      int nt = p.M - m0;
      nt = nt >= p.NT ? p.NT : ((nt + 31) & ~31);
      const int half = nt >> 1, col0 = h * half;
      const int n = n0 + 32 * q + lane;
      const float b0 = sd.bias ? DType<T>::to_float(sd.bias[n]) : 0.f;
      tc::mbar_wait(bar_dfull, uint32_t(t) & 1u, abort_flag, &g_gemm_status, tc::kStatusWaitDone, p.wait_cycles);
      tc::fence_after_sync();
      const uint32_t d0 = tmem + (uint32_t(32 * q) << 16) + uint32_t(col0);
      float* wt = cut ? p.ws + size_t(cut_slot(tile)) * p.split * (256 * kTileRows) : nullptr;
      // slices of up to 48 tokens: three loads in flight, one wait, staging, 16-byte stores
      for (int s0 = 0; s0 < half; s0 += kPStageTokens) {
        const int sn = half - s0 < kPStageTokens ? half - s0 : kPStageTokens;
        uint32_t r[3][16];
#pragma unroll
        for (int ch = 0; ch < 3; ++ch)
          if (16 * ch < sn) tc::tmem_ld_32x32b_x16(d0 + uint32_t(s0 + 16 * ch), r[ch]);
        tc::wait_ld();
        if (s0 + sn >= half) {   // the accumulator is free as soon as it has been read
          tc::fence_before_sync();
          if (lane == 0) {
            if constexpr (PAIR) tc::mbar_arrive_cluster(bar_dempty & tc::kPeerBitMask);
            else tc::mbar_arrive(bar_dempty);
          }
        }
        if (cut) {   // this block's k-range of a cut tile: raw fp32 sums to its workspace slot
          float* mine = wt + size_t(cut_part) * (256 * kTileRows) + 32 * q + lane;
#pragma unroll
          for (int ch = 0; ch < 3; ++ch)
            if (16 * ch < sn)
#pragma unroll
              for (int j = 0; j < 16; ++j)
                __stcg(mine + size_t(col0 + s0 + 16 * ch + j) * kTileRows, __uint_as_float(r[ch][j]));
          continue;
        }
        if (p.acc_out) {   // first stream of two: raw fp32 sums, no bias, no rounding
          float* dst = p.acc_out + size_t(m0 + col0 + s0) * p.ld_acc + n0 + 32 * q + lane;
#pragma unroll
          for (int ch = 0; ch < 3; ++ch)
            if (16 * ch < sn)
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (m0 + col0 + s0 + 16 * ch + j < p.M)
                  __stcg(dst + size_t(16 * ch + j) * p.ld_acc, __uint_as_float(r[ch][j]));
          continue;
        }
        if (p.acc_in) {    // second stream: the first stream's sums join before bias and rounding
          const float* src = p.acc_in + size_t(m0 + col0 + s0) * p.ld_acc + n0 + 32 * q + lane;
#pragma unroll
          for (int ch = 0; ch < 3; ++ch)
            if (16 * ch < sn)
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float a = m0 + col0 + s0 + 16 * ch + j < p.M
                                    ? __ldcg(src + size_t(16 * ch + j) * p.ld_acc) : 0.f;
                r[ch][j] = __float_as_uint(a + __uint_as_float(r[ch][j]));
              }
        }
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          if (16 * ch < sn) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float v = __uint_as_float(r[ch][j]) + b0;
              const int tok = s0 + 16 * ch + j;
              if (sd.out_aligned) stg[(16 * ch + j) * kTileRows + 32 * q + lane] = DType<T>::from_float(v);
              else if (m0 + col0 + tok < p.M)
                sd.out[size_t(m0 + col0 + tok) * sd.ldo + n] = DType<T>::from_float(v);
            }
          }
        }
        if (sd.out_aligned) {
          asm volatile("bar.sync %0, 128;" ::"r"(2 + h) : "memory");
          const uint4* src = reinterpret_cast<const uint4*>(stg);
          for (int idx = et; idx < sn * 16; idx += 128) {
            const int r_ = col0 + s0 + (idx >> 4), c = idx & 15;
            if (m0 + r_ < p.M)
              *reinterpret_cast<uint4*>(sd.out + size_t(m0 + r_) * sd.ldo + n0 + 8 * c) = src[idx];
          }
          asm volatile("bar.sync %0, 128;" ::"r"(2 + h) : "memory");   // the slice is reused
        }
      }
      if (cut) {
        // All `split` blocks of the tile store their partial tiles, meet on a counter (bounded
        // wait: the grid is one block per SM and every block does its cut piece first), and
        // each finishes the token pairs g with g % split == its part: the partial sums are
        // added in part (= ascending k) order, bias, one rounding, element stores.
        int* cnt = p.tickets + 2 * cut_slot(tile);
        __threadfence();
        asm volatile("bar.sync 4, %0;" ::"r"(kPEpiWarps * 32) : "memory");
        if (warp == kLookupWarps + 2 && lane == 0) {
          atomicAdd(cnt, 1);
          int ok = 1;
          const long long w0 = clock64();
          while (*reinterpret_cast<volatile int*>(cnt) < p.split) {
            if (*abort_flag || clock64() - w0 > p.wait_cycles) { ok = 0; break; }
          }
          if (!ok) { *abort_flag = 1; atomicCAS(&g_gemm_status, tc::kStatusOk, tc::kStatusWaitDone); }
          *cut_flag = ok;
        }
        asm volatile("bar.sync 4, %0;" ::"r"(kPEpiWarps * 32) : "memory");
        if (*cut_flag) {
          __threadfence();
          // pairs of tokens, dealt round-robin over the parts and the two column halves; all
          // `split` partial values of a pair are requested before the first is used
          const int ngrp = nt >> 1;
          for (int g2 = cut_part + p.split * h; g2 < ngrp; g2 += 2 * p.split) {
            float v[8][2];
#pragma unroll
            for (int ci = 0; ci < 8; ++ci) {
              if (ci < p.split) {
                const float* src = wt + (size_t(ci) * 256 + 2 * g2) * kTileRows + 32 * q + lane;
                v[ci][0] = __ldcg(src);
                v[ci][1] = __ldcg(src + kTileRows);
              }
            }
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int ci = 0; ci < 8; ++ci)
              if (ci < p.split) { a0 += v[ci][0]; a1 += v[ci][1]; }
            const int tok = m0 + 2 * g2;
            if (tok < p.M) sd.out[size_t(tok) * sd.ldo + n] = DType<T>::from_float(a0 + b0);
            if (tok + 1 < p.M) sd.out[size_t(tok + 1) * sd.ldo + n] = DType<T>::from_float(a1 + b0);
          }
        }
        asm volatile("bar.sync 4, %0;" ::"r"(kPEpiWarps * 32) : "memory");
        if (warp == kLookupWarps + 2 && lane == 0) {
          __threadfence();
          if (atomicAdd(cnt + 1, 1) == p.split - 1) { cnt[0] = 0; cnt[1] = 0; }   // ready for the next launch
        }
      }
    }
  }
  tc::fence_before_sync();
  if constexpr (PAIR) tc::cluster_sync();      // neither CTA's memories are in use by the other any more
  else __syncthreads();
  if (warp == kLookupWarps) {
    tc::fence_after_sync();
    if constexpr (PAIR) tc::tmem_dealloc_pair(tmem, kTmemCols);
    else tc::tmem_dealloc(tmem, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

template <typename T>
int launch(const CUtensorMap& map, const GemmParams& p, int n_tiles, bool pdl, cudaStream_t stream) {
  auto kern = gemm_tc_kernel<T>;
  static bool configured[64] = {false};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(kMaxDynSmem)));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(n_tiles * p.m_tiles), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(na);
  B200LUT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, map, p));
  return B200LUT_OK;
}

// Split planning for `tiles` output tiles of G k-blocks on `sms` blocks: whole rounds of tiles
// stay whole; each tile of the partly filled last round is cut along K into `split` parts.
struct SplitPlan { int split, full, left; size_t bytes; };
constexpr size_t kTicketBytes = 4096;   // counters first, at a fixed place: they outlive a shape change

SplitPlan plan_split(long long tiles, int G, int sms) {
  SplitPlan sp = {0, 0, 0, 0};
  if (tiles <= 0 || sms <= 0) return sp;
  const long long full = tiles / sms, left = tiles - full * sms;
  if (left == 0 || left > (long long)(kTicketBytes / 8)) return sp;
  long long S = sms / left;
  if (S > 8) S = 8;
  while (S >= 2 && G < 2 * S) --S;       // every part keeps at least two k-blocks
  if (S < 2) return sp;
  sp.split = int(S); sp.full = int(full); sp.left = int(left);
  sp.bytes = kTicketBytes + size_t(left) * size_t(S) * 256 * kTileRows * sizeof(float);
  return sp;
}

template <typename T, int BITS, int MODE, bool PAIR>
int launch_persistent(const CUtensorMap& map, const CUtensorMap& tmap, const PersistParams& p,
                      int grid, bool pdl, cudaStream_t stream) {
  auto kern = gemm_tc_persistent_kernel<T, BITS, MODE, PAIR>;
  static bool configured[64] = {false};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(kMaxDynSmem)));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(grid), 1, 1);
  cfg.blockDim = dim3(kPThreads, 1, 1);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (PAIR) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(na);
  B200LUT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, map, tmap, p));
  return B200LUT_OK;
}

// Whether a launch of `rows` row tiles and M activation rows runs as CTA pairs: whole 256-token
// tiles are worth it, the row tiles must pair up, and so must the SMs.
bool pairs_serve(int rows, int M, int sms) { return M >= kPMaxNT && rows >= 2 && rows % 2 == 0 && sms % 2 == 0; }

int encode_x_map(CUtensorMap* map, const void* x, int64_t ldx, int M, int K, int dtype, int NT) {
  EncodeTiledFn enc = encode_fn();
  B200LUT_REQUIRE(enc != nullptr, B200LUT_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(M)};
  const cuuint64_t strides[1] = {cuuint64_t(ldx) * 2};
  const cuuint32_t box[2] = {cuuint32_t(kChunkK), cuuint32_t(NT)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dtype == B200LUT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         2, const_cast<void*>(x), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200LUT_REQUIRE(r == CUDA_SUCCESS, B200LUT_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", int(r));
  return B200LUT_OK;
}

}  // namespace

}  // namespace b200lut

using namespace b200lut;


// Device-side status of the library's kernels on the current device (0 = none). A
// non-zero value means a bounded wait ran out inside a kernel (tensor-core pipeline codes,
// or 0x7000 + rank for an exchange wait on that rank's push); cleared by this call.
extern "C" int b200lut_device_status(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
  const int e = b200lut::exchange_status_take();
  const int g = b200lut::embed_status_take();
  return v != 0 ? v : (e != 0 ? e : g);
}

namespace {
// Host side of the persistent kernel: `nseg` projections that share x (one code stream each,
// the same code width and group size, at most two palettes per 128-row tile) as one launch
// whose row tiles are the concatenation of the projections' row tiles.
int persistent_gemm(const void* x, int64_t ldx, int M, int K, int dtype, const b200lut_segment* segs,
                    int nseg, bool pdl, void* workspace, size_t workspace_bytes,
                    void* stream, float* acc_out = nullptr, const float* acc_in = nullptr,
                    long long ld_acc = 0, int kg_rows = 0, bool cta_pairs = false) {
  PersistParams pp = {};
  pp.acc_out = acc_out; pp.acc_in = acc_in; pp.ld_acc = ld_acc;
  const bool kgrouped = kg_rows > 0;     // segs[0].lut is lut_k [K / 128][kg_rows][2^bits]
  pp.kg_N = kg_rows;
  int rows = 0, extra = 0;
  const uint16_t* t_base = nullptr;
  long long t_ld = 0;
  for (int i = 0; i < nseg; ++i) {
    const b200lut_segment& s = segs[i];
    PersistSeg& d = pp.seg[i];
    d.packed = static_cast<const uint8_t*>(s.packed);
    d.lut = static_cast<const uint16_t*>(s.lut);
    d.bias = static_cast<const uint16_t*>(s.bias);
    d.out = static_cast<uint16_t*>(s.out);
    d.ldo = s.ldo;
    d.out_aligned = (aligned16(s.out) && s.ldo % 8 == 0) ? 1 : 0;
    d.row0 = rows;
    d.n_groups = s.n_groups;
    rows += s.N / kTileRows;
    if (s.res_rank > 0) {
      // all residual projections of a launch read column blocks of ONE t matrix
      if (!t_base) { t_base = static_cast<const uint16_t*>(s.res_t); t_ld = s.res_ldt; }
      const long long col0 = static_cast<const uint16_t*>(s.res_t) - t_base;
      const int blocks = (s.res_rank + kChunkK - 1) / kChunkK;
      B200LUT_REQUIRE(s.res_ldt == t_ld && col0 >= 0 && col0 % 8 == 0 &&
                          col0 + (long long)blocks * kChunkK <= t_ld,
                      B200LUT_ERR_INVALID,
                      "the res_t blocks of a merged prefill launch must lie in one [M, res_ldt] matrix, "
                      "16-byte aligned and 64 * ceil(rank / 64) columns wide each (segment %d)", i);
      d.resA = static_cast<const uint16_t*>(s.resA);
      d.res_rank = s.res_rank;
      d.t_col0 = int(col0);
      if (blocks > extra) extra = blocks;
    }
  }
  pp.E = extra;
  pp.nsegs = nseg;
  const b200lut_segment& s = segs[0];
  pp.M = M; pp.K = K; pp.G = K / kChunkK;
  pp.gs = s.group_size;
  int sms = 148;
  {
    int dev = 0;
    B200LUT_CUDA_OK(cudaGetDevice(&dev));
    B200LUT_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  // CTA pairs (cta_group::2), on request (B200LUT_FLAG_CTA_PAIRS): the plain lookup mode only.
  // Measured 1.47x SLOWER than one CTA per tile at every prefill shape (bit-identical results),
  // so the library never picks it by itself.
  const bool pair = cta_pairs && pairs_serve(rows, M, sms) && !acc_out && !acc_in && !extra && !kgrouped;
  pp.NT = M >= kPMaxNT ? kPMaxNT : ((M + 31) / 32) * 32;
  pp.m_tiles = (M + pp.NT - 1) / pp.NT;
  pp.n_tiles = pair ? rows / 2 : rows;      // a pair schedules pairs of row tiles
  pp.W = (pp.m_tiles - 1) * pp.NT + ((M - (pp.m_tiles - 1) * pp.NT + 31) / 32) * 32;
  pp.smem_bytes = uint32_t(kMaxDynSmem);
  // Waits inside the kernel give up after ~10 ms. A profiler that replays the kernel with
  // heavy instrumentation can stretch a healthy wait beyond that; B200LUT_WAIT_MS raises the
  // bound for such runs (capped at one second).
  pp.wait_cycles = tc::kWaitCycles;
  if (const char* e = getenv("B200LUT_WAIT_MS")) {
    long ms = atol(e);
    if (ms < 1) ms = 1;
    if (ms > 1000) ms = 1000;
    pp.wait_cycles = (long long)ms * 2000000ll;
  }
  CUtensorMap pmap, tmap;
  const int box_rows = pair ? pp.NT / 2 : pp.NT;     // each CTA of a pair fetches half of the tile's tokens
  if (int rc = encode_x_map(&pmap, x, ldx, M, K, dtype, box_rows)) return rc;
  if (extra) {
    if (int rc = encode_x_map(&tmap, t_base, t_ld, M, int(t_ld), dtype, box_rows)) return rc;
  } else {
    tmap = pmap;
  }
  // the schedule's blocks: CTAs, or pairs of them over pairs of row tiles
  const int units = pair ? sms / 2 : sms;
  const long long tiles = (long long)pp.n_tiles * pp.m_tiles;
  int grid = int(tiles < units ? tiles : units);
  SplitPlan sp = plan_split(tiles, pp.G + pp.E, units);
  if (pair) sp.bytes = sp.split ? kTicketBytes + 2 * (sp.bytes - kTicketBytes) : 0;   // a slot per CTA
  if (pair && sp.left > int(kTicketBytes / 16)) sp.split = 0;
  if (sp.split && workspace && workspace_bytes >= sp.bytes && aligned16(workspace) &&
      !acc_out && !acc_in) {
    pp.split = sp.split; pp.full = sp.full; pp.left = sp.left;
    pp.tickets = static_cast<int*>(workspace);
    pp.ws = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kTicketBytes);
    grid = units;
  }
  if (pair) grid *= 2;
#define B200LUT_PERSIST_AS(B, MODE, PAIR)                                                                 \
  (dtype == B200LUT_BF16                                                                                   \
       ? launch_persistent<__nv_bfloat16, B, MODE, PAIR>(pmap, tmap, pp, grid, pdl, cudaStream_t(stream)) \
       : launch_persistent<__half, B, MODE, PAIR>(pmap, tmap, pp, grid, pdl, cudaStream_t(stream)))
#define B200LUT_PERSIST(B)                                                         \
  (kgrouped ? B200LUT_PERSIST_AS(B, kModeKGrouped, false)                          \
            : (extra ? B200LUT_PERSIST_AS(B, kModeResidual, false)                 \
                     : (pair ? B200LUT_PERSIST_AS(B, kModePlain, true) : B200LUT_PERSIST_AS(B, kModePlain, false))))
  switch (s.bits) {
    case 4: return B200LUT_PERSIST(4);
    case 3: return B200LUT_PERSIST(3);
    case 2: return B200LUT_PERSIST(2);
    default: return B200LUT_PERSIST(1);
  }
#undef B200LUT_PERSIST
#undef B200LUT_PERSIST_AS
}

// the checks every projection of a prefill GEMM passes, whichever kernel serves it
int check_gemm_segment(const b200lut_segment& s) {
  B200LUT_REQUIRE(s.packed && s.lut && s.out, B200LUT_ERR_INVALID, "null codes, palette or output");
  B200LUT_REQUIRE(s.N > 0 && s.N % kTileRows == 0 && s.ldo >= s.N, B200LUT_ERR_INVALID,
                  "N must be a positive multiple of 128 and ldo >= N (N=%d)", s.N);
  B200LUT_REQUIRE(s.res_rank >= 0 && s.res_rank <= 1024 && s.res_rank % 8 == 0, B200LUT_ERR_UNSUPPORTED,
                  "the rank of a fused low-rank residual is a multiple of 8, at most 1024 (got %d)",
                  s.res_rank);
  B200LUT_REQUIRE(s.res_rank == 0 || (s.resA && s.res_t && aligned16(s.resA) && aligned16(s.res_t) &&
                                      s.res_ldt % 8 == 0),
                  B200LUT_ERR_INVALID,
                  "a fused low-rank residual needs resA and res_t (from b200lut_residual_project_rows), "
                  "16-byte aligned, and a res_ldt that is a multiple of 8");
  B200LUT_REQUIRE(s.group_size >= 32 && s.n_groups >= 1 &&
                      ((s.group_size < 128 && (s.group_size & (s.group_size - 1)) == 0) ||
                       s.group_size % 128 == 0),
                  B200LUT_ERR_UNSUPPORTED, "group_size %d not served (32, 64 or a multiple of 128)",
                  s.group_size);
  return B200LUT_OK;
}

}  // namespace

extern "C" size_t b200lut_gemm_workspace_bytes(int M, int N, int K) {
  if (M < 1 || N < kTileRows || K < 2 * kChunkK) return 0;
  const int nt = M >= kPMaxNT ? kPMaxNT : ((M + 31) / 32) * 32;
  const long long tiles = (long long)(N / kTileRows) * ((M + nt - 1) / nt);
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // what either form of the launch may ask for: single CTAs, or (on request) CTA pairs over pairs of row tiles
  size_t need = plan_split(tiles, K / kChunkK, sms).bytes;
  if (pairs_serve(N / kTileRows, M, sms)) {
    const SplitPlan sp = plan_split(tiles / 2, K / kChunkK, sms / 2);
    const size_t pair_need = sp.split ? kTicketBytes + 2 * (sp.bytes - kTicketBytes) : 0;
    if (pair_need > need) need = pair_need;
  }
  return need;
}

extern "C" int b200lut_gemm(const void* x, int64_t ldx, int M, int K, int dtype,
                            const b200lut_segment* seg, int epilogue, int flags, void* stream) {
  return b200lut_gemm_ws(x, ldx, M, K, dtype, seg, epilogue, flags, nullptr, 0, stream);
}

extern "C" int b200lut_gemm_multi(const void* x, int64_t ldx, int M, int K, int dtype,
                                  const b200lut_segment* segs, int nseg, int flags,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  B200LUT_REQUIRE(x && segs, B200LUT_ERR_INVALID, "null x or segment table");
  B200LUT_REQUIRE(nseg >= 1 && nseg <= kPMaxSeg, B200LUT_ERR_UNSUPPORTED,
                  "1 <= nseg <= %d projections per launch, got %d", kPMaxSeg, nseg);
  B200LUT_REQUIRE(M >= 1, B200LUT_ERR_INVALID, "M must be >= 1, got %d", M);
  B200LUT_REQUIRE(K >= 2 * kChunkK && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a multiple of 64 and at least 128, got %d", K);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, B200LUT_ERR_ALIGN,
                  "x must be 16-byte aligned with a row stride that is a multiple of 8 and >= K");
  for (int i = 0; i < nseg; ++i) {
    const b200lut_segment& s = segs[i];
    if (int rc = check_gemm_segment(s)) return rc;
    B200LUT_REQUIRE(!s.packed2, B200LUT_ERR_UNSUPPORTED,
                    "a merged prefill launch serves one code stream per projection");
    B200LUT_REQUIRE(s.bits >= 1 && s.bits <= 4 && s.bits == segs[0].bits &&
                        s.group_size == segs[0].group_size && s.group_size >= 64,
                    B200LUT_ERR_UNSUPPORTED,
                    "the projections of a merged prefill launch share one code width (1..4) and "
                    "one group size >= 64 (segment %d: %d bits, group %d)", i, s.bits, s.group_size);
    B200LUT_REQUIRE(aligned16(s.packed), B200LUT_ERR_ALIGN, "code buffers must be 16-byte aligned");
  }
  return persistent_gemm(x, ldx, M, K, dtype, segs, nseg, (flags & 1) != 0, workspace,
                         workspace_bytes, stream, nullptr, nullptr, 0, 0,
                         (flags & B200LUT_FLAG_CTA_PAIRS) != 0);
}

extern "C" int b200lut_gemm_kgrouped(const void* x, int64_t ldx, int M, int K, int dtype,
                                     const void* packed, const void* lut_k, const void* bias, int N,
                                     int bits, void* out, int64_t ldo, int flags, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  B200LUT_REQUIRE(x && packed && lut_k && out, B200LUT_ERR_INVALID, "null x, codes, palettes or output");
  B200LUT_REQUIRE(M >= 1, B200LUT_ERR_INVALID, "M must be >= 1, got %d", M);
  B200LUT_REQUIRE(K >= 128 && K % 128 == 0, B200LUT_ERR_INVALID,
                  "K must be a positive multiple of 128 (one palette per 128 input columns), got %d", K);
  B200LUT_REQUIRE(N > 0 && N % kTileRows == 0 && ldo >= N, B200LUT_ERR_INVALID,
                  "N must be a positive multiple of 128 and ldo >= N (N=%d)", N);
  B200LUT_REQUIRE(bits >= 1 && bits <= 4, B200LUT_ERR_INVALID, "code width must be 1..4, got %d", bits);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(x) && aligned16(packed) && aligned16(lut_k) && ldx % 8 == 0 && ldx >= K,
                  B200LUT_ERR_ALIGN,
                  "x, codes and palettes must be 16-byte aligned, the x row stride a multiple of 8 and >= K");
  b200lut_segment s = {};
  s.packed = packed;
  s.lut = lut_k;
  s.bias = bias;
  s.out = out;
  s.ldo = ldo;
  s.N = N;
  s.group_size = kTileRows;     // not used by the K-grouped lookup
  s.n_groups = N / kTileRows;
  s.bits = bits;
  return persistent_gemm(x, ldx, M, K, dtype, &s, 1, (flags & 1) != 0, workspace, workspace_bytes, stream,
                         nullptr, nullptr, 0, N, (flags & B200LUT_FLAG_CTA_PAIRS) != 0);
}

extern "C" size_t b200lut_gemm_two_stream_bytes(int M, int N) {
  if (M < 1 || N < 1) return 0;
  return size_t(M) * size_t(N) * sizeof(float);
}

extern "C" int b200lut_gemm_two_stream(const void* x, int64_t ldx, int M, int K, int dtype,
                                       const b200lut_segment* seg, int flags, void* scratch,
                                       size_t scratch_bytes, void* stream) {
  B200LUT_REQUIRE(x && seg, B200LUT_ERR_INVALID, "null x or segment");
  B200LUT_REQUIRE(M >= 1, B200LUT_ERR_INVALID, "M must be >= 1, got %d", M);
  B200LUT_REQUIRE(K >= 2 * kChunkK && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a multiple of 64 and at least 128, got %d", K);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, B200LUT_ERR_ALIGN,
                  "x must be 16-byte aligned with a row stride that is a multiple of 8 and >= K");
  const b200lut_segment& s = *seg;
  if (int rc = check_gemm_segment(s)) return rc;
  B200LUT_REQUIRE(s.packed2 && s.lut2, B200LUT_ERR_INVALID, "the second stream (packed2 / lut2) is missing");
  B200LUT_REQUIRE(s.bits >= 1 && s.bits <= 4 && s.bits2 >= 1 && s.bits2 <= 4 && s.group_size >= 64,
                  B200LUT_ERR_UNSUPPORTED,
                  "code widths must be 1..4 and the group size >= 64 (got %d / %d bits, group %d)",
                  s.bits, s.bits2, s.group_size);
  B200LUT_REQUIRE(aligned16(s.packed) && aligned16(s.packed2), B200LUT_ERR_ALIGN,
                  "code buffers must be 16-byte aligned");
  B200LUT_REQUIRE(scratch && scratch_bytes >= b200lut_gemm_two_stream_bytes(M, s.N) && aligned16(scratch),
                  B200LUT_ERR_WORKSPACE, "the two-stream GEMM needs a 16-byte aligned scratch of %zu bytes",
                  b200lut_gemm_two_stream_bytes(M, s.N));
  float* acc = static_cast<float*>(scratch);
  b200lut_segment first = s, second = s;
  first.packed2 = first.lut2 = nullptr; first.bits2 = 0; first.bias = nullptr;
  first.res_rank = 0; first.resA = nullptr; first.res_t = nullptr;   // the second launch carries it
  second.packed = s.packed2; second.lut = s.lut2; second.bits = s.bits2;
  second.packed2 = second.lut2 = nullptr; second.bits2 = 0;
  const bool pdl = (flags & 1) != 0;
  if (int rc = persistent_gemm(x, ldx, M, K, dtype, &first, 1, pdl, nullptr, 0, stream, acc,
                               nullptr, s.N))
    return rc;
  return persistent_gemm(x, ldx, M, K, dtype, &second, 1, pdl, nullptr, 0, stream, nullptr, acc,
                         s.N);
}

extern "C" int b200lut_gemm_ws(const void* x, int64_t ldx, int M, int K, int dtype,
                               const b200lut_segment* seg, int epilogue, int flags,
                               void* workspace, size_t workspace_bytes, void* stream) {
  B200LUT_REQUIRE(x && seg, B200LUT_ERR_INVALID, "null x or segment");
  B200LUT_REQUIRE(M >= 1, B200LUT_ERR_INVALID, "M must be >= 1, got %d", M);
  B200LUT_REQUIRE(K > 0 && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a positive multiple of 64, got %d", K);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(epilogue == B200LUT_EPI_NONE || epilogue == B200LUT_EPI_SILU_MUL,
                  B200LUT_ERR_INVALID, "unknown epilogue %d", epilogue);
  B200LUT_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, B200LUT_ERR_ALIGN,
                  "x must be 16-byte aligned with a row stride that is a multiple of 8 and >= K");
  const b200lut_segment& s = *seg;
  if (int rc = check_gemm_segment(s)) return rc;
  const bool silu = epilogue == B200LUT_EPI_SILU_MUL;
  const bool two = s.packed2 != nullptr;
  B200LUT_REQUIRE(!silu || two, B200LUT_ERR_INVALID,
                  "the silu-mul epilogue needs the up projection in packed2 / lut2");
  B200LUT_REQUIRE(s.bits >= 1 && s.bits <= 4 && (!two || (s.lut2 && s.bits2 >= 1 && s.bits2 <= 4)),
                  B200LUT_ERR_INVALID, "code widths must be 1..4 (got %d / %d)", s.bits, s.bits2);
  B200LUT_REQUIRE(aligned16(s.packed) && (!two || aligned16(s.packed2)), B200LUT_ERR_ALIGN,
                  "code buffers must be 16-byte aligned");

  const bool pdl = (flags & 1) != 0;
  const int nl = s.group_size >= 128 ? 1 : 128 / s.group_size;
  if (!two && nl <= 2 && K / kChunkK >= 2) {
    return persistent_gemm(x, ldx, M, K, dtype, seg, 1, pdl, workspace, workspace_bytes, stream,
                           nullptr, nullptr, 0, 0, (flags & B200LUT_FLAG_CTA_PAIRS) != 0);
  }

  // what is left for the one-tile kernel: two code streams, the fused gate/up form, four
  // palettes per tile — it looks 4-bit codes up
  B200LUT_REQUIRE(s.res_rank == 0, B200LUT_ERR_UNSUPPORTED,
                  "the low-rank residual is fused into one-stream prefill launches with at most two "
                  "palettes per tile, and into b200lut_gemm_two_stream");
  B200LUT_REQUIRE(s.bits == 4 && (!two || s.bits2 == 4), B200LUT_ERR_UNSUPPORTED,
                  "two-stream, gate/up-fused and group-size-32 prefill GEMMs serve 4-bit codes "
                  "(got %d / %d)", s.bits, s.bits2);
  GemmParams p = {};
  p.packed[0] = static_cast<const uint8_t*>(s.packed);
  p.lut[0] = static_cast<const uint16_t*>(s.lut);
  p.bias[0] = static_cast<const uint16_t*>(s.bias);
  p.packed[1] = static_cast<const uint8_t*>(s.packed2);
  p.lut[1] = static_cast<const uint16_t*>(s.lut2);
  p.out = static_cast<uint16_t*>(s.out);
  p.ldo = s.ldo;
  p.out_aligned = (aligned16(s.out) && s.ldo % 8 == 0) ? 1 : 0;
  p.M = M; p.N = s.N; p.K = K; p.G = K / kChunkK;
  p.gs = s.group_size; p.n_groups = s.n_groups;
  p.npass = two ? 2 : 1;
  p.plane[0] = 0;
  p.plane[1] = silu ? 1 : 0;
  p.silu = silu ? 1 : 0;
  const int nt_max = silu ? 128 : 256;
  int NT = ((M + 31) / 32) * 32;           // even halves of whole 16-column epilogue chunks
  if (NT > nt_max) NT = nt_max;
  p.NT = NT;
  p.m_tiles = (M + NT - 1) / NT;
  const int tables = (p.npass * nl + 1) / 2;
  // Activation stages fill what the control block and the 64 KB-aligned tables leave
  // free. The dynamic window starts 1 KB into the shared window on sm_100; the kernel
  // recomputes the stage count from its real base and drains with a status if fewer
  // than two fit.
  {
    const size_t stage = size_t(NT) * 128, win0 = 1024, tbl0 = 65536;
    const size_t below = (tbl0 - ((win0 + kCtrlBytes + 1023) & ~size_t(1023))) / stage;
    const size_t top = win0 + kMaxDynSmem, tbl1 = tbl0 + size_t(tables) * kTableBytes;
    const size_t above = top > tbl1 ? (top - tbl1) / stage : 0;
    B200LUT_REQUIRE(tbl1 <= top && below + above >= 2, B200LUT_ERR_UNSUPPORTED,
                    "group_size %d with %d code stream(s) leaves no room for two activation "
                    "stages in shared memory", s.group_size, p.npass);
  }
  p.smem_bytes = uint32_t(kMaxDynSmem);

  CUtensorMap map;
  if (int rc = encode_x_map(&map, x, ldx, M, K, dtype, NT)) return rc;
  if (dtype == B200LUT_BF16)
    return launch<__nv_bfloat16>(map, p, s.N / kTileRows, pdl, cudaStream_t(stream));
  return launch<__half>(map, p, s.N / kTileRows, pdl, cudaStream_t(stream));
}
