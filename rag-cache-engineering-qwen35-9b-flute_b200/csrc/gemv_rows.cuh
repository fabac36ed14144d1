// Row-range decode GEMV (M <= 8, 4-bit codes, one code stream) for sm_100a.
// Included by gemv.cu (shares the segment structs, the epilogue pieces and the exchange).
//
// Replaces, for the shapes it serves, the tile x K-split form of the kernel above (reference:
// src/flute_extended/src/kernel_gemv.cu:92-253, kernel_gemv_splitk.cu:135-409,
// kernel_gemv_multi.cu:101-334, kernel_gemv_mlp.cu:92-450).
//
// Why a second form. At 4 bits one 1 KB plane of a chunk holds 32 output rows x 64 k, so 32
// rows over ALL of K are a stream of 1 KB pieces, 4 KB apart. A block here owns a contiguous
// range of such 32-row units over the whole of K: nothing is folded across blocks, a launch
// of N rows fills min(N / 32, SMs) SMs whatever N / 128 is, and the work per block is even
// to within one unit. (K is only split, across a thread-block cluster folded through
// distributed shared memory, when a launch has fewer units than half the SMs.)
//
// One block of 16 warps per SM. Per warp: a ring of four 1 KB pieces in registers (one 256-bit
// load per lane each); slot j of the next round is requested as soon as slot j of the current one
// has been looked up. A piece is 2 slabs x 4 k-steps: 32 pair-table lookups (one byte permute +
// one ld.shared each, the 16 of a slab issued back to back) feed 8 mma.m16n8k16. Warps take
// k-chunks round-robin, so when the block's K range is 64 chunks (K = 4096) a warp's slot j is
// always its chunk j and its activation fragments stay in registers for the whole launch;
// otherwise they are read per piece from the rows staged in shared memory. Every n8 column of the
// accumulator carries batch row (column mod M'), M' = M rounded up to 1, 2, 4, 8, so no select
// is spent on columns. The warps' sums meet in shared memory in warp order (deterministic), then
// bias / residual / SiLU*mul and ONE rounding.
//
// Prologue, in the order that matters under programmatic dependent launch: every warp requests
// its first round of codes; then half of the warps fetch the palettes and write the pair tables
// while the other half waits for the previous kernel and stages the activation rows, so the two
// memory round trips overlap each other and the code fetch.
//
// The pair table sits at a fixed offset of the block's shared window (kRowsTableAbs), so a lookup
// address is the byte permute plus an immediate offset in the load; no 64 KB alignment is needed.
//
// What the staging half can do on the way (b200lut_input / b200lut_exchange): multiply the rows
// into silu(x) * x_mul, rotate them (one fold for the launch, or one per segment — the blocks are
// then dealt to the segments so that none crosses one), wait for the peers of a column-parallel
// exchange (flags, or the rows themselves as the arrival signal).
#pragma once

namespace b200lut {
namespace {

constexpr int kRowsWarps = 16;
constexpr int kRowsThreads = kRowsWarps * 32;
constexpr int kRowsRing = 4;            // 1 KB pieces in flight per warp
constexpr int kUnitRows = 32;           // output rows of one 1 KB plane at 4 bits
constexpr int kRowsMaxPlanes = 16;      // planes (units x streams) per block: one lane each
constexpr int kRowsMaxSlots = 4;        // palettes a block can hold (two 64 KB tables)
constexpr uint32_t kRowsTableAbs = 2048;   // offset of the first pair table inside the block's shared window
constexpr uint32_t kRowsWindowMask = 0x3FFFFu;   // a block's shared window is smaller than 256 KB
constexpr int kRowsStatusBadWindow = 0x5000;
constexpr int kRowsMaxFhtSegs = 8;

struct RowsParams {
  const uint16_t* x;
  const uint16_t* x2;      // non-null: the activation is silu(x) * x2 (both [M, ldx])
  long long ldx;
  int M, Mp, K, G, nseg, epilogue;
  int units_total;         // 32-row units (pairs of units under the SiLU*mul epilogue)
  int row_blocks, split, ntables, red_planes;
  // incr (M' = 8, K of exactly 64 chunks): the warps' sums of a unit are folded as soon as its
  // last plane is done (one block barrier per plane) out of 2 (4 under SiLU*mul) rotating plane
  // buffers that take the place of the staged rows (which live in registers by then), instead of
  // all planes after the loop out of a buffer of their own: eight rows of K = 4096 then fit next
  // to four palettes, and a block's planes are bounded only by the lanes that hold their metadata
  int incr;
  uint32_t xs_abs, red_abs, part_abs;    // offsets inside the block's shared window
  uint32_t meta_abs;                     // RowsUnitMeta[units of the block]
  // Hadamard rotation of the activation rows inside the launch (rot_signs != null): descending
  // power-of-two segments of K, as b200lut_fht runs them; fht_abs: fp32 scratch of one segment
  const float* rot_signs;
  const float* awq_scale;
  // per_seg: every segment has its own fold (seg_signs[i] null = that segment's input is used
  // as it is); blocks then never cross a segment: segment i owns blocks [blk0[i], blk0[i + 1])
  int per_seg;
  int blk0[kMaxSeg + 1];
  const float* seg_signs[kMaxSeg];
  const float* seg_awq[kMaxSeg];
  uint32_t fht_abs;
  int fht_nseg;
  int fht_off[kRowsMaxFhtSegs], fht_len[kRowsMaxFhtSegs], fht_stages[kRowsMaxFhtSegs];
  float fht_inv[kRowsMaxFhtSegs];
  int* status;
  // Inside a persistent plan (gemv_rows_plan_kernel; all null / zero in a plain launch): the
  // completion counter of the job that produces the activation rows and the value it has when
  // every block of that job has stored its rows; this job's own counter; the plan's abort word.
  const int* dep_done;
  int dep_target;
  int xreg;                // which instantiation serves the job (see XREG below)
  int* done;
  int* abort_word;
  SegDev seg[kMaxSeg];
  ExchangeDev ex;
};

__device__ __forceinline__ uint32_t lds32_tbl(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+2048];" : "=r"(v) : "r"(addr));
  return v;
}
static_assert(kRowsTableAbs == 2048, "the immediate in lds32_tbl is the table address");

// Activation fragments out of shared memory. Not volatile (the scheduler may hoist it across
// lookups); ordered against the staging barrier by the token every address carries.
__device__ __forceinline__ void lds128(uint32_t (&r)[4], uint32_t addr) {
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
      : "r"(addr));
}

__device__ __forceinline__ unsigned long long shfl_u64(unsigned long long v, int src) {
  return __shfl_sync(0xffffffffu, v, src);
}

// out = silu(g) * u on 8 packed 16-bit values, fp32 inside, one rounding
template <typename T>
__device__ __forceinline__ uint4 silu_mul8(uint4 g, uint4 u) {
  uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w}, o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float g0 = DType<T>::to_float(uint16_t(gw[i] & 0xFFFFu)), g1 = DType<T>::to_float(uint16_t(gw[i] >> 16));
    const float u0 = DType<T>::to_float(uint16_t(uw[i] & 0xFFFFu)), u1 = DType<T>::to_float(uint16_t(uw[i] >> 16));
    const uint32_t lo = DType<T>::from_float(g0 / (1.f + __expf(-g0)) * u0);
    const uint32_t hi = DType<T>::from_float(g1 / (1.f + __expf(-g1)) * u1);
    o[i] = lo | (hi << 16);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Exchange without flags ("the data is its own flag"): the rows a waiting launch stages live in a
// buffer that its last block refills with 0xFFFF after use (no finite bf16 / f16 value, nor the
// NaN a conversion produces, has that pattern), and the producers on every rank store their
// elements into it with plain 2-byte stores, which are atomic. A 16-byte piece is therefore
// complete exactly when none of its eight elements is 0xFFFF: the waiting launch polls the piece
// itself (bounded; on expiry status 0x7000 + the rank that owns the missing column, and the launch
// carries on). The producer needs no system-wide fence and no flag stores.
__device__ __forceinline__ bool has_sentinel(const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  bool any = false;
#pragma unroll
  for (int i = 0; i < 4; ++i) any = any || (w[i] & 0xFFFFu) == 0xFFFFu || (w[i] >> 16) == 0xFFFFu;
  return any;
}
__device__ __forceinline__ uint4 load_rows_piece(const RowsParams& p, const uint16_t* ptr, int col) {
  uint4 v = __ldcg(reinterpret_cast<const uint4*>(ptr));
  if (p.ex.wait && p.ex.sentinel && has_sentinel(v)) {
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
      asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "l"(ptr)
                   : "memory");
      if (!has_sentinel(v)) break;
      if ((i & 15u) == 0u) {
        if (*reinterpret_cast<volatile int*>(p.ex.status) != 0) break;
        if (clock64() - t0 > p.ex.wait_cycles) {
          atomicExch(p.ex.status, 0x7000 + col / (p.K / p.ex.world));
          break;
        }
      }
    }
  }
  return v;
}

// 4096-point Hadamard butterfly (no scaling) by 256 threads, 16 values per thread, the stages
// in the order len = 1, 2, 4, ... 2048 — the order of b200lut_fht, so every value goes through
// the same additions and subtractions and has the same bits. Stages 0-3, 4-7 and 8-11 each run
// on 16 registers; between them the values are regrouped through `buf` (4096 floats; value i
// lives in the 16-byte piece (i >> 2) ^ ((i >> 5) & 3), which keeps the 16-byte stores of the
// first pass and the strided reads of the last one free of bank conflicts).
// In: v[j] = value 16 t + j. Out: v[j] = value 256 j + t. `bar` = barrier id of the 256 threads.
__device__ __forceinline__ void fht16_regs(float (&v)[16]) {
#pragma unroll
  for (int len = 1; len < 16; len <<= 1)
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (!(i & len)) {
        const float a = v[i], b = v[i + len];
        v[i] = a + b;
        v[i + len] = a - b;
      }
}

__device__ __forceinline__ int fht4096_slot(int i) { return (((i >> 2) ^ ((i >> 5) & 3)) << 2) | (i & 3); }

__device__ __forceinline__ void fht4096_regs(float (&v)[16], float* buf, int t) {
  fht16_regs(v);                                                   // stages 0-3
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<float4*>(buf + fht4096_slot(16 * t + 4 * c)) =
        make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  asm volatile("bar.sync 1, 256;" ::: "memory");
  const int mid = ((t >> 4) << 8) | (t & 15);
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = buf[fht4096_slot(mid + 16 * j)];
  fht16_regs(v);                                                   // stages 4-7
#pragma unroll
  for (int j = 0; j < 16; ++j) buf[fht4096_slot(mid + 16 * j)] = v[j];
  asm volatile("bar.sync 1, 256;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = buf[fht4096_slot(256 * j + t)];
  fht16_regs(v);                                                   // stages 8-11
  asm volatile("bar.sync 1, 256;" ::: "memory");                   // buf may be written again
}

// The 32-row units [u0, u1) of row block rb. Plain: `row_blocks` even ranges of the launch's
// units. Per-segment folds: even ranges of the units of the segment that owns the block.
__host__ __device__ inline void rows_block_units(int per_seg, const int* blk0, const SegDev* seg, int nseg,
                                                 int units_total, int row_blocks, int rb, int* u0, int* u1,
                                                 int* owner) {
  if (!per_seg) {
    // floor(units * rb / blocks); a 32-bit division whenever the product allows (same quotient)
    const unsigned long long a = (unsigned long long)(units_total) * unsigned(rb);
    const unsigned long long b = a + (unsigned long long)(units_total);
    *u0 = (b >> 32) == 0 ? int(uint32_t(a) / uint32_t(row_blocks)) : int(a / unsigned(row_blocks));
    *u1 = (b >> 32) == 0 ? int(uint32_t(b) / uint32_t(row_blocks)) : int(b / unsigned(row_blocks));
    *owner = 0;
    return;
  }
  int s = 0;
  for (int i = 1; i < nseg; ++i)
    if (rb >= blk0[i]) s = i;
  const int ub = 4 * seg[s].tile_begin;
  const int ue = s + 1 < nseg ? 4 * seg[s + 1].tile_begin : units_total;
  const int nb = blk0[s + 1] - blk0[s], lb = rb - blk0[s];
  *u0 = ub + int((long long)(ue - ub) * lb / nb);
  *u1 = ub + int((long long)(ue - ub) * (lb + 1) / nb);
  *owner = s;
}

// What the epilogue needs to know about one 32-row unit of the block, worked out once in the
// prologue (segment search and parameter loads off the tail of the launch) and kept in shared memory.
struct RowsUnitMeta {
  uint16_t* out;            // &out[0][n0] of the unit (gate segment under SiLU*mul)
  const uint16_t* bias;     // &bias[n0] or null
  const uint16_t* bias2;    // up segment's, under SiLU*mul
  long long ldo;
  int seg;                  // segment index (gate segment under SiLU*mul)
  int n0;                   // first row of the unit inside its segment
  int has_res;              // bit 0: segment has a fused residual; bit 1: the up segment has one
  int pad;
};

// Bias, residual, SiLU*mul, the one rounding, the store (and its mirrors on the peers).
template <typename T>
__device__ __forceinline__ void rows_finish(const RowsParams& p, const RowsUnitMeta& um, bool silu,
                                            int m, int row, float a, float b) {
  if (um.has_res & 1) a += residual_dot<T>(p.seg[um.seg], m, um.n0 + row);
  if (um.bias) a += DType<T>::to_float(um.bias[row]);
  float v = a;
  if (silu) {
    if (um.has_res & 2) b += residual_dot<T>(p.seg[um.seg + 1], m, um.n0 + row);
    if (um.bias2) b += DType<T>::to_float(um.bias2[row]);
    v = a / (1.f + __expf(-a)) * b;
  }
  uint16_t* dst = um.out + size_t(m) * um.ldo + row;
  const uint16_t bits16 = DType<T>::from_float(v);
  *dst = bits16;
  if (p.ex.push) {
    for (int q = 0; q < p.ex.world; ++q)
      if (q != p.ex.rank)
        *reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(dst) + p.ex.delta[q]) = bits16;
  }
}

// One 1 KB piece: 2 slabs x 4 k-steps. The 16 lookups of a slab are issued before its four
// mma so that the shared-memory latency is paid once per slab, not once per k-step.
template <typename T>
__device__ __forceinline__ void rows_item(float (&acc)[2][4], const uint32_t (&w)[8], uint32_t base,
                                          const uint32_t (&xb)[2][4]) {
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    uint32_t a[4][4];
#pragma unroll
    for (int kt = 0; kt < 4; ++kt)
#pragma unroll
      for (int f = 0; f < 4; ++f)
        a[kt][f] = lds32_tbl(__byte_perm(w[4 * s + kt], base, 0x7604u | (uint32_t(f) << 4)));
#pragma unroll
    for (int kt = 0; kt < 4; ++kt)
      mma16816<T>(acc[s], a[kt], xb[kt >> 1][2 * (kt & 1)], xb[kt >> 1][2 * (kt & 1) + 1]);
  }
}

// The same with the activation fragments fetched from the staged rows in shared memory.
template <typename T>
__device__ __forceinline__ void rows_item_smem(float (&acc)[2][4], const uint32_t (&w)[8],
                                               uint32_t base, uint32_t xs_addr) {
  uint32_t xb[2][4];
  lds128(xb[0], xs_addr);
  lds128(xb[1], xs_addr + 16);
  rows_item<T>(acc, w, base, xb);
}

// XREG: the block's K range is exactly kRowsWarps * kRowsRing chunks, so a warp's ring slot j is
// always its chunk j and the warp keeps the activation fragments of its chunks in registers.
// `bid` of `nblk`: the block's place in the launch (its place among the job's blocks inside a plan).
template <typename T, bool XREG, bool PLAN>
__device__ __forceinline__ void rows_block(const RowsParams& p, uint8_t* smem, const int bid, const int nblk) {
  constexpr int NW = kRowsWarps, NT = kRowsThreads, R = kRowsRing;
  constexpr uint32_t kFull = 0xffffffffu;
  constexpr unsigned long long kHop = (unsigned long long)(NW) * 4096ull;   // a warp's next chunk
  // Shared-state-space addresses of this block: `win` is the start of its window (zero for a
  // plain launch, the block's slice of the cluster window otherwise), `low` where the dynamic
  // array starts inside it. Everything below sits at fixed offsets from `win`.
  const uint32_t smem_abs = smem_u32(smem);
  const uint32_t low = smem_abs & kRowsWindowMask, win = smem_abs - low;
  // Never seen; reported instead of trusted. A block in this state does no work but still meets
  // its cluster at the barriers below.
  const bool bad_window = low > kRowsTableAbs;
  if (bad_window && threadIdx.x == 0) atomicExch(p.status, kRowsStatusBadWindow);
  auto generic = [&](uint32_t off) { return smem + (off - low); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int split = p.split;
  const int rb = bid / split, sp = bid % split;
  const int c0 = (p.G * sp) / split, c1 = (p.G * (sp + 1)) / split;
  const int kc = c1 - c0;
  const bool silu = p.epilogue == B200LUT_EPI_SILU_MUL;
  const int ppu = silu ? 2 : 1;
  int u0, u1, owner;
  rows_block_units(p.per_seg, p.blk0, p.seg, p.nseg, p.units_total, p.row_blocks, rb, &u0, &u1, &owner);
  const float* rot_signs = p.per_seg ? p.seg_signs[owner] : p.rot_signs;
  const float* awq_scale = p.per_seg ? p.seg_awq[owner] : p.awq_scale;
  const int nplanes = bad_window ? 0 : (u1 - u0) * ppu;
  const int M = p.M, Mp = p.Mp;

  asm volatile("griddepcontrol.launch_dependents;");

  // ---- plane j of the block lives in lane j of every warp -----------------------------------
  unsigned long long my_ptr = 0, my_lut = 0;
  const int which = silu ? (lane & 1) : 0;
  int si = 0, lu = 0;
  if (lane < nplanes) {   // where the plane's codes start: all the first loads need
    const int u = u0 + lane / ppu;
    for (int s = 0; s < p.nseg; s += ppu)
      if ((u >> 2) >= p.seg[s].tile_begin) si = s;
    lu = u - 4 * p.seg[si].tile_begin;
    my_ptr = reinterpret_cast<unsigned long long>(
        p.seg[si + which].packed + (size_t(lu >> 2) * p.G + c0 + warp) * 4096 + size_t(lu & 3) * 1024);
  }


  // ---- rounds: up to R consecutive chunks of one plane. The first round is requested now,
  //      before anything else; afterwards slot j of the next round is requested as soon as
  //      slot j of the current one has been looked up. -------------------------------------------
  const int cnt = kc > warp ? (kc - warp + NW - 1) / NW : 0;    // this warp's chunks per plane
  const unsigned long long lane_off = (unsigned long long)(lane) * 32ull;
  uint32_t w[R][8];
  int cur_plane = 0, cur_k = 0;
  int cur_n = (cnt > 0 && nplanes > 0) ? (cnt < R ? cnt : R) : 0;
  {
    const uint8_t* first = reinterpret_cast<const uint8_t*>(shfl_u64(my_ptr, 0) + lane_off);
#pragma unroll
    for (int j = 0; j < R; ++j) {
#pragma unroll
      for (int i = 0; i < 8; ++i) w[j][i] = 0u;
      ldg_stream256_if(w[j], first + j * kHop, j < cur_n ? 1u : 0u);
    }
  }

  // ---- the plane's palette and what the epilogue needs to know about its unit ------------------
  if (lane < nplanes) {
    const SegDev& sg = p.seg[si + which];
    int grp = (lu * kUnitRows) / sg.gs;
    if (grp > sg.n_groups - 1) grp = sg.n_groups - 1;
    my_lut = reinterpret_cast<unsigned long long>(sg.lut + size_t(grp) * 16);
    if (warp == 0 && which == 0) {
      const SegDev& s0 = p.seg[si];
      RowsUnitMeta um;
      um.n0 = lu * kUnitRows;
      um.out = s0.out + um.n0;
      um.bias = s0.bias ? s0.bias + um.n0 : nullptr;
      um.bias2 = (silu && p.seg[si + 1].bias) ? p.seg[si + 1].bias + um.n0 : nullptr;
      um.ldo = s0.ldo;
      um.seg = si;
      um.has_res = (s0.res_rank ? 1 : 0) | ((silu && p.seg[si + 1].res_rank) ? 2 : 0);
      um.pad = 0;
      reinterpret_cast<RowsUnitMeta*>(generic(p.meta_abs))[lane / ppu] = um;
    }
  }

  // ---- palettes: one slot per run of planes that share a palette -------------------------------
  const unsigned long long prev_lut = __shfl_up_sync(kFull, my_lut, ppu);
  const bool change = lane < nplanes && (lane < ppu || prev_lut != my_lut);
  const uint32_t m0 = __ballot_sync(kFull, change && which == 0);
  const uint32_t m1 = __ballot_sync(kFull, change && which == 1);
  const uint32_t upto = (2u << lane) - 1u;
  const int my_slot = which ? __popc(m0) + __popc(m1 & upto) - 1 : __popc(m0 & upto) - 1;
  const int nslots = __popc(m0) + __popc(m1);

  // The lower half of the warps fetches the palettes and writes the pair tables while the upper
  // half waits for the producer of the activation rows and stages them: the two round trips
  // (palette entries from DRAM, activations from L2) run side by side.
  if (warp < NW / 2) {
    constexpr int NTB = NT / 2;   // threads that build
    uint32_t lutv[2] = {0u, 0u};
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int want = 2 * t + (lane >> 4);
      unsigned long long lp = 0;
#pragma unroll
      for (int s = 2 * t; s < 2 * t + 2; ++s) {
        const uint32_t owner = __ballot_sync(kFull, change && my_slot == s);
        const unsigned long long v = shfl_u64(my_lut, owner ? __ffs(owner) - 1 : 0);
        if (want == s) lp = v;
      }
      if (want < nslots) lutv[t] = uint32_t(__ldg(reinterpret_cast<const uint16_t*>(lp) + (lane & 15)));
    }
    // pair tables: entry e of slot s at table(s >> 1) + e * 256 + (s & 1) * 128 + 4 * lane
    if (!bad_window) {
      uint8_t* tbl = generic(kRowsTableAbs);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int nsl = nslots - 2 * t < 2 ? nslots - 2 * t : 2;
        if (nsl > 0) {   // block-uniform
#pragma unroll
          for (int k = 0; k < 4096 / NTB; ++k) {
            const int idx = threadIdx.x + k * NTB;
            if (idx < nsl * 2048) {   // warp-uniform
              const int q = idx & 7, e = (idx >> 3) & 255, sl = idx >> 11;
              const uint32_t lo = __shfl_sync(kFull, lutv[t], 16 * sl + (e & 15));
              const uint32_t hi = __shfl_sync(kFull, lutv[t], 16 * sl + (e >> 4));
              const uint32_t v = lo | (hi << 16);
              *reinterpret_cast<uint4*>(tbl + size_t(t) * kTableBytes + e * 256 + sl * 128 + q * 16) =
                  make_uint4(v, v, v, v);
            }
          }
        }
      }
    }
  } else {
    constexpr int NTS = NT / 2;   // threads that stage
    const int tid = int(threadIdx.x) - NTS;
    // the rotation's signs (and scales) do not depend on the previous kernel: pull their lines
    // into L1 while waiting for it
    if (rot_signs) {
      for (int i = tid * 32; i < p.K; i += NTS * 32) {
        asm volatile("prefetch.global.L1 [%0];" ::"l"(rot_signs + i));
        if (awq_scale) asm volatile("prefetch.global.L1 [%0];" ::"l"(awq_scale + i));
      }
    }
    // the dependency: the previous kernel of the stream, or the peers' pushes
    if (PLAN && p.dep_done) {
      // every block of the producing job has stored its rows and bumped the job's counter
      if (tid == 0) dep_poll(DepWait{2, p.dep_done, p.dep_target, p.abort_word, nullptr});
      asm volatile("bar.sync 1, %0;" ::"n"(NTS) : "memory");
    } else if (p.ex.wait && p.ex.sentinel) {
      // nothing to wait for up front: every staged piece is polled until it is complete
    } else if (p.ex.wait) {
      for (int i = tid; i < p.ex.world * p.ex.blocks; i += NTS) peer_poll(p.ex, i);
      asm volatile("bar.sync 1, %0;" ::"n"(NTS) : "memory");
    } else {
      asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    // activation rows of this block's K range into shared memory, B-fragment order:
    // element (chunk g, tig, kt, j) at g*128 + tig*32 + kt*8 + 2j bytes = x[64g + 16kt + 4tig + j]
    if (!bad_window && rot_signs) {
      // Rotated rows (the boundary fold of the reference's rotated artifacts, fused like its
      // gemv_fht_prologue, src/flute_extended/include/flute/gemv.cuh:305-351): per row and
      // segment, fp32 butterfly in shared memory in the stage order of b200lut_fht (same
      // expression tree, same bits), then signs, 1/sqrt(b) (and the AWQ scale on both sides),
      // ONE rounding to the activation dtype, written in B-fragment order. K is never split here.
      uint8_t* xs = generic(p.xs_abs);
      float* buf = reinterpret_cast<float*>(generic(p.fht_abs));
      for (int m = 0; m < Mp; ++m) {
        for (int sg = 0; sg < p.fht_nseg; ++sg) {
          const int off = p.fht_off[sg], n = p.fht_len[sg], stages = p.fht_stages[sg];
          const float inv = p.fht_inv[sg];
          if (n == 4096 || n == 8192) {
            // register form: one or two 4096-point transforms; for 8192 values the first half
            // waits in the upper part of the scratch (every thread reads back its own slots) and
            // the last stage (len = 4096) joins the two halves on the way out
            static_assert(NTS == 256, "fht4096_regs is written for 256 threads");
            const int halves = n >> 12;
            float v[16];
            for (int h = 0; h < halves; ++h) {
              uint4 raw[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
              const int i0 = 4096 * h + 16 * tid;
              if (m < M) {
                const size_t at = size_t(m) * p.ldx + size_t(off + i0);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                  raw[c] = load_rows_piece(p, p.x + at + 8 * c, off + i0 + 8 * c);
                  if (p.x2) raw[c] = silu_mul8<T>(raw[c], __ldcg(reinterpret_cast<const uint4*>(p.x2 + at + 8 * c)));
                }
              }
              const uint32_t wv[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float f = DType<T>::to_float(uint16_t(wv[j >> 1] >> (16 * (j & 1))));
                if (awq_scale) f = f * awq_scale[off + i0 + j];
                v[j] = f;
              }
              fht4096_regs(v, buf, tid);
              if (h + 1 < halves) {
#pragma unroll
                for (int j = 0; j < 16; ++j) buf[4096 + 256 * j + tid] = v[j];
              }
            }
            // value j of this thread is element 256 j + tid of the segment (and of its upper half):
            // its place in the staged rows moves by 512 bytes per j, its sign by 256 floats
            const int k0 = off + tid;
            uint8_t* dst0 = xs + (size_t(m) * kc + (k0 >> 6)) * 128 + (((k0 & 63) & 15) >> 2) * 32 +
                            ((k0 & 63) >> 4) * 8 + (k0 & 3) * 2;
            auto emit = [&](int j, int half, float val) {
              const int k = k0 + 4096 * half + 256 * j;
              float r = val * __ldg(rot_signs + k);
              r = r * inv;
              if (awq_scale) r = __fdiv_rn(r, __ldg(awq_scale + k));
              *reinterpret_cast<uint16_t*>(dst0 + size_t(half) * (64 * 128) + size_t(j) * 512) = DType<T>::from_float(r);
            };
            if (halves == 2) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float a = buf[4096 + 256 * j + tid], b = v[j];
                emit(j, 0, a + b);
                emit(j, 1, a - b);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) emit(j, 0, v[j]);
            }
            continue;
          }
          for (int i = tid * 8; i < n; i += NTS * 8) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < M) {
              const size_t at = size_t(m) * p.ldx + size_t(off + i);
              v = load_rows_piece(p, p.x + at, off + i);
              if (p.x2) v = silu_mul8<T>(v, __ldcg(reinterpret_cast<const uint4*>(p.x2 + at)));
            }
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float f = DType<T>::to_float(uint16_t(wv[j >> 1] >> (16 * (j & 1))));
              if (awq_scale) f = f * awq_scale[off + i + j];
              buf[i + j] = f;
            }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(NTS) : "memory");
          for (int st = 0; st < stages; ++st) {
            const int len = 1 << st;
            for (int i = tid; i < n / 2; i += NTS) {
              const int lo = ((i >> st) << (st + 1)) + (i & (len - 1));
              const float a = buf[lo], b = buf[lo + len];
              buf[lo] = a + b;
              buf[lo + len] = a - b;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NTS) : "memory");
          }
          for (int i = tid * 4; i < n; i += NTS * 4) {
            uint32_t o[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t pair = 0;
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int k = off + i + 2 * h + e;
                float r = buf[i + 2 * h + e] * rot_signs[k];
                r = r * inv;
                if (awq_scale) r = __fdiv_rn(r, awq_scale[k]);
                pair |= uint32_t(DType<T>::from_float(r)) << (16 * e);
              }
              o[h] = pair;
            }
            const int k = off + i, g = k >> 6, w64 = k & 63, kt = w64 >> 4, tg = (w64 & 15) >> 2;
            *reinterpret_cast<uint2*>(xs + (size_t(m) * kc + g) * 128 + tg * 32 + kt * 8) = make_uint2(o[0], o[1]);
          }
          asm volatile("bar.sync 1, %0;" ::"n"(NTS) : "memory");
        }
      }
    } else if (!bad_window) {
      uint8_t* xs = generic(p.xs_abs);
      const int per_row = kc * 8;   // 16-byte pieces of one row
      const int total = Mp * per_row;
#pragma unroll 8
      for (int idx = tid; idx < total; idx += NTS) {
        const int m = idx / per_row, pc = idx - m * per_row;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (m < M) {
          const size_t off = size_t(m) * p.ldx + size_t(c0) * kChunkK + size_t(pc) * 8;
          v = load_rows_piece(p, p.x + off, c0 * kChunkK + pc * 8);
          if (p.x2) v = silu_mul8<T>(v, __ldcg(reinterpret_cast<const uint4*>(p.x2 + off)));
        }
        const int g = pc >> 3, o = pc & 7, kt = o >> 1, tg = (o & 1) * 2;
        uint8_t* dst = xs + (size_t(m) * kc + g) * 128 + tg * 32 + kt * 8;
        *reinterpret_cast<uint2*>(dst) = make_uint2(v.x, v.y);
        *reinterpret_cast<uint2*>(dst + 32) = make_uint2(v.z, v.w);
      }
    }
  }
  __syncthreads();   // tables and activation rows are in place

  // ---- main loop ------------------------------------------------------------------------------
  uint32_t token;   // defined after the barrier; part of every shared-memory address below
  asm volatile("mov.u32 %0, 0;" : "=r"(token));
  float acc[2][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[s][r] = 0.f;
  float* red = reinterpret_cast<float*>(generic(p.red_abs));
  const int nwa = kc < NW ? kc : NW;   // warps that held chunks
  const RowsUnitMeta* meta = reinterpret_cast<const RowsUnitMeta*>(generic(p.meta_abs));
  // sum of the 16 warps' partial results of one (plane buffer, batch row, row): loads first, adds in warp order
  auto warp_sum = [&](int plane, int m, int row) {
    const float* r0 = red + (plane * Mp + m) * kUnitRows + row;
    const int stride = p.red_planes * Mp * kUnitRows;
    float part_v[NW];
#pragma unroll
    for (int wi = 0; wi < NW; ++wi) part_v[wi] = wi < nwa ? r0[wi * stride] : 0.f;
    float v = 0.f;
#pragma unroll
    for (int wi = 0; wi < NW; ++wi) v += part_v[wi];
    return v;
  };
  const uint32_t xs_lane = token + win + p.xs_abs + uint32_t(gid & (Mp - 1)) * uint32_t(kc) * 128u +
                           uint32_t(tig) * 32u + uint32_t(warp) * 128u;
  auto slot_base = [&](int plane) {
    const int sl = __shfl_sync(kFull, my_slot, plane & 31);
    return token + win + uint32_t(lane) * 4u + uint32_t(sl & 1) * 128u + uint32_t(sl >> 1) * kTableBytes;
  };
  uint32_t base = slot_base(0);
  uint32_t xr[XREG ? R : 1][2][4];
  if (XREG) {
#pragma unroll
    for (int j = 0; j < R; ++j) {
      lds128(xr[j][0], xs_lane + uint32_t(j) * uint32_t(NW * 128));
      lds128(xr[j][1], xs_lane + uint32_t(j) * uint32_t(NW * 128) + 16);
    }
    if (p.incr) {
      // the plane buffers take the place of the staged rows: nobody may write a sum before
      // every warp holds its fragments (the values are pinned here, ahead of the barrier)
#pragma unroll
      for (int j = 0; j < R; ++j)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 4; ++i) asm volatile("" : "+r"(xr[j][h][i]));
      __syncthreads();
    }
  }

  while (cur_n > 0) {   // warp-uniform
    // the round after this one
    int nxt_plane = cur_plane, nxt_k = cur_k + cur_n;
    if (nxt_k >= cnt) { nxt_k = 0; ++nxt_plane; }
    int nxt_n = cnt - nxt_k < R ? cnt - nxt_k : R;
    if (nxt_plane >= nplanes) nxt_n = 0;
    const uint8_t* nxt_ptr = reinterpret_cast<const uint8_t*>(
        shfl_u64(my_ptr, nxt_plane & 31) + lane_off + (unsigned long long)(nxt_k) * kHop);
    const uint32_t xs_cur = xs_lane + uint32_t(cur_k) * uint32_t(NW * 128);
    if (XREG) {   // every round is a whole plane: cur_n == R
      if (nxt_n == R) {
#pragma unroll
        for (int j = 0; j < R; ++j) {
          rows_item<T>(acc, w[j], base, xr[j]);
          ldg_stream256(w[j], nxt_ptr + j * kHop);
        }
      } else {
#pragma unroll
        for (int j = 0; j < R; ++j) rows_item<T>(acc, w[j], base, xr[j]);
      }
    } else if (cur_n == R && nxt_n == R) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        rows_item_smem<T>(acc, w[j], base, xs_cur + uint32_t(j) * uint32_t(NW * 128));
        ldg_stream256(w[j], nxt_ptr + j * kHop);
      }
    } else if (cur_n == R) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        rows_item_smem<T>(acc, w[j], base, xs_cur + uint32_t(j) * uint32_t(NW * 128));
        ldg_stream256_if(w[j], nxt_ptr + j * kHop, j < nxt_n ? 1u : 0u);
      }
    } else {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        if (j < cur_n) rows_item_smem<T>(acc, w[j], base, xs_cur + uint32_t(j) * uint32_t(NW * 128));
        ldg_stream256_if(w[j], nxt_ptr + j * kHop, j < nxt_n ? 1u : 0u);
      }
    }
    if (nxt_plane != cur_plane) {   // this warp's share of the plane is done
      const int buf = (XREG && p.incr) ? (cur_plane & (p.red_planes - 1)) : cur_plane;
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int col = 2 * tig + (r & 1);
          if (col < Mp)
            red[((warp * p.red_planes + buf) * Mp + col) * kUnitRows + 16 * s + gid + 8 * (r >> 1)] =
                acc[s][r];
          acc[s][r] = 0.f;
        }
      base = slot_base(nxt_plane);
      if (XREG && p.incr) {
        // Every warp passes here once per plane (all sixteen hold chunks). After the barrier the
        // plane's sums are complete; when it closes a unit, the unit is finished right away. A
        // buffer is written again two (four) planes later, i.e. behind the next barrier, which
        // the folding threads reach only after this fold.
        asm volatile("bar.sync 3, %0;" ::"n"(NT) : "memory");
        if ((cur_plane % ppu) == ppu - 1) {
          const int ul = cur_plane / ppu, b0 = (cur_plane - (ppu - 1)) & (p.red_planes - 1);
          for (int idx = threadIdx.x; idx < M * kUnitRows; idx += NT) {
            const int row = idx & 31, m = idx >> 5;
            const float a = warp_sum(b0, m, row);
            const float b = silu ? warp_sum(b0 + 1, m, row) : 0.f;
            rows_finish<T>(p, meta[ul], silu, m, row, a, b);
          }
        }
      }
    }
    cur_plane = nxt_plane;
    cur_k = nxt_k;
    cur_n = nxt_n;
  }
  __syncthreads();

  // ---- fold the warps' sums (warp order), then the K parts of a cluster (rank order) -----------
  const int nu = nplanes / ppu;
  const int total_out = nu * M * kUnitRows;
  if (XREG && p.incr) {
    // every unit was finished behind its last plane
  } else if (PLAN || split == 1) {   // (a plan never splits K)
    for (int idx = threadIdx.x; idx < total_out; idx += NT) {
      const int row = idx & 31, m = (idx >> 5) % M, ul = (idx >> 5) / M;
      const float a = warp_sum(ul * ppu, m, row);
      const float b = silu ? warp_sum(ul * ppu + 1, m, row) : 0.f;
      rows_finish<T>(p, meta[ul], silu, m, row, a, b);
    }
  } else {
    float* part = reinterpret_cast<float*>(generic(p.part_abs));   // [plane][m][row]
    for (int idx = threadIdx.x; idx < nplanes * M * kUnitRows; idx += NT) {
      const int row = idx & 31, m = (idx >> 5) % M, pl = (idx >> 5) / M;
      part[idx] = warp_sum(pl, m, row);
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int rank = int(cluster.block_rank());
    const int i0 = (total_out * rank) / split, i1 = (total_out * (rank + 1)) / split;
    for (int idx = i0 + int(threadIdx.x); idx < i1; idx += NT) {
      const int row = idx & 31, m = (idx >> 5) % M, ul = (idx >> 5) / M;
      float a = 0.f, b = 0.f;
      for (int q = 0; q < split; ++q) {   // fixed rank order = ascending k
        const float* peer = cluster.map_shared_rank(part, q);
        a += peer[((ul * ppu) * M + m) * kUnitRows + row];
        if (silu) b += peer[((ul * ppu + 1) * M + m) * kUnitRows + row];
      }
      rows_finish<T>(p, meta[ul], silu, m, row, a, b);
    }
    cluster.sync();   // keep shared memory alive until every peer has read it
  }

  if (p.ex.wait) {
    __syncthreads();
    // the fold buffer is free by now: its first word tells the block whether it is the last one
    volatile int& last_block = *reinterpret_cast<volatile int*>(generic(p.red_abs));
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(p.ex.wait_ticket, 1u);
      last_block = old == uint32_t(nblk) - 1u ? 1 : 0;
      if (last_block) {
        *reinterpret_cast<volatile uint32_t*>(p.ex.wait_ticket) = 0u;
        *reinterpret_cast<volatile uint32_t*>(p.ex.wait_count) += 1u;
      }
    }
    if (p.ex.sentinel) {
      // every block has staged its rows: the last one marks them as not yet arrived again
      __syncthreads();
      if (last_block) {
        const uint4 ones = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
        uint16_t* rows = const_cast<uint16_t*>(p.x);
        for (int idx = threadIdx.x; idx < M * (p.K / 8); idx += NT) {
          const int m = idx / (p.K / 8), pc = idx - m * (p.K / 8);
          *reinterpret_cast<uint4*>(rows + size_t(m) * p.ldx + size_t(pc) * 8) = ones;
        }
      }
    }
  }
  if (p.ex.push && !p.ex.sentinel) {
    // one system-wide fence per block, then this block's flag in every rank's flag array
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.ex.epoch) + 1u;
      __threadfence_system();
      const uint32_t slot = uint32_t(p.ex.rank) * uint32_t(nblk) + uint32_t(bid);
      for (int q = 0; q < p.ex.world; ++q)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.ex.peer_flag[q] + slot), "r"(e)
                     : "memory");
      const uint32_t old = atomicAdd(p.ex.ticket, 1u);
      if (old == uint32_t(nblk) - 1u) {
        *reinterpret_cast<volatile uint32_t*>(p.ex.ticket) = 0u;
        *reinterpret_cast<volatile uint32_t*>(p.ex.epoch) = e;
      }
    }
  }
  if (PLAN && p.done) {
    // the rows of this block are stored: one fence for the block, then the job's counter
    __syncthreads();
    if (threadIdx.x == 0)
      asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.done) : "memory");
  }
}

template <typename T, bool XREG>
__global__ void __launch_bounds__(kRowsThreads, 1) gemv_rows_kernel(const __grid_constant__ RowsParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  rows_block<T, XREG, false>(p, smem, int(blockIdx.x), int(gridDim.x));
}

// Persistent form: a list of jobs (the projections of a model step, each depending on the one
// before it or on none) in ONE launch of one block per SM. Every block walks the list; a job's
// parameters sit in shared memory (the next job's are copied in while this one runs), and block b
// works on job j when b is below the job's block count. Because the body requests its first
// round of codes and builds its pair tables BEFORE it looks at the producer's counter, code
// bytes are in flight across every dependency, and no launch, drain or ramp separates two jobs.
// The only waits are the bounded polls of a producer's counter; when one runs out the plan's
// abort word is set, every later poll returns at once and the launch ends.
struct RowsPlanHeader {
  unsigned long long magic;
  int njobs, grid;
  uint32_t smem_bytes, params_abs;     // dynamic shared memory of the launch; where the two job slots sit
  long long jobs_off, done_off, misc_off, total_bytes;
};
constexpr unsigned long long kRowsPlanMagic = 0xB200'1A7E'D0C0'DE02ull;
constexpr uint32_t kRowsPlanSlot = (uint32_t(sizeof(RowsParams)) + 15u) & ~15u;

template <typename T>
__global__ void __launch_bounds__(kRowsThreads, 1) gemv_rows_plan_kernel(uint8_t* plan_bytes) {
  extern __shared__ __align__(16) uint8_t smem[];
  const RowsPlanHeader& hdr = *reinterpret_cast<const RowsPlanHeader*>(plan_bytes);
  const uint8_t* jobs = plan_bytes + hdr.jobs_off;
  int* done = reinterpret_cast<int*>(plan_bytes + hdr.done_off);
  int* misc = reinterpret_cast<int*>(plan_bytes + hdr.misc_off);   // [0] exit count, [1] abort
  const int njobs = hdr.njobs;
  const uint32_t low = smem_u32(smem) & kRowsWindowMask;
  uint8_t* slots = smem + (hdr.params_abs - low);
  auto fetch = [&](int j) {   // 16 bytes per thread, no register round trip
    const uint32_t dst = smem_u32(slots) + uint32_t(j & 1) * kRowsPlanSlot;
    const uint8_t* src = jobs + size_t(j) * kRowsPlanSlot;
    for (uint32_t o = threadIdx.x * 16u; o < kRowsPlanSlot; o += kRowsThreads * 16u)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + o), "l"(src + o) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0);
  for (int j = 0; j < njobs; ++j) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();             // job j's parameters are in; nobody still works on job j - 1
    if (j + 1 < njobs) fetch(j + 1);
    const RowsParams& p = *reinterpret_cast<const RowsParams*>(slots + size_t(j & 1) * kRowsPlanSlot);
    const int nblk = p.row_blocks;
    if (int(blockIdx.x) < nblk) {
      if (p.xreg) rows_block<T, true, true>(p, smem, int(blockIdx.x), nblk);
      else rows_block<T, false, true>(p, smem, int(blockIdx.x), nblk);
    }
  }
  // the last block out resets the completion counters for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int old = atomicAdd(misc, 1);
    if (old == int(gridDim.x) - 1) {
      for (int j = 0; j < njobs; ++j) done[j] = 0;
      misc[0] = 0;
      __threadfence();
    }
  }
}

// ---- host side: geometry of a launch ------------------------------------------------------------

struct RowsGeom {
  int units_total, row_blocks, split, ntables, red_planes, Mp, xreg, incr;
  int per_seg, blk0[kMaxSeg + 1];
  uint32_t xs_abs, red_abs, part_abs, fht_abs, meta_abs, end_abs;
};

// Palette slots the busiest block needs when `units` units are cut into `row_blocks` ranges
// (the device assigns one slot per run of consecutive planes with the same palette, per stream).
int rows_max_slots(const SegDev* seg, int nseg, bool silu, int units, int row_blocks, int per_seg = 0,
                   const int* blk0 = nullptr, int* most_units = nullptr) {
  const int ppu = silu ? 2 : 1;
  int worst = 0, widest = 0;
  for (int rb = 0; rb < row_blocks; ++rb) {
    int u0, u1, owner;
    rows_block_units(per_seg, blk0, seg, nseg, units, row_blocks, rb, &u0, &u1, &owner);
    if (u1 - u0 > widest) widest = u1 - u0;
    int slots = 0;
    for (int wh = 0; wh < ppu; ++wh) {
      const void* prev = nullptr;
      for (int u = u0; u < u1; ++u) {
        int si = 0;
        for (int s = 0; s < nseg; s += ppu)
          if ((u >> 2) >= seg[s].tile_begin) si = s;
        const SegDev& sg = seg[si + wh];
        const int lu = u - 4 * seg[si].tile_begin;
        int grp = (lu * kUnitRows) / sg.gs;
        if (grp > sg.n_groups - 1) grp = sg.n_groups - 1;
        const void* key = sg.lut + size_t(grp) * 16;
        if (u == u0 || key != prev) ++slots;
        prev = key;
      }
    }
    if (slots > worst) worst = slots;
  }
  if (most_units) *most_units = widest;
  return worst;
}

// Per-segment folds: `blocks` row blocks dealt to the segments in proportion to their units
// (at least one each, never more than a segment has units). Returns the blocks dealt.
int rows_deal_blocks(const SegDev* seg, int nseg, int units, int blocks, int* blk0) {
  int nb[kMaxSeg], us[kMaxSeg], dealt = 0;
  for (int i = 0; i < nseg; ++i) {
    us[i] = (i + 1 < nseg ? 4 * seg[i + 1].tile_begin : units) - 4 * seg[i].tile_begin;
    nb[i] = 1;
    ++dealt;
  }
  while (dealt < blocks) {
    int best = -1;
    for (int i = 0; i < nseg; ++i)
      if (nb[i] < us[i] && (best < 0 || (long long)us[i] * nb[best] > (long long)us[best] * nb[i])) best = i;
    if (best < 0) break;
    ++nb[best];
    ++dealt;
  }
  blk0[0] = 0;
  for (int i = 0; i < nseg; ++i) blk0[i + 1] = blk0[i] + nb[i];
  return dealt;
}

// Decide whether the row-range kernel serves this launch and lay it out. Returns false when the
// tile x split kernel has to run (other code widths, a second stream, M > 8, a K range whose
// activation rows do not fit in shared memory).
bool rows_plan(const SegDev* seg, int nseg, bool silu, int tiles_total, int M, int K, int sms,
               uint32_t fht_bytes, int per_seg, bool may_split, RowsGeom* g) {
  if (M < 1 || M > 8) return false;
  if (per_seg && silu) return false;    // a (gate, up) pair is one unit and has one input
  for (int i = 0; i < nseg; ++i)
    if (seg[i].bits != 4 || seg[i].packed2 != nullptr || seg[i].gs < kUnitRows) return false;
  const int ppu = silu ? 2 : 1;
  const int Mp = M == 1 ? 1 : (M == 2 ? 2 : (M <= 4 ? 4 : 8));
  const int G = K / kChunkK;
  const int U = tiles_total * 4;
  int cap_planes = 32 / Mp;                       // fold buffer <= 32 KB
  if (cap_planes > kRowsMaxPlanes) cap_planes = kRowsMaxPlanes;
  // Eight rows of a K of exactly 64 chunks: the units are folded as they finish out of 2 * ppu
  // rotating plane buffers in the place of the staged rows (see RowsParams::incr), so the fold
  // buffer neither caps the planes of a block nor takes shared memory of its own.
  const bool incr_ok = Mp == 8 && G == kRowsWarps * kRowsRing;
  const int upb_max = (incr_ok ? kRowsMaxPlanes : cap_planes) / ppu;
  if (upb_max < 1) return false;
  int split = 1, row_blocks, slots;
  g->per_seg = per_seg;
  for (int i = 0; i <= kMaxSeg; ++i) g->blk0[i] = 0;
  int widest = 0;
  if (per_seg) {
    // blocks never cross a segment: one block per SM dealt over the segments (or the next
    // multiple that fits the palette slots and the fold buffer), one unit per block at most
    row_blocks = 0;
    slots = 0;
    for (int k = 1; !row_blocks; ++k) {
      const int want = k * sms < U ? k * sms : U;
      const int got = rows_deal_blocks(seg, nseg, U, want, g->blk0);
      const int sl = rows_max_slots(seg, nseg, silu, U, got, 1, g->blk0, &widest);
      if ((widest <= upb_max && sl <= kRowsMaxSlots) || want == U) { row_blocks = got; slots = sl; }
    }
  } else if (U > sms) {
    // One block per SM, or the next multiple of that whose blocks fit the palette slots and
    // the fold buffer.
    row_blocks = 0;
    slots = 0;
    for (int k = 1; k * sms <= U && !row_blocks; ++k) {
      const int rbk = k * sms;
      if ((U + rbk - 1) / rbk > upb_max) continue;
      const int sl = rows_max_slots(seg, nseg, silu, U, rbk);
      if (sl <= kRowsMaxSlots) { row_blocks = rbk; slots = sl; }
    }
    if (!row_blocks) { row_blocks = U; slots = ppu; }
  } else if (2 * U > sms) {
    row_blocks = U;
    slots = ppu;
  } else {
    row_blocks = U;
    slots = ppu;
    // K is split over a cluster only down to 64 chunks per part: a part then still streams
    // 64 KB per unit (about as long as the cluster fold costs) and keeps its activation
    // fragments in registers.
    split = sms / U;
    if (split > kMaxClusterSplit) split = kMaxClusterSplit;
    if (split > G / (kRowsWarps * kRowsRing)) split = G / (kRowsWarps * kRowsRing);
    if (split < 1 || fht_bytes || !may_split) split = 1;
  }
  g->units_total = U;
  g->row_blocks = row_blocks;
  g->split = split;
  g->ntables = slots > 2 ? 2 : 1;
  g->Mp = Mp;
  g->xreg = (G % split == 0 && G / split == kRowsWarps * kRowsRing) ? 1 : 0;
  if (!per_seg) widest = (U + row_blocks - 1) / row_blocks;
  g->incr = (incr_ok && split == 1) ? 1 : 0;
  if (!g->incr && widest * ppu > cap_planes) return false;
  g->red_planes = g->incr ? 2 * ppu : widest * ppu;
  const int kc_max = (G + split - 1) / split;
  g->xs_abs = kRowsTableAbs + uint32_t(g->ntables) * kTableBytes;
  g->red_abs = g->xs_abs + uint32_t(Mp) * uint32_t(kc_max) * 128u;
  g->part_abs = g->red_abs + uint32_t(kRowsWarps) * uint32_t(g->red_planes) * uint32_t(Mp) * 128u;
  if (g->incr) {   // 16 warps x 2 ppu planes x M' x 128 bytes <= M' x 64 chunks x 128 bytes
    g->part_abs = g->red_abs;
    g->red_abs = g->xs_abs;
  }
  g->fht_abs = g->part_abs + (split > 1 ? uint32_t(g->red_planes) * uint32_t(Mp) * 128u : 0u);
  g->meta_abs = g->fht_abs + ((fht_bytes + 15u) & ~15u);
  g->end_abs = g->meta_abs + uint32_t(widest) * uint32_t(sizeof(RowsUnitMeta));
  return g->end_abs <= 227u * 1024u;
}

}  // namespace
}  // namespace b200lut
