// Decode-time LUT GEMV (M <= 16) for sm_100a.
//
// y[m, n] = sum_k x[m, k] * LUT[n / gs][code(n, k)], fp32 accumulation, one rounding.
// Replaces the reference's M = 1 streamers and their split-K / merged variants
// (src/flute_extended/src/kernel_gemv.cu:92-253, kernel_gemv_splitk.cu:135-409,
// kernel_gemv_multi.cu:101-334, kernel_gemv_mlp.cu:92-450).
//
// Design (one block per (128-row tile, K split), one block per SM):
//  * The packed codes are streamed once from HBM with 256-bit loads per lane, fully
//    coalesced (a warp reads 1 KB contiguous per instruction), straight into
//    registers, one 128-row x 64-k chunk (4 KB at 4 bits) ahead of the math.
//  * A pair of codes (2*bits bits) is turned into a packed pair of 16-bit palette
//    entries by ONE shared-memory load from a "pair table" (4^bits entries). The
//    table is replicated 32 times so that lane L only ever touches bank L: entry e
//    of slot s lives at table + e*256 + s*128 + 4*L. The table is 64 KB aligned in
//    the shared window, so the load address is formed by a single byte permute of
//    (code word, lane base) — no shift, mask or add per lookup.
//  * The looked-up pairs ARE the A fragments of mma.m16n8k16 (the slab layout is
//    that register order); x supplies the B fragment (batch rows in the n8 columns).
//    Tensor-core math is far off the critical path; it removes the 16->32-bit
//    conversions and FMAs a scalar GEMV would spend its issue slots on.
//  * Warps split the block's K range chunk by chunk; partial sums meet in shared
//    memory in a fixed order. K splits of one tile form a thread-block cluster and
//    are folded through distributed shared memory in rank order (deterministic, no
//    atomics on data, no scratch). Splits wider than a cluster (9..16) use an fp32
//    workspace and a last-arrival ticket, also folded in index order.
//  * The kernel is written for programmatic dependent launch: code prefetch and
//    table build run before griddepcontrol.wait, so they overlap the previous
//    kernel's tail; only x depends on the predecessor.
#include <cooperative_groups.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "pairtable.cuh"

namespace cg = cooperative_groups;

namespace b200lut {
namespace {

__device__ int g_exchange_status = 0;

constexpr int kMaxSeg = 8;
constexpr int kMaxM = 16;
constexpr uint32_t kPartBytes = 2 * kMaxM * kTileRows * 4;  // two result planes (gate/up)
constexpr int kMaxClusterSplit = 8;

struct SegDev {
  const uint8_t* packed;
  const uint16_t* lut;
  const uint8_t* packed2;
  const uint16_t* lut2;
  const uint16_t* bias;
  uint16_t* out;
  long long ldo;
  int N, gs, n_groups, bits, bits2, tile_begin;
  const uint16_t* resA;     // fused low-rank residual: [N, res_rank], or null
  const float* res_t;       // [M, res_ldt] fp32 = x @ resB^T
  long long res_ldt;
  int res_rank, pad;
};

// Column-parallel exchange (see b200lut_exchange): where to mirror outputs, whom to signal,
// what to wait for.
struct ExchangeDev {
  int world, rank, push, wait;
  int blocks;           // blocks of the producing grid = flags per rank
  long long delta[B200LUT_MAX_PEERS];
  uint32_t* peer_flag[B200LUT_MAX_PEERS];
  uint32_t* ticket;
  uint32_t* epoch;
  const uint32_t* flags;
  uint32_t* wait_ticket;
  uint32_t* wait_count;
  int* status;          // device status word of the library (set when a wait runs out)
  long long wait_cycles;   // bound of the flag wait in SM clock cycles
  int sentinel, pad;    // no flags: the waiting launch polls its rows for 0xFFFF (see gemv_rows.cuh)
};

struct GemvParams {
  const uint16_t* x;
  long long ldx;
  int M, K, G, nseg, split, epilogue, tiles_total, cluster;
  float* ws;       // workspace fold: [split][tiles_total][planes][M][128] fp32
  int* tickets;    // workspace fold: [tiles_total]
  SegDev seg[kMaxSeg];
  ExchangeDev ex;
  // what the launch does to the activation rows first (row-range kernel only)
  const uint16_t* x_mul;     // x := silu(x) * x_mul
  const float* rot_signs;    // x := Hadamard rotation of x (segments + signs)
  const float* awq_scale;    // ... in the AWQ-compensated form
  int per_seg;               // every segment has its own fold (seg_signs / seg_awq, null = none)
  const float* seg_signs[kMaxSeg];
  const float* seg_awq[kMaxSeg];
};

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4],
                                                        uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4],
                                                 uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared-memory address of the pair-table entry of field i of slab s.
// base = 64 KB-aligned table address + slot*128 + lane*4 (bits 8..15 zero).
template <int BITS>
__device__ __forceinline__ uint32_t field_addr(const uint32_t (&w)[8 * BITS], int s, int i,
                                               uint32_t base) {
  if constexpr (BITS == 4) {
    // field = byte (i & 3) of word 4s + (i >> 2): place it in address bits 8..15
    return __byte_perm(w[4 * s + (i >> 2)], base, 0x7604u | (uint32_t(i & 3) << 4));
  } else {
    constexpr uint32_t kMask = ((1u << (2 * BITS)) - 1u) << 8;
    const int pos = 32 * BITS * s + 2 * BITS * i, m = pos >> 5, sh = pos & 31;
    uint32_t v;
    if (sh + 2 * BITS > 32) v = __funnelshift_r(w[m], w[(m + 1) % (8 * BITS)], sh - 8);
    else if (sh >= 8) v = w[m] >> (sh - 8);
    else v = w[m] << (8 - sh);
    return (v & kMask) | base;
  }
}

template <int BITS>
__device__ __forceinline__ void load_chunk(uint32_t (&w)[8 * BITS], const uint8_t* chunk_lane) {
#pragma unroll
  for (int p = 0; p < BITS; ++p) ldg_stream256(&w[8 * p], chunk_lane + p * 1024);
}

// What a pass must wait for before it may read the activation rows: nothing, the previous
// kernel in the stream (programmatic dependent launch), or a completion counter of the
// producing job inside a persistent launch.
struct DepWait {
  int mode;                 // 0 none, 1 griddepcontrol.wait, 2 counter
  const int* counter;       // mode 2: tiles of the producer finished so far
  int target;               // mode 2: proceed when *counter >= target
  int* abort_word;          // mode 2: global word set when any block gave up waiting
  const ExchangeDev* ex;    // mode 1: also wait for the peers' pushes (null: no exchange)
};

constexpr long long kDepWaitCycles = 40000000;   // ~20 ms: far beyond any healthy wait
// Waits on OTHER processes' kernels get a second: ranks drift apart by host-side work
// (allocation, page locking, a late start) far more than blocks of one launch do.
constexpr long long kPeerWaitCycles = 2000000000;

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait on a producer's completion counter (one thread polls). Gives up after a
// fixed number of cycles, or at once when another block already gave up, and records it.
__device__ __forceinline__ void dep_poll(const DepWait& dep) {
  if (ld_acquire(dep.counter) >= dep.target) return;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (ld_acquire(dep.counter) >= dep.target) return;
    if ((i & 15u) == 0u) {
      if (ld_acquire(dep.abort_word) != 0) return;
      if (clock64() - t0 > kDepWaitCycles) break;
    }
  }
  atomicExch(dep.abort_word, 1);
}

// Bounded wait for one block of one rank's push: its flag (written over NVLink by that
// block of that rank's producer) must have reached the number of waits this rank has completed on the channel, plus one (that
// count is bumped by the last block of the waiting grid, after every block has read it).
// On expiry the status word is set and the launch
// carries on, so the context stays usable and the host can see what happened.
__device__ __forceinline__ void peer_poll(const ExchangeDev& ex, int idx) {
  const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(ex.wait_count) + 1u;
  const uint32_t* f = ex.flags + idx;
  auto arrived = [&]() {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    return int(v - want) >= 0;
  };
  if (arrived()) return;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (arrived()) return;
    if ((i & 15u) == 0u) {
      if (*reinterpret_cast<volatile int*>(ex.status) != 0) return;
      if (clock64() - t0 > ex.wait_cycles) break;
    }
  }
  atomicExch(ex.status, 0x7000 + idx / ex.blocks);
}

// Batch-column plan. The n8 columns of the m16n8k16 accumulator are shared between
// batch rows and row slabs: with CP batch columns per slab (CP = 1, 2, 4, 8), one
// accumulator fragment serves 8/CP slabs — slab j of the group accumulates into columns
// [j*CP, (j+1)*CP), because its B fragment carries x only in those columns (zero
// elsewhere). At M = 1 the whole 128-row tile lives in ONE fragment (4 registers),
// which frees the register file for codes in flight. CP = 16 is the two-fragment
// form for 9..16 batch rows.
template <int CP> struct Plan {
  static constexpr int kCols = CP > 8 ? 8 : CP;          // batch columns per slab and fragment
  static constexpr int kNB = CP > 8 ? 2 : 1;             // B fragments (batch rows gid, gid + 8)
  static constexpr int kSlabsPerAcc = 8 / kCols;
  static constexpr int kAcc = kCols * kNB;               // accumulator fragments
};

template <int CP>
__device__ __forceinline__ void load_x(uint2 (&xf)[Plan<CP>::kNB][4],
                                       const uint16_t* __restrict__ x, long long ldx, int M,
                                       int k0, int gid, int tig) {
#pragma unroll
  for (int nb = 0; nb < Plan<CP>::kNB; ++nb) {
    const int m = gid % Plan<CP>::kCols + 8 * nb;
#pragma unroll
    for (int kt = 0; kt < 4; ++kt) {
      xf[nb][kt] = make_uint2(0u, 0u);
      if (m < M)
        xf[nb][kt] = __ldcg(reinterpret_cast<const uint2*>(x + size_t(m) * ldx + k0 + 16 * kt + 4 * tig));
    }
  }
}

// Look up and multiply one chunk held in w; refill each 1 KB plane of w from `next`
// (when `more`) as soon as its last field has been used.
template <typename T, int BITS, int CP>
__device__ __forceinline__ void chunk_math(float (&acc)[Plan<CP>::kAcc][4], uint32_t (&w)[8 * BITS],
                                           const uint2 (&xf)[Plan<CP>::kNB][4], uint32_t tbl_lane,
                                           int slot_shift, int gid, const uint8_t* next,
                                           uint32_t more) {
  using P = Plan<CP>;
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const int slot = s >> slot_shift;
    const uint32_t base = tbl_lane + uint32_t(slot >> 1) * kTableBytes + uint32_t(slot & 1) * 128u;
    const bool mine = (gid / P::kCols) == (s % P::kSlabsPerAcc);
#pragma unroll
    for (int kt = 0; kt < 4; ++kt) {
      uint32_t a[4];
#pragma unroll
      for (int f = 0; f < 4; ++f) a[f] = lds32(field_addr<BITS>(w, s, 4 * kt + f, base));
#pragma unroll
      for (int nb = 0; nb < P::kNB; ++nb) {
        const uint32_t b0 = (P::kSlabsPerAcc == 1 || mine) ? xf[nb][kt].x : 0u;
        const uint32_t b1 = (P::kSlabsPerAcc == 1 || mine) ? xf[nb][kt].y : 0u;
        mma16816<T>(acc[(s / P::kSlabsPerAcc) * P::kNB + nb], a, b0, b1);
      }
    }
#pragma unroll
    for (int pl = (s * BITS) / 8; pl < ((s + 1) * BITS) / 8; ++pl)
      ldg_stream256_if(&w[8 * pl], next + pl * 1024, more);
  }
}

// One pass: stream the codes of one (segment stream, tile) over the block's chunk
// range, fold the warps' sums and add the result into part[m][row] (the block's
// K-range contribution). Each warp keeps RC chunks in flight in registers; the
// first ones are requested before the pair tables are built, so the palette fetch
// and the first code fetches overlap.
template <typename T, int BITS, int CP, int NWARPS, int RC>
__device__ __forceinline__ void stream_pass(float* part_plane, bool accumulate, uint8_t* tbl_ptr,
                                            uint32_t tbl_addr, const uint8_t* __restrict__ packed,
                                            const uint16_t* __restrict__ lut, int n_groups, int gs,
                                            int tile, int G, int c0, int c1,
                                            const uint16_t* __restrict__ x, long long ldx, int M,
                                            bool sync_before, DepWait dep) {
  using P = Plan<CP>;
  constexpr int NT = NWARPS * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const size_t chunk_bytes = size_t(1024) * BITS;
  const size_t hop = chunk_bytes * NWARPS;            // bytes between a warp's consecutive chunks
  const uint8_t* lane_base = packed + (size_t(tile) * G) * chunk_bytes + lane * 32;
  float* red = reinterpret_cast<float*>(tbl_ptr);   // aliases the tables after the loop

  uint32_t w[RC][8 * BITS];
  int c = c0 + warp;
#pragma unroll
  for (int u = 0; u < RC; ++u) {
#pragma unroll
    for (int i = 0; i < 8 * BITS; ++i) w[u][i] = 0u;
#pragma unroll
    for (int pl = 0; pl < BITS; ++pl)
      ldg_stream256_if(&w[u][8 * pl], lane_base + size_t(c) * chunk_bytes + u * hop + pl * 1024,
                       c + u * NWARPS < c1 ? 1u : 0u);
  }

  int nl = kTileRows / gs;
  if (nl < 1) nl = 1;
  const int slot_shift = nl == 1 ? 3 : (nl == 2 ? 2 : 1);
  if (sync_before) __syncthreads();   // the previous pass's fold buffer aliases the tables
  // Palette entries are requested now and written into the table only after the activation
  // rows have been requested too: the two global round trips overlap, and both sit behind
  // the code fetches issued above.
  const bool split_build = nl <= 2;
  uint32_t lutv = 0u;
  if (split_build) lutv = palette_fetch(lut, BITS, n_groups, tile * kTileRows, gs, nl);
  else build_tables(tbl_ptr, lut, BITS, n_groups, tile * kTileRows, gs, nl, NT);
  if (dep.mode == 2) {
    if (threadIdx.x == 0) dep_poll(dep);   // producer job's tiles, bounded
    __syncthreads();
  }
  if (dep.mode == 1) {
    // everything above is independent of the previous kernel in the stream
    if (dep.ex) {   // block-uniform
      // The activation rows come from this and the other ranks' producers: their flags are
      // the whole dependency (they also order this rank's own slice), so the launch does
      // not wait for the previous grid to drain.
      for (int i = int(threadIdx.x); i < dep.ex->world * dep.ex->blocks; i += int(blockDim.x))
        peer_poll(*dep.ex, i);
      __syncthreads();
    } else {
      asm volatile("griddepcontrol.wait;" ::: "memory");
    }
  }
  // x fragments ride the code ring: the rows of a chunk are requested RC chunks ahead of their
  // use (a first touch of x misses L1 and pays an L2 round trip).
  uint2 xf[RC][P::kNB][4];
#pragma unroll
  for (int u = 0; u < RC; ++u)
    load_x<CP>(xf[u], x, ldx, (c + u * NWARPS < c1) ? M : 0, (c + u * NWARPS) * kChunkK, gid, tig);
  if (split_build) table_store_shfl<NT>(tbl_ptr, lutv, BITS, nl);
  __syncthreads();
  float acc[P::kAcc][4];
#pragma unroll
  for (int a = 0; a < P::kAcc; ++a)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[a][r] = 0.f;

  uint32_t token;   // defined after the build barrier; part of every lookup address
  asm volatile("mov.u32 %0, 0;" : "=r"(token));
  const uint32_t tbl_lane = tbl_addr + lane * 4 + token;
  for (; c < c1; c += RC * NWARPS) {
#pragma unroll
    for (int u = 0; u < RC; ++u) {
      const int cu = c + u * NWARPS;
      if (cu < c1) {   // warp-uniform
        const bool more = cu + RC * NWARPS < c1;
        chunk_math<T, BITS, CP>(acc, w[u], xf[u], tbl_lane, slot_shift, gid,
                                lane_base + size_t(cu) * chunk_bytes + RC * hop, more ? 1u : 0u);
        load_x<CP>(xf[u], x, ldx, more ? M : 0, (cu + RC * NWARPS) * kChunkK, gid, tig);
      }
    }
  }
#pragma unroll
  for (int a = 0; a < P::kAcc; ++a)
#pragma unroll
    for (int r = 0; r < 4; ++r) asm volatile("" ::"f"(acc[a][r]));   // lookups end here
  __syncthreads();   // all warps are done with the tables
  // cross-warp fold, 8 batch columns at a time: red[warp][m & 7][row], fixed warp order
#pragma unroll
  for (int nb = 0; nb < P::kNB; ++nb) {
    if (nb) __syncthreads();
#pragma unroll
    for (int a = 0; a < P::kCols; ++a)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int col = 2 * tig + (r & 1);
        const int s = a * P::kSlabsPerAcc + col / P::kCols, mm = col % P::kCols;
        const int row = 16 * s + gid + 8 * (r >> 1);
        red[(warp * P::kCols + mm) * kTileRows + row] = acc[a * P::kNB + nb][r];
      }
    __syncthreads();
    for (int idx = threadIdx.x; idx < P::kCols * kTileRows; idx += NT) {
      const int mm = idx >> 7, row = idx & 127, m = mm + 8 * nb;
      if (m < M) {
        float v = 0.f;
#pragma unroll
        for (int wi = 0; wi < NWARPS; ++wi) v += red[(wi * P::kCols + mm) * kTileRows + row];
        float* dst = part_plane + m * kTileRows + row;
        *dst = accumulate ? *dst + v : v;
      }
    }
  }
}

// sum_r t[m, r] * resA[n, r]: the second factor of the low-rank residual, 8 ranks per step.
template <typename T>
__device__ __forceinline__ float residual_dot(const SegDev& sg, int m, int n) {
  const uint16_t* a = sg.resA + size_t(n) * sg.res_rank;
  const float* t = sg.res_t + size_t(m) * sg.res_ldt;
  float v = 0.f;
  for (int r = 0; r < sg.res_rank; r += 8) {
    const uint4 aw = __ldg(reinterpret_cast<const uint4*>(a + r));
    const float4 t0 = __ldcg(reinterpret_cast<const float4*>(t + r));
    const float4 t1 = __ldcg(reinterpret_cast<const float4*>(t + r + 4));
    v = fmaf(t0.x, DType<T>::to_float(uint16_t(aw.x & 0xFFFFu)), v);
    v = fmaf(t0.y, DType<T>::to_float(uint16_t(aw.x >> 16)), v);
    v = fmaf(t0.z, DType<T>::to_float(uint16_t(aw.y & 0xFFFFu)), v);
    v = fmaf(t0.w, DType<T>::to_float(uint16_t(aw.y >> 16)), v);
    v = fmaf(t1.x, DType<T>::to_float(uint16_t(aw.z & 0xFFFFu)), v);
    v = fmaf(t1.y, DType<T>::to_float(uint16_t(aw.z >> 16)), v);
    v = fmaf(t1.z, DType<T>::to_float(uint16_t(aw.w & 0xFFFFu)), v);
    v = fmaf(t1.w, DType<T>::to_float(uint16_t(aw.w >> 16)), v);
  }
  return v;
}

// Fold the K splits of one tile and write the outputs. part[plane][m][row] holds this
// block's K-range contribution. split == 1: direct; cluster: ranks fold disjoint row
// ranges through distributed shared memory in rank order; otherwise fp32 partials go
// to the workspace and the last-arrival block (ticket) folds them in split order.
// Deterministic in every mode. Returns to the caller with all of the block's threads.
template <typename T, int NT>
__device__ __forceinline__ void fold_and_store(const GemvParams& p, float* part, int si, int tile,
                                               int tile_g, int sp) {
  const int split = p.split, M = p.M;
  const bool silu = p.epilogue == B200LUT_EPI_SILU_MUL;
  const int nplanes = silu ? 2 : 1;
  const SegDev& s0 = p.seg[si];
  const int n0 = tile * kTileRows;
  auto finish = [&](int m, int row, float a, float b) {
    const int n = n0 + row;
    if (s0.res_rank) a += residual_dot<T>(s0, m, n);
    if (s0.bias) a += DType<T>::to_float(s0.bias[n]);
    float v = a;
    if (silu) {
      const SegDev& s1 = p.seg[si + 1];
      if (s1.res_rank) b += residual_dot<T>(s1, m, n);
      if (s1.bias) b += DType<T>::to_float(s1.bias[n]);
      v = a / (1.f + __expf(-a)) * b;
    }
    uint16_t* dst = s0.out + size_t(m) * s0.ldo + n;
    const uint16_t bits16 = DType<T>::from_float(v);
    *dst = bits16;
    if (p.ex.push) {   // the same element of every peer's buffer, over NVLink
      for (int q = 0; q < p.ex.world; ++q)
        if (q != p.ex.rank)
          *reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(dst) + p.ex.delta[q]) = bits16;
    }
  };

  if (split == 1) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < M * kTileRows; idx += NT) {
      const int m = idx >> 7, row = idx & 127;
      finish(m, row, part[m * kTileRows + row],
             silu ? part[(kMaxM + m) * kTileRows + row] : 0.f);
    }
    return;
  }

  if (p.cluster) {
    // Pull fold. (A push variant — every rank stores its partial rows into the owners' shared
    // memory and ONE cluster barrier follows — was measured slower: 7.3 vs 6.6 us per launch
    // of the 4096 x 4096 projection.)
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();   // every rank's part[] is complete and visible
    const int rank = int(cluster.block_rank());
    const int r0 = (kTileRows * rank) / split, r1 = (kTileRows * (rank + 1)) / split;
    const int nrows = r1 - r0;
    for (int idx = threadIdx.x; idx < M * nrows; idx += NT) {
      const int m = idx / nrows, row = r0 + idx % nrows;
      float a = 0.f, b = 0.f;
      for (int q = 0; q < split; ++q) {   // fixed rank order
        const float* peer = cluster.map_shared_rank(part, q);
        a += peer[m * kTileRows + row];
        if (silu) b += peer[(kMaxM + m) * kTileRows + row];
      }
      finish(m, row, a, b);
    }
    cluster.sync();   // keep shared memory alive until every peer has read it
    return;
  }

  // workspace fold: partials to global, last-arrival block folds in split order
  {
    __syncthreads();
    const size_t plane_elems = size_t(M) * kTileRows;
    const size_t tile_elems = size_t(nplanes) * plane_elems;
    float* mine = p.ws + (size_t(sp) * p.tiles_total + tile_g) * tile_elems;
    for (int idx = threadIdx.x; idx < int(tile_elems); idx += NT) {
      const int pl = idx / int(plane_elems), rem = idx % int(plane_elems);
      mine[idx] = part[(pl * kMaxM + rem / kTileRows) * kTileRows + rem % kTileRows];
    }
    __threadfence();
    __syncthreads();
    __shared__ int is_last;
    if (threadIdx.x == 0) {
      const int old = atomicAdd(p.tickets + tile_g, 1);
      is_last = (old == split - 1);
      if (is_last) p.tickets[tile_g] = 0;   // self-resetting: ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < M * kTileRows; idx += NT) {
      const int m = idx >> 7, row = idx & 127;
      float a = 0.f, b = 0.f;
      for (int q = 0; q < split; ++q) {
        const float* src = p.ws + (size_t(q) * p.tiles_total + tile_g) * tile_elems;
        a += __ldcg(src + m * kTileRows + row);
        if (silu) b += __ldcg(src + plane_elems + m * kTileRows + row);
      }
      finish(m, row, a, b);
    }
  }
}

template <typename T, int CP, int NWARPS, int RC>
__global__ void __launch_bounds__(NWARPS * 32, 1) gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int NT = NWARPS * 32;

  float* part = reinterpret_cast<float*>(smem);   // [plane][m][row]
  const uint32_t part_addr = smem_u32(smem);
  const uint32_t tbl_addr = (part_addr + kPartBytes + 0xFFFFu) & ~0xFFFFu;
  uint8_t* tbl_ptr = smem + (tbl_addr - part_addr);

  // which tile / split is this block
  const int split = p.split;
  const int tile_g = blockIdx.x / split, sp = blockIdx.x % split;
  const int c0 = (p.G * sp) / split, c1 = (p.G * (sp + 1)) / split;

  const bool silu = p.epilogue == B200LUT_EPI_SILU_MUL;
  // plain: one segment per tile. silu-mul: segments come in (gate, up) pairs that
  // share the tile index; both are computed by this block, one after the other.
  int si = 0;
  {
    const int step = silu ? 2 : 1;
    for (int s = 0; s < p.nseg; s += step)
      if (tile_g >= p.seg[s].tile_begin) si = s;
  }
  const int tile = tile_g - p.seg[si].tile_begin;
  const int nplanes = silu ? 2 : 1;

  asm volatile("griddepcontrol.launch_dependents;");

  const int M = p.M;
  bool first = true;
  for (int plane = 0; plane < nplanes; ++plane) {
    const SegDev& sg = p.seg[si + plane];
    const int npass = sg.packed2 ? 2 : 1;
    for (int pass = 0; pass < npass; ++pass) {
      const uint8_t* packed = pass ? sg.packed2 : sg.packed;
      const uint16_t* lut = pass ? sg.lut2 : sg.lut;
      const int bits = pass ? sg.bits2 : sg.bits;
      float* dst = part + plane * kMaxM * kTileRows;
#define B200LUT_PASS(B)                                                                       \
  stream_pass<T, B, CP, NWARPS, RC>(dst, pass != 0, tbl_ptr, tbl_addr, packed, lut, sg.n_groups,  \
                                    sg.gs, tile, p.G, c0, c1, p.x, p.ldx, M, !first,              \
                                    DepWait{first ? 1 : 0, nullptr, 0, nullptr, (first && p.ex.wait) ? &p.ex : nullptr})
      switch (bits) {   // block-uniform
        case 4: B200LUT_PASS(4); break;
        case 3: B200LUT_PASS(3); break;
        case 2: B200LUT_PASS(2); break;
        default: B200LUT_PASS(1); break;
      }
#undef B200LUT_PASS
      first = false;
    }
  }
  fold_and_store<T, NT>(p, part, si, tile, tile_g, sp);
  if (p.ex.wait) {
    // The last block of a waiting grid counts the wait as done (every block read the count
    // when it polled, before it came here).
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(p.ex.wait_ticket, 1u);
      if (old == gridDim.x - 1) {
        *reinterpret_cast<volatile uint32_t*>(p.ex.wait_ticket) = 0u;
        *reinterpret_cast<volatile uint32_t*>(p.ex.wait_count) += 1u;
      }
    }
  }
  if (p.ex.push) {
    // Every block signals for itself: the barrier orders its threads' (remote) stores before
    // thread 0, whose single system-wide fence makes them visible everywhere before it writes
    // this block's flag into every rank's flag array. System-wide fences are slow (several
    // microseconds), so there is exactly one per block, all blocks pay it in parallel, and
    // nothing is serialised behind a last block. The ticket only maintains the push count
    // for the next launch and is off the peers' critical path.
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.ex.epoch) + 1u;
      __threadfence_system();
      const uint32_t slot = uint32_t(p.ex.rank) * gridDim.x + blockIdx.x;
      for (int q = 0; q < p.ex.world; ++q)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.ex.peer_flag[q] + slot), "r"(e)
                     : "memory");
      const uint32_t old = atomicAdd(p.ex.ticket, 1u);
      if (old == gridDim.x - 1) {   // every block has read the count by now
        *reinterpret_cast<volatile uint32_t*>(p.ex.ticket) = 0u;
        *reinterpret_cast<volatile uint32_t*>(p.ex.epoch) = e;
      }
    }
  }
}

constexpr int kWarpsM8 = 16, kWarpsM16 = 8;

}  // namespace
}  // namespace b200lut

#include "gemv_plan.cuh"
#include "gemv_rows.cuh"

namespace b200lut {
namespace {

size_t smem_bytes_for(int max_tables) {
  return size_t(kPartBytes) + 65536 + size_t(max_tables) * kTableBytes;
}

template <typename T, int CP, int NWARPS, int RC>
int launch(const GemvParams& p, int max_tables, bool pdl, cudaStream_t stream) {
  auto kern = gemv_kernel<T, CP, NWARPS, RC>;
  const size_t smem = smem_bytes_for(max_tables);
  static size_t configured[64] = {0};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && configured[dev] < smem) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(smem_bytes_for(2))));
    configured[dev] = smem_bytes_for(2);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(p.tiles_total * p.split), 1, 1);
  cfg.blockDim = dim3(NWARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = unsigned(p.split);
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(na);
  B200LUT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
  return B200LUT_OK;
}

// Validate the caller's segments and convert them to the device form. Shared by the
// per-launch entry and the plan builder.
int convert_segments(const b200lut_segment* segs, int nseg, bool silu, SegDev* out, int* tiles,
                     int* max_tables) {
  for (int i = 0; i < nseg; ++i) {
    const b200lut_segment& s = segs[i];
    B200LUT_REQUIRE(s.packed && s.lut, B200LUT_ERR_INVALID, "segment %d: null codes or palette", i);
    B200LUT_REQUIRE(s.N > 0 && s.N % kTileRows == 0, B200LUT_ERR_INVALID,
                    "segment %d: N must be a positive multiple of 128, got %d", i, s.N);
    B200LUT_REQUIRE(s.bits >= 1 && s.bits <= 4, B200LUT_ERR_INVALID,
                    "segment %d: stream-1 width must be 1..4, got %d", i, s.bits);
    const bool has2 = s.packed2 != nullptr;
    B200LUT_REQUIRE(!has2 || (s.lut2 && s.bits2 >= 1 && s.bits2 <= 4), B200LUT_ERR_INVALID,
                    "segment %d: stream-2 needs a palette and a width of 1..4 (got %d)", i,
                    s.bits2);
    B200LUT_REQUIRE(s.group_size >= 32 && s.n_groups >= 1 &&
                        ((s.group_size < 128 && (s.group_size & (s.group_size - 1)) == 0) ||
                         s.group_size % 128 == 0),
                    B200LUT_ERR_UNSUPPORTED,
                    "segment %d: group_size %d not served (32, 64 or a multiple of 128)", i,
                    s.group_size);
    B200LUT_REQUIRE(aligned16(s.packed) && (!has2 || aligned16(s.packed2)), B200LUT_ERR_ALIGN,
                    "segment %d: code buffers must be 16-byte aligned", i);
    const bool writes = !silu || (i % 2 == 0);
    B200LUT_REQUIRE(!writes || (s.out && s.ldo >= s.N), B200LUT_ERR_INVALID,
                    "segment %d: null output or row stride < N", i);
    if (silu && (i % 2 == 1))
      B200LUT_REQUIRE(s.N == segs[i - 1].N, B200LUT_ERR_INVALID,
                      "gate and up segments must have the same N (%d vs %d)", segs[i - 1].N, s.N);
    SegDev& d = out[i];
    d.packed = static_cast<const uint8_t*>(s.packed);
    d.lut = static_cast<const uint16_t*>(s.lut);
    d.packed2 = static_cast<const uint8_t*>(s.packed2);
    d.lut2 = static_cast<const uint16_t*>(s.lut2);
    d.bias = static_cast<const uint16_t*>(s.bias);
    d.out = static_cast<uint16_t*>(s.out);
    d.ldo = s.ldo;
    d.N = s.N;
    d.gs = s.group_size;
    d.n_groups = s.n_groups;
    d.bits = s.bits;
    d.bits2 = has2 ? s.bits2 : 0;
    B200LUT_REQUIRE(s.res_rank >= 0 && s.res_rank <= 4096 && s.res_rank % 8 == 0,
                    B200LUT_ERR_UNSUPPORTED,
                    "segment %d: residual rank must be a multiple of 8 up to 4096, got %d", i,
                    s.res_rank);
    if (s.res_rank > 0) {
      B200LUT_REQUIRE(s.resA && s.res_t && s.res_ldt >= s.res_rank, B200LUT_ERR_INVALID,
                      "segment %d: the residual needs resA, res_t and res_ldt >= rank", i);
      B200LUT_REQUIRE(aligned16(s.resA) && aligned16(s.res_t) && s.res_ldt % 4 == 0,
                      B200LUT_ERR_ALIGN,
                      "segment %d: resA and res_t must be 16-byte aligned, res_ldt a multiple of 4", i);
    }
    d.resA = static_cast<const uint16_t*>(s.resA);
    d.res_t = static_cast<const float*>(s.res_t);
    d.res_ldt = s.res_ldt;
    d.res_rank = s.res_rank;
    d.pad = 0;
    if (silu && (i % 2 == 1)) {
      d.tile_begin = out[i - 1].tile_begin;
    } else {
      d.tile_begin = *tiles;
      *tiles += s.N / kTileRows;
    }
    const int nl = s.group_size >= 128 ? 1 : 128 / s.group_size;
    if ((nl + 1) / 2 > *max_tables) *max_tables = (nl + 1) / 2;
  }
  return B200LUT_OK;
}

template <typename T>
int dispatch(const GemvParams& p, int max_tables, bool pdl, cudaStream_t st) {
  if (p.M == 1) return launch<T, 1, kWarpsM8, 1>(p, max_tables, pdl, st);
  if (p.M == 2) return launch<T, 2, kWarpsM8, 2>(p, max_tables, pdl, st);
  if (p.M <= 4) return launch<T, 4, kWarpsM8, 2>(p, max_tables, pdl, st);
  if (p.M <= 8) return launch<T, 8, kWarpsM8, 1>(p, max_tables, pdl, st);
  return launch<T, 16, kWarpsM16, 1>(p, max_tables, pdl, st);
}


template <typename T, bool XREG>
int launch_rows_as(const RowsParams& p, const RowsGeom& g, bool pdl, cudaStream_t stream) {
  auto kern = gemv_rows_kernel<T, XREG>;
  static bool configured[64] = {false};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  B200LUT_REQUIRE(dev >= 0 && dev < 64, B200LUT_ERR_UNSUPPORTED, "device index %d not served", dev);
  if (!configured[dev]) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(g.row_blocks * g.split), 1, 1);
  cfg.blockDim = dim3(kRowsThreads, 1, 1);
  cfg.dynamicSmemBytes = g.end_abs;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g.split > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = unsigned(g.split);
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = unsigned(na);
  B200LUT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
  return B200LUT_OK;
}

template <typename T>
int launch_rows(const RowsParams& p, const RowsGeom& g, bool pdl, cudaStream_t stream) {
  return g.xreg ? launch_rows_as<T, true>(p, g, pdl, stream) : launch_rows_as<T, false>(p, g, pdl, stream);
}

int sm_count_cached();

// Device address of the library's status word on the current device (looked up once per device).
int* device_status_addr(int* rc) {
  static int* status_addr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = fail(B200LUT_ERR_UNSUPPORTED, "device index %d not served", dev);
    return nullptr;
  }
  if (!status_addr[dev]) {
    void* a = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&a, g_exchange_status);
    if (e != cudaSuccess) {
      *rc = fail(B200LUT_ERR_CUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    status_addr[dev] = static_cast<int*>(a);
  }
  return status_addr[dev];
}

// Which decode kernel the library policy picks: the flag bits decide when set, else the
// process-wide default — the row-range kernel, unless B200LUT_GEMV_KERNEL=tile is in the
// environment (read once).
bool rows_kernel_wanted(int flags) {
  if (flags & B200LUT_FLAG_TILE_KERNEL) return false;
  if (flags & B200LUT_FLAG_ROWS_KERNEL) return true;
  static const bool dflt = [] {
    const char* e = getenv("B200LUT_GEMV_KERNEL");
    return !(e != nullptr && e[0] == 't');
  }();
  return dflt;
}

// Library policy between the two decode kernels for a launch both serve (no kernel flag, no
// input transform, no flag-less exchange). The row-range kernel stages all M rows of its K range
// in shared memory before its first lookup. With ONE unit per block and a K range whose
// fragments cannot stay in registers (K != 4096) nothing amortises that from two rows on, and
// the tile kernel (activation fragments straight from L2, chunk by chunk) is faster. Measured,
// rows / tile: 4096 x 12288 per launch, M=1 10.2 / 10.2 us, M=2 12.9 / 11.5, M=3 14.5 / 11.6,
// M=4 15.2 / 11.8; the 9B stack per step with this rule off / on, M=2 1.50 / 1.39 ms, M=3
// 1.81 / 1.64, M=4 1.89 / 1.69. (The same rule for one-unit launches of K = 4096 from three
// rows on wins per launch, 7.4 / 6.7 us at M=4, but loses in the stack, 1.69 -> 1.78 ms: the
// launch chain then alternates between the two kernels four times per layer instead of twice.)
bool rows_kernel_faster(const RowsGeom& g, int M) {
  if (g.split != 1 || g.per_seg || g.units_total > g.row_blocks) return true;
  return g.xreg || M < 2;
}

// The layout of the row-range kernel for a launch, or false when the kernel does not serve it.
// It depends only on the segment geometry; it is planned once per distinct launch shape (the
// planner walks every 32-row unit) and looked up afterwards.
bool rows_geometry(const GemvParams& gp, int tiles, bool may_split, RowsGeom* out) {
  const bool silu = gp.epilogue == B200LUT_EPI_SILU_MUL;
  struct Entry { unsigned long long key; bool ok; RowsGeom g; };
  static Entry cache[64];
  static int used = 0;
  static std::mutex mu;
  unsigned long long h = 1469598103934665603ull;
  auto mix = [&](unsigned long long v) { h = (h ^ v) * 1099511628211ull; };
  mix(unsigned(gp.nseg)); mix(unsigned(gp.epilogue)); mix(unsigned(gp.M)); mix(unsigned(gp.K));
  mix(unsigned(tiles)); mix(unsigned(sm_count_cached())); mix(may_split ? 1u : 0u);
  uint32_t fht_bytes = 0;
  if (gp.rot_signs || gp.per_seg) {   // fp32 scratch of the largest power-of-two segment of K
    int b = 1;
    while (b * 2 <= gp.K) b *= 2;
    fht_bytes = uint32_t(b) * 4u;
  }
  mix(fht_bytes);
  mix(unsigned(gp.per_seg));
  for (int i = 0; i < gp.nseg; ++i) {
    mix(unsigned(gp.seg[i].N)); mix(unsigned(gp.seg[i].gs)); mix(unsigned(gp.seg[i].n_groups));
    mix(unsigned(gp.seg[i].bits)); mix(gp.seg[i].packed2 ? 1u : 0u);
    mix(reinterpret_cast<unsigned long long>(gp.seg[i].lut));
  }
  std::lock_guard<std::mutex> lock(mu);
  int hit = -1;
  for (int i = 0; i < used; ++i)
    if (cache[i].key == h) { hit = i; break; }
  if (hit < 0) {
    hit = used < 64 ? used++ : int(h % 64);
    cache[hit].key = h;
    cache[hit].ok = rows_plan(gp.seg, gp.nseg, silu, tiles, gp.M, gp.K, sm_count_cached(), fht_bytes,
                              gp.per_seg, may_split, &cache[hit].g);
  }
  if (cache[hit].ok) *out = cache[hit].g;
  return cache[hit].ok;
}

// The kernel parameters of a launch with geometry g.
int fill_rows_params(const GemvParams& gp, const uint16_t* x2, const RowsGeom& g, RowsParams* out) {
  RowsParams& p = *out;
  p = RowsParams{};
  p.x = gp.x;
  p.x2 = x2 ? x2 : gp.x_mul;
  if (gp.rot_signs || gp.per_seg) {
    p.rot_signs = gp.rot_signs;
    p.awq_scale = gp.awq_scale;
    p.per_seg = g.per_seg;
    for (int i = 0; i <= kMaxSeg; ++i) p.blk0[i] = g.blk0[i];
    for (int i = 0; i < kMaxSeg; ++i) {
      p.seg_signs[i] = gp.seg_signs[i];
      p.seg_awq[i] = gp.seg_awq[i];
    }
    p.fht_abs = g.fht_abs;
    int off = 0;
    while (off < gp.K) {
      int b = 1, stages = 0;
      while (b * 2 <= gp.K - off) b *= 2;
      while ((1 << stages) < b) ++stages;
      B200LUT_REQUIRE(p.fht_nseg < kRowsMaxFhtSegs, B200LUT_ERR_UNSUPPORTED,
                      "K=%d splits into more than %d power-of-two segments: rotate with b200lut_fht first",
                      gp.K, kRowsMaxFhtSegs);
      p.fht_off[p.fht_nseg] = off;
      p.fht_len[p.fht_nseg] = b;
      p.fht_stages[p.fht_nseg] = stages;
      p.fht_inv[p.fht_nseg] = float(1.0 / sqrt(double(b)));
      ++p.fht_nseg;
      off += b;
    }
  }
  p.ldx = gp.ldx;
  p.M = gp.M;
  p.Mp = g.Mp;
  p.K = gp.K;
  p.G = gp.G;
  p.nseg = gp.nseg;
  p.epilogue = gp.epilogue;
  p.units_total = g.units_total;
  p.row_blocks = g.row_blocks;
  p.split = g.split;
  p.ntables = g.ntables;
  p.red_planes = g.red_planes;
  p.incr = g.incr;
  p.xs_abs = g.xs_abs;
  p.red_abs = g.red_abs;
  p.part_abs = g.part_abs;
  p.meta_abs = g.meta_abs;
  p.xreg = g.xreg;
  int rc = B200LUT_OK;
  p.status = device_status_addr(&rc);
  if (rc) return rc;
  for (int i = 0; i < gp.nseg; ++i) p.seg[i] = gp.seg[i];
  p.ex = gp.ex;
  return B200LUT_OK;
}

// The row-range kernel when it serves the launch (4-bit, one stream, M <= 8).
template <typename T>
int try_rows(const GemvParams& gp, const uint16_t* x2, int tiles, bool pdl, bool must, cudaStream_t st,
             bool* served) {
  *served = false;
  RowsGeom g;
  if (!rows_geometry(gp, tiles, true, &g)) return B200LUT_OK;
  if (!must && !rows_kernel_faster(g, gp.M)) return B200LUT_OK;
  RowsParams p;
  if (int rc = fill_rows_params(gp, x2, g, &p)) return rc;
  // (a flag-less exchange has no flags to count)
  B200LUT_REQUIRE(!p.ex.push || p.ex.sentinel || p.ex.blocks == g.row_blocks * g.split, B200LUT_ERR_INVALID,
                  "exchange: producer_blocks is %d but this launch has %d blocks "
                  "(b200lut_gemv_launch_blocks gives the count)", p.ex.blocks, g.row_blocks * g.split);
  *served = true;
  return launch_rows<T>(p, g, pdl, st);
}

int sm_count_cached() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}


// Split policy: one block per SM is resident. A wave of blocks costs a fixed part (launch
// ramp, palette fetch and table build, first code fetch, cluster fold: about three chunk
// rounds of time, measured) plus the chunk rounds of its busiest warp; clusters of `s`
// blocks place a little under one block per SM.
int pick_split(int tiles, int G, int sms, int warps) {
  constexpr long kWaveFixed = 3;
  int best = 1;
  long best_cost = -1;
  for (int s = 1; s <= kMaxClusterSplit; ++s) {
    if (s > G) break;
    const long blocks = long(tiles) * s;
    long cap = s == 1 ? sms : long(sms / s) * s * 9 / 10;
    if (cap < s) cap = s;
    const long waves = (blocks + cap - 1) / cap;
    const long per_block = (G + s - 1) / s;
    const long per_warp = (per_block + warps - 1) / warps;
    const long cost = waves * (per_warp + kWaveFixed) * 8 + s;   // ties: the smaller split
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
  }
  return best;
}

}  // namespace
}  // namespace b200lut

using namespace b200lut;

extern "C" int b200lut_sm_count(void) { return sm_count_cached(); }


extern "C" int b200lut_gemv_pick_split(int tiles, int K) {
  if (tiles <= 0 || K <= 0) return 1;
  return pick_split(tiles, K / kChunkK, sm_count_cached(), kWarpsM8);
}

extern "C" size_t b200lut_gemv_workspace_bytes(int total_rows, int M, int split) {
  if (split <= kMaxClusterSplit || total_rows <= 0 || M <= 0) return 0;
  const size_t tiles = size_t(total_rows) / kTileRows;
  // two planes (gate/up) of fp32 partials per split and tile, then the tickets
  return size_t(split) * tiles * 2 * size_t(M) * kTileRows * 4 + tiles * 4;
}

namespace b200lut {
int exchange_status_take() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_exchange_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_exchange_status, &zero, sizeof(int));
  return v;
}
}  // namespace b200lut

namespace {

// Validate an exchange descriptor and turn it into the device form.
int convert_exchange(const b200lut_exchange* ex, ExchangeDev* out) {
  *out = ExchangeDev{};
  if (!ex || (!ex->push && !ex->wait)) return B200LUT_OK;
  B200LUT_REQUIRE(ex->world >= 1 && ex->world <= B200LUT_MAX_PEERS && ex->rank >= 0 &&
                      ex->rank < ex->world,
                  B200LUT_ERR_INVALID, "exchange: world must be 1..%d and rank inside it (got %d, %d)",
                  B200LUT_MAX_PEERS, ex->world, ex->rank);
  B200LUT_REQUIRE(ex->producer_blocks >= 1 && ex->producer_blocks <= 4096, B200LUT_ERR_INVALID,
                  "exchange: producer_blocks must be 1..4096, got %d", ex->producer_blocks);
  out->world = ex->world;
  out->rank = ex->rank;
  out->blocks = ex->producer_blocks;
  if (ex->push) {
    B200LUT_REQUIRE(ex->ticket && ex->epoch && ((uintptr_t(ex->ticket) | uintptr_t(ex->epoch)) & 3) == 0,
                    B200LUT_ERR_INVALID, "exchange: push needs its ticket and count words");
    out->epoch = static_cast<uint32_t*>(ex->epoch);
    for (int q = 0; q < ex->world; ++q) {
      B200LUT_REQUIRE(ex->peer_flag[q] && (uintptr_t(ex->peer_flag[q]) & 3) == 0,
                      B200LUT_ERR_INVALID, "exchange: null or misaligned flag of rank %d", q);
      B200LUT_REQUIRE(ex->peer_delta[q] % 2 == 0, B200LUT_ERR_ALIGN,
                      "exchange: odd buffer offset to rank %d", q);
      out->delta[q] = ex->peer_delta[q];
      out->peer_flag[q] = static_cast<uint32_t*>(ex->peer_flag[q]);
    }
    out->ticket = static_cast<uint32_t*>(ex->ticket);
    out->push = 1;
  }
  if (ex->wait) {
    B200LUT_REQUIRE(ex->flags && (uintptr_t(ex->flags) & 3) == 0, B200LUT_ERR_INVALID,
                    "exchange: wait needs the local flag array");
    B200LUT_REQUIRE(ex->wait_ticket && ex->wait_count &&
                        ((uintptr_t(ex->wait_ticket) | uintptr_t(ex->wait_count)) & 3) == 0,
                    B200LUT_ERR_INVALID, "exchange: wait needs its ticket and count words");
    out->flags = static_cast<const uint32_t*>(ex->flags);
    out->wait_ticket = static_cast<uint32_t*>(ex->wait_ticket);
    out->wait_count = static_cast<uint32_t*>(ex->wait_count);
    out->wait = 1;
    B200LUT_REQUIRE(ex->wait_ms >= 0 && ex->wait_ms <= 1000, B200LUT_ERR_INVALID,
                    "exchange: wait_ms must be 0 (default) or 1..1000, got %d", ex->wait_ms);
    out->wait_cycles = ex->wait_ms ? (long long)ex->wait_ms * 2000000ll : kPeerWaitCycles;
  }
  out->sentinel = ex->sentinel ? 1 : 0;
  if (!out->wait_cycles) out->wait_cycles = kPeerWaitCycles;
  int rc = B200LUT_OK;
  out->status = b200lut::device_status_addr(&rc);
  if (rc) return rc;
  return B200LUT_OK;
}

}  // namespace

extern "C" int b200lut_gemv_multi(const void* x, int64_t ldx, int M, int K, int dtype,
                                  const b200lut_segment* segs, int nseg, int epilogue, int split,
                                  void* workspace, size_t workspace_bytes, int flags,
                                  void* stream) {
  return b200lut_gemv_exchange(x, ldx, M, K, dtype, segs, nseg, epilogue, split, workspace,
                               workspace_bytes, flags, nullptr, stream);
}

extern "C" int b200lut_gemv_exchange(const void* x, int64_t ldx, int M, int K, int dtype,
                                     const b200lut_segment* segs, int nseg, int epilogue,
                                     int split, void* workspace, size_t workspace_bytes, int flags,
                                     const b200lut_exchange* ex, void* stream) {
  return b200lut_gemv_input(x, ldx, M, K, dtype, segs, nseg, epilogue, split, workspace,
                            workspace_bytes, flags, ex, nullptr, stream);
}

extern "C" int b200lut_gemv_input(const void* x, int64_t ldx, int M, int K, int dtype,
                                  const b200lut_segment* segs, int nseg, int epilogue, int split,
                                  void* workspace, size_t workspace_bytes, int flags,
                                  const b200lut_exchange* ex, const b200lut_input* in, void* stream) {
  B200LUT_REQUIRE(x && segs, B200LUT_ERR_INVALID, "null x or segment table");
  B200LUT_REQUIRE(M >= 1 && M <= kMaxM, B200LUT_ERR_UNSUPPORTED,
                  "decode GEMV serves 1 <= M <= 16, got M=%d (use b200lut_gemm)", M);
  B200LUT_REQUIRE(K > 0 && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a positive multiple of 64, got %d", K);
  B200LUT_REQUIRE(nseg >= 1 && nseg <= kMaxSeg, B200LUT_ERR_INVALID,
                  "1..%d segments per launch, got %d", kMaxSeg, nseg);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(epilogue == B200LUT_EPI_NONE || epilogue == B200LUT_EPI_SILU_MUL,
                  B200LUT_ERR_INVALID, "unknown epilogue %d", epilogue);
  B200LUT_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, B200LUT_ERR_ALIGN,
                  "x must be 16-byte aligned with a row stride that is a multiple of 8 and >= K");
  const bool silu = epilogue == B200LUT_EPI_SILU_MUL;
  B200LUT_REQUIRE(!silu || nseg % 2 == 0, B200LUT_ERR_INVALID,
                  "the silu-mul epilogue needs (gate, up) segment pairs");

  GemvParams p = {};
  p.x = static_cast<const uint16_t*>(x);
  p.ldx = ldx;
  p.M = M;
  p.K = K;
  p.G = K / kChunkK;
  p.nseg = nseg;
  p.epilogue = epilogue;
  if (int rc = convert_exchange(ex, &p.ex)) return rc;
  int tiles = 0, max_tables = 1;
  if (int rc = convert_segments(segs, nseg, silu, p.seg, &tiles, &max_tables)) return rc;
  p.tiles_total = tiles;
  const bool transformed = in && (in->x_mul || in->rot_signs || in->awq_scale || in->per_segment);
  if (transformed) {
    B200LUT_REQUIRE(!in->awq_scale || in->rot_signs, B200LUT_ERR_INVALID,
                    "input transform: an AWQ scale needs the rotation signs");
    if (in->per_segment) {
      B200LUT_REQUIRE(!in->rot_signs && !silu, B200LUT_ERR_INVALID,
                      "input transform: per-segment folds exclude a launch-wide fold and the silu-mul "
                      "epilogue (a gate/up pair shares its input)");
      p.per_seg = 1;
      for (int i = 0; i < nseg; ++i) {
        B200LUT_REQUIRE(!in->seg_awq_scale[i] || in->seg_rot_signs[i], B200LUT_ERR_INVALID,
                        "input transform: segment %d has an AWQ scale but no rotation signs", i);
        p.seg_signs[i] = in->seg_rot_signs[i];
        p.seg_awq[i] = in->seg_awq_scale[i];
      }
    }
    B200LUT_REQUIRE(!in->x_mul || aligned16(in->x_mul), B200LUT_ERR_ALIGN,
                    "input transform: x_mul must be 16-byte aligned");
    B200LUT_REQUIRE(split <= 0 && !(flags & B200LUT_FLAG_TILE_KERNEL), B200LUT_ERR_UNSUPPORTED,
                    "an input transform is served by the row-range kernel only (split = 0, no tile-kernel flag)");
    p.x_mul = static_cast<const uint16_t*>(in->x_mul);
    p.rot_signs = in->rot_signs;
    p.awq_scale = in->awq_scale;
  }
  const bool pdl = (flags & B200LUT_FLAG_PDL) != 0;
  cudaStream_t st = cudaStream_t(stream);
  // Library policy (split == 0): the row-range kernel when it serves the shapes. An explicit
  // split or B200LUT_FLAG_TILE_KERNEL selects the tile x split kernel.
  if (split <= 0 && rows_kernel_wanted(flags)) {
    bool served = false;
    const bool must = transformed || p.ex.sentinel || (flags & B200LUT_FLAG_ROWS_KERNEL);
    const int rc = dtype == B200LUT_BF16
                       ? try_rows<__nv_bfloat16>(p, nullptr, tiles, pdl, must, st, &served)
                       : try_rows<__half>(p, nullptr, tiles, pdl, must, st, &served);
    if (rc || served) return rc;
  }
  B200LUT_REQUIRE(!transformed, B200LUT_ERR_UNSUPPORTED,
                  "an input transform needs 4-bit single-stream segments and M <= 8 (the row-range "
                  "kernel); transform the rows with b200lut_fht / b200lut_silu_mul first");
  B200LUT_REQUIRE(!p.ex.sentinel, B200LUT_ERR_UNSUPPORTED,
                  "an exchange without flags (sentinel) is served by the row-range kernel only: 4-bit "
                  "single-stream segments, M <= 8, split = 0 and rows that fit its shared memory");
  const int warps = M <= 8 ? kWarpsM8 : kWarpsM16;
  if (split <= 0) split = pick_split(tiles, p.G, sm_count_cached(), warps);
  B200LUT_REQUIRE(split >= 1 && split <= 16 && split <= p.G, B200LUT_ERR_INVALID,
                  "split must be 1..16 and <= K/64, got %d", split);
  p.split = split;
  p.cluster = (split > 1 && split <= kMaxClusterSplit) ? 1 : 0;
  if (split > kMaxClusterSplit) {
    size_t rows = size_t(tiles) * kTileRows;
    const size_t need = b200lut_gemv_workspace_bytes(int(rows), M, split);
    B200LUT_REQUIRE(workspace && workspace_bytes >= need, B200LUT_ERR_WORKSPACE,
                    "split %d needs %zu workspace bytes, got %zu", split, need, workspace_bytes);
    B200LUT_REQUIRE(aligned16(workspace), B200LUT_ERR_ALIGN, "workspace must be 16-byte aligned");
    p.ws = static_cast<float*>(workspace);
    p.tickets = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) +
                                       size_t(split) * tiles * 2 * size_t(M) * kTileRows * 4);
  }
  B200LUT_REQUIRE(!p.ex.push || p.ex.blocks == tiles * split, B200LUT_ERR_INVALID,
                  "exchange: producer_blocks is %d but this launch has %d tiles x split %d blocks",
                  p.ex.blocks, tiles, split);
  if (dtype == B200LUT_BF16) return dispatch<__nv_bfloat16>(p, max_tables, pdl, st);
  return dispatch<__half>(p, max_tables, pdl, st);
}


extern "C" int b200lut_gemv_launch_blocks(int M, int K, const b200lut_segment* segs, int nseg,
                                          int epilogue, int flags) {
  if (!segs || nseg < 1 || nseg > kMaxSeg || M < 1 || M > kMaxM || K <= 0 || K % kChunkK) return 0;
  const bool silu = epilogue == B200LUT_EPI_SILU_MUL;
  if (silu && nseg % 2) return 0;
  GemvParams p = {};
  p.M = M;
  p.K = K;
  p.G = K / kChunkK;
  p.nseg = nseg;
  p.epilogue = epilogue;
  b200lut_segment tmp[kMaxSeg];
  for (int i = 0; i < nseg; ++i) {
    tmp[i] = segs[i];
    if (!tmp[i].out) { tmp[i].out = reinterpret_cast<void*>(uintptr_t(16)); tmp[i].ldo = tmp[i].N; }
  }
  int tiles = 0, max_tables = 1;
  if (convert_segments(tmp, nseg, silu, p.seg, &tiles, &max_tables)) return 0;
  if (rows_kernel_wanted(flags)) {
    RowsGeom g;
    if (rows_geometry(p, tiles, true, &g) &&
        ((flags & B200LUT_FLAG_ROWS_KERNEL) || rows_kernel_faster(g, M)))
      return g.row_blocks * g.split;
  }
  return tiles * pick_split(tiles, p.G, sm_count_cached(), M <= 8 ? kWarpsM8 : kWarpsM16);
}

extern "C" int b200lut_gemv(const void* x, const void* packed, const void* lut, void* out, int M,
                            int N, int K, int bits, int group_size, int n_groups, int dtype,
                            int split, void* workspace, size_t workspace_bytes, void* stream) {
  b200lut_segment s = {};
  s.packed = packed;
  s.lut = lut;
  s.out = out;
  s.ldo = N;
  s.N = N;
  s.group_size = group_size;
  s.n_groups = n_groups;
  s.bits = bits;
  return b200lut_gemv_multi(x, K, M, K, dtype, &s, 1, B200LUT_EPI_NONE, split, workspace,
                            workspace_bytes, 0, stream);
}

// ------------------------------------------------------------------------------------------
// Persistent decode plan
// ------------------------------------------------------------------------------------------
namespace {

struct PlanLayout {
  PlanHeader hdr;
  std::vector<JobDev> jobs;
};

int plan_layout(const b200lut_job* jobs, int njobs, int M, int dtype, int grid, PlanLayout* out) {
  B200LUT_REQUIRE(jobs && njobs >= 1 && njobs <= 4096, B200LUT_ERR_INVALID,
                  "a plan holds 1..4096 jobs, got %d", njobs);
  B200LUT_REQUIRE(M >= 1 && M <= kMaxM, B200LUT_ERR_UNSUPPORTED,
                  "a decode plan serves 1 <= M <= 16, got M=%d", M);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  out->jobs.assign(size_t(njobs), JobDev{});
  long long ws_floats = 0;
  int ntickets = 0;
  for (int j = 0; j < njobs; ++j) {
    const b200lut_job& src = jobs[j];
    JobDev& d = out->jobs[size_t(j)];
    B200LUT_REQUIRE(src.x && src.K > 0 && src.K % kChunkK == 0, B200LUT_ERR_INVALID,
                    "job %d: null x or K not a positive multiple of 64", j);
    B200LUT_REQUIRE(aligned16(src.x) && src.ldx % 8 == 0 && src.ldx >= src.K, B200LUT_ERR_ALIGN,
                    "job %d: x must be 16-byte aligned, row stride a multiple of 8 and >= K", j);
    B200LUT_REQUIRE(src.nseg >= 1 && src.nseg <= kMaxSeg, B200LUT_ERR_INVALID,
                    "job %d: 1..%d segments, got %d", j, kMaxSeg, src.nseg);
    B200LUT_REQUIRE(src.epilogue == B200LUT_EPI_NONE || src.epilogue == B200LUT_EPI_SILU_MUL,
                    B200LUT_ERR_INVALID, "job %d: unknown epilogue %d", j, src.epilogue);
    B200LUT_REQUIRE(src.dep >= -1 && src.dep < j, B200LUT_ERR_INVALID,
                    "job %d: dep must name an earlier job or be -1 (got %d)", j, src.dep);
    const bool silu = src.epilogue == B200LUT_EPI_SILU_MUL;
    B200LUT_REQUIRE(!silu || src.nseg % 2 == 0, B200LUT_ERR_INVALID,
                    "job %d: the silu-mul epilogue needs (gate, up) segment pairs", j);
    int tiles = 0, max_tables = 1;
    if (int rc = convert_segments(src.segs, src.nseg, silu, d.seg, &tiles, &max_tables)) return rc;
    for (int q = 0; q < src.nseg; ++q)
      B200LUT_REQUIRE(src.segs[q].res_rank == 0, B200LUT_ERR_UNSUPPORTED,
                      "job %d: the fused residual is served by b200lut_gemv_multi, not by a plan", j);
    B200LUT_REQUIRE(max_tables <= 1, B200LUT_ERR_UNSUPPORTED,
                    "job %d: a plan serves group sizes >= 64 (two palettes per tile at most)", j);
    d.x = static_cast<const uint16_t*>(src.x);
    d.ldx = src.ldx;
    d.K = src.K;
    d.G = src.K / kChunkK;
    d.nseg = src.nseg;
    d.epilogue = src.epilogue;
    d.tiles_total = tiles;
    d.planes = silu ? 2 : 1;
    d.dep = src.dep;
    d.dep_target = src.dep >= 0 ? out->jobs[size_t(src.dep)].tiles_total : 0;
    const long long total = (long long)tiles * d.G;
    d.per = int((total + grid - 1) / grid);
    d.maxc = (d.G + d.per - 1) / d.per + 1;
    d.ws_off = ws_floats;
    d.ticket_off = ntickets;
    ws_floats += (long long)tiles * d.maxc * d.planes * M * kTileRows;
    ntickets += tiles;
  }
  PlanHeader& h = out->hdr;
  h.magic = kPlanMagic;
  h.njobs = njobs; h.M = M; h.dtype = dtype; h.grid = grid;
  long long off = (sizeof(PlanHeader) + 255) & ~255ll;
  h.jobs_off = off;      off += ((long long)njobs * sizeof(JobDev) + 255) & ~255ll;
  h.done_off = off;      off += ((long long)njobs * 4 + 255) & ~255ll;
  h.tickets_off = off;   off += ((long long)ntickets * 4 + 255) & ~255ll;
  h.misc_off = off;      off += 65536;   // exit count, abort word; profiling builds log here
  h.ws_off = off;        off += (ws_floats * 4 + 255) & ~255ll;
  h.total_bytes = off;
  h.ntickets = ntickets;
  return B200LUT_OK;
}

// ---- the row-range form of a plan --------------------------------------------------------------
// When every job is served by the row-range kernel (4-bit, one stream, M <= 8, rows that fit its
// shared memory, at most one block per SM) the plan runs gemv_rows_plan_kernel: the same block
// body as a single launch of that kernel, job after job. B200LUT_PLAN_KERNEL=tile in the
// environment (read once) keeps the tile-share kernel for every plan.
struct RowsPlanLayout {
  RowsPlanHeader hdr;
  std::vector<uint8_t> jobs;    // njobs slots of kRowsPlanSlot bytes
};

bool rows_plan_wanted() {
  static const bool wanted = [] {
    const char* e = getenv("B200LUT_PLAN_KERNEL");
    return !(e != nullptr && e[0] == 't');
  }();
  return wanted;
}

// `base`: device address of the plan buffer (null when only the size is asked for). Call after
// plan_layout has validated the jobs. *served = false: some job needs the tile-share kernel.
int rows_plan_layout(const b200lut_job* jobs, int njobs, int M, uint8_t* base, RowsPlanLayout* out,
                     bool* served) {
  *served = false;
  if (!rows_plan_wanted() || M > 8) return B200LUT_OK;
  const int sms = sm_count_cached();
  RowsPlanHeader& h = out->hdr;
  h = RowsPlanHeader{};
  h.magic = kRowsPlanMagic;
  h.njobs = njobs;
  long long off = (sizeof(RowsPlanHeader) + 255) & ~255ll;
  h.jobs_off = off;   off += ((long long)njobs * kRowsPlanSlot + 255) & ~255ll;
  h.done_off = off;   off += ((long long)njobs * 4 + 255) & ~255ll;
  h.misc_off = off;   off += 256;
  h.total_bytes = off;
  out->jobs.assign(size_t(njobs) * kRowsPlanSlot, uint8_t(0));
  std::vector<int> blocks(size_t(njobs), 0);
  int* done = reinterpret_cast<int*>(base + h.done_off);
  int* misc = reinterpret_cast<int*>(base + h.misc_off);
  uint32_t max_end = 0;
  int grid = 1;
  for (int j = 0; j < njobs; ++j) {
    const b200lut_job& src = jobs[j];
    const bool silu = src.epilogue == B200LUT_EPI_SILU_MUL;
    GemvParams gp = {};
    gp.x = static_cast<const uint16_t*>(src.x);
    gp.ldx = src.ldx;
    gp.M = M;
    gp.K = src.K;
    gp.G = src.K / kChunkK;
    gp.nseg = src.nseg;
    gp.epilogue = src.epilogue;
    int tiles = 0, max_tables = 1;
    if (int rc = convert_segments(src.segs, src.nseg, silu, gp.seg, &tiles, &max_tables)) return rc;
    gp.tiles_total = tiles;
    RowsGeom g;
    if (!rows_geometry(gp, tiles, false, &g) || g.split != 1 || g.row_blocks > sms) return B200LUT_OK;
    RowsParams p;
    if (int rc = fill_rows_params(gp, nullptr, g, &p)) return rc;
    blocks[size_t(j)] = g.row_blocks;
    if (src.dep >= 0) {
      p.dep_done = done + src.dep;
      p.dep_target = blocks[size_t(src.dep)];
    }
    p.done = done + j;
    p.abort_word = misc + 1;
    memcpy(out->jobs.data() + size_t(j) * kRowsPlanSlot, &p, sizeof(p));
    if (g.end_abs > max_end) max_end = g.end_abs;
    if (g.row_blocks > grid) grid = g.row_blocks;
  }
  h.grid = grid;
  h.params_abs = (max_end + 15u) & ~15u;
  h.smem_bytes = h.params_abs + 2u * kRowsPlanSlot;
  if (h.smem_bytes > 227u * 1024u) return B200LUT_OK;
  *served = true;
  return B200LUT_OK;
}

// What b200lut_plan_run must know about a row-range plan, kept on the host by the build call
// (the run call gets the device buffer only).
struct RowsPlanInfo { const void* plan; int dev, grid; uint32_t smem; };
std::mutex g_rows_plan_mu;
std::vector<RowsPlanInfo> g_rows_plans;     // one entry per live row-range plan buffer

void rows_plan_forget(const void* plan, int dev) {
  for (size_t i = 0; i < g_rows_plans.size();)
    if (g_rows_plans[i].plan == plan && g_rows_plans[i].dev == dev) {
      g_rows_plans[i] = g_rows_plans.back();
      g_rows_plans.pop_back();
    } else {
      ++i;
    }
}

template <typename T>
int launch_rows_plan(void* plan, const RowsPlanInfo& info, cudaStream_t stream) {
  auto kern = gemv_rows_plan_kernel<T>;
  static bool configured[64] = {false};
  if (info.dev < 64 && !configured[info.dev]) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured[info.dev] = true;
  }
  uint8_t* arg = static_cast<uint8_t*>(plan);
  void* args[] = {&arg};
  // cooperative: every block of the grid is resident, so a block that waits for a producer
  // never holds the SM the producer needs
  B200LUT_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), dim3(unsigned(info.grid)),
                                              dim3(kRowsThreads), args, info.smem, stream));
  return B200LUT_OK;
}

template <typename T, int CP, int NWARPS>
int launch_plan(void* plan, int grid, cudaStream_t stream) {
  auto kern = gemv_plan_kernel<T, CP, NWARPS>;
  const size_t smem = smem_bytes_for(2);
  static bool configured[64] = {false};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    B200LUT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(smem)));
    configured[dev] = true;
  }
  uint8_t* arg = static_cast<uint8_t*>(plan);
  void* args[] = {&arg};
  B200LUT_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), dim3(unsigned(grid)),
                                              dim3(NWARPS * 32), args, smem, stream));
  return B200LUT_OK;
}

template <typename T>
int dispatch_plan(void* plan, int M, int grid, cudaStream_t st) {
  if (M == 1) return launch_plan<T, 1, kWarpsM8>(plan, grid, st);
  if (M == 2) return launch_plan<T, 2, kWarpsM8>(plan, grid, st);
  if (M <= 4) return launch_plan<T, 4, kWarpsM8>(plan, grid, st);
  if (M <= 8) return launch_plan<T, 8, kWarpsM8>(plan, grid, st);
  return launch_plan<T, 16, kWarpsM16>(plan, grid, st);
}

}  // namespace

extern "C" size_t b200lut_plan_bytes(const b200lut_job* jobs, int njobs, int M, int dtype) {
  PlanLayout lay;
  if (plan_layout(jobs, njobs, M, dtype, sm_count_cached(), &lay) != B200LUT_OK) return 0;
  RowsPlanLayout rows;
  bool served = false;
  if (rows_plan_layout(jobs, njobs, M, nullptr, &rows, &served) != B200LUT_OK) return 0;
  return served ? size_t(rows.hdr.total_bytes) : size_t(lay.hdr.total_bytes);
}

extern "C" int b200lut_plan_build(void* plan, size_t plan_bytes, const b200lut_job* jobs, int njobs,
                                  int M, int dtype, void* stream) {
  B200LUT_REQUIRE(plan && aligned16(plan), B200LUT_ERR_ALIGN, "plan buffer must be 16-byte aligned");
  PlanLayout lay;
  if (int rc = plan_layout(jobs, njobs, M, dtype, sm_count_cached(), &lay)) return rc;
  cudaStream_t st = cudaStream_t(stream);
  uint8_t* base = static_cast<uint8_t*>(plan);
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(g_rows_plan_mu);
    rows_plan_forget(plan, dev);
  }
  RowsPlanLayout rows;
  bool served = false;
  if (int rc = rows_plan_layout(jobs, njobs, M, base, &rows, &served)) return rc;
  if (served) {
    const RowsPlanHeader& h = rows.hdr;
    B200LUT_REQUIRE(plan_bytes >= size_t(h.total_bytes), B200LUT_ERR_WORKSPACE,
                    "plan needs %lld bytes, got %zu", h.total_bytes, plan_bytes);
    B200LUT_CUDA_OK(cudaMemsetAsync(base, 0, size_t(h.total_bytes), st));
    B200LUT_CUDA_OK(cudaMemcpyAsync(base, &h, sizeof(h), cudaMemcpyHostToDevice, st));
    B200LUT_CUDA_OK(cudaMemcpyAsync(base + h.jobs_off, rows.jobs.data(), rows.jobs.size(),
                                    cudaMemcpyHostToDevice, st));
    B200LUT_CUDA_OK(cudaStreamSynchronize(st));   // the host staging dies with this call
    std::lock_guard<std::mutex> lock(g_rows_plan_mu);
    g_rows_plans.push_back(RowsPlanInfo{plan, dev, h.grid, h.smem_bytes});
    return B200LUT_OK;
  }
  B200LUT_REQUIRE(plan_bytes >= size_t(lay.hdr.total_bytes), B200LUT_ERR_WORKSPACE,
                  "plan needs %lld bytes, got %zu", lay.hdr.total_bytes, plan_bytes);
  // counters, tickets and the abort word start at zero; partials need no initial value
  B200LUT_CUDA_OK(cudaMemsetAsync(base, 0, size_t(lay.hdr.ws_off), st));
  B200LUT_CUDA_OK(cudaMemcpyAsync(base, &lay.hdr, sizeof(PlanHeader), cudaMemcpyHostToDevice, st));
  B200LUT_CUDA_OK(cudaMemcpyAsync(base + lay.hdr.jobs_off, lay.jobs.data(),
                                  lay.jobs.size() * sizeof(JobDev), cudaMemcpyHostToDevice, st));
  B200LUT_CUDA_OK(cudaStreamSynchronize(st));   // the host staging dies with this call
  return B200LUT_OK;
}

extern "C" int b200lut_plan_run(void* plan, int M, int dtype, void* stream) {
  B200LUT_REQUIRE(plan, B200LUT_ERR_INVALID, "null plan");
  B200LUT_REQUIRE(M >= 1 && M <= kMaxM && (dtype == B200LUT_BF16 || dtype == B200LUT_F16),
                  B200LUT_ERR_INVALID, "M and dtype must be those the plan was built with");
  {
    int dev = 0;
    B200LUT_CUDA_OK(cudaGetDevice(&dev));
    RowsPlanInfo info = {};
    {
      std::lock_guard<std::mutex> lock(g_rows_plan_mu);
      for (const RowsPlanInfo& e : g_rows_plans)
        if (e.plan == plan && e.dev == dev) info = e;
    }
    if (info.plan) {
      if (dtype == B200LUT_BF16) return launch_rows_plan<__nv_bfloat16>(plan, info, cudaStream_t(stream));
      return launch_rows_plan<__half>(plan, info, cudaStream_t(stream));
    }
  }
  const int grid = sm_count_cached();
  if (dtype == B200LUT_BF16) return dispatch_plan<__nv_bfloat16>(plan, M, grid, cudaStream_t(stream));
  return dispatch_plan<__half>(plan, M, grid, cudaStream_t(stream));
}

extern "C" int b200lut_plan_release(const void* plan) {
  if (!plan) return B200LUT_OK;
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_rows_plan_mu);
  rows_plan_forget(plan, dev);
  return B200LUT_OK;
}

extern "C" int b200lut_plan_form(const void* plan) {
  if (!plan) return -1;
  unsigned long long magic = 0;
  if (cudaMemcpy(&magic, plan, sizeof(magic), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return magic == kRowsPlanMagic ? 1 : (magic == kPlanMagic ? 0 : -1);
}

extern "C" int b200lut_plan_status(const void* plan) {
  B200LUT_REQUIRE(plan, B200LUT_ERR_INVALID, "null plan");
  unsigned long long magic = 0;
  B200LUT_CUDA_OK(cudaMemcpy(&magic, plan, sizeof(magic), cudaMemcpyDeviceToHost));
  if (magic == kRowsPlanMagic) {
    RowsPlanHeader rh;
    B200LUT_CUDA_OK(cudaMemcpy(&rh, plan, sizeof(rh), cudaMemcpyDeviceToHost));
    int words[2] = {0, 0};
    B200LUT_CUDA_OK(cudaMemcpy(words, static_cast<const uint8_t*>(plan) + rh.misc_off, sizeof(words),
                               cudaMemcpyDeviceToHost));
    if (words[1] != 0) return fail(B200LUT_ERR_DEVICE, "a dependency wait inside the plan ran out");
    return B200LUT_OK;
  }
  PlanHeader h;
  B200LUT_CUDA_OK(cudaMemcpy(&h, plan, sizeof(h), cudaMemcpyDeviceToHost));
  B200LUT_REQUIRE(h.magic == kPlanMagic, B200LUT_ERR_INVALID, "not a plan buffer");
  int misc[2] = {0, 0};
  B200LUT_CUDA_OK(cudaMemcpy(misc, static_cast<const uint8_t*>(plan) + h.misc_off, sizeof(misc),
                             cudaMemcpyDeviceToHost));
  if (misc[1] != 0) return fail(B200LUT_ERR_DEVICE, "a dependency wait inside the plan ran out");
  return B200LUT_OK;
}

// ------------------------------------------------------------------------------------------
// Allocation-free entry point
// ------------------------------------------------------------------------------------------
// Some hosts of this library cannot give it memory: a runtime that hands out its device
// pool once at start-up and forbids cudaMalloc afterwards, a plug-in called from inside a
// region where allocation is banned, an embedding in a process that has no allocator of
// its own. For them the split-K fold's scratch (fp32 partial tiles + tickets) lives in a
// fixed array inside the library image instead of a caller buffer. Every device that loads
// the library holds these 8 MiB until the process exits.
namespace {
constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;
constexpr size_t kNoAllocTicketBytes = 4096;   // 1024 tiles
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
}  // namespace

namespace {
// Device address of the built-in scratch on the current device. The array's name is only a
// host-side handle; kernels and memsets need the address behind it, looked up once per device
// with that device current. Concurrent first calls from several host threads all store the same
// value.
int noalloc_scratch(unsigned char** out) {
  static unsigned char* scratch_addr[64] = {nullptr};
  int dev = 0;
  B200LUT_CUDA_OK(cudaGetDevice(&dev));
  B200LUT_REQUIRE(dev >= 0 && dev < 64, B200LUT_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  if (!scratch_addr[dev]) {
    void* ptr = nullptr;
    B200LUT_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    B200LUT_REQUIRE(ptr != nullptr, B200LUT_ERR_CUDA, "no device address for the built-in scratch");
    scratch_addr[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = scratch_addr[dev];
  return B200LUT_OK;
}
}  // namespace

// Zero the tickets of the built-in scratch (its first 4 KiB), stream-ordered. The tickets return to
// zero by themselves at the end of every healthy launch; a launch that never finished (a sticky
// CUDA error on the stream, a lost context) can leave some set, and every later call on those
// tiles would then fold early. A host that has recovered from such an error calls this once.
extern "C" int b200lut_gemv_noalloc_reset(void* stream) {
  unsigned char* base = nullptr;
  if (int rc = noalloc_scratch(&base)) return rc;
  B200LUT_CUDA_OK(cudaMemsetAsync(base, 0, kNoAllocTicketBytes, cudaStream_t(stream)));
  return B200LUT_OK;
}

extern "C" int b200lut_gemv_noalloc(const void* x, const void* packed, const void* lut, void* out,
                                    int M, int N, int K, int bits, int group_size, int n_groups,
                                    int dtype, int split, void* stream) {
  B200LUT_REQUIRE(x && packed && lut && out, B200LUT_ERR_INVALID, "null x, codes, palette or output");
  B200LUT_REQUIRE(M >= 1 && M <= kMaxM, B200LUT_ERR_UNSUPPORTED,
                  "decode GEMV serves 1 <= M <= 16, got M=%d", M);
  B200LUT_REQUIRE(K > 0 && K % kChunkK == 0, B200LUT_ERR_INVALID,
                  "K must be a positive multiple of 64, got %d", K);
  B200LUT_REQUIRE(dtype == B200LUT_BF16 || dtype == B200LUT_F16, B200LUT_ERR_INVALID,
                  "dtype must be B200LUT_BF16 or B200LUT_F16");
  B200LUT_REQUIRE(aligned16(x), B200LUT_ERR_ALIGN, "x must be 16-byte aligned");
  b200lut_segment seg = {};
  seg.packed = packed;
  seg.lut = lut;
  seg.out = out;
  seg.ldo = N;
  seg.N = N;
  seg.group_size = group_size;
  seg.n_groups = n_groups;
  seg.bits = bits;

  GemvParams p = {};
  p.x = static_cast<const uint16_t*>(x);
  p.ldx = K;
  p.M = M;
  p.K = K;
  p.G = K / kChunkK;
  p.nseg = 1;
  p.epilogue = B200LUT_EPI_NONE;
  int tiles = 0, max_tables = 1;
  if (int rc = convert_segments(&seg, 1, false, p.seg, &tiles, &max_tables)) return rc;
  p.tiles_total = tiles;
  if (split <= 0) split = pick_split(tiles, p.G, sm_count_cached(), M <= 8 ? kWarpsM8 : kWarpsM16);
  B200LUT_REQUIRE(split >= 1 && split <= 16 && split <= p.G, B200LUT_ERR_INVALID,
                  "split must be 1..16 and <= K/64, got %d", split);
  // the built-in scratch bounds the problem: partial tiles of every split, plus tickets
  const size_t need = size_t(split) * size_t(tiles) * 2 * size_t(M) * kTileRows * sizeof(float);
  B200LUT_REQUIRE(size_t(tiles) * sizeof(int) <= kNoAllocTicketBytes &&
                      need <= kNoAllocScratchBytes - kNoAllocTicketBytes,
                  B200LUT_ERR_WORKSPACE,
                  "N=%d, M=%d, split=%d needs %zu bytes of fold scratch; the allocation-free entry "
                  "has %zu (lower split, or use b200lut_gemv with a caller workspace)",
                  N, M, split, need, kNoAllocScratchBytes - kNoAllocTicketBytes);

  // set-up, once per device, with that device current (see noalloc_scratch)
  unsigned char* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  p.split = split;
  p.cluster = 0;     // always the scratch fold: partials to the array, last arrival sums them
  p.tickets = reinterpret_cast<int*>(scratch);            // zero at load, self-resetting
  p.ws = reinterpret_cast<float*>(scratch + kNoAllocTicketBytes);   // fully rewritten per call
  cudaStream_t st = cudaStream_t(stream);
  if (dtype == B200LUT_BF16) return dispatch<__nv_bfloat16>(p, max_tables, false, st);
  return dispatch<__half>(p, max_tables, false, st);
}
