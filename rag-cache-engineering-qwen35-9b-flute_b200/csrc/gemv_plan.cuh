// Persistent decode executor: a whole list of decode GEMV jobs (the projections of a
// model step) in ONE cooperative launch, one block per SM.
// Included by gemv.cu (shares stream_pass, the pair tables and the parameter structs).
//
// Why: a 4096 x 4096 4-bit projection is 8 MB — 1.3 us of HBM time — while a kernel
// boundary costs several microseconds of drain, launch, palette fetch and first-byte
// latency. Here the boundary disappears: every block walks the job list, and for each job
// takes an equal, contiguous share of the job's (tile, k-chunk) space (so all SMs stream
// the same number of bytes whatever the tile count), requests its first codes, builds its
// pair table, and only then waits — on a completion counter — for the job that produces
// its activation rows. Code bytes are therefore in flight across the dependency. The walk
// is a flat sequence of passes (one code stream of one tile share) pipelined one ahead:
// while a pass folds, the first codes of the next pass — of the next tile or the next job —
// are already requested and its pair table is already built in the other table region.
//
// Shares of one tile held by different blocks are folded through an fp32 workspace: each
// contributor writes its partial tile, takes a ticket, and the last arrival sums the
// partials in contributor (= ascending k) order, applies the epilogue, stores, and bumps
// the job's completion counter. No block ever waits for a ticket; the only waits are the
// dependency polls, which are bounded (they give up, raise a plan-wide abort word and let
// every block drain). Results are deterministic: shares and fold order are pure functions
// of the job shapes and the grid size.
#pragma once

namespace b200lut {
namespace {

struct JobDev {
  const uint16_t* x;
  long long ldx;
  long long ws_off;         // floats from the start of the plan's workspace
  int K, G, nseg, epilogue, tiles_total, planes;
  int dep, dep_target;      // producer job (-1: none) and its tile count
  int per;                  // chunks per block (last block may hold fewer)
  int maxc;                 // most contributors a tile can have
  int ticket_off;
  int pad;
  SegDev seg[kMaxSeg];
};

struct PlanHeader {
  unsigned long long magic;
  int njobs, M, dtype, grid;
  long long jobs_off, done_off, tickets_off, misc_off, ws_off, total_bytes;   // byte offsets
  int ntickets, pad;
};
constexpr unsigned long long kPlanMagic = 0xB200'1A7E'D0C0'DE01ull;

template <typename T>
__device__ __forceinline__ void plan_store(const SegDev& s0, const SegDev* s1, int m, int n,
                                           float a, float b) {
  if (s0.bias) a += DType<T>::to_float(s0.bias[n]);
  float v = a;
  if (s1) {
    if (s1->bias) b += DType<T>::to_float(s1->bias[n]);
    v = a / (1.f + __expf(-a)) * b;
  }
  s0.out[size_t(m) * s0.ldo + n] = DType<T>::from_float(v);
}

// ---- pieces of one pass (one code stream of one tile share) --------------------------------

// First chunk of a pass into the (width-agnostic) register buffer.
__device__ __forceinline__ void first_chunk(uint32_t (&w)[32], const uint8_t* __restrict__ packed,
                                            int bits, int tile, int G, int c, int c1, int lane) {
  const size_t chunk_bytes = size_t(1024) * bits;
  const uint8_t* p = packed + (size_t(tile) * G + c) * chunk_bytes + lane * 32;
#pragma unroll
  for (int pl = 0; pl < 4; ++pl)
    ldg_stream256_if(&w[8 * pl], p + pl * 1024, (pl < bits && c < c1) ? 1u : 0u);
}

// The chunk loop of a pass: one chunk of codes in flight per warp, activations one chunk ahead.
template <typename T, int BITS, int CP, int NWARPS>
__device__ __forceinline__ void plan_kloop(float (&acc)[Plan<CP>::kAcc][4], uint32_t (&w32)[32],
                                           const uint8_t* __restrict__ packed, int tile, int G,
                                           int c0, int c1, const uint16_t* __restrict__ x,
                                           long long ldx, int M, uint32_t tbl_lane, int slot_shift) {
  using P = Plan<CP>;
  uint32_t(&w)[8 * BITS] = reinterpret_cast<uint32_t(&)[8 * BITS]>(w32);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const size_t chunk_bytes = size_t(1024) * BITS;
  const uint8_t* lane_base = packed + (size_t(tile) * G) * chunk_bytes + lane * 32;
  int c = c0 + warp;
  uint2 xa[P::kNB][4], xb[P::kNB][4];
  load_x<CP>(xa, x, ldx, c < c1 ? M : 0, c * kChunkK, gid, tig);
  for (; c < c1; c += 2 * NWARPS) {
    {
      const bool more = c + NWARPS < c1;
      load_x<CP>(xb, x, ldx, more ? M : 0, (c + NWARPS) * kChunkK, gid, tig);
      chunk_math<T, BITS, CP>(acc, w, xa, tbl_lane, slot_shift, gid,
                              lane_base + size_t(c + NWARPS) * chunk_bytes, more ? 1u : 0u);
    }
    if (c + NWARPS < c1) {
      const bool more = c + 2 * NWARPS < c1;
      load_x<CP>(xa, x, ldx, more ? M : 0, (c + 2 * NWARPS) * kChunkK, gid, tig);
      chunk_math<T, BITS, CP>(acc, w, xb, tbl_lane, slot_shift, gid,
                              lane_base + size_t(c + 2 * NWARPS) * chunk_bytes, more ? 1u : 0u);
    }
  }
#pragma unroll
  for (int a = 0; a < P::kAcc; ++a)
#pragma unroll
    for (int r = 0; r < 4; ++r) asm volatile("" ::"f"(acc[a][r]));   // lookups end here
}

// Cross-warp fold of the accumulator fragments through `red`, fixed warp order, into
// part_plane[m][row] (+= when accumulate). Caller guarantees `red` is free (a barrier after
// the last lookup of the table it aliases).
template <int CP, int NWARPS>
__device__ __forceinline__ void plan_warp_fold(const float (&acc)[Plan<CP>::kAcc][4], float* red,
                                               float* part_plane, bool accumulate, int M) {
  using P = Plan<CP>;
  constexpr int NT = NWARPS * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
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

// One pass of a block's walk through the plan (block-uniform values).
struct PassDesc {
  bool valid;
  int j, slot;                 // job index and the shared-memory copy that holds it
  int tile_g, tile, si, c0, c1, plane, pass;
  bool first_of_job, last_of_tile;
  const uint8_t* packed;
  const uint16_t* lut;
  int bits, gs, n_groups, nl;
};

template <typename T, int CP, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32, 1) gemv_plan_kernel(uint8_t* plan_bytes) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int NT = NWARPS * 32;
  using P = Plan<CP>;
  __shared__ JobDev jobbuf[2];
  __shared__ int is_last;

  const PlanHeader& hdr = *reinterpret_cast<const PlanHeader*>(plan_bytes);
  const JobDev* jobs = reinterpret_cast<const JobDev*>(plan_bytes + hdr.jobs_off);
  int* done = reinterpret_cast<int*>(plan_bytes + hdr.done_off);
  int* tickets = reinterpret_cast<int*>(plan_bytes + hdr.tickets_off);
  int* misc = reinterpret_cast<int*>(plan_bytes + hdr.misc_off);   // [0] exit count, [1] abort
  float* ws = reinterpret_cast<float*>(plan_bytes + hdr.ws_off);

  float* part = reinterpret_cast<float*>(smem);
  const uint32_t part_addr = smem_u32(smem);
  const uint32_t tbl_addr = (part_addr + kPartBytes + 0xFFFFu) & ~0xFFFFu;   // two regions follow
  uint8_t* tbl_ptr = smem + (tbl_addr - part_addr);
  const int b = blockIdx.x, M = hdr.M, njobs = hdr.njobs;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // ---- the walk: jobs in order, this block's share of each, its tiles, planes, streams -------
  int it_j = 0, it_lin = 0, it_lin1 = 0, it_plane = 0, it_pass = 0;
  bool it_loaded = false, it_first = false;
  auto advance = [&](PassDesc& d) {
    d.valid = false;
    for (;;) {
      if (it_j >= njobs) return;
      JobDev& job = jobbuf[it_j & 1];
      if (!it_loaded) {
        __syncthreads();   // nobody still reads the copy this one replaces
        const uint32_t* src = reinterpret_cast<const uint32_t*>(jobs + it_j);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&job);
        for (int i = threadIdx.x; i < int(sizeof(JobDev) / 4); i += NT) dst[i] = __ldcg(src + i);
        __syncthreads();
        const int total = job.tiles_total * job.G;
        it_lin = b * job.per;
        it_lin1 = it_lin + job.per;
        if (it_lin1 > total) it_lin1 = total;
        it_plane = it_pass = 0;
        it_loaded = true;
        it_first = true;
      }
      if (it_lin >= it_lin1) { ++it_j; it_loaded = false; continue; }
      const int G = job.G;
      const bool silu = job.epilogue == B200LUT_EPI_SILU_MUL;
      d.j = it_j; d.slot = it_j & 1;
      d.tile_g = it_lin / G;
      d.c0 = it_lin - d.tile_g * G;
      d.c1 = d.c0 + (it_lin1 - it_lin);
      if (d.c1 > G) d.c1 = G;
      int si = 0;
      for (int s = 0; s < job.nseg; s += silu ? 2 : 1)
        if (d.tile_g >= job.seg[s].tile_begin) si = s;
      d.si = si;
      d.tile = d.tile_g - job.seg[si].tile_begin;
      d.plane = it_plane; d.pass = it_pass;
      const SegDev& sg = job.seg[si + it_plane];
      const int npass = sg.packed2 ? 2 : 1;
      d.packed = it_pass ? sg.packed2 : sg.packed;
      d.lut = it_pass ? sg.lut2 : sg.lut;
      d.bits = it_pass ? sg.bits2 : sg.bits;
      d.gs = sg.gs; d.n_groups = sg.n_groups;
      d.nl = sg.gs >= kTileRows ? 1 : kTileRows / sg.gs;
      d.first_of_job = it_first;
      it_first = false;
      // step
      d.last_of_tile = false;
      if (++it_pass >= npass) {
        it_pass = 0;
        if (++it_plane >= job.planes) {
          it_plane = 0;
          d.last_of_tile = true;
          it_lin += d.c1 - d.c0;
        }
      }
      d.valid = true;
      return;
    }
  };

#define TM_MARK()
#define TM_ADD(v)
  PassDesc cur, nxt;
  uint32_t w[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) w[i] = 0u;
  uint32_t lutv[LutRegs<NT>::n];
  advance(cur);
  int region = 0;
  if (cur.valid) {
    first_chunk(w, cur.packed, cur.bits, cur.tile, jobbuf[cur.slot].G, cur.c0 + warp, cur.c1, lane);
    table_fetch<NT>(lutv, cur.lut, cur.bits, cur.n_groups, cur.tile * kTileRows, cur.gs, cur.nl);
    table_store<NT>(tbl_ptr, lutv, cur.bits, cur.nl);
  }

  while (cur.valid) {
    const JobDev& job = jobbuf[cur.slot];
    uint8_t* my_tbl = tbl_ptr + size_t(region) * kTableBytes;
    const uint32_t my_tbl_addr = tbl_addr + uint32_t(region) * kTableBytes;
    TM_MARK();
    // look one pass ahead first (may load the next job's descriptor; block-uniform) and
    // request that pass's palette: none of it depends on the producer of this job's rows
    advance(nxt);
    if (nxt.valid)
      table_fetch<NT>(lutv, nxt.lut, nxt.bits, nxt.n_groups, nxt.tile * kTileRows, nxt.gs, nxt.nl);
    // the producer of this job's activation rows must have finished (bounded poll)
    if (cur.first_of_job && job.dep >= 0 && threadIdx.x == 0)
      dep_poll(DepWait{2, done + job.dep, job.dep_target, misc + 1});
    __syncthreads();                       // table of this pass is complete; dependency met
    TM_ADD(tm_head);
    TM_MARK();
    float acc[P::kAcc][4];
#pragma unroll
    for (int a = 0; a < P::kAcc; ++a)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[a][r] = 0.f;
    uint32_t token;
    asm volatile("mov.u32 %0, 0;" : "=r"(token));
    const uint32_t tbl_lane = my_tbl_addr + lane * 4 + token;
    const int slot_shift = cur.nl == 1 ? 3 : 2;
#define B200LUT_KLOOP(B)                                                                        \
  plan_kloop<T, B, CP, NWARPS>(acc, w, cur.packed, cur.tile, job.G, cur.c0, cur.c1, job.x, job.ldx, \
                               M, tbl_lane, slot_shift)
    switch (cur.bits) {   // block-uniform
      case 4: B200LUT_KLOOP(4); break;
      case 3: B200LUT_KLOOP(3); break;
      case 2: B200LUT_KLOOP(2); break;
      default: B200LUT_KLOOP(1); break;
    }
#undef B200LUT_KLOOP

    TM_ADD(tm_loop);
    TM_MARK();
    // codes and table of the next pass go out before this pass folds
    if (nxt.valid) {
      first_chunk(w, nxt.packed, nxt.bits, nxt.tile, jobbuf[nxt.slot].G, nxt.c0 + warp, nxt.c1, lane);
      table_store<NT>(tbl_ptr + size_t(region ^ 1) * kTableBytes, lutv, nxt.bits, nxt.nl);
    }
    __syncthreads();                       // every warp is done with this pass's table
    plan_warp_fold<CP, NWARPS>(acc, reinterpret_cast<float*>(my_tbl),
                               part + cur.plane * kMaxM * kTileRows, cur.pass != 0, M);

    TM_ADD(tm_fold);
    TM_MARK();
    if (cur.last_of_tile) {
      // ---- fold the shares of this tile across blocks and store -----------------------------
      const bool silu = job.epilogue == B200LUT_EPI_SILU_MUL;
      const SegDev& s0 = job.seg[cur.si];
      const SegDev* s1 = silu ? &job.seg[cur.si + 1] : nullptr;
      const int G = job.G, n0 = cur.tile * kTileRows, tile_g = cur.tile_g;
      const int first = (tile_g * G) / job.per, last = (tile_g * G + G - 1) / job.per;
      const int nctr = last - first + 1, ci = b - first;
      const int plane_elems = M * kTileRows, tile_elems = job.planes * plane_elems;
      __syncthreads();
      bool wrote = true;
      if (nctr == 1) {
        for (int idx = threadIdx.x; idx < plane_elems; idx += NT) {
          const int m = idx >> 7, row = idx & 127;
          plan_store<T>(s0, s1, m, n0 + row, part[m * kTileRows + row],
                        silu ? part[(kMaxM + m) * kTileRows + row] : 0.f);
        }
      } else {
        float* tile_ws = ws + job.ws_off + size_t(tile_g) * job.maxc * tile_elems;
        float* mine = tile_ws + size_t(ci) * tile_elems;
        for (int idx = threadIdx.x; idx < tile_elems; idx += NT) {
          const int pl = idx / plane_elems, rem = idx - pl * plane_elems;
          __stcg(mine + idx, part[(pl * kMaxM + (rem >> 7)) * kTileRows + (rem & 127)]);
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
          const int old = atomicAdd(tickets + job.ticket_off + tile_g, 1);
          is_last = (old == nctr - 1);
          if (is_last) tickets[job.ticket_off + tile_g] = 0;   // ready for the next launch
        }
        __syncthreads();
        wrote = is_last != 0;
        if (wrote) {
          __threadfence();
          for (int idx = threadIdx.x; idx < plane_elems; idx += NT) {
            const int m = idx >> 7, row = idx & 127;
            float a = 0.f, bb = 0.f;
            for (int qi = 0; qi < nctr; ++qi) {   // contributor order = ascending k
              const float* src = tile_ws + size_t(qi) * tile_elems;
              a += __ldcg(src + idx);
              if (silu) bb += __ldcg(src + plane_elems + idx);
            }
            plan_store<T>(s0, s1, m, n0 + row, a, bb);
          }
        }
      }
      if (wrote) {
        __syncthreads();
        if (threadIdx.x == 0) {
          __threadfence();
          atomicAdd(done + cur.j, 1);
        }
      }
    }
    TM_ADD(tm_tile);
    cur = nxt;
    region ^= 1;
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

}  // namespace
}  // namespace b200lut
