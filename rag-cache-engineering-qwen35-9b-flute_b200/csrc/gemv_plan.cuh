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
// its activation rows. Code bytes are therefore in flight across the dependency.
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

template <typename T, int CP, int NWARPS, int RC>
__global__ void __launch_bounds__(NWARPS * 32, 1) gemv_plan_kernel(uint8_t* plan_bytes) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int NT = NWARPS * 32;
  __shared__ JobDev job;
  __shared__ int is_last;

  const PlanHeader& hdr = *reinterpret_cast<const PlanHeader*>(plan_bytes);
  const JobDev* jobs = reinterpret_cast<const JobDev*>(plan_bytes + hdr.jobs_off);
  int* done = reinterpret_cast<int*>(plan_bytes + hdr.done_off);
  int* tickets = reinterpret_cast<int*>(plan_bytes + hdr.tickets_off);
  int* misc = reinterpret_cast<int*>(plan_bytes + hdr.misc_off);   // [0] exit count, [1] abort
  float* ws = reinterpret_cast<float*>(plan_bytes + hdr.ws_off);

  float* part = reinterpret_cast<float*>(smem);
  const uint32_t part_addr = smem_u32(smem);
  const uint32_t tbl_addr = (part_addr + kPartBytes + 0xFFFFu) & ~0xFFFFu;
  uint8_t* tbl_ptr = smem + (tbl_addr - part_addr);
  const int b = blockIdx.x, M = hdr.M;
#ifdef B200LUT_PLAN_TIMING
  long long tm_copy = 0, tm_pass = 0, tm_fold = 0, tm_total0 = clock64(), tm_mark;
#define TM_MARK() tm_mark = clock64()
#define TM_ADD(v) v += clock64() - tm_mark
#else
#define TM_MARK()
#define TM_ADD(v)
#endif

  for (int j = 0; j < hdr.njobs; ++j) {
    TM_MARK();
    __syncthreads();
    {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(jobs + j);
      uint32_t* dst = reinterpret_cast<uint32_t*>(&job);
      for (int i = threadIdx.x; i < int(sizeof(JobDev) / 4); i += NT) dst[i] = __ldcg(src + i);
    }
    __syncthreads();
    TM_ADD(tm_copy);
    const int G = job.G, total = job.tiles_total * G;
    const int lin0 = b * job.per;
    int lin1 = lin0 + job.per;
    if (lin1 > total) lin1 = total;
    const bool silu = job.epilogue == B200LUT_EPI_SILU_MUL;
    bool waited = job.dep < 0;
    for (int lin = lin0; lin < lin1;) {
      const int tile_g = lin / G, c0 = lin - tile_g * G;
      int c1 = c0 + (lin1 - lin);
      if (c1 > G) c1 = G;
      int si = 0;
      for (int s = 0; s < job.nseg; s += silu ? 2 : 1)
        if (tile_g >= job.seg[s].tile_begin) si = s;
      const int tile = tile_g - job.seg[si].tile_begin;

      TM_MARK();
      for (int plane = 0; plane < job.planes; ++plane) {
        const SegDev& sg = job.seg[si + plane];
        const int npass = sg.packed2 ? 2 : 1;
        for (int pass = 0; pass < npass; ++pass) {
          const uint8_t* packed = pass ? sg.packed2 : sg.packed;
          const uint16_t* lut = pass ? sg.lut2 : sg.lut;
          const int bits = pass ? sg.bits2 : sg.bits;
          float* dst = part + plane * kMaxM * kTileRows;
          const DepWait dep{waited ? 0 : 2, done + (job.dep < 0 ? 0 : job.dep), job.dep_target,
                            misc + 1};
#define B200LUT_PASS(B)                                                                          \
  stream_pass<T, B, CP, NWARPS, RC>(dst, pass != 0, tbl_ptr, tbl_addr, packed, lut, sg.n_groups, \
                                    sg.gs, tile, G, c0, c1, job.x, job.ldx, M, true, dep)
          switch (bits) {   // block-uniform
            case 4: B200LUT_PASS(4); break;
            case 3: B200LUT_PASS(3); break;
            case 2: B200LUT_PASS(2); break;
            default: B200LUT_PASS(1); break;
          }
#undef B200LUT_PASS
          waited = true;
        }
      }

      TM_ADD(tm_pass);
      TM_MARK();
      // ---- fold the shares of this tile and store ------------------------------------------
      const SegDev& s0 = job.seg[si];
      const SegDev* s1 = silu ? &job.seg[si + 1] : nullptr;
      const int n0 = tile * kTileRows;
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
          atomicAdd(done + j, 1);
        }
      }
      TM_ADD(tm_fold);
      lin += c1 - c0;
    }
  }
#ifdef B200LUT_PLAN_TIMING
  if (threadIdx.x == 0 && b < 4) {
    long long* t = reinterpret_cast<long long*>(misc + 16) + b * 4;
    t[0] = tm_copy; t[1] = tm_pass; t[2] = tm_fold; t[3] = clock64() - tm_total0;
  }
#endif

  // the last block out resets the completion counters for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int old = atomicAdd(misc, 1);
    if (old == int(gridDim.x) - 1) {
      for (int j = 0; j < hdr.njobs; ++j) done[j] = 0;
      misc[0] = 0;
      __threadfence();
    }
  }
}

}  // namespace
}  // namespace b200lut
