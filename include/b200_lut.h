/*
 * b200_lut.h — C ABI of the B200 (sm_100a) LUT-palettized linear library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL = the legacy default stream) and returns
 * an integer status (B200LUT_OK = 0). No function allocates device memory unless
 * its comment says so; the caller owns every buffer. After a non-zero status,
 * b200lut_last_error() returns a message for the calling thread.
 *
 * Each declaration names the interface of the reference project
 * (pkhairkh/rag-cache-engineering-qwen35-9b-flute) that it replaces.
 *
 * Semantics shared by all compute entry points
 *   W[n, k] = LUT[min(n / group_size, n_groups - 1)][code(n, k)]   (exact lookup)
 *   y[m, n] = sum_k x[m, k] * W[n, k]   accumulated in fp32, rounded once
 * dtype: element type of x, LUT entries and outputs (B200LUT_BF16 / B200LUT_F16).
 */
#ifndef B200_LUT_H_
#define B200_LUT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200LUT_OK = 0,
  B200LUT_ERR_INVALID = 1,      /* bad argument (shape, null pointer, range) */
  B200LUT_ERR_UNSUPPORTED = 2,  /* valid request outside the compiled kernel table */
  B200LUT_ERR_CUDA = 3,         /* a CUDA runtime call or launch failed */
  B200LUT_ERR_WORKSPACE = 4,    /* caller's workspace is too small */
  B200LUT_ERR_ALIGN = 5,        /* a pointer misses its required alignment */
  B200LUT_ERR_DEVICE = 6        /* a kernel reported a device-side status (bounded wait ran out) */
};

enum { B200LUT_BF16 = 0, B200LUT_F16 = 1 };

/* Launch flags of the compute entry points (`flags` argument). */
enum {
  B200LUT_FLAG_PDL = 1,          /* programmatic dependent launch: everything that does not depend
                                    on the previous kernel of the stream (code prefetch, palette
                                    fetch, table build) runs before the launch waits for it */
  B200LUT_FLAG_TILE_KERNEL = 2,  /* decode GEMV: run the tile x K-split kernel */
  B200LUT_FLAG_ROWS_KERNEL = 4,  /* decode GEMV: run the row-range kernel where it serves the shapes
                                    (4-bit codes, one stream, M <= 8, split = 0, no exchange). It
                                    is the library's choice for those shapes anyway, unless the
                                    process runs with B200LUT_GEMV_KERNEL=tile */
  B200LUT_FLAG_CTA_PAIRS = 8     /* prefill GEMM: run launches of M >= 256 rows with an even number of
                                    128-row tiles as pairs of CTAs (tcgen05 cta_group::2: one MMA
                                    covers 256 weight rows, each CTA fetches half of the activation
                                    tile; no multicast load). Same results bit for bit, measured
                                    slower than one CTA per tile, so it is never the default */
};

/* Epilogue selector of b200lut_gemv_multi / b200lut_gemm. */
enum {
  B200LUT_EPI_NONE = 0,
  B200LUT_EPI_SILU_MUL = 1      /* segments come in (gate, up) pairs: out = silu(gate) * up */
};

/* Library version (major * 100 + minor). */
int b200lut_version(void);

/* Message of the calling thread's last failure ("" if none). Replaces the
 * TORCH_CHECK exception text of the reference's host wrappers
 * (src/flute_extended/src/kernel_gemv.cu:338-454). */
const char* b200lut_last_error(void);

/* Device-side status of the tensor-core kernels on the current device: 0 = none;
 * non-zero = a bounded wait inside a kernel ran out (the kernel then returned early
 * with its tensor memory freed and its output undefined). Synchronises the device
 * read; clears the word. No counterpart in the reference (its kernels never wait).
 * 0x6000: an embedding gather met an id outside its table (that row was written as zeros). */
int b200lut_device_status(void);

/* Number of SMs of the current device (used by the split policy). */
int b200lut_sm_count(void);

/* ------------------------------------------------------------------------- *
 * Weight layout
 * ------------------------------------------------------------------------- */

/* Bytes of the slab-layout code buffer for an [N, K] matrix at `bits` per code
 * (= N*K*bits/8, the same count as the idxN blob; reference:
 * src/flute_extended/flute_extended/idxN.py:111-114). 0 on invalid shape. */
size_t b200lut_packed_bytes(int N, int K, int bits);

/* One-time conversion of an idxN blob (device) into this library's slab layout
 * (device, 16-byte aligned, b200lut_packed_bytes long). Replaces the consumer
 * side of the idxN format: src/flute_extended/flute_extended/idxN.py:37-55,
 * 267-291 (unpack_idxn) and the fragment-direct readers of
 * src/flute_extended/include/flute/gemv.cuh:50-96. Requires N % 128 == 0,
 * K % 64 == 0, bits in 1..4. */
int b200lut_repack_from_idxn(const void* idxn_blob, void* packed, int N, int K, int bits,
                             void* stream);

/* Inverse conversion (slab layout -> idxN blob), for artifact export and
 * round-trip checks. Reference: idxN.py:235-264 (pack_idxn). */
int b200lut_repack_to_idxn(const void* packed, void* idxn_blob, int N, int K, int bits,
                           void* stream);

/* Logical code matrix [N, K] uint8 from the slab layout. Reference:
 * src/scripts/palettized_modules.py:658-666 (_logical_indices_numpy). */
int b200lut_unpack_codes(const void* packed, uint8_t* codes, int N, int K, int bits, void* stream);

/* Dequantised weight export: out[n*K + k] = the 16-bit LUT entry of W[n, k]
 * (raw bits, dtype of the LUT). Replaces reference_dequant
 * (src/scripts/palettized_modules.py:125-162) as the bit-exactness probe. */
int b200lut_dequant(const void* packed, const void* lut, int n_groups, void* out,
                    int N, int K, int bits, int group_size, void* stream);

/* ------------------------------------------------------------------------- *
 * Decode GEMV (M <= 16)
 * ------------------------------------------------------------------------- */

/* One palettized projection ("segment") of a decode launch. Replaces one row
 * of the reference's CPU int64 [count, 15] segment table
 * (src/flute_extended/include/flute/entrypoints.h:105-122). */
typedef struct b200lut_segment {
  const void* packed;    /* stream-1 codes, slab layout */
  const void* lut;       /* stream-1 palette [n_groups, 2^bits], dtype */
  const void* packed2;   /* stream-2 codes or NULL */
  const void* lut2;      /* stream-2 palette [n_groups, 2^bits2] or NULL */
  const void* bias;      /* [N] dtype or NULL; added in fp32 before the one rounding */
  void* out;             /* [M, ldo] dtype; with EPI_SILU_MUL only the gate segment's out is written */
  int64_t ldo;           /* elements between consecutive rows of out */
  int N;                 /* output features of this segment (multiple of 128) */
  int group_size;        /* rows per palette (power of two >= 32, or any multiple of 128) */
  int n_groups;          /* palette rows actually present (row-group index is clamped) */
  int bits;              /* stream-1 width (1..4) */
  int bits2;             /* stream-2 width, 0 if absent */
  int res_rank;          /* R of the fused low-rank residual (a multiple of 8), 0 if absent */
  const void* resA;      /* [N, R] dtype, row-major: out[m, n] += sum_r res_t[m, r] * resA[n, r] */
  const void* res_t;     /* x @ resB^T. Decode GEMV: fp32 [M, res_ldt] from
                            b200lut_residual_project. Prefill GEMM: dtype [M, res_ldt] from
                            b200lut_residual_project_rows, a block of 64 * ceil(R / 64) columns
                            whose columns beyond R are zero; the blocks of the projections of a
                            merged launch lie side by side in one matrix (one res_ldt). */
  int64_t res_ldt;       /* elements between consecutive rows of res_t */
} b200lut_segment;

/* First factor of the low-rank residual of the decode path: t[m, r] = sum_k x[m, k] *
 * resB[r, k] in fp32, M <= 16. resB is [R, K] dtype, row-major; the rB factors of projections
 * that share x (Q/K/V, gate/up) may be stacked along r so that one call serves a merged
 * launch. The GEMV that follows adds sum_r t[m, r] * resA[n, r] to its fp32 sums before bias
 * and the single rounding (segment fields res_rank / resA / res_t / res_ldt). Replaces the
 * residual branch the reference's split-K GEMV computes inside its launch
 * (src/flute_extended/src/kernel_gemv_splitk.cu:260-292, 340-349; R <= 256 there).
 * flags bit 0: programmatic dependent launch. */
int b200lut_residual_project(const void* x, int64_t ldx, int M, int K, int dtype,
                             const void* resB, int R, float* t, int64_t ldt, int flags,
                             void* stream);

/* The same first factor for the prefill GEMM, any M: t[m, c] = round_dtype(sum_k x[m, k] *
 * resB[c, k]) for c < R and 0 for R <= c < cols, t a [M, ldt] dtype matrix; cols is a multiple
 * of 64, ldt >= cols a multiple of 8. The rounding of t to the factors' dtype is the
 * reference route's (src/scripts/palettized_modules.py:1363-1364). The prefill GEMM then
 * feeds t and the projection's resA rows to its accumulator as extra k-blocks
 * (segment fields res_rank / resA / res_t / res_ldt), so the residual, the bias and the code
 * streams are rounded once, together — the reference's streaming kernel accumulates the
 * residual inside its launch the same way
 * (src/flute_extended/src/kernel_streaming.cu:1438-1463). flags bit 0: programmatic
 * dependent launch. */
int b200lut_residual_project_rows(const void* x, int64_t ldx, int M, int K, int dtype,
                                  const void* resB, int R, void* t, int64_t ldt, int cols,
                                  int flags, void* stream);

/* Scratch bytes b200lut_gemv_multi needs for (segments, M, split): zero when the
 * split is reduced through thread-block-cluster shared memory (split <= 8),
 * else the fp32 partial buffer + tickets of the workspace fold. Reference:
 * gemv_workspace_for, src/flute_extended/src/gemv_host.cpp:45-78. */
size_t b200lut_gemv_workspace_bytes(int total_rows, int M, int split);

/* Split-K factor the library would pick for `tiles` 128-row tiles over K.
 * Reference: gemv_pick_split, src/flute_extended/src/gemv_host.cpp:29-38
 * (re-derived for 148 SMs x 2 resident blocks). */
int b200lut_gemv_pick_split(int tiles, int K);

/* y_s = x @ W_s^T for 1..8 segments that share the activation rows x [M, K]
 * (row stride ldx elements), M <= 16. Replaces qgemm_cutlass_gemv_stream,
 * qgemm_cutlass_gemv_splitk_stream, qgemm_cutlass_gemv_multi and (with
 * B200LUT_EPI_SILU_MUL) qgemm_cutlass_gemv_mlp
 * (src/flute_extended/include/flute/entrypoints.h:49-122).
 * split: 0 = library policy, else 1..16. workspace: needed only when
 * b200lut_gemv_workspace_bytes(...) > 0; must be zero-filled once before first
 * use (tickets reset themselves) and is used by one launch at a time.
 * flags bit 0: launch with programmatic dependent launch, so the weight
 * prefetch overlaps the tail of the previous kernel in the stream. */
int b200lut_gemv_multi(const void* x, int64_t ldx, int M, int K, int dtype,
                       const b200lut_segment* segs, int nseg, int epilogue, int split,
                       void* workspace, size_t workspace_bytes, int flags, void* stream);

/* Single-projection convenience form of b200lut_gemv_multi (one stream, no bias).
 * Replaces qgemm_cutlass_gemv_stream (entrypoints.h:49-60). */
int b200lut_gemv(const void* x, const void* packed, const void* lut, void* out,
                 int M, int N, int K, int bits, int group_size, int n_groups, int dtype,
                 int split, void* workspace, size_t workspace_bytes, void* stream);

/* b200lut_gemv for callers that cannot hand the library any memory — a host whose device
 * pool is carved up once at start-up, a plug-in invoked where cudaMalloc is forbidden, a
 * process without an allocator. Same arithmetic as b200lut_gemv, but the split-K fold always
 * goes through scratch, and that scratch is an 8 MiB array built into the library image
 * (every device that loads the library holds it until exit); the call allocates and frees
 * nothing. Limit: split * (N/128) * M * 1024 bytes of partial tiles must fit 8 MiB - 4 KiB
 * and N <= 131072; larger requests return B200LUT_ERR_WORKSPACE with the sizes in the
 * message. split: 0 = library policy, else 1..16. The first call on each device looks up
 * the array's device address (make that call before any stream capture). All calls share
 * the array: launches that overlap on the GPU race; stream-ordered calls are safe (partials
 * are fully rewritten by each call, tickets return to zero by themselves).
 * This entry point has no counterpart in the reference. */
int b200lut_gemv_noalloc(const void* x, const void* packed, const void* lut, void* out,
                         int M, int N, int K, int bits, int group_size, int n_groups, int dtype,
                         int split, void* stream);

/* Stream-ordered reset of the tickets of the built-in scratch of b200lut_gemv_noalloc (a
 * cudaMemsetAsync over its first 4 KiB; allocates nothing). The tickets return to zero at the end
 * of every healthy launch, so ordinary use never needs this. A launch that did not finish (a
 * sticky CUDA error on its stream, a lost context that the host recovered from) can leave some
 * set, and later calls on those tiles would then fold their partial sums too early; a caller-
 * owned workspace is re-zeroed with a memset in that situation, the built-in array with this
 * call. This entry point has no counterpart in the reference. */
int b200lut_gemv_noalloc_reset(void* stream);

/* ---- column-parallel exchange: the all-gather folded into the GEMV ---------------------
 *
 * On G GPUs of one box every rank owns N/G output rows of a projection; a consumer with a
 * full-K input (down_proj after the SiLU*mul of gate/up) needs all ranks' slices. The
 * reference has no multi-GPU path; the plain form of this step is an NCCL all-gather between
 * two launches. The fused form removes that launch: the producing GEMV stores every output
 * element into its own buffer AND, over NVLink, at the same position of every peer's buffer;
 * every block of the grid then writes this rank's push count into its own flag word in every
 * rank's flag array (one system-wide fence per block, no serialisation behind a last
 * block); the consuming GEMV waits (bounded, about one second; on expiry the launch carries on
 * and b200lut_device_status() turns nonzero) until all world x producer_blocks flags have
 * reached the number of waits done on the channel plus one, and only then reads its
 * activation rows. With programmatic dependent launch the waiting launch does not wait for
 * the previous grid to drain — the flags (its own rank's included) are its whole dependency,
 * so its code prefetch and table build overlap the producer's tail and the NVLink latency.
 *
 * Contract: all ranks issue the same sequence of pushes and waits on the same exchange
 * words; a buffer that is pushed into must not be pushed into again before every rank's
 * consumer of the previous contents has finished (two or more layers with a buffer each
 * give that for free, because a rank cannot get a step ahead of a peer's consumer).
 * peer memory is only ever written with plain stores by this library's own kernels. */
#define B200LUT_MAX_PEERS 8

typedef struct b200lut_exchange {
  int world, rank;        /* 1 <= world <= 8 */
  int push;               /* nonzero: mirror outputs to the peers and signal them */
  int wait;               /* nonzero: wait for all ranks' signals before reading x */
  int producer_blocks;    /* blocks of the pushing launch (b200lut_gemv_launch_blocks for split = 0,
                             tiles x split for an explicit split); the same on every rank;
                             push: checked against the launch; wait: flags per rank */
  int wait_ms;            /* wait: bound of the flag wait in milliseconds, 1..1000; 0 = the default
                             (about one second). When it runs out the launch carries on with
                             whatever its activation buffer holds, b200lut_device_status()
                             returns 0x7000 + the rank whose flag was missing, and every later
                             wait on the device returns at once until that call has cleared the
                             word: outputs are undefined from the first expiry until the host
                             has read the status and re-zeroed the exchange words. */
  int64_t peer_delta[B200LUT_MAX_PEERS];  /* bytes from a local output address to the same
                                             element of rank q's buffer (entry `rank` unused) */
  void* peer_flag[B200LUT_MAX_PEERS];     /* rank q's flag array u32[world][producer_blocks]
                                             (entry `rank`: the local one) */
  void* ticket;           /* local u32, zero before first use (push) */
  void* epoch;            /* local u32, zero before first use: pushes done (push) */
  const void* flags;      /* the local flag array, zero before first use (wait) */
  void* wait_ticket;      /* local u32, zero before first use (wait) */
  void* wait_count;       /* local u32, zero before first use: waits done (wait) */
  int sentinel;           /* nonzero on BOTH launches of a channel: no flags and no system-wide fence.
                             The exchanged rows themselves say what has arrived: the buffer starts
                             filled with 0xFFFF (a pattern no finite value and no converted NaN
                             has), every rank's producer stores its elements into it with plain
                             16-bit stores, the waiting launch polls each 16-byte piece it stages
                             until none of its elements is 0xFFFF (bounded by wait_ms), and its
                             last block refills the rows with 0xFFFF when every block has staged
                             them. Served by the row-range kernel only (4-bit single-stream
                             segments, M <= 8 and rows that fit its shared memory); other launches
                             return B200LUT_ERR_UNSUPPORTED. */
  int reserved;
} b200lut_exchange;

/* Blocks of the launch that b200lut_gemv_multi / b200lut_gemv_exchange would make for these
 * segments with split = 0 (the library's policy) — the producer_blocks of an exchange whose
 * pushing launch they describe. Output pointers of the segments may be NULL here. 0 on invalid
 * arguments. The policy picks between the two decode kernels by shape and M; a launch that
 * carries an input transform or a flag-less (sentinel) exchange always runs the row-range
 * kernel, so pass B200LUT_FLAG_ROWS_KERNEL here for such a launch. No counterpart in the
 * reference. */
int b200lut_gemv_launch_blocks(int M, int K, const b200lut_segment* segs, int nseg, int epilogue,
                               int flags);

/* b200lut_gemv_multi with the exchange described above (ex == NULL: identical to it).
 * No counterpart in the reference. */
int b200lut_gemv_exchange(const void* x, int64_t ldx, int M, int K, int dtype,
                          const b200lut_segment* segs, int nseg, int epilogue, int split,
                          void* workspace, size_t workspace_bytes, int flags,
                          const b200lut_exchange* ex, void* stream);

/* What a decode launch does to its activation rows before it multiplies, inside the launch
 * (every block transforms the rows it stages; no extra kernel, no round trip through memory):
 *   x_mul      non-NULL: x := silu(x) * x_mul, element-wise, fp32 inside, one rounding — the
 *              act_fn(gate) * up in front of down_proj (src/scripts/modeling.py:1001-1003) when
 *              gate and up were left as two plain outputs; x_mul has x's shape and row stride;
 *   rot_signs  non-NULL: x := Hadamard rotation of x, descending power-of-two segments of K,
 *              signs on the output, 1/sqrt(b) — bit-identical to b200lut_fht(FORWARD). Replaces
 *              the reference's fused prologue gemv_fht_prologue
 *              (src/flute_extended/include/flute/gemv.cuh:305-351; kernel_gemv.cu:579-776);
 *   awq_scale  with rot_signs: the compensated form ((x * s) H * signs / sqrt(b)) / s
 *              (b200lut_fht mode AWQ). (K,) fp32 each.
 * x_mul is applied first. Served for 4-bit single-stream segments, M <= 8, split = 0 (the
 * row-range kernel); other requests return B200LUT_ERR_UNSUPPORTED and the caller transforms the
 * rows with b200lut_silu_mul / b200lut_fht first. */
typedef struct b200lut_input {
  const void* x_mul;
  const float* rot_signs;
  const float* awq_scale;
  /* Non-zero: every segment of the launch has its own fold — seg_rot_signs[i] (NULL: segment
   * i takes the rows as they are) and seg_awq_scale[i] — as the segment table of the
   * reference's merged kernels carries a rotation per segment
   * (src/flute_extended/include/flute/gemv.cuh:112-133,
   * src/flute_extended/src/kernel_gemv_multi.cu:101-334). rot_signs / awq_scale must then be
   * NULL and the epilogue B200LUT_EPI_NONE; a launch block never crosses a segment. */
  int per_segment;
  const float* seg_rot_signs[8];
  const float* seg_awq_scale[8];
} b200lut_input;

/* b200lut_gemv_exchange with an input transform (in == NULL: identical to it). */
int b200lut_gemv_input(const void* x, int64_t ldx, int M, int K, int dtype,
                       const b200lut_segment* segs, int nseg, int epilogue, int split,
                       void* workspace, size_t workspace_bytes, int flags,
                       const b200lut_exchange* ex, const b200lut_input* in, void* stream);

/* Sharing a device buffer between the ranks (processes) of one box. export: fills a 64-byte
 * handle for the allocation that contains ptr and the offset of ptr inside it (the buffer
 * must come from cudaMalloc, directly or through a caching allocator). open: maps another
 * process's allocation into this one (peer access over NVLink) and returns its base; close
 * unmaps it. Handles travel between the processes by any host channel. */
int b200lut_peer_export(const void* ptr, unsigned char handle[64], int64_t* offset);
int b200lut_peer_open(const unsigned char handle[64], void** base);
int b200lut_peer_close(void* base);

/* One decode GEMV launch inside a persistent plan: what b200lut_gemv_multi takes, plus
 * the index of the earlier job that produces this job's activation rows (-1: none). */
typedef struct b200lut_job {
  const void* x;          /* [M, ldx] activation rows (device) */
  int64_t ldx;
  int K;
  int nseg;               /* 1..8 */
  int epilogue;           /* B200LUT_EPI_* */
  int dep;                /* producer job index (< this job's index) or -1 */
  b200lut_segment segs[8];
} b200lut_job;

/* A plan runs a whole list of decode jobs (all projections of a model step) in ONE
 * cooperative launch with one block per SM: code bytes stay in flight across job
 * boundaries, and a job starts its math when the job it depends on has finished
 * (bounded wait on a completion counter). Replaces the reference's per-module launch
 * chain under CUDA-graph replay (src/docs/ARCHITECTURE.md section 3,
 * src/scripts/palettized_modules.py:870-983).
 * b200lut_plan_bytes: size of the caller-owned device buffer that holds the job table,
 * counters and the split-fold workspace (0 on invalid input).
 * b200lut_plan_build: validates and uploads the jobs (synchronises the stream).
 * b200lut_plan_run: one launch; may be captured in a CUDA graph; launches of one plan
 * must not overlap. b200lut_plan_status: B200LUT_ERR_DEVICE if a wait ever ran out. */
size_t b200lut_plan_bytes(const b200lut_job* jobs, int njobs, int M, int dtype);
int b200lut_plan_build(void* plan, size_t plan_bytes, const b200lut_job* jobs, int njobs, int M,
                       int dtype, void* stream);
int b200lut_plan_run(void* plan, int M, int dtype, void* stream);
int b200lut_plan_status(const void* plan);
/* Which kernel a built plan runs: 1 = the row-range block body, job after job (every job
 * 4-bit, single-stream, M <= 8, one block per SM at most); 0 = the tile-share kernel (any other
 * mix, or B200LUT_PLAN_KERNEL=tile in the environment); negative = not a plan buffer. */
int b200lut_plan_form(const void* plan);
/* Call before the buffer of a built plan is freed or reused for something else (with the
 * buffer's device current): the library keeps one small host-side record per row-range plan
 * (what b200lut_plan_run must know to launch it) and drops it here. Rebuilding a plan in the
 * same buffer replaces the record by itself. NULL is accepted. */
int b200lut_plan_release(const void* plan);

/* ------------------------------------------------------------------------- *
 * Prefill GEMM (M > 16), tcgen05 / TMEM
 * ------------------------------------------------------------------------- */

/* out[M, N] = x[M, K] @ W^T (+ bias). Replaces qgemm_cutlass_streaming
 * (src/flute_extended/include/flute/entrypoints.h:31-37, kernels
 * src/flute_extended/src/kernel_streaming.cu:987-1108). x rows must be
 * 16-byte aligned (K % 8 == 0 and ldx % 8 == 0). With B200LUT_EPI_SILU_MUL,
 * packed/lut are the gate projection and packed2/lut2 the up projection of the
 * same shape and out = silu(x Wg^T) * (x Wu^T); otherwise a non-NULL packed2 is
 * a second stream summed into the same accumulator. */
int b200lut_gemm(const void* x, int64_t ldx, int M, int K, int dtype,
                 const b200lut_segment* seg, int epilogue, int flags, void* stream);

/* b200lut_gemm with a caller-owned scratch buffer. When the tile count (N/128 x ceil(M/256))
 * leaves a partly filled last round of SMs, each tile of that round is cut along K into 2..8
 * parts, one per SM; the parts exchange fp32 partial tiles through the workspace and each
 * finishes a share of the tile's columns, adding the partial sums in ascending-k order
 * (deterministic). b200lut_gemm_workspace_bytes gives the size for a shape on the current
 * device (0: the shape gains nothing); with a NULL or smaller buffer the whole-tile schedule
 * runs. The buffer must be zero-filled once before first use (its first 4 KiB are counters
 * that return to zero by themselves), 16-byte aligned, and serves one launch at a time; it may
 * be reused across shapes. No counterpart in the reference (its GEMM is one tile per block). */
size_t b200lut_gemm_workspace_bytes(int M, int N, int K);
int b200lut_gemm_ws(const void* x, int64_t ldx, int M, int K, int dtype,
                    const b200lut_segment* seg, int epilogue, int flags,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Several projections that share x as ONE prefill launch: Q/K/V(/z) of an attention block, or
 * gate and up of an MLP (out[i] = x @ W_i^T + bias_i, every projection into its own out / ldo).
 * The row tiles of the projections are concatenated, so the launch fills the SMs like one wide
 * projection (and the split schedule of b200lut_gemm_ws applies to the sum; size the workspace
 * with b200lut_gemm_workspace_bytes(M, sum of N, K)). 1 <= nseg <= 4; one code stream per
 * projection, one code width and one group size (>= 64) for all; K >= 128. Counterpart of
 * the merged decode launch (b200lut_gemv_multi) at prefill width; the reference runs one
 * streaming GEMM per projection (src/scripts/palettized_modules.py:1468-1641 at M > 16). */
int b200lut_gemm_multi(const void* x, int64_t ldx, int M, int K, int dtype,
                       const b200lut_segment* segs, int nseg, int flags,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Prefill GEMM of ONE projection with two code streams of any widths (the mixed-radix recipes,
 * e.g. 4 + 2 bits): out = x @ (W1 + W2)^T + bias with fp32 sums and ONE rounding, as two
 * tensor-core launches — the first leaves its fp32 sums in `scratch` ([M][N] floats,
 * b200lut_gemm_two_stream_bytes), the second adds them to its own before bias and rounding
 * (stream 1 first, the reference's order, src/scripts/palettized_modules.py:1241-1251).
 * group_size >= 64, K >= 128; b200lut_gemm serves the 4 + 4 bit pair and group size 32 in one
 * launch. Replaces the second-stream branch of the reference's streaming GEMM
 * (src/flute_extended/src/kernel_streaming.cu:1246-). */
size_t b200lut_gemm_two_stream_bytes(int M, int N);
int b200lut_gemm_two_stream(const void* x, int64_t ldx, int M, int K, int dtype,
                            const b200lut_segment* seg, int flags, void* scratch,
                            size_t scratch_bytes, void* stream);

/* ---- K-grouped palettes ---------------------------------------------------------------------
 *
 * out[m, n] = sum_k x[m, k] * lut_k[k / 128][n][code(n, k)] (+ bias[n]), M <= 16: one
 * 2^bits-entry palette per (block of 128 input columns, output row); lut_k is
 * [K / 128][N][2^bits] in dtype, the codes are in the slab layout. fp32 sums, one rounding.
 * The reference groups palettes along the output rows and has no kernel of this form; its
 * reference route expresses it as K / 128 modules of 128 columns with group_size = 1
 * (src/scripts/palettized_modules.py:125-162), summed in fp32. split = 0 lets the library pick
 * the number of K ranges (b200lut_gemv_kgrouped_split); with split > 1 the caller passes a
 * zero-initialised workspace of b200lut_gemv_kgrouped_workspace_bytes(N, M, split) bytes
 * (fp32 partial sums folded in range order by the last block; the tickets reset themselves).
 * The N / 128 tickets sit at the start of the workspace and the partial sums behind them: a
 * caller that reuses one workspace for different N zeroes its first N / 128 * 4 + 256 bytes when
 * N grows. With split = 0 and 4-bit codes at M <= 8 the library runs the row-range form of the
 * kernel instead (one block per range of 32-row units over all of K, no workspace). */
int b200lut_gemv_kgrouped_split(int N, int K);
size_t b200lut_gemv_kgrouped_workspace_bytes(int N, int M, int split);
int b200lut_gemv_kgrouped(const void* x, int64_t ldx, int M, int K, int dtype,
                          const void* packed, const void* lut_k, const void* bias,
                          int N, int bits, void* out, int64_t ldo, int split,
                          void* workspace, size_t workspace_bytes, void* stream);

/* The same projection at any M on the tensor cores (the prefill form): the persistent tcgen05
 * kernel of b200lut_gemm with a lookup that reads every weight out of its row's palette — the
 * palettes of a lookup warp's 32 rows travel with the codes through a shared-memory ring. fp32
 * sums, one rounding. workspace: optional scratch of the split schedule, as b200lut_gemm_ws takes
 * it (b200lut_gemm_workspace_bytes(M, N, K) bytes, zero-filled once); NULL runs whole tiles.
 * flags bit 0: programmatic dependent launch. */
int b200lut_gemm_kgrouped(const void* x, int64_t ldx, int M, int K, int dtype,
                          const void* packed, const void* lut_k, const void* bias, int N,
                          int bits, void* out, int64_t ldo, int flags, void* workspace,
                          size_t workspace_bytes, void* stream);

/* ---- embedding gather ----------------------------------------------------------------------
 *
 * out[t, :] = W[ids[t], :] for n_ids int64 ids on the device, W the palettized [N, K] table
 * described by `table` (packed / lut / bits, optional packed2 / lut2 / bits2, group_size,
 * n_groups, N; resA + res_rank with `resB` [R, K] for the low-rank residual; out / ldo; bias and
 * res_t are ignored). Arithmetic of the reference's PalettizedEmbedding.forward
 * (src/scripts/palettized_modules.py:2276-2335): stream 1 palette entry, plus the stream 2
 * entry in ONE add rounded to the palette dtype (stream 1 first), widened to fp32, plus
 * sum_r resA[id, r] * resB[r, k] in fp32 (ascending r), then one rounding to dtype — or no
 * rounding with out_fp32 != 0 (fp32 rows, for the un-rotation of a tied table:
 * b200lut_fht(mode ADJOINT, dtype fp32) then b200lut_round_rows). The rows are read out of the
 * slab layout, so a tied lm_head / embedding pair shares one copy of the codes; the reference
 * keeps an unpacked [N, K] uint8 cache instead (:2181-2205).
 * An id outside [0, N) writes a row of zeros and raises the device status
 * (b200lut_device_status() != 0); the reference aborts the context with a device-side
 * assertion (:1957-1976). */
int b200lut_embed_gather(const int64_t* ids, int64_t n_ids, int K, int dtype,
                         const b200lut_segment* table, const void* resB, int out_fp32,
                         void* stream);

/* out[m, k] = round_to_dtype(in[m, k]) for fp32 rows (the `.to(lut.dtype)` that ends the
 * reference's embedding forward, :2335). */
int b200lut_round_rows(const float* in, int64_t ldi, void* out, int64_t ldo, int64_t M, int K,
                       int dtype, void* stream);

/* gate[m, n] = silu(gate[m, n]) * up[m, n] over 16-bit [M, N] matrices (fp32 inside, one
 * rounding), in place on the gate buffer: the pass between two full-width prefill GEMMs (gate,
 * up) and the down projection. Replaces the act_fn(gate) * up of the reference's MLP at M > 1
 * (src/scripts/palettized_modules.py:1643-1723). N % 8 == 0; rows 16-byte aligned. */
int b200lut_silu_mul(void* gate, const void* up, int M, int N, int64_t ld_gate, int64_t ld_up,
                     int dtype, void* stream);

/* ------------------------------------------------------------------------- *
 * Hadamard rotation of the activations
 * ------------------------------------------------------------------------- */

enum {
  B200LUT_FHT_FORWARD = 0,   /* ((x H) * signs) / sqrt(b)         per segment */
  B200LUT_FHT_ADJOINT = 1,   /* ((x * signs) H) / sqrt(b)         per segment */
  B200LUT_FHT_AWQ = 2        /* (((x * scale) H) * signs / sqrt(b)) / scale   */
};

/* Row-wise transform of x [M, K] into out [M, K] (out may equal x: in place).
 * block == 0: descending power-of-two segments of K (4096 -> one 4096-point
 * transform; 12288 -> 8192 + 4096); block > 0 (power of two dividing K, <= 8192):
 * independent `block`-point transforms. signs: (K,) fp32 +-1 or NULL (= all +1);
 * scale: (K,) fp32, AWQ mode only. fp32 butterfly whatever the I/O dtype.
 * dtype: B200LUT_BF16, B200LUT_F16 or 2 = fp32.
 * Replaces fht_forward / fht_backward / fht_inplace_ / fht_forward_awq
 * (src/flute_extended/src/kernel_fht.cu:70-255, src/flute_extended/fht.py:206-238). */
int b200lut_fht(const void* x, void* out, const float* signs, const float* scale,
                int M, int K, int64_t ldx, int64_t ldo, int dtype, int mode, int block,
                void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* B200_LUT_H_ */
