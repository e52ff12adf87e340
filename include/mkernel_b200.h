/*
 * mkernel_b200 -- C ABI of the B200 (sm_100a) tensor-parallel GEMM + collective operators.
 *
 * This is the boundary a host language binds (ctypes, cgo, JNI, pybind).  Every entry point takes
 * plain pointers and sizes, returns 0 on success or a negative mk_status, never exits the
 * process and never throws.  mk_last_error() returns a thread-local message for the last failure.
 *
 * One process drives one GPU.  "Symmetric" buffers are allocated collectively by all ranks of a
 * node, each rank holding its own copy plus mapped addresses of every peer's copy and, when
 * requested and supported, one NVSwitch multicast address that aliases all copies.
 *
 * Each operator entry below names the reference interface it stands in for
 * (paths inside uccl-project/mKernel).
 */
#ifndef MKERNEL_B200_H_
#define MKERNEL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MK_MAX_WORLD 8

typedef enum mk_status {
  MK_OK = 0,
  MK_ERR_INVALID = -1,      /* bad argument / unsupported shape (reference: TORCH_CHECK failure) */
  MK_ERR_CUDA = -2,         /* a CUDA runtime or driver call failed */
  MK_ERR_TRANSPORT = -3,    /* rendezvous between ranks failed or timed out */
  MK_ERR_UNSUPPORTED = -4,  /* feature not available on this system (e.g. multicast) */
  MK_ERR_DEVICE_WAIT = -5   /* a device-side bounded wait expired (see mk_op_status) */
} mk_status;

/* Layout of operand B. */
#define MK_B_NK 0 /* B stored [N, K], K contiguous (AllGather+GEMM, GEMM+ReduceScatter) */
#define MK_B_KN 1 /* B stored [K, N], N contiguous (GEMM+AllReduce) */

typedef struct mk_comm mk_comm; /* per-process rendezvous + device context           */
typedef struct mk_symm mk_symm; /* one symmetric allocation                          */

/* View of a symmetric allocation that the operators consume.  A caller with its own symmetric
 * heap can fill this struct by hand instead of using mk_symm_alloc. */
typedef struct mk_symm_view {
  int rank;
  int world;
  size_t bytes;
  void* peer[MK_MAX_WORLD]; /* peer[rank] is the local copy */
  void* mc;                 /* multicast alias or NULL */
} mk_symm_view;

const char* mk_last_error(void);
int mk_version(void);

/* ---- transport: replaces include/comm/local_broker.cuh:362-534 (shm + unix-socket broker),
 *      include/comm/ipc.cuh:100-122 (fd import) and include/comm/vmm.cuh:29-119 (VMM, multicast).
 * `key` names the rendezvous; all ranks of one job pass the same key.  Collective calls must be
 * made by every rank in the same order. */
int mk_comm_create(const char* key, int rank, int world, int device, mk_comm** out);
int mk_comm_destroy(mk_comm* comm);
int mk_comm_rank(const mk_comm* comm);
int mk_comm_world(const mk_comm* comm);
int mk_comm_barrier(mk_comm* comm);
/* Every rank contributes `bytes` (<= 256) bytes; out receives world * bytes. */
int mk_comm_allgather(mk_comm* comm, const void* in, size_t bytes, void* out);
/* Every rank contributes one file descriptor; out_fds[r] is a descriptor in this process that
 * refers to rank r's file (out_fds[rank] is a dup of fd).  The caller closes them. */
int mk_comm_allgather_fd(mk_comm* comm, int fd, int* out_fds);

/* ---- symmetric memory: replaces dist::ParallelBuffer, include/dist/parallel_buffer.cuh:87-338 */
int mk_symm_alloc(mk_comm* comm, size_t bytes, int want_multicast, mk_symm** out);
int mk_symm_free(mk_symm* buf);
int mk_symm_get_view(const mk_symm* buf, mk_symm_view* out);

/* ---- operators.  `stream` is a cudaStream_t.  All launches are asynchronous. ---------------- */

/* Words (uint32) an operator's synchronisation buffer must hold.  The buffers are symmetric,
 * multicast not required, and must be zeroed once before the first launch, on every rank, with
 * all ranks synchronised afterwards: mk_gemm_rs_prepare does the zeroing; the AllGather `ready`
 * and the AllReduce `barrier` buffers are zeroed by the caller (as in the reference's drivers).
 * A buffer that was never zeroed gives each rank an arbitrary epoch and the first launch ends in
 * a wait timeout.  After a device wait has expired (mk_op_status returns MK_ERR_DEVICE_WAIT)
 * the status words stay set and every later launch on that buffer gives up at its first slow
 * wait until mk_op_status_clear is called.
 * Reference: ag_gemm_warp_specialized_ready_words, gemm_rs_blackwell_sync_shape
 * (include/operators/ag_gemm/ag_gemm_warp_specialized_session.cuh:12-47,
 *  include/operators/gemm_rs/gemm_rs_blackwell_session.cuh:11-15), barrier (2,1024,1024). */
#define MK_AG_READY_WORDS 65536
#define MK_RS_SYNC_WORDS 524288
#define MK_AR_BARRIER_WORDS (2 * 1024 * 1024)

/* Plain C[M,N] = A[M,K] * B on one GPU (bf16 in, fp32 accumulate, bf16 out).  The W = 1 case of
 * every fused operator; no counterpart entry point in the reference.  `status4` may be NULL or
 * point to 4 zeroed device words that receive a failure record. */
int mk_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int b_layout,
                 uint32_t* status4, void* stream);

/* AllGather + GEMM.  Replaces ag_gemm_warp_specialized_prepare / _launch
 * (include/operators/ag_gemm/ag_gemm_warp_specialized.cuh:331-406,
 *  src/ag_gemm_warp_specialized.cu:115-134, 610-696).
 * A: symmetric [W, M/W, K] bf16, rank r has filled slab r.  ready: symmetric MK_AG_READY_WORDS.
 * B: [N, K] bf16.  C: [W, M/W, N] bf16 (M = total rows).  The reference's prepare is an all-rank
 * entry barrier kernel; here the launch itself carries that ordering (every rank announces
 * "entered launch e" to its peers and nobody writes into a peer's gathered buffer before seeing
 * it), so prepare only validates `ready` and may be called or skipped; it does NOT zero
 * `ready`. */
int mk_ag_gemm_prepare(const mk_symm_view* ready, void* stream);
int mk_ag_gemm_launch(const mk_symm_view* A, const mk_symm_view* ready, const void* B, void* C,
                      int M, int N, int K, void* stream);

/* Same with B in either layout and an optional caller-supplied epoch (0 = device epoch; otherwise
 * strictly increasing per launch on this `ready` buffer).  Replaces the shape of
 * ag_gemm_multinode (include/operators/ag_gemm/session.cuh:210-229), whose B is [K, N] and whose
 * epoch comes from the host, for a single node. */
int mk_ag_gemm_launch_ex(const mk_symm_view* A, const mk_symm_view* ready, const void* B, void* C,
                         int M, int N, int K, int b_layout, uint32_t epoch, void* stream);

/* AllGather + GEMM with a fused SwiGLU epilogue: H[M, N2/2] = silu(X G^T) * (X U^T), where X is
 * the gathered A and B_gate_up [N2, K] holds, per block of 256 rows, 128 rows of the gate
 * projection G followed by the 128 rows of the up projection U for the same 128 outputs.
 * The first half of the tensor-parallel MLP (its second half is mk_gemm_rs_launch on H).  The
 * reference fuses the same activation into the epilogue of its gate/up GEMM
 * (src/dispatch_gemm_glu_combine.cu:21-25).  N2 must be a multiple of 256.  H: [W, M/W, N2/2]. */
int mk_ag_gemm_swiglu_launch(const mk_symm_view* A, const mk_symm_view* ready,
                             const void* B_gate_up, void* H, int M, int N2, int K, void* stream);

/* GEMM + ReduceScatter.  Replaces gemm_rs_blackwell_prepare / _launch
 * (src/gemm_rs_blackwell.cu:642-732).  A: [M, K_local], B: [N, K_local], C: symmetric [M, N]
 * (workspace: rank s's partial rows of owner o land in slab s of o's copy; after the launch rows
 * [rank*M/W, (rank+1)*M/W) hold the reduced result).  sync: symmetric MK_RS_SYNC_WORDS.  prepare zeroes sync once; the caller
 * then synchronises the stream and barriers all ranks before the first launch. */
int mk_gemm_rs_prepare(const mk_symm_view* sync, void* stream);
int mk_gemm_rs_launch(const void* A, const void* B, const mk_symm_view* C,
                      const mk_symm_view* sync, int M, int N, int K, void* stream);

/* Same with B in either layout and an optional caller-supplied epoch (0 = device epoch).
 * Replaces the shape of gemm_rs_fused (include/operators/gemm_rs/session.cuh:128-153) for a
 * single node. */
int mk_gemm_rs_launch_ex(const void* A, const void* B, const mk_symm_view* C,
                         const mk_symm_view* sync, int M, int N, int K, int b_layout,
                         uint32_t epoch, void* stream);

/* One-GPU GEMM + ReduceScatter that allocates nothing: C[M,N] = A[M,K] * B[N,K]^T with the
 * kernel's synchronisation words held in a 64 KiB device array built into the library, for
 * callers that cannot allocate device memory where they need the product (a process whose GPU
 * memory is fully owned by a pre-sized arena, or a path that must not hit cudaMalloc's device
 * synchronisation).  No counterpart in the reference.  Limits and rules:
 *  - world size 1 only; output tiles (128 x block_n) plus row-blocks (128 rows) may number at
 *    most 16320 together (e.g. 8192 x 8192 is fine, 32768 x 28672 is rejected with
 *    MK_ERR_INVALID);
 *  - the first call on each device looks up the array's device address; make that call
 *    before starting any stream capture;
 *  - all calls on a device share the one array: calls that overlap on the GPU (two streams)
 *    race; calls on one stream are safe;
 *  - calls no cudaMalloc/cudaFree; the array stays resident on every GPU that loads the library. */
int mk_gemm_rs_launch_noalloc(const void* A, const void* B, void* C, int M, int N, int K,
                              void* stream);

/* GEMM + AllReduce.  Replaces gemm_ar_intranode_blackwell
 * (include/operators/gemm_ar/gemm_ar_blackwell.cuh:205-246, src/gemm_ar_blackwell.cu:57-610).
 * A: [M, K_local], B: [K_local, N] (MK_B_KN) or [N, K_local] (MK_B_NK).  C: symmetric [M, N]
 * partial product.  C_final: symmetric [M, N], complete on every rank when the launch ends.
 * barrier: symmetric MK_AR_BARRIER_WORDS, zeroed once.  epoch: strictly increasing from 1 (the
 * reference's contract), or 0 to let the library keep the epoch in `barrier` itself, which makes
 * the launch replayable from a CUDA graph. */
int mk_gemm_ar_launch(const void* A, const void* B, const mk_symm_view* C,
                      const mk_symm_view* barrier, const mk_symm_view* C_final, int M, int N,
                      int K, uint32_t epoch, int b_layout, void* stream);

/* Reads the 4 status words {code, where, detail0, detail1} of an operator's synchronisation
 * buffer (synchronous device-to-host copy).  Returns MK_ERR_DEVICE_WAIT when code != 0. */
int mk_op_status(const mk_symm_view* sync, uint32_t out4[4]);
/* Clears the status words (asynchronous memset on `stream`). */
int mk_op_status_clear(const mk_symm_view* sync, void* stream);

/* ---- options (process-wide): "wait_limit_ms" (device wait budget, default 4000),
 *      "n_comm" (dedicated exchange CTAs, -1 = heuristic), "block_n" (0 = heuristic), "group_rows" / "group_cols"
 *      (raster group in row / column blocks, 0 = heuristic; column groups apply on one GPU only),
 *      "use_nvls" (0/1, default 0: exchange through NVSwitch multicast when the buffers have an
 *      alias; the in-switch sum of the AllReduce is not rounded to nearest, so its error can
 *      exceed the 1e-2 parity tolerance slightly),
 *      "cta_pair" (0/1, default 1: two-SM MMA over CTA pairs when the shape allows),
 *      "ar_one_shot" (GEMM+AR: 0 = two-shot, owners reduce and broadcast; 1 = one-shot, every
 *      rank reduces all rows for itself), "ag_fanout" (AllGather push: 0 = one work item per
 *      receiver, 1 = an item loads its rows once and stores them to every peer), "push_bulk"
 *      (AllGather push through bulk shared-to-global stores), "ag_chunks" (AllGather push: 0 =
 *      an item is 4 full rows and consumers wait for whole row-blocks; 1 = an item is every row
 *      of a row-block over one K-range and consumers wait range by range inside the K loop), "ag_lead" (AllGather push pacing:
 *      rows are pushed at most this many quarter raster groups before the GEMM reaches the group
 *      that consumes them; default 6, 0 = push as fast as possible), "pdl" (0/1, default 1: launch with
 *      programmatic stream serialization so a kernel's set-up overlaps the previous kernel's
 *      tail), "ar_push" (GEMM+AR: 2/1/0 = staging slabs with epoch words / with flags / owners
 *      fetch partials), "split_tail" (0/1, default 1: cut the tiles
 *      of a partial last round along K over all CTAs -- plain GEMM and AllGather+GEMM; uses a
 *      scratch buffer per device and stream that the library allocates at the first such launch,
 *      never during stream capture), "max_stages" (cap on the
 *      operand ring depth, 0 = as many as fit), "l2_promo" (L2 promotion of the operand tensor
 *      maps, 0..3 = none/64/128/256 bytes).  Values are range-checked (wait_limit_ms in
 *      [1, 60000]; only n_comm accepts -1).  The environment variable
 *      MKERNEL_B200_OPTIONS="name=value,..." sets start-up defaults when the library is loaded,
 *      through the same checks.  Builds made with -DMKB_DIAG add "debug_flags" and "trace_ptr"
 *      (timing diagnostics; results undefined); the default build rejects them. */
int mk_set_option(const char* name, long long value);
long long mk_get_option(const char* name);

/* ---- introspection used by host-side tests and tools (no GPU needed) ---------------------- */
typedef struct mk_plan {
  int block_n, stages, n_comm, grid, smem_bytes;
  int row_blocks, col_blocks, k_blocks, part_rows, part_blocks, interleave, group_rows;
  long long sync_words;
  int group_cols;
} mk_plan;
/* Launch plan for op (0 GEMM, 1 AG, 2 RS, 3 AR) without touching a device; num_sms <= 0 means
 * 148. */
int mk_plan_op(int op, int rank, int world, int M, int N, int K, int b_layout, int num_sms,
               mk_plan* out);
/* Tile visiting order of a compute CTA set: writes row0/rows/col0 per tile, returns tile count
 * (or a negative status).  `cap` is the capacity of each output array. */
int mk_sched_tiles(int op, int rank, int world, int M, int N, int block_n, int group_rows,
                   int group_cols, int* row0, int* rows, int* col0, int* rowblock, int cap);
/* Work list of compute CTA `cta` (of n_comp; cg = 2: CTAs work as pairs on consecutive tiles):
 * whole tiles, then at most one piece [kb0, kb1) of a tile of a partial last round when
 * splitting applies (max_parts >= 2; piece = -1 for whole tiles).  Returns the item count. */
int mk_sched_work_items(int total_tiles, int n_comp, int cg, int k_blocks, int max_parts, int cta,
                        int* tile, int* kb0, int* kb1, int* piece, int cap);
/* Rows [row0,row1) that owner `owner` reduces for its k-th item; returns number of items. */
int mk_sched_owner_items(int op, int world, int M, int N, int block_n, int owner, int* row0,
                         int* row1, int cap);

#ifdef __cplusplus
}
#endif
#endif /* MKERNEL_B200_H_ */
