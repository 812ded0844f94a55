/*
 * ckl_gemm.h -- C ABI of the B200 (sm_100a) tensor-core GEMM library.
 *
 *     C = alpha * (A * B) + beta * C        FP16 or BF16 A and B, FP32 accumulate
 *
 * Conventions are the reference library's (include/ckl/gemm.hpp:7-15 there):
 * row-major storage, A is m x k, B is k x n, C is m x n, no transposes, no
 * batching, device pointers owned by the caller, work is enqueued on `stream`
 * and the call returns without synchronising (NULL = the legacy default
 * stream).  Unlike the reference's C++ launchers the leading dimensions are
 * explicit, because an N-sharded B or C is a column block of a wider matrix.
 *
 * Every function returns a ckl_status (0 = success) and never throws or
 * aborts; ckl_last_error() gives the message for the calling thread's last
 * failure.  Degenerate shapes follow the reference
 * (include/ckl/detail/wmma_gemm.cuh:142-159, src/gemm/cublas_gemm_ex.cpp:41-50):
 * m <= 0 or n <= 0 is a no-op, k <= 0 computes C = beta * C.  As in BLAS, C is
 * not read when beta == 0.
 *
 * The library links only the CUDA runtime.  There is no CPU fallback: a call
 * on a machine without an sm_100 GPU fails with CKL_ERR_CUDA /
 * CKL_ERR_UNSUPPORTED.
 */
#ifndef CKL_GEMM_H_
#define CKL_GEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ckl_status {
    CKL_OK = 0,
    CKL_ERR_INVALID_ARG = 1, /* null pointer, bad dtype, leading dimension too small */
    CKL_ERR_CUDA = 2,        /* a CUDA runtime or driver call failed */
    CKL_ERR_UNSUPPORTED = 3, /* device is not sm_100, or forced algo cannot run the shape */
    CKL_ERR_DEVICE = 4,      /* a kernel reported a bounded wait that ran out */
    CKL_ERR_TOO_LARGE = 5    /* request exceeds a fixed capacity of the entry point */
} ckl_status;

/* Element types.  A and B are CKL_F16 or CKL_BF16; C may be any of the three. */
typedef enum ckl_dtype { CKL_F32 = 0, CKL_F16 = 1, CKL_BF16 = 2 } ckl_dtype;

/* Kernel selection.  CKL_ALGO_AUTO is what every reference-named entry point
 * uses; the others exist so tests and benchmarks can pin one kernel. */
typedef enum ckl_algo {
    CKL_ALGO_AUTO = 0,
    CKL_ALGO_SIMT = 1,       /* general-shape CUDA-core kernel (any size, any alignment) */
    CKL_ALGO_UMMA_1CTA = 2,  /* TMA + tcgen05.mma, one CTA per 128x256 tile, data-parallel */
    CKL_ALGO_UMMA_SK = 3,    /* same kernel with the stream-K split of the tile remainder */
    CKL_ALGO_UMMA_2CTA = 4,  /* CTA-pair tcgen05.mma (cta_group::2), 256x256 tile per pair */
    CKL_ALGO_UMMA_2CTA_SK = 5,
    CKL_ALGO_UMMA_2CTA_WIDE = 6, /* CTA pair, 256x512 tile filling all of tensor memory */
    CKL_ALGO_UMMA_2CTA_WIDE_SK = 7,
    CKL_ALGO_UMMA_1CTA_N128 = 8, /* the single-CTA kernel on 128x128 tiles: twice the tiles for
                                    problems too small to fill the SMs with 128x256 ones */
    CKL_ALGO_UMMA_1CTA_N128_SK = 9
} ckl_algo;

/* Stream handle: a cudaStream_t passed as an opaque pointer so this header
 * needs no CUDA include. */
typedef void* ckl_stream_t;

/* FP16 inputs.  Replaces ckl::gemm_wmma_fp16 / gemm_mma_ptx / gemm_mma_ldm /
 * gemm_mma_opt of the reference (include/ckl/gemm.hpp:68-69,75-76,80-81,85-86;
 * definitions src/gemm/gemm_wmma_fp16.cu:8-11, gemm_mma_ptx.cu:144-158,
 * gemm_mma_ldmatrix.cu:141-153, gemm_mma_opt.cu:214-226), which all compute
 * the same function with c_dtype = CKL_F32, lda = k, ldb = ldc = n. */
int ckl_gemm_f16(const void* a, const void* b, void* c, int c_dtype, int m, int n, int k, int lda,
                 int ldb, int ldc, float alpha, float beta, ckl_stream_t stream);

/* BF16 inputs.  Replaces ckl::gemm_wmma_bf16 (include/ckl/gemm.hpp:70-71,
 * src/gemm/gemm_wmma_bf16.cu:10-13). */
int ckl_gemm_bf16(const void* a, const void* b, void* c, int c_dtype, int m, int n, int k, int lda,
                  int ldb, int ldc, float alpha, float beta, ckl_stream_t stream);

/* Same computation with the input type and the kernel chosen by argument.
 * Forcing a tensor-core algo on a shape it cannot take (A or B not 16-byte
 * aligned, lda or ldb not a multiple of 8 elements, k <= 0) returns
 * CKL_ERR_UNSUPPORTED.  CKL_ALGO_AUTO routes such shapes to CKL_ALGO_SIMT the
 * way the reference routes them to its scalar kernel
 * (include/ckl/detail/wmma_gemm.cuh:148-158) while they are small; from
 * m*n*k = 2^28 on it copies the offending operand(s) into a per-stream scratch
 * buffer with an aligned pitch (one copy kernel each, scratch allocated on first
 * use: make that call outside stream capture) and runs the tensor-core kernel
 * on the copies, so an odd leading dimension no longer costs the tensor cores.
 * On such problems a C that rules out 16-byte accesses (base or ldc*sizeof)
 * is likewise computed into an aligned copy and copied out by one more pass. */
int ckl_gemm_ex(int ab_dtype, const void* a, const void* b, void* c, int c_dtype, int m, int n,
                int k, int lda, int ldb, int ldc, float alpha, float beta, int algo,
                ckl_stream_t stream);

/* Fused epilogue C = relu(alpha * A*B + bias[col]) (C is not read), and the
 * unfused second pass C = relu(C + bias[col]) over an FP32 C.  Replace
 * ckl::gemm_mma_opt_bias and ckl::gemm_bias_relu (include/ckl/gemm.hpp:91-93,
 * src/gemm/gemm_mma_opt.cu:228-246).  bias is n floats on the device. */
int ckl_gemm_bias_relu_ex(int ab_dtype, const void* a, const void* b, void* c, int c_dtype,
                          const float* bias, int m, int n, int k, int lda, int ldb, int ldc,
                          float alpha, int algo, ckl_stream_t stream);
int ckl_bias_relu_f32(float* c, const float* bias, int m, int n, int ldc, ckl_stream_t stream);

/* Single-precision GEMM, C = alpha*A*B + beta*C with FP32 inputs, FP32 multiply-add
 * and FP32 C (no tensor cores: the reference's FP32 tests demand agreement with
 * SGEMM to 1e-4, tests/test_gemm.cpp:50,98-101).  Replaces the reference's four
 * FP32 rungs ckl::gemm_naive / gemm_tiled / gemm_register / gemm_cp_async
 * (include/ckl/gemm.hpp:40-58; src/gemm/gemm_naive.cu, gemm_tiled.cu,
 * gemm_register.cu, gemm_cp_async.cu), which all compute this with the same
 * signature.  Row-major, explicit leading dimensions, any shape and alignment;
 * m <= 0 or n <= 0 is a no-op, k <= 0 scales C by beta; C is not read when
 * beta == 0.  Stream-ordered, allocates nothing. */
int ckl_sgemm(const float* a, const float* b, float* c, int m, int n, int k, int lda, int ldb,
              int ldc, float alpha, float beta, ckl_stream_t stream);

/* Triangular solve with many right-hand sides, L X = alpha B: L is m x m lower
 * triangular with a non-unit diagonal (its upper part is not read), B is m x n
 * and is overwritten by X; FP32, row-major, explicit leading dimensions.
 * Recursive halving: solve the upper half of the rows, subtract its contribution
 * from the lower half with one ckl_sgemm call, solve the lower half; halves of at
 * most 64 rows are solved directly.  The bulk of the flops run in the GEMMs.
 * Replaces ckl::trsm_naive and ckl::trsm_blocked (include/ckl/trsm.hpp:19-24;
 * src/trsm/trsm_naive.cu, src/trsm/trsm_blocked.cu:64-92), whose blocked form
 * updates the trailing rows with a one-thread-per-element loop instead of a
 * GEMM.  m <= 0 or n <= 0 is a no-op.  Stream-ordered, allocates nothing. */
int ckl_strsm_lower(const float* l, float* b, int m, int n, int lda, int ldb, float alpha,
                    ckl_stream_t stream);

/* Whole call with HOST buffers: copies A, B (and C when beta != 0) to device
 * memory the library keeps per device, runs the GEMM, copies C back and waits.
 * This is what a caller holding host matrices pays end to end; it is the
 * host-side counterpart of the upload / launch / download sequence in the
 * reference's test driver (tests/test_gemm_tensor.cpp:69-85).  Pinned host
 * buffers make the copies run at full link rate.  Large problems travel in row
 * panels so that uploads, the multiplication and downloads overlap; one call
 * at a time per device (calls from several threads queue). */
int ckl_gemm_host(int ab_dtype, const void* a_host, const void* b_host, void* c_host, int c_dtype,
                  int m, int n, int k, float alpha, float beta);

/* Host-side planning, no GPU needed: what ckl_gemm_ex would launch for this
 * shape on a device with `sm_count` SMs.  Mirrors the role of the reference's
 * launch_wmma dispatch test (include/ckl/detail/wmma_gemm.cuh:148) as a pure
 * function so it can be unit-tested on a CPU.  The plan is the one for a 16-bit
 * C or beta == 0; with an FP32 C and beta != 0, CKL_ALGO_AUTO keeps the 256x256
 * tile up to k = 8192 instead of 4096 (the only output-dependent choice). */
typedef struct ckl_plan {
    int algo;           /* resolved ckl_algo */
    int tile_m, tile_n; /* output tile of one work unit (per CTA pair for 2-CTA) */
    int tile_k;         /* k elements per pipeline stage */
    int tiles_m, tiles_n, k_blocks;
    int grid;           /* CTAs launched */
    int units;          /* schedulable workers: CTAs, or CTA pairs for the 2-CTA kernel */
    int group_m;        /* tile rows per raster group */
    int dp_tiles;       /* tiles computed whole by one CTA (or pair) */
    int sk_tiles;       /* tiles whose k range is split across CTAs */
    int sk_units;       /* CTAs (or pairs) sharing the split tiles */
    long long sk_iters; /* total k-block iterations in the split region */
    size_t workspace_bytes;
    int repack;         /* 1: A, B and/or C travel through copies with a 128-byte-aligned pitch */
} ckl_plan;
int ckl_plan_gemm(int m, int n, int k, int lda, int ldb, int ldc, int a_align, int b_align,
                  int algo, int sm_count, ckl_plan* out);

/* The same with everything the dispatcher looks at: the C type, whether C is read
 * (beta != 0 without the bias epilogue) and the number of CTA pairs the device can keep
 * resident (max_pairs <= 0 means sm_count / 2, the usual value). */
int ckl_plan_gemm_ex(int m, int n, int k, int lda, int ldb, int ldc, int a_align, int b_align,
                     int algo, int sm_count, int max_pairs, int c_dtype, int c_is_read,
                     ckl_plan* out);

/* The plan of the calling thread's most recent ckl_gemm_* call that reached the dispatcher:
 * what was actually launched, on the actual device. */
int ckl_last_plan(ckl_plan* out);

/* The k-block range of split tile work owned by unit `u` of a plan:
 * iterations [*begin, *end) of the sk_iters total.  Exposed for tests. */
int ckl_plan_sk_range(const ckl_plan* plan, int u, long long* begin, long long* end);

/* The work list of unit `u`, in execution order, produced by the very
 * functions the kernels run.  Each segment is 6 ints: linear tile, tile row,
 * tile column, first k block, one-past-last k block, workspace slot (-1 when
 * the unit owns the whole tile and writes C itself).  Writes at most
 * `max_segments` segments and returns the full count, or a negative
 * ckl_status.  Exposed for tests. */
int ckl_plan_unit_segments(const ckl_plan* plan, int u, int* out, int max_segments);

/* The workspace slots the fix-up pass adds, in order, for split tile `sk_tile`
 * (0 <= sk_tile < sk_tiles); 0 slots means one unit owned the tile whole.
 * Returns the count or a negative ckl_status.  Exposed for tests. */
int ckl_plan_fixup_slots(const ckl_plan* plan, int sk_tile, int* out, int max_slots);

/* Device-side health word.  Kernels never trap or spin forever: a wait that
 * exceeds its limit records a code here and the kernel drains and exits.
 * Synchronises the current device, returns CKL_OK or CKL_ERR_DEVICE and
 * clears the word; info (4 words: code, block, role, detail) may be NULL. */
int ckl_device_status(unsigned int* info);

/* Stream-copy bandwidth probe used by the roofline tools (replaces
 * stream_copy in src/tools/device_probe.cu:25-70): copies `bytes` from src
 * to dst on the device with a grid sized for HBM3e. */
int ckl_stream_copy(void* dst, const void* src, size_t bytes, ckl_stream_t stream);

/* Multi-GPU helper for the N-sharded GEMM (no counterpart in the reference,
 * which is single-GPU): after an all-gather of per-rank column blocks,
 * src holds parts x m x n_shard elements ([rank][row][col]); this writes the
 * row-major m x (parts * n_shard) matrix dst.  elem_size is 2 or 4 bytes. */
int ckl_assemble_column_blocks(void* dst, const void* src, int elem_size, int m, int n_shard,
                               int parts, ckl_stream_t stream);

/* ---- several GPUs of one box (no counterpart in the reference, which is single-GPU and
 * never calls cudaSetDevice; its upload / launch / download sequence,
 * tests/test_gemm_tensor.cpp:69-85, is what these generalise) ---------------------------
 *
 * One rank per GPU, each a process or a host thread with its device current.  Output columns
 * are independent, so rank r of `world` owns the column block ckl_column_shard() gives it of
 * B and C, and A is replicated.  The ranks meet through a communicator that wraps NCCL
 * (loaded with dlopen at first use: the library itself still links only the CUDA runtime;
 * CKL_NCCL_LIB names the file if "libnccl.so.2" is not on the loader's path).  Every NCCL
 * call gets buffers of the calling rank's own memory; the only accesses to another GPU's
 * memory are plain stores of this library's copy kernel into buffers made with
 * ckl_comm_alloc_shared. */

/* Column block of rank `rank`: block widths are multiples of `align` columns (8 keeps every
 * block 16-byte aligned for 16-bit types), the tail rank takes what is left, ranks past the
 * end get width 0. */
int ckl_column_shard(int n, int world, int rank, int align, int* col0, int* width);

typedef struct ckl_comm ckl_comm;
#define CKL_COMM_ID_BYTES 128

/* Rank 0 draws an id (CKL_COMM_ID_BYTES bytes) and hands it to the other ranks by any means
 * the job has; then every rank calls ckl_comm_init with its device current.  Collective. */
int ckl_comm_get_unique_id(void* id);
int ckl_comm_init(ckl_comm** comm, int world, int rank, const void* id);
int ckl_comm_world(const ckl_comm* comm);
int ckl_comm_rank(const ckl_comm* comm);
/* Frees the communicator's streams, staging and shared buffers.  Collective when world > 1. */
int ckl_comm_destroy(ckl_comm* comm);

/* A device buffer of `bytes` bytes on every rank, each rank's copy mapped into all the others
 * (CUDA IPC between processes, peer access between threads of one process).  Collective: all
 * ranks call it with the same size, in the same order.  *local is this rank's copy. */
int ckl_comm_alloc_shared(ckl_comm* comm, size_t bytes, void** local);
int ckl_comm_free_shared(ckl_comm* comm, void* local);

/* How ckl_gemm_host_sharded deals the m rows of A: rank r uploads rows
 * [row0, row0 + rows) (rows_per_rank each, the tail rank fewer), in `panels` panels of
 * panel_rows rows; on the device A and C live as [panel][rank][panel_rows] rows
 * (padded_rows in all).  Pure host arithmetic. */
typedef struct ckl_host_shard_plan {
    int rows_per_rank;
    int row0, rows;
    int panels, panel_rows;
    int padded_rows;
} ckl_host_shard_plan;
int ckl_plan_host_sharded(int m, int world, int rank, ckl_host_shard_plan* out);

/* The N-sharded GEMM on HOST buffers, end to end: C[:, block] = alpha*A*B[:, block] +
 * beta*C[:, block].  a_rows_host is THIS rank's rows of A (plan.rows x k, packed), so the m x k
 * matrix crosses the host links once in total, not once per GPU; b_shard_host is the rank's
 * k x n_shard block and c_shard_host its m x n_shard block (both packed).  Each rank uploads
 * over its own link, the row panels of A are all-gathered over NVLink, and panel j is
 * multiplied and sent back while panel j+1 is still arriving.  Collective; returns when this
 * rank's block of C is in c_shard_host.  With world == 1 it does what ckl_gemm_host does. */
int ckl_gemm_host_sharded(ckl_comm* comm, int ab_dtype, const void* a_rows_host,
                          const void* b_shard_host, void* c_shard_host, int c_dtype, int m,
                          int n_shard, int k, float alpha, float beta);

/* The N-sharded GEMM on DEVICE buffers with the whole C assembled on every rank.  a is the
 * replicated m x k matrix (lda), b_shard the rank's k x width block (ldb), c_shard its packed
 * m x width block (C_in on entry when beta != 0, the rank's result on return), c_full a buffer
 * from ckl_comm_alloc_shared that receives the row-major m x n matrix; width and the column
 * offset are ckl_column_shard(n, world, rank, 8).  The local GEMM runs in row panels on
 * `stream`; behind each panel a copy kernel writes the panel's column block into every rank's
 * c_full with plain 16-byte stores over NVLink, on a stream of the communicator, so the
 * transfer overlaps the next panel's multiplication.  Collective and stream-ordered: later
 * work on `stream` sees the complete c_full of all ranks' blocks. */
int ckl_gemm_gathered(ckl_comm* comm, int ab_dtype, const void* a, const void* b_shard,
                      void* c_shard, void* c_full, int c_dtype, int m, int n, int k, int lda,
                      int ldb, float alpha, float beta, ckl_stream_t stream);

/* The copy kernel on its own: writes the packed rows x width block src to columns
 * [col0, col0 + width) of `parts` row-major matrices of n columns (dsts[i], any mix of local
 * and mapped peer buffers).  elem_size is 2 or 4 bytes. */
int ckl_scatter_column_block(void* const* dsts, int parts, const void* src, int elem_size,
                             int rows, int width, int n, int col0, ckl_stream_t stream);

/* No counterpart in the reference.  The stream-K tensor-core GEMM for callers that
 * must not allocate device memory: hosts that have given all device memory to an
 * arena of their own (a cudaMalloc inside a library would fail or break their
 * budget) and latency-critical loops that cannot take cudaMalloc's device-wide
 * synchronisation.  Same arguments and result as ckl_gemm_ex with
 * CKL_ALGO_UMMA_SK, but the partial-tile workspace and the status word are arrays
 * built into the library image (ckl_noalloc_scratch_bytes() = 38,797,312 bytes,
 * held by every GPU that loads the library until the process exits) and no
 * cudaMalloc, cudaFree or allocating routine is ever called.
 *   - Only the tensor-core kernel: A and B 16-byte aligned, lda and ldb multiples
 *     of 8, k > 0; anything else returns CKL_ERR_UNSUPPORTED (m <= 0 or n <= 0 is
 *     still a no-op).
 *   - The scratch serves schedules of up to 148 CTAs; a device that would need
 *     more returns CKL_ERR_TOO_LARGE.
 *   - All calls on a device share the scratch, which keeps the previous call's
 *     contents (harmless: every slot is rewritten before it is read).  Calls
 *     that overlap on the GPU race on it: use one stream per device or order
 *     them with events.
 *   - The first call on each device does one-time set-up with that device
 *     current (symbol address look-ups, kernel attributes, driver entry point);
 *     make it before any stream capture starts.  It is also the moment the
 *     CUDA runtime loads this library's device code on that GPU and backs the
 *     built-in scratch with device memory (about 37 MiB): a host that gives
 *     all device memory to its own arena makes this first call before it does.
 *   - A wait that ran out inside one of this entry point's kernels is reported
 *     by ckl_noalloc_device_status() (same contract as ckl_device_status():
 *     synchronises the current device, fills the optional 4 words, clears the
 *     word, returns CKL_OK or CKL_ERR_DEVICE), which allocates nothing either.
 *     ckl_device_status() does not see it: that one reads the regular entry
 *     points' word and creates their per-device context with cudaMalloc.
 * Errors of these functions are described by ckl_noalloc_last_error(). */
int ckl_gemm_streamk_noalloc(int ab_dtype, const void* a, const void* b, void* c, int c_dtype,
                             int m, int n, int k, int lda, int ldb, int ldc, float alpha,
                             float beta, ckl_stream_t stream);
int ckl_noalloc_device_status(unsigned int* info);
const char* ckl_noalloc_last_error(void);
size_t ckl_noalloc_scratch_bytes(void);

/* Test hook for the bounded waits (no fault is raised, nothing traps, no wait exceeds the
 * limit given here): makes ONE wait of the calling thread's next tensor-core launch run out.
 *   kind 1: the TMA producer of the first CTA announces 16 bytes more than it loads for its
 *           first pipeline stage, so that stage's barrier never completes and the MMA warp's
 *           wait gives up;
 *   kind 2: the owner of a split tile (fused stream-K launches only) waits for a flag value
 *           that no CTA publishes.
 * The waiting role records (code, block, role, detail) in the device status word, every role
 * of the CTA leaves its loop, copies and MMAs in flight are drained, tensor memory is freed
 * and the kernel returns; C of that launch is incomplete, ckl_device_status() then returns
 * CKL_ERR_DEVICE, and the next launch runs normally.  wait_limit_ns replaces the 2 s limit
 * for that launch (0 keeps it).  kind 0 disarms. */
int ckl_test_arm_wait_fault(int kind, unsigned long long wait_limit_ns);

/* Counters for tests: "tensor_map_encodes" = TMA descriptors encoded by this process so far
 * (descriptors are cached per device, keyed by address, shape, pitch, type and box, so a
 * repeated call encodes none).  Unknown names give ~0. */
unsigned long long ckl_debug_counter(const char* name);

/* Message of the calling thread's most recent non-zero status ("" if none). */
const char* ckl_last_error(void);

/* Name of a ckl_algo value, e.g. "umma_1cta". */
const char* ckl_algo_name(int algo);

/* Frees every per-device cache (workspaces, staging buffers). */
void ckl_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* CKL_GEMM_H_ */
