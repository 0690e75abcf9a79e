/*
 * C ABI of libsgemm_runner.so — the drop-in boundary of the sm_100a SGEMM backend.
 *
 * The reference keeps the corresponding steps as internal C++ functions of its runner program
 * (runner/generator_runner.cpp); each entry point below names the one it replaces.  A caller in
 * any language binds these symbols (plain pointers and sizes, no C++ or torch types).
 *
 * Conventions
 *   - every function returns 0 (SGEMM_OK) or a negative sgemm_error code; nothing throws or aborts;
 *   - matrices are FP32, column-major: A is M x K (lda >= M), B is K x N (ldb >= K), C and D are M x N
 *     (ldc, ldd >= M);  D = alpha * A * B + beta * C;  C may be NULL when beta == 0.  A cubin generated with
 *     trans_a (trans_b) expects A stored as K x M with lda >= K (B stored as N x K with ldb >= N) instead;
 *   - the caller owns A, B, C, D; the handle owns the loaded module, its kernels, a status buffer, the
 *     tensor-map cache and (unless the caller lends one) the scratch workspace;
 *   - one handle belongs to one device; a handle is not thread-safe, distinct handles are;
 *   - sgemm_launch is asynchronous on the given stream (NULL = the default stream);
 *   - there is no CPU path: every compute entry point fails with SGEMM_ERR_NO_DRIVER / SGEMM_ERR_CUDA
 *     when no CUDA driver or device is present.
 */
#ifndef SGEMM_RUNNER_H
#define SGEMM_RUNNER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sgemm_handle sgemm_handle;

typedef enum sgemm_error {
    SGEMM_OK = 0,
    SGEMM_ERR_INVALID_ARGUMENT = -1, /* NULL handle/pointer, ld smaller than the rows it must hold, ... */
    SGEMM_ERR_TOML = -2,             /* config file missing, unreadable, or a required key absent/ill-typed */
    SGEMM_ERR_NO_DRIVER = -3,        /* libcuda.so.1 could not be loaded */
    SGEMM_ERR_CUDA = -4,             /* a CUDA driver call failed; see sgemm_last_error */
    SGEMM_ERR_MODULE = -5,           /* cubin missing / not loadable / entry point not found */
    SGEMM_ERR_UNSUPPORTED = -6,      /* the loaded kernel cannot serve this request (e.g. forced variant) */
    SGEMM_ERR_WORKSPACE = -7,        /* lent workspace too small, or allocation failed */
    SGEMM_ERR_DEVICE_STATUS = -8,    /* a kernel reported a bounded wait that ran out (sgemm_last_status) */
    SGEMM_ERR_SCRATCH_LIMIT = -9,    /* problem needs more scratch than sgemm_launch_noalloc's fixed array holds */
    SGEMM_ERR_COMM = -10             /* NCCL not loadable, no communicator on the handle, or a collective failed */
} sgemm_error;

/* Kernel configuration as read from the generator's TOML (generator/generator.py:1001-1017 writes it,
 * runner/generator_runner.cpp:85-124 `AsmKernelConfig` / `getAsmKernelConfig` reads it there). */
typedef struct sgemm_config {
    int32_t a_type, b_type, cd_type, scalar_type;
    int32_t mfma[4];
    int32_t wave_group[2];
    int32_t wave_tiling[2];
    int32_t depth_k;
    int32_t vmem_stage;
    int32_t wavefront_size;
    int32_t lds_usage_bytes;
    int32_t trans_a, trans_b;
    /* sm_100a additions (0 / empty when the file has only the legacy keys) */
    int32_t variant;            /* 0 = SIMT FFMA, 1 = tcgen05 3xTF32 */
    int32_t num_threads;
    int32_t dynamic_smem_bytes;
    int32_t stages;
    int32_t a_kmajor;           /* tensor variant reads A from a K-major packed copy */
    int32_t split_inkernel;     /* tensor variant: 1 = the kernel makes the 3xTF32 lo tiles itself (no pre-pass), 2 = only B's (A's lo copy by the pre-pass) */
    int32_t fallback_tile[3];
    int32_t fallback_threads;
    char entry[64];
    char fallback_entry[64];
    /* companion tcgen05 kernel for low-intensity shapes (tensor-variant cubins; empty entry: none) */
    int32_t skinny_tile[3];
    int32_t skinny_threads;
    int32_t skinny_smem_bytes;
    char skinny_entry[64];
    /* tensor variant: k accumulated inside the tensor core before the partial sum moves to FP32 registers, as the
     * kernels were generated (0: the kernel has no such path and accumulates all of K in one chain) */
    int32_t acc_chain;
    int32_t skinny_acc_chain;
    /* twin of the main tensor kernel that accumulates all of K in one chain (empty: none); same tile, threads and
     * shared memory as the main kernel */
    char wholek_entry[64];
    /* the companion's narrow sibling (128 x 32 tiles) for N of a few columns (empty entry: none) */
    int32_t thin_tile[3];
    int32_t thin_threads;
    int32_t thin_smem_bytes;
    int32_t thin_acc_chain;
    char thin_entry[64];
    /* FFMA variant: 1 = the main kernel is the TMA-fed, warp-specialised one (TOML feed = "tma"); operands TMA cannot
     * describe go to the register-fed kernel named by fallback_entry, as in a tensor-variant cubin */
    int32_t feed_tma;
} sgemm_config;

/* Replaces getAsmKernelConfig (runner/generator_runner.cpp:100-124).  Host only, needs no GPU. */
int sgemm_config_parse(const char *toml_path, sgemm_config *out);

/* Tile of D one launch unit covers: mfma[i] * wave_group[i] * wave_tiling[i], the product rule of
 * makeKernelArguments (runner/generator_runner.cpp:128-129).  Host only. */
int sgemm_config_tile(const sgemm_config *cfg, uint32_t *tile_m, uint32_t *tile_n);

/* Replaces prepareASMKernel + getAsmKernelConfig (runner/generator_runner.cpp:69-73, 193-197):
 * loads the cubin with cuModuleLoad on `device` (its primary context) and resolves the entry points. */
int sgemm_open(const char *cubin_path, const char *toml_path, int device, sgemm_handle **out);

/* Replaces hipModuleUnload + the frees at the end of main (runner/generator_runner.cpp:318-322). */
int sgemm_close(sgemm_handle *h);

/* Replaces makeKernelArguments + launchASMKernel (runner/generator_runner.cpp:126-190) with device
 * pointers.  (A and B are declared `const float *` as in the reference's FP32-only runner; with a cubin generated
 * for FP16 or BF16 operands — `a_type` 1 or 2 in its TOML — they point to 16-bit elements, and lda, ldb count
 * those elements.  C, D, alpha and beta are always FP32.)  Chooses the kernel variant and split-K factor (see sgemm_set_option), runs the 3xTF32
 * split pre-pass and the split-K reduction when they apply.  May allocate or grow the handle-owned
 * workspace (a synchronising cuMemAlloc) unless a workspace was lent with sgemm_set_workspace. */
int sgemm_launch(sgemm_handle *h, const float *dA, const float *dB, const float *dC, float *dD,
                 float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                 uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, void *stream);

/* No counterpart in the reference (its runner allocates freely with hipMalloc).  sgemm_launch for callers
 * that cannot allocate device memory at call time: a serving loop with a frozen memory budget, a real-time path
 * that cannot take a blocking driver call, or a process whose device memory belongs to another allocator.  Same arguments and
 * results as sgemm_launch, but the scratch (3xTF32 lo copies, split-K partials) comes from a fixed array of
 * SGEMM_NOALLOC_SCRATCH_BYTES that is part of the library image on every GPU that loads it; no cudaMalloc,
 * cuMemAlloc or other allocating call is made.  Problems needing more scratch fail with
 * SGEMM_ERR_SCRATCH_LIMIT before anything is launched (sgemm_workspace_bytes_for tells the need, copies of
 * operands that TMA cannot read where they lie included).  The first call on a handle resolves the array's device
 * address in the handle's own context (one-time set-up; make it before any stream capture; the calling thread's
 * current device and context are left untouched).  All calls on a device share the array: kernels of two such
 * calls must not overlap in time on one GPU. */
#define SGEMM_NOALLOC_SCRATCH_BYTES (32u << 20)
int sgemm_launch_noalloc(sgemm_handle *h, const float *dA, const float *dB, const float *dC, float *dD,
                         float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                         uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, void *stream);
/* Size of that array in bytes (= SGEMM_NOALLOC_SCRATCH_BYTES of the library that was actually loaded). */
size_t sgemm_noalloc_scratch_bytes(void);

/* The same call with HOST buffers: uploads A, B (and C when beta != 0), launches, downloads D and
 * synchronises — what the reference's main does around its kernel with hipMalloc / hipMemcpyHtoD /
 * hipMemcpyDtoH (runner/generator_runner.cpp:236-242, 289-291).  Device staging buffers are cached in
 * the handle.  Host buffers may be pageable or pinned.  Large problems (>= 64 MiB of operands, N >= 4 tiles) are
 * pipelined over column chunks on three internal streams so that uploads, GEMM and downloads overlap (this needs
 * pinned host memory to take effect; option "pipeline_host" = 0 turns it off); results are the same either way. */
int sgemm_run_host(sgemm_handle *h, const float *hA, const float *hB, const float *hC, float *hD,
                   float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                   uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd);

/* ---- one SGEMM over several GPUs of a box: column shards --------------------------------------------------------
 * No counterpart in the reference, which is single-GPU (its runner never selects a device,
 * runner/generator_runner.cpp:192-324).  D's columns are independent: GPU r of g computes D[:, n0:n1] from a
 * replicated A and B[:, n0:n1]; in column-major storage these are contiguous ranges, so a shard is a pointer offset
 * and each GPU runs the ordinary single-GPU call (sgemm_launch) on n1 - n0 columns.  No collective sits on the
 * compute path.  One handle per GPU, in one process (sgemm_comm_init_all) or one process per GPU (sgemm_comm_init with
 * an id made by one rank and handed to the others by the host program).  The communicator is NCCL's, bound at run
 * time; it is used in exactly two places: to complete the replicated A on the host-buffer path, and for the optional
 * all-gather of D.  Only NCCL touches peer memory. */

/* Columns [*n0, *n1) of rank `rank` of `world`: whole tiles of tile_n columns, as even as possible, earlier ranks take
 * the extra tile, the last non-empty shard absorbs a ragged tail.  Host only. */
int sgemm_shard_columns(uint32_t n, uint32_t world, uint32_t rank, uint32_t tile_n, uint32_t *n0, uint32_t *n1);

#define SGEMM_COMM_ID_BYTES 128
/* Make the id of a new communicator (one rank calls this; the host program hands the bytes to all ranks). */
int sgemm_comm_unique_id(uint8_t id[SGEMM_COMM_ID_BYTES]);
/* Join the communicator as rank `rank` of `world` with this handle's GPU.  Collective: returns when all ranks joined. */
int sgemm_comm_init(sgemm_handle *h, const uint8_t id[SGEMM_COMM_ID_BYTES], int rank, int world);
/* One process, `count` handles on distinct GPUs: make one communicator over them, handle i = rank i. */
int sgemm_comm_init_all(sgemm_handle *const *handles, int count);
/* Leave it (sgemm_close does this too). */
int sgemm_comm_destroy(sgemm_handle *h);

/* sgemm_run_host for one rank of a sharded call: hB, hC, hD are this rank's column shards (n_local columns, may be 0),
 * hA is the whole replicated A as every rank holds it in host memory — of which only this rank's 1/world slice of
 * the columns is uploaded; the ranks then complete each other's device copies over NVLink (in-place all-gather of the
 * slices into each GPU's own memory, before any kernel reads it), so A crosses the host link once per box, not once
 * per GPU.  Collective: every rank of the communicator must make the call.  The result equals sgemm_run_host's bit
 * for bit. */
int sgemm_run_host_sharded(sgemm_handle *h, const float *hA, const float *hB, const float *hC, float *hD,
                           float alpha, float beta, uint32_t m, uint32_t n_local, uint32_t k,
                           uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd);

/* Optional all-gather of D: dD_full is a full M x N matrix (pitch ldd) on every rank, in which this rank's shard —
 * columns sgemm_shard_columns(n, world, rank, tile_n) — has been computed in place (pass dD_full + n0 * ldd to
 * sgemm_launch).  Afterwards every rank holds all of D.  In place: equal shards go as one ncclAllGather, ragged ones
 * as grouped broadcasts; no padding, no temporary.  Asynchronous on `stream`; collective. */
int sgemm_allgather_columns(sgemm_handle *h, float *dD_full, uint32_t m, uint32_t n, uint32_t ldd, uint32_t tile_n,
                            void *stream);

/* Replaces the timed loop of main (runner/generator_runner.cpp:270-280): `warmup` untimed launches, then
 * `runs` back-to-back launches between two events on `stream`; *ms_mean = elapsed / runs. Synchronises. */
int sgemm_bench(sgemm_handle *h, const float *dA, const float *dB, const float *dC, float *dD,
                float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
                uint32_t warmup, uint32_t runs, void *stream, float *ms_mean);

/* Device status words of the last kernels (synchronises the device).  status[0] == 0: no kernel gave up
 * on a wait.  Otherwise status[0] = 1 (a bounded wait ran out), [1] = role/barrier tag, [2] = tile,
 * [3] = k-block, [4] = block index, [5] = parity; the words are cleared by the call.  The reference has
 * no counterpart (it ignores every hipError_t, runner/generator_runner.cpp:194-322). */
int sgemm_last_status(sgemm_handle *h, uint32_t status[8]);

/* Failure-detection self-test (no counterpart in the reference, which never inspects an error): launches a
 * one-block kernel that waits, with the GEMM kernel's own bounded-wait routine and a limit of `timeout_ms`
 * (1..1000), on a barrier nothing arrives on.  The wait runs out, the kernel records the status words and ends
 * normally; the following sgemm_last_status must return SGEMM_ERR_DEVICE_STATUS with status[1] == tag, and the
 * handle must keep working.  Cubins whose main kernel is fed by TMA (tensor variant, TMA-fed FFMA) only: the
 * register-fed FFMA kernel waits on nothing. */
int sgemm_wait_selftest(sgemm_handle *h, uint32_t timeout_ms, uint32_t tag);

/* Options: "force_variant" 0 auto, 1 tensor (main kernel), 2 simt, 3 tensor (companion kernel for skinny shapes);
 * "skinny_below_intensity": in auto mode problems with fewer flop per byte of A and B than this (default 200: a
 * skinny M or N with a long K) run on the companion kernel (128 x 128 tiles, lo terms made in the kernel, no pre-pass;
 * with N <= 32 on its sibling with 128 x 32 tiles);
 * "skinny_below_flops": so do problems with 2*M*N*K below this (default 2^33: the pre-pass would be one more dependent
 * launch in a call that only lasts a few); "split_k" 0 auto, n >= 1 fixed;
 * "simt_below_flops" problems with 2*M*N*K below this use the SIMT kernel (auto mode);
 * "repitch" 1 (default): FP32 operands TMA cannot read where they lie (base not 16-byte aligned, leading dimension
 * not a multiple of 4) are copied to an aligned pitch in the workspace so that the tensor kernel serves them — in auto
 * mode for problems of at least "repitch_above_flops" (default 2^31), always when the tensor variant is forced; 0: such
 * problems run on the FFMA kernel, and forcing the tensor variant on them is SGEMM_ERR_UNSUPPORTED;
 * "pdl" 1 (default) launches every kernel with programmatic stream serialisation so that launch latency and per-CTA
 * set-up overlap with the tail of the previous kernel (all kernels wait on the grid dependency before touching memory);
 * "wave_sync" 1 (default) lets the persistent CTAs of the tensor kernel wait briefly for each other at tile
 * boundaries so that they keep sharing operand panels in L2 (a bounded, soft wait: performance only);
 * "pipeline_host" 1 (default) lets sgemm_run_host overlap transfers and compute over column chunks,
 * "pipeline_chunks" (2..64, default 16) says how many;
 * "profile" 1 brackets every main-GEMM-kernel launch with an event pair (read with "profile_main_ns");
 * "acc_chain": k per tensor-core accumulation chain, -1 (default) = as the kernel was generated (128 unless its
 * TOML says otherwise), 0 = all of K in one chain (fastest; the tensor core's truncating adds then drift toward zero
 * in proportion to K), otherwise a multiple of the kernel's k-block; a kernel generated without the register path
 * (acc_chain = 0 in its TOML) accepts only -1 and 0.  Problems whose K is at most two chains long are accumulated
 * in one chain in any case, and, like acc_chain 0, run on the cubin's whole-K twin of the main kernel. */
int sgemm_set_option(sgemm_handle *h, const char *key, int64_t value);

/* Facts: "variant" (of the cubin), "last_variant" (1 tensor main / 2 simt / 3 tensor companion), "last_split_k", "last_grid",
 * "last_tile_n" (columns of the tile of the last launch: tells the companion, 128, from its narrow sibling, 32),
 * "last_feed_tma" (1 when the main kernel of the last launch was fed by TMA: any tensor kernel, or the TMA-fed FFMA
 * kernel; 0 for the register-fed FFMA kernel),
 * "last_acc_chain" (k per accumulation chain of the last tensor launch, 0 = whole K), "acc_chain" and
 * "skinny_acc_chain" (the chains the main and the companion tensor kernel were generated with),
 * "launches" (kernel launches issued so far), "tile_m", "tile_n", "sm_count", "workspace_bytes",
 * "comm_rank" / "comm_world" (-1 / 0 without a communicator),
 * "sm_khz_effective" (SM clock the tensor-kernel launches since the last read of this key really ran at, counted on
 * the device as SM cycles per nanosecond of block 0; 0 without such a launch; synchronises and clears the tally),
 * "profile_count" (bracketed launches since the last read), "profile_main_ns" (their summed device time in
 * nanoseconds; synchronises on them and resets the tally). */
int sgemm_get_info(sgemm_handle *h, const char *key, int64_t *value);

/* Scratch bytes sgemm_launch needs for this problem under the current options (0 = none), for operands whose base
 * addresses are 16-byte aligned.  (No counterpart in the reference, whose kernel needs no scratch.) */
int sgemm_workspace_bytes(sgemm_handle *h, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb,
                          size_t *bytes);
/* The same for the operands a call will really get: an FP32 operand TMA cannot read where it lies (base not 16-byte
 * aligned, or leading dimension not a multiple of 4) is first copied to an aligned pitch inside the workspace, which
 * adds to the need.  dA / dB are only inspected, never dereferenced; NULL means "aligned". */
int sgemm_workspace_bytes_for(sgemm_handle *h, const void *dA, const void *dB, uint32_t m, uint32_t n, uint32_t k,
                              uint32_t lda, uint32_t ldb, size_t *bytes);

/* Lend device scratch (256-byte aligned) so that sgemm_launch never allocates; NULL returns to the
 * handle-owned, grow-on-demand workspace. */
int sgemm_set_workspace(sgemm_handle *h, void *dptr, size_t bytes);

/* Seeded U[-1,1) fill on the device: element i gets the index-hash value of (first_index + i, stream_id).
 * Replaces `randomize` (runner/Utils/BufferUtils.hpp:6-14), which is unseeded in the reference. */
int sgemm_fill_uniform(sgemm_handle *h, float *dptr, uint64_t count, uint64_t first_index,
                       uint64_t stream_id, void *stream);

/* No counterpart in the reference (FP32 only).  Device conversion of `count` FP32 values to the 16-bit operand type of
 * the loaded cubin (FP16 or BF16, round to nearest even); SGEMM_ERR_UNSUPPORTED on an FP32 cubin. */
int sgemm_narrow16(sgemm_handle *h, const float *dsrc, void *ddst, uint64_t count, void *stream);

/* Tile rasterisation of the loaded kernel: xy[2*z], xy[2*z+1] = (tile x, tile y) of launch unit z for an
 * nx x ny tile grid, computed on the device by the kernel's own mapping function (the workgroup remap of
 * generator/generator.py:1437-1464). */
int sgemm_tile_map(sgemm_handle *h, int32_t *host_xy, uint32_t nx, uint32_t ny);

/* Plain device-memory helpers so that a caller without its own CUDA binding (the runner program, a
 * ctypes harness) can stage buffers: hipMalloc / hipFree / hipMemcpy / hipMemset / hipDeviceSynchronize
 * of runner/generator_runner.cpp:236-242, 267, 289, 319-322. */
int sgemm_dev_alloc(sgemm_handle *h, size_t bytes, void **dptr);
int sgemm_dev_free(sgemm_handle *h, void *dptr);
int sgemm_dev_upload(sgemm_handle *h, void *dptr, const void *host, size_t bytes);
int sgemm_dev_download(sgemm_handle *h, void *host, const void *dptr, size_t bytes);
int sgemm_dev_memset(sgemm_handle *h, void *dptr, int byte_value, size_t bytes);
int sgemm_dev_sync(sgemm_handle *h);

/* Short text for an error code; detail of the last failure on a handle (NULL handle: last open error). */
const char *sgemm_strerror(int code);
const char *sgemm_last_error(sgemm_handle *h);

/* Number of CUDA devices (<= 0: none or no driver). Host-side probe used by the runner program. */
int sgemm_device_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SGEMM_RUNNER_H */
