// ---------------------------------------------------------------------------------------------
// TMA-fed, warp-specialised pure-FFMA SGEMM (strict FP32).  Same arithmetic, thread tiles and epilogue as the FFMA kernel
// of sgemm_simt.cuh (which must precede this file in the translation unit: ffma_outer_product2 and ffma_epilogue are
// defined there), but the operand tiles are not carried through registers: one producer thread issues two TMA box
// copies per k-step into a ring of FT_STAGES shared-memory stages and the FT_CONSUMERS consumer threads only read
// fragments and multiply.  Stages are handed over with mbarriers ("full": the copies' bytes have landed; "ready": the
// B tile has been transposed, where that is needed; "empty": every consumer warp has read the stage), so the block has
// no block-wide barrier in its main loop, no global loads or shared stores in the multiplying warps, and copies run
// FT_STAGES - 1 steps ahead of the arithmetic.
//
// What TMA can describe decides who may use this kernel: FP32 operands with 16-byte aligned bases and leading
// dimensions that are multiples of 4; A stored untransposed.  The runner launches the register-fed kernel of the same
// cubin for everything else.  M, N and K themselves are arbitrary: a box that reaches past the matrix is zero-filled by
// TMA, and the epilogue guards rows and columns.
//
// Stage layout (floats):  A tile [FT_BK][FT_BM] (box {BM, BK} of the M x K matrix: row = one k), then the B tile
// [FT_BK][FT_BN] (row = one k) in which every thread finds the FT_TN values of a k-slice in 16-byte vectors:
//   B transposed (N contiguous):   TMA writes it (box {BN, BK} of the N x K matrix).
//   B untransposed (K contiguous): TMA cannot transpose.  It writes the box {BK, BN} of the K x N matrix (row = one n)
//     into a third, raw buffer of the stage, and the three warps that share the producer's warp group copy it,
//     transposed, into the B tile: 16-byte reads along k with the k-quad rotated over the lanes, 4-byte writes with
//     32 consecutive n per warp, both free of bank conflicts.  (Reading a K-contiguous tile straight from the
//     multiplying threads, eight rows per k-slice, measured 13 % slower than the register-fed kernel.)
//
// Every mbarrier wait is bounded: after FT_TIMEOUT_NS without progress the waiting thread records what it waited for
// in the status words, raises a block-wide flag, every role leaves its loop, the block waits for copies that may still
// be in flight and returns without writing D.
//
// Warps: the first group of four holds the producer (warp 0, one lane) and the transposing warps 1 to 3 (idle when B
// needs no transposing), the consumers follow.  Registers can be handed from one role to another only in groups of
// four warps (setmaxnreg), and every scheduler partition holds one warp of each group: the first group shrinks to
// FT_REGS_PRODUCER registers per thread and the consumers grow to FT_REGS_CONSUMER, which is what lets 256 consumers hold
// 16 x 8 accumulators each.  One block per SM (a tile lasts about a millisecond at K = 8192, its prologue and epilogue
// a few microseconds).
//
// Generator-supplied macros: FT_ENTRY, FT_BM, FT_BN, FT_BK (block tile), FT_TM, FT_TN (thread tile: 4 x 4 blocks strided
// over the block tile, as in the register-fed kernel), FT_STAGES.
// Launch: grid (tiles_m * tiles_n, 1, split_k), block FT_THREADS, FT_SMEM_BYTES of dynamic shared memory.
// ---------------------------------------------------------------------------------------------
#ifndef FT_STAGES
#define FT_STAGES 4
#endif
#ifndef FT_TIMEOUT_NS
#define FT_TIMEOUT_NS 2000000000ull
#endif
#define FT_TX (FT_BM / FT_TM)
#define FT_TY (FT_BN / FT_TN)
#define FT_GM (FT_TM / 4)
#define FT_GN (FT_TN / 4)
#define FT_CONSUMERS (FT_TX * FT_TY)
#define FT_CONSUMER_WARPS (FT_CONSUMERS / 32)
#define FT_FIRST_CONSUMER 128                 // threads of the first warp group (producer + three transposing warps)
#define FT_THREADS (FT_FIRST_CONSUMER + FT_CONSUMERS)
// Register hand-over.  Every scheduler partition holds one warp of the first group and FT_CONSUMERS / 128 consumer warps,
// and owns 512 registers per lane; __launch_bounds__ lets ptxas give every thread FT_REGS_LAUNCH of them, which is what
// it does for a kernel that contains setmaxnreg.  The block can only ever redistribute what it was launched with
// (setmaxnreg.inc waits, without limit, for registers that other warps of the block release): the consumers' gain
// must not exceed what the first group gives up, which the static_assert below holds the numbers to.  With 128
// consumers the launch allocation already is the per-thread maximum and nothing is handed over.
#define FT_WARPS_PER_PARTITION (FT_THREADS / 128)
#define FT_REGS_LAUNCH ((512 / FT_WARPS_PER_PARTITION) / 8 * 8)
#define FT_REG_HANDOVER (FT_CONSUMERS >= 256)
#define FT_REGS_PRODUCER 40
#define FT_REGS_CONSUMER_RAW ((FT_WARPS_PER_PARTITION * FT_REGS_LAUNCH - FT_REGS_PRODUCER) / (FT_WARPS_PER_PARTITION - 1) / 8 * 8)
#define FT_REGS_CONSUMER (FT_REGS_CONSUMER_RAW > 232 ? 232 : FT_REGS_CONSUMER_RAW)
#define FT_XFORM (!GEMM_TRANS_B)              // B arrives K-contiguous and is transposed in shared memory
#define FT_XFORM_WARPS 3
#define FT_A_FLOATS (FT_BK * FT_BM)
#define FT_B_FLOATS (FT_BK * FT_BN)
#define FT_RAW_FLOATS (FT_XFORM ? FT_BK * FT_BN : 0)
#define FT_STAGE_FLOATS (FT_A_FLOATS + FT_B_FLOATS + FT_RAW_FLOATS)
#define FT_TMA_BYTES ((FT_A_FLOATS + FT_B_FLOATS) * 4)           // what the two copies of a stage deliver
#define FT_SMEM_BYTES (FT_STAGES * FT_STAGE_FLOATS * 4 + 128 + 512)   // ring + alignment slack + barriers and abort flag
#define FT_KQ (FT_BK / 4)                     // 16-byte vectors along k in a row of the raw B tile

static_assert(FT_TM % 4 == 0 && FT_TN % 4 == 0 && FT_BM % FT_TM == 0 && FT_BN % FT_TN == 0 && FT_BK % 4 == 0, "tile shapes");
static_assert(FT_CONSUMERS % 128 == 0, "consumers are whole groups of four warps");
static_assert(!GEMM_TRANS_A, "the TMA-fed FFMA kernel reads an untransposed A");
static_assert(FT_BM <= 256 && FT_BN <= 256 && FT_BK <= 256, "a TMA box has at most 256 elements per dimension");
static_assert(!FT_XFORM || (FT_BN % 32 == 0 && (FT_KQ & (FT_KQ - 1)) == 0), "the transposing warps take 32 columns at a time and rotate a power-of-two number of k-quads");
static_assert(FT_STAGES >= 2 && FT_STAGES <= 12, "ring depth");
static_assert(!FT_REG_HANDOVER || ((FT_WARPS_PER_PARTITION - 1) * FT_REGS_CONSUMER + FT_REGS_PRODUCER <= FT_WARPS_PER_PARTITION * FT_REGS_LAUNCH &&
                                   FT_REGS_CONSUMER > FT_REGS_LAUNCH && FT_REGS_PRODUCER < FT_REGS_LAUNCH),
              "register hand-over: the consumers may only take what the first warp group releases");
static_assert(FT_SMEM_BYTES <= 232448, "shared memory budget of one CTA");

struct alignas(64) FtTensorMap { uint64_t opaque[16]; };

__device__ __forceinline__ uint32_t ft_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t ft_globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void ft_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void ft_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ft_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t ft_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// TMA box copy into this CTA's shared memory; the bytes are counted on the mbarrier `bar`
__device__ __forceinline__ void ft_tma_load_2d(uint32_t dst, const FtTensorMap *map, uint32_t bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

struct FtWait {
    volatile uint32_t *abort_flag;  // shared memory, block-wide
    uint32_t *status;               // global memory, SGEMM_STATUS_WORDS words
    uint64_t timeout_ns;            // how long one wait may go without the barrier completing
};
// tags of the status record: which role gave up
#define FT_TAG_PRODUCER 0x46540001u   // producer waiting for a stage to be read ("empty")
#define FT_TAG_CONSUMER 0x46540002u   // a consumer waiting for a stage's copies ("full")
#define FT_TAG_XFORM 0x46540003u      // a transposing warp waiting for a stage's copies ("full")
#define FT_TAG_READY 0x46540004u      // a consumer waiting for the transposed B tile ("ready")

__device__ __forceinline__ bool ft_wait_slow(const FtWait &w, uint32_t bar, uint32_t parity, uint32_t tag, uint32_t step) {
    const uint64_t t0 = ft_globaltimer();
    uint32_t spins = 0;
    for (;;) {
        if (ft_mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0u) {
            if (*w.abort_flag) return false;
            if (ft_globaltimer() - t0 > w.timeout_ns) {
                *w.abort_flag = 1u;
                if (atomicCAS(w.status, SGEMM_STATUS_OK, SGEMM_STATUS_TIMEOUT) == SGEMM_STATUS_OK) {
                    w.status[1] = tag;
                    w.status[2] = blockIdx.x;
                    w.status[3] = step;
                    w.status[4] = blockIdx.z;
                    w.status[5] = parity;
                }
                __threadfence();
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool ft_wait(const FtWait &w, uint32_t bar, uint32_t parity, uint32_t tag, uint32_t step) {
    if (ft_mbar_try_wait(bar, parity)) return true;
    return ft_wait_slow(w, bar, parity, tag, step);
}

// Fragments of k-slice kk of a stage, 16-byte vectors along M and N.  as: this thread's first A element of the stage
// (tile + tx*4); bs: its first B element (tile + ty*4).
__device__ __forceinline__ void ft_load_fragments(int kk, const float *__restrict__ as, const float *__restrict__ bs,
                                                  float (&fa)[FT_TM], float (&fb)[FT_TN]) {
#pragma unroll
    for (int g = 0; g < FT_GM; ++g) {
        const float4 v = *reinterpret_cast<const float4 *>(as + kk * FT_BM + g * FT_TX * 4);
        fa[g * 4 + 0] = v.x; fa[g * 4 + 1] = v.y; fa[g * 4 + 2] = v.z; fa[g * 4 + 3] = v.w;
    }
#pragma unroll
    for (int g = 0; g < FT_GN; ++g) {
        const float4 v = *reinterpret_cast<const float4 *>(bs + kk * FT_BN + g * FT_TY * 4);
        fb[g * 4 + 0] = v.x; fb[g * 4 + 1] = v.y; fb[g * 4 + 2] = v.z; fb[g * 4 + 3] = v.w;
    }
}

// One stage: FT_BK k-slices, the fragments of slice kk + 1 requested before the multiplications of slice kk are issued.
__device__ __forceinline__ void ft_stage(uint64_t (&acc2)[FT_TN][FT_TM / 2], const float *__restrict__ as,
                                         const float *__restrict__ bs) {
    float fa[2][FT_TM], fb[2][FT_TN];
    ft_load_fragments(0, as, bs, fa[0], fb[0]);
#pragma unroll
    for (int kk = 0; kk < FT_BK; ++kk) {
        if (kk + 1 < FT_BK) ft_load_fragments(kk + 1, as, bs, fa[(kk + 1) & 1], fb[(kk + 1) & 1]);
        ffma_outer_product2<FT_TM, FT_TN>(acc2, fa[kk & 1], fb[kk & 1]);
    }
}

#if FT_XFORM
// raw [FT_BN][FT_BK] (row = one n) -> tile [FT_BK][FT_BN] (row = one k), by one of the FT_XFORM_WARPS transposing warps.
// A work item is 32 columns x one k-quad per lane: lane l reads the 16 bytes of column n0 + l at k-quad
// (l * min(KQ, 8) / 8 + c) mod KQ — within the 8 lanes of a shared-memory wavefront the rows are 4*FT_BK bytes apart,
// and rotating the k-quad spreads them over the banks — and writes its four values to four rows of the tile, where the
// 32 lanes of the warp hit 32 consecutive words.
__device__ __forceinline__ void ft_transpose_b(const float *__restrict__ raw, float *__restrict__ tile, uint32_t xwarp, uint32_t lane) {
    constexpr uint32_t kItems = (FT_BN / 32) * FT_KQ;
    constexpr uint32_t kSpread = FT_KQ < 8 ? FT_KQ : 8;
    for (uint32_t item = xwarp; item < kItems; item += FT_XFORM_WARPS) {
        const uint32_t n = (item / FT_KQ) * 32 + lane;
        const uint32_t kq = ((lane % 8) * kSpread / 8 + item % FT_KQ) % FT_KQ;
        const float4 v = *reinterpret_cast<const float4 *>(raw + n * FT_BK + kq * 4);
        float *dst = tile + (kq * 4) * FT_BN + n;
        dst[0] = v.x;
        dst[FT_BN] = v.y;
        dst[2 * FT_BN] = v.z;
        dst[3 * FT_BN] = v.w;
    }
}
#endif

extern "C" __global__ void __launch_bounds__(FT_THREADS, 1)
FT_ENTRY(const float *__restrict__ a, const float *__restrict__ b, const float *c, float *d,
         uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
         float alpha, float beta, int32_t num_wg_x, int32_t num_wg_y,
         float *ws, uint32_t *status, uint32_t split_k,
         uint32_t *wave_sync, uint32_t wave_sync_base,
         const __grid_constant__ FtTensorMap map_a, const __grid_constant__ FtTensorMap map_b) {
    extern __shared__ uint8_t ft_smem_raw[];
    (void)a; (void)b; (void)lda; (void)ldb;   // the operands are reached through the tensor maps
    (void)wave_sync; (void)wave_sync_base;    // one tile per block: nothing to align

    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(ft_smem_raw) + 127) & ~(uintptr_t)127);
    float *ring = reinterpret_cast<float *>(base);
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + FT_STAGES * FT_STAGE_FLOATS * 4);   // full[S] | empty[S] | ready[S]
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(bars + 3 * FT_STAGES);
    const uint32_t full0 = ft_smem_u32(bars), empty0 = ft_smem_u32(bars + FT_STAGES), ready0 = ft_smem_u32(bars + 2 * FT_STAGES);
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < FT_STAGES; ++s) {
            ft_mbar_init(full0 + 8 * s, 1);
            ft_mbar_init(empty0 + 8 * s, FT_CONSUMER_WARPS);
            ft_mbar_init(ready0 + 8 * s, FT_XFORM_WARPS);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const FtWait waiter{abort_flag, status, FT_TIMEOUT_NS};

    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    uint32_t tile_x, tile_y;
    sgemm_tile_raster(blockIdx.x, (uint32_t)num_wg_x, (uint32_t)num_wg_y, OPT_WGM, tile_x, tile_y);
    const uint32_t m0 = tile_x * FT_BM, n0 = tile_y * FT_BN;

    // K range of this split (whole FT_BK steps per split; the last split takes the tail, which TMA zero-fills)
    const uint32_t steps_total = (k + FT_BK - 1) / FT_BK;
    const uint32_t steps_per = (steps_total + split_k - 1) / split_k;
    const uint32_t k_begin = min(k, blockIdx.z * steps_per * FT_BK);
    const uint32_t k_end = min(k, k_begin + steps_per * FT_BK);
    const uint32_t steps = (k_end - k_begin + FT_BK - 1) / FT_BK;

    if (threadIdx.x < FT_FIRST_CONSUMER) {
#if FT_REG_HANDOVER
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FT_REGS_PRODUCER));
#endif
        // ------------------------------------------------------------------ producer: one lane issues the copies
        if (warp == 0 && lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            for (uint32_t t = 0; t < steps; ++t) {
                const uint32_t s = t % FT_STAGES, round = t / FT_STAGES;
                // a stage is free once the consumers have read its previous contents (first round: free from the start)
                if (!ft_wait(waiter, empty0 + 8 * s, (round & 1u) ^ 1u, FT_TAG_PRODUCER, t)) break;
                const uint32_t full = full0 + 8 * s;
                const uint32_t dst_a = ft_smem_u32(ring + (size_t)s * FT_STAGE_FLOATS);
                const int32_t k0 = (int32_t)(k_begin + t * FT_BK);
                ft_mbar_expect_tx(full, FT_TMA_BYTES);
                ft_tma_load_2d(dst_a, &map_a, full, (int32_t)m0, k0);
#if FT_XFORM
                ft_tma_load_2d(dst_a + (FT_A_FLOATS + FT_B_FLOATS) * 4, &map_b, full, k0, (int32_t)n0);   // the raw buffer
#else
                ft_tma_load_2d(dst_a + FT_A_FLOATS * 4, &map_b, full, (int32_t)n0, k0);
#endif
            }
        }
#if FT_XFORM
        // -------------------------------------------------------------- warps 1 to 3: transpose the B tile of every stage
        // (the raw buffer and the tile of a stage are free when its copies land: the producer issued them only after
        // the consumers had released the stage, and these warps finished with its raw buffer before the consumers began)
        if (warp >= 1) {
            for (uint32_t t = 0; t < steps; ++t) {
                const uint32_t s = t % FT_STAGES, round = t / FT_STAGES;
                if (!ft_wait(waiter, full0 + 8 * s, round & 1u, FT_TAG_XFORM, t)) break;
                float *stage = ring + (size_t)s * FT_STAGE_FLOATS;
                ft_transpose_b(stage + FT_A_FLOATS + FT_B_FLOATS, stage + FT_A_FLOATS, warp - 1, lane);
                __syncwarp();
                if (lane == 0) ft_mbar_arrive(ready0 + 8 * s);
            }
        }
#endif
    } else {
#if FT_REG_HANDOVER
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FT_REGS_CONSUMER));
#endif
        // ------------------------------------------------------------------ consumers: fragments and packed FMAs
        const uint32_t ct = threadIdx.x - FT_FIRST_CONSUMER;
        const uint32_t tx = ct % FT_TX, ty = ct / FT_TX;
        uint64_t acc2[FT_TN][FT_TM / 2];
#pragma unroll
        for (int j = 0; j < FT_TN; ++j)
#pragma unroll
            for (int i = 0; i < FT_TM / 2; ++i) acc2[j][i] = 0ull;

        const uint32_t a_off = tx * 4, b_off = FT_A_FLOATS + ty * 4;
        bool ok = true;
        for (uint32_t t = 0; t < steps; ++t) {
            const uint32_t s = t % FT_STAGES, round = t / FT_STAGES;
            // the A tile is TMA's: wait for the copies themselves, then (where B is transposed here) for the B tile
            if (!ft_wait(waiter, full0 + 8 * s, round & 1u, FT_TAG_CONSUMER, t)) { ok = false; break; }
#if FT_XFORM
            if (!ft_wait(waiter, ready0 + 8 * s, round & 1u, FT_TAG_READY, t)) { ok = false; break; }
#endif
            const float *stage = ring + (size_t)s * FT_STAGE_FLOATS;
            ft_stage(acc2, stage + a_off, stage + b_off);
            __syncwarp();
            if (lane == 0) ft_mbar_arrive(empty0 + 8 * s);
        }
        if (ok && !*abort_flag) {
            float acc[FT_TN][FT_TM];
#pragma unroll
            for (int j = 0; j < FT_TN; ++j)
#pragma unroll
                for (int i = 0; i < FT_TM / 2; ++i)
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[j][2 * i]), "=f"(acc[j][2 * i + 1]) : "l"(acc2[j][i]));
            ffma_epilogue<FT_TM, FT_TN, FT_TX, FT_TY>(acc, c, d, ws, m, n, ldc, ldd, alpha, beta, split_k, m0, n0, tx, ty);
        }
    }

    // teardown: every thread gets here on both the normal and the abort path
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // copies that were issued but never waited for may still be in flight: the block's shared memory must not be
        // given to another block before they have landed
        const uint64_t t0 = ft_globaltimer();
        while (ft_globaltimer() - t0 < 2000000ull) __nanosleep(1000);
    }
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait (same entry name and arguments as the tensor kernels' self-test, of which a cubin
// holds one or the other): one block initialises an mbarrier that nothing will ever arrive on and waits on it with this
// kernel's own wait routine and a short limit.  The wait must run out, record the status words and return, the kernel
// must end normally and the context must stay usable.
// ---------------------------------------------------------------------------------------------
extern "C" __global__ void sgemm_wait_selftest(uint32_t *status, uint64_t timeout_ns, uint32_t tag) {
    __shared__ __align__(8) uint64_t barrier_storage;
    __shared__ uint32_t abort_flag;
    sgemm_grid_dependency_wait();
    if (threadIdx.x == 0) {
        ft_mbar_init(ft_smem_u32(&barrier_storage), 1);
        abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const FtWait waiter{&abort_flag, status, timeout_ns};
    // every thread waits; the first whose limit runs out reports, the others leave through the abort flag
    const bool completed = ft_wait(waiter, ft_smem_u32(&barrier_storage), 0u, tag, threadIdx.x);
    if (completed && threadIdx.x == 0) status[6] = 0xBAD0BAD0u;   // cannot happen: nobody arrives
    __syncthreads();
}
