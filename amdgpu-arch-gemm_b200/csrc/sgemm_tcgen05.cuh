// ---------------------------------------------------------------------------------------------
// 3xTF32 split-precision SGEMM on the sm_100a tensor cores (tcgen05.mma, accumulators in TMEM).
//
//   A*B  ~=  A_lo*B_hi + A_hi*B_lo + A_hi*B_hi          (the lo*lo term is below FP32 rounding)
//
// hi is the raw FP32 operand (the tensor core reads only its top 19 bits), lo = x - trunc_tf32(x)
// is written once per call by sgemm_split_lo.  All three products accumulate into one FP32 TMEM
// accumulator, k ascending, in chains of a fixed length that are added up in a fixed order (see
// "chunked accumulation"), so results do not depend on scheduling (bit-reproducible).
//
// Roles of the warps of a CTA (persistent over output tiles, tile = blockIdx + i*gridDim).  Roles are laid out in
// groups of four warps, the unit in which registers can be handed from one role to another (setmaxnreg):
//   warp 0, one lane : TMA producer. Per k-block it fills one ring stage with four operand tiles
//                      (A_hi, A_lo, B_hi, B_lo) and arms the stage's "full" mbarrier with the bytes.
//   warp 1, one lane : MMA issuer. Waits "full", issues 3 * TC_BK/8 tcgen05.mma (K = 8 each) and
//                      commits them to the stage's "empty" mbarrier; after the last k-block of a
//                      tile it commits to the accumulator's "tmem_full" mbarrier. Warp 1 also owns
//                      the TMEM allocation (two accumulator buffers, so the epilogue of tile i
//                      overlaps the main loop of tile i+1).
//   warps 2, 3       : no work (they complete the first group of four).
//   warps 4..7 (..11): epilogue, TC_EPI_WARPS = 4 or 8 warps. Warp w reads TMEM lanes 32*(w%4)..+31
//                      (= rows of the tile) with tcgen05.ld, applies alpha/beta and stores straight to
//                      global memory: D is column-major, so the 32 lanes of a warp write 128 contiguous
//                      bytes per column.  With 8 warps the two warps of a lane quarter take half of the
//                      tile's columns each, which doubles the loads/stores in flight (it matters when K
//                      is small or C is read).
//   4 more warps     : (TC_SPLIT_INKERNEL) transform warps that write the lo tiles in shared memory.
//
// Chunked accumulation (kernels generated with TC_ACC_CHUNK > 0, launched with acc_chunk > 0).  The tensor core
// adds products into its accumulator with truncation (toward zero, two guard bits), so an unbroken chain of MMAs
// drifts toward zero in proportion to its length.  The issuer therefore starts a fresh accumulator, in the other
// TMEM buffer, every acc_chunk k-blocks (the first two chunks of a tile are twice as long), and the epilogue warps
// add the finished chunks, in chunk order and with round-to-nearest FP32 adds, to a running sum in registers; the
// epilogue proper then runs from registers.  The running sum needs TC_EPI_COLS registers per epilogue thread; with
// 8 epilogue warps the other warp groups give registers up and the epilogue groups take them.  The generator emits
// this template a second time with TC_ACC_CHUNK = 0 (entry generated_gemm_wholek: one chain per launch unit, the
// accumulator written out straight from TMEM) for problems whose k range per unit is a single chunk anyway.
//
// Operand tiles in shared memory (128-byte swizzle, written by TMA, read by the tensor core):
//   A (column-major, M contiguous => "MN-major" operand): per 32 rows of M one chunk of TC_BK rows
//     of 128 bytes (row = one k, 32 consecutive m).  32-bit MN-major operands must use the 128-byte
//     swizzle with 32-byte atoms (descriptor layout 1; TMA mode SWIZZLE_128B_ATOM_32B), whose
//     repeating unit is 4 rows: LBO = chunk stride (next 32 rows of M), SBO = 4 rows = 512 B (next
//     4 k); one K=8 MMA step spans two units and advances the start address by 1024 B.
//   B (K contiguous per column => "K-major" operand): per 32 k one sub-tile of BN rows of 128 bytes
//     (row = one n, 32 consecutive k);                SBO = 8 rows = 1024 B;
//     one K=8 MMA step advances the start address by 32 B inside the swizzle span.
//     TC_BK = 16 uses 64-byte rows with the 64-byte swizzle instead (SBO = 512 B).
//   With TC_A_KMAJOR the A operand is K-major — the caller's A is stored transposed (K contiguous), or
//   packed copies made by sgemm_pack_a_kmajor are read — and uses B's layout.  With TC_B_MNMAJOR the
//   caller's B is stored transposed (N contiguous) and uses A's MN-major layout (32-column chunks).
//   16-bit operands (TC_ELEM_BYTES = 2) use the same two layouts with twice the elements per 128-byte row:
//   K-major rows of 64 k, MN-major chunks of 64 rows of M (or columns of N) with the ordinary 128-byte swizzle
//   of 16-byte units (repeating unit 8 rows: SBO = 1024 B; one K=16 MMA step spans two units, 2048 B).
//
// TC_CTA_GROUP = 2 pairs two CTAs (a 2x1 cluster, two neighbouring SMs) on one 256 x TC_BN tile with
// tcgen05.mma.cta_group::2: CTA r of the pair loads rows 128r.. of the A tile and columns (TC_BN/2)r.. of
// the B tile into its OWN shared memory (no cluster-wide copies), so per SM the B traffic halves and a
// stage shrinks to 2*(128 + TC_BN/2)*TC_BK*4 bytes.  Only the leader (rank 0) issues MMAs; they read both
// CTAs' shared memory and write both CTAs' TMEM (each CTA holds its 128 rows x TC_BN columns).  Barriers:
//   full[s]      lives in the leader; both CTAs' TMA loads report their bytes to it
//   empty[s]     one per CTA; the leader commits to its own and to the peer's copy (two plain commits)
//   tmem_full[b] one per CTA, committed the same way;  tmem_empty[b] in the leader, the epilogue warps of both CTAs arrive
//
// TC_SPLIT_INKERNEL = 1 drops the pre-pass: TMA brings only the raw (hi) tiles, four extra "transform" warps
// (the last warp group) compute lo = x - trunc_tf32(x) from the landed tile into the stage's lo tile (element-wise,
// so the swizzle does not matter), publish the writes to the tensor core's proxy with fence.proxy.async and
// arrive on the stage's "ready" barrier, which the MMA issuer then waits on instead of "full".  In a CTA pair
// "full" is then local to each CTA (each transforms what it loaded) and "ready" lives in the leader
// (4 warps x 2 CTAs arrive).  Operand traffic from L2/HBM halves and no lo copies exist in global memory.
// TC_SPLIT_HYBRID = 1 (with TC_SPLIT_INKERNEL) is the middle way: A's lo tile still comes from the pre-pass by TMA,
// only B's lo tile is made by the transform warps — three quarters of the TMA traffic of the pre-pass scheme, half of
// the transform traffic of the in-kernel scheme.
//
// Split-K (split_k > 1): every launch unit covers one K range of one tile and stores its raw partial to the
// workspace; the host runs sgemm_splitk_reduce afterwards (fixed summation order, no atomics).
//
// Every mbarrier wait is bounded: after TC_TIMEOUT_NS without progress the waiting role records a
// status word, raises a CTA-wide abort flag and all roles leave their loops, release TMEM and
// return; the host reads the status after synchronising.
//
// Generator-supplied macros: TC_BN (tile columns), TC_BK (k per stage: 16 or a multiple of 32), TC_STAGES,
// TC_CTA_GROUP (1/2), TC_EPI_WARPS (4/8), TC_SPLIT_INKERNEL (0/1), TC_A_KMAJOR (0/1), TC_B_MNMAJOR (0/1),
// TC_TERMS (3 = 3xTF32, 1 = one MMA per k-slice: plain TF32 for bring-up, or 16-bit operands), TC_ELEM_BYTES (4 / 2),
// TC_AB_FORMAT (operand type code of the instruction descriptor), TC_ACC_CHUNK (default accumulation chain in k-blocks, 0 = the
// kernel has no running sum), OPT_WGM.
// ---------------------------------------------------------------------------------------------
#ifndef TC_TERMS
#define TC_TERMS 3
#endif
#ifndef TC_ELEM_BYTES
#define TC_ELEM_BYTES 4   // operand element size: 4 = FP32 (kind::tf32, split precision), 2 = FP16 / BF16 (kind::f16)
#endif
#ifndef TC_AB_FORMAT
#define TC_AB_FORMAT 2u   // operand type code of the instruction descriptor: 2 = TF32; with kind::f16: 0 = F16, 1 = BF16
#endif
#define TC_MMA_K (32 / TC_ELEM_BYTES)              // k extent of one MMA instruction: 32 bytes of K per operand row
#define TC_OPERAND_TILES (TC_TERMS == 3 ? 2 : 1)   // tiles per operand and stage: hi and lo, or the operand alone
#ifndef TC_TIMEOUT_NS
#define TC_TIMEOUT_NS 2000000000ull
#endif
#ifndef TC_WAVE_SYNC_NS
#define TC_WAVE_SYNC_NS 100000ull   // longest a unit waits for the others at a tile boundary (soft, see the producer)
#endif

#ifndef TC_ACC_CHUNK
#define TC_ACC_CHUNK 0   // != 0: the kernel can cut the accumulation into chains of `acc_chunk` k-blocks (a kernel argument) and add the
                         // chains up in FP32 registers; the value is the generator's default chain, in k-blocks
#endif
#ifndef TC_CTA_GROUP
#define TC_CTA_GROUP 1
#endif
#ifndef TC_B_MNMAJOR
#define TC_B_MNMAJOR 0   // 1: B is stored N-contiguous (the caller's B is transposed), read as an MN-major operand
#endif
#define TC_BM 128                              // rows of A (and of the accumulator) per CTA
#define TC_UMMA_M (TC_BM * TC_CTA_GROUP)       // rows of the launch unit's tile = UMMA M
#define TC_BN_CTA (TC_BN / TC_CTA_GROUP)       // columns of B this CTA keeps in shared memory
#ifndef TC_SPLIT_INKERNEL
#define TC_SPLIT_INKERNEL 0
#endif
#ifndef TC_SPLIT_HYBRID
#define TC_SPLIT_HYBRID 0
#endif
#ifndef TC_EPI_WARPS
#define TC_EPI_WARPS 4
#endif
#define TC_XFORM_WARPS (TC_SPLIT_INKERNEL ? 4 : 0)
#define TC_THREADS (128 + 32 * TC_EPI_WARPS + 32 * TC_XFORM_WARPS)
#define TC_FIRST_EPI_WARP 4u
#ifndef TC_CW
#define TC_CW 16  // columns of C per fetch in the epilogue that runs from registers (three buffers of this size)
#endif
#define TC_EPI_COLS (TC_BN / (TC_EPI_WARPS / 4))   // accumulator columns one epilogue warp drains per tile
static_assert(TC_EPI_WARPS == 4 || TC_EPI_WARPS == 8, "one or two epilogue warps per TMEM lane quarter");
// Registers.  A scheduler partition owns 512 registers per lane and runs TC_THREADS/128 warps of this CTA, one of
// each group of four.  With 8 epilogue warps and a running sum (chunked accumulation) an even share is too small for
// the epilogue threads, so the other groups shrink to TC_REGS_SMALL and the two epilogue groups grow to TC_REGS_EPI.
#define TC_WARPS_PER_PARTITION (TC_THREADS / 128)
#define TC_REGS_LAUNCH ((512 / TC_WARPS_PER_PARTITION) / 8 * 8)           // what __launch_bounds__ lets ptxas use
#define TC_REG_HANDOVER (TC_ACC_CHUNK > 0 && TC_EPI_WARPS == 8)
#define TC_REGS_SMALL 40
#define TC_REGS_EPI (((TC_WARPS_PER_PARTITION * TC_REGS_LAUNCH - (TC_WARPS_PER_PARTITION - 2) * TC_REGS_SMALL) / 2) / 8 * 8)
static_assert(!TC_REG_HANDOVER || (2 * TC_REGS_EPI + (TC_WARPS_PER_PARTITION - 2) * TC_REGS_SMALL <= TC_WARPS_PER_PARTITION * TC_REGS_LAUNCH &&
                                   TC_REGS_EPI <= 232 && TC_REGS_EPI > TC_REGS_LAUNCH && TC_REGS_SMALL < TC_REGS_LAUNCH),
              "the register hand-over must not ask for more than the launch allocated");
static_assert(TC_EPI_COLS % 32 == 0, "an epilogue warp drains whole 32-column chunks");
#define TC_A_BYTES (TC_BM * TC_BK * TC_ELEM_BYTES)
#define TC_B_BYTES (TC_BN_CTA * TC_BK * TC_ELEM_BYTES)
#define TC_STAGE_BYTES (TC_OPERAND_TILES * (TC_A_BYTES + TC_B_BYTES))   // [A | A_lo] [B | B_lo]
#define TC_KSPAN (TC_BK * TC_ELEM_BYTES >= 128 ? 128 / TC_ELEM_BYTES : TC_BK)   // k per swizzled row of a K-major tile (128- or 64-byte rows)
#define TC_KROW_BYTES (TC_KSPAN * TC_ELEM_BYTES)
#define TC_KSUBS (TC_BK / TC_KSPAN)            // K-major sub-tiles per stage
#define TC_MN_CHUNK (128 / TC_ELEM_BYTES)      // MN-major: rows of M (columns of N) per chunk = elements per 128-byte row
#define TC_A_CHUNK_BYTES (TC_BK * 128)         // MN-major: TC_MN_CHUNK rows of M x TC_BK
#define TC_MN_SBO (TC_ELEM_BYTES == 4 ? 512 : 1024)      // MN-major: bytes between the swizzle's repeating units along K
#define TC_MN_STEP (TC_MMA_K * 128)            // MN-major: bytes one MMA's k extent spans
#define TC_A_SUB_BYTES (TC_BM * TC_KROW_BYTES) // K-major : TC_BM rows x TC_KSPAN k
#define TC_B_SUB_BYTES (TC_BN_CTA * TC_KROW_BYTES) // K-major : TC_BN_CTA rows x TC_KSPAN k
#define TC_TMEM_COLS_NEEDED (2 * TC_BN)
#define TC_TMEM_COLS (TC_TMEM_COLS_NEEDED <= 32 ? 32 : TC_TMEM_COLS_NEEDED <= 64 ? 64 : \
                      TC_TMEM_COLS_NEEDED <= 128 ? 128 : TC_TMEM_COLS_NEEDED <= 256 ? 256 : 512)
#define TC_SMEM_BYTES (TC_STAGES * TC_STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/)

static_assert(TC_ELEM_BYTES == 4 || TC_ELEM_BYTES == 2, "FP32 or 16-bit operands");
static_assert(TC_BK * TC_ELEM_BYTES == 64 || (TC_BK * TC_ELEM_BYTES) % 128 == 0, "k per stage: one 64-byte span or whole 128-byte swizzle spans");
static_assert(TC_ELEM_BYTES == 4 || (TC_TERMS == 1 && !TC_SPLIT_INKERNEL), "16-bit operands: one MMA per k-slice, no lo tiles");
static_assert(!TC_SPLIT_INKERNEL || TC_TERMS == 3, "the in-kernel split makes the lo tiles of the 3xTF32 scheme");
static_assert(!TC_SPLIT_HYBRID || TC_SPLIT_INKERNEL, "the hybrid split is the in-kernel pipeline with A's lo tile loaded by TMA");
static_assert(TC_CTA_GROUP == 1 || TC_CTA_GROUP == 2, "one CTA or a CTA pair per tile");
static_assert(!TC_B_MNMAJOR || (TC_BN / TC_CTA_GROUP) % TC_MN_CHUNK == 0, "MN-major B is staged in chunks of 128 bytes of N");
static_assert(TC_BN % (16 * TC_CTA_GROUP) == 0 && TC_BN >= 16 * TC_CTA_GROUP && TC_BN <= 256, "UMMA N");
static_assert(TC_SMEM_BYTES <= 232448, "shared memory budget of one CTA");

struct alignas(64) TcTensorMap { uint64_t opaque[16]; };

// --------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t tc_smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t tc_globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t tc_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// TMA tile load into this CTA's shared memory.  In a CTA pair the completion bytes are reported to the
// leader's mbarrier (`bar` is then a shared::cluster address), which the cta_group::2 form permits.
__device__ __forceinline__ void tc_tma_load_2d(uint32_t dst, const TcTensorMap *map, uint32_t bar,
                                               int32_t x, int32_t y) {
#if TC_CTA_GROUP == 2
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
#else
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
#endif
}
// TMA tile load whose completion is reported to a barrier of this same CTA (any cluster shape).
__device__ __forceinline__ void tc_tma_load_2d_local(uint32_t dst, const TcTensorMap *map, uint32_t bar,
                                                     int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t tc_map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void tc_mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_prefetch_map(const TcTensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
#if TC_ELEM_BYTES == 4
#define TC_MMA_KIND "kind::tf32"
#else
#define TC_MMA_KIND "kind::f16"
#endif
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
#if TC_CTA_GROUP == 2
        "tcgen05.mma.cta_group::2." TC_MMA_KIND " [%0], %1, %2, %3, p;\n\t}"
#else
        "tcgen05.mma.cta_group::1." TC_MMA_KIND " [%0], %1, %2, %3, p;\n\t}"
#endif
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.  In a CTA pair the same
// barrier exists in both CTAs: the leader commits to its own copy and to the peer's (rank 1) copy.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
#if TC_CTA_GROUP == 2
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(tc_map_to_cta(bar, 1u)) : "memory");
#else
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
#endif
}
__device__ __forceinline__ void tc_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------------------ bounded waiting
struct TcWait {
    volatile uint32_t *abort_flag;  // shared memory, CTA-wide
    uint32_t *status;               // global memory, SGEMM_STATUS_WORDS words
    uint64_t timeout_ns;            // how long one wait may go without the barrier completing
};

__device__ __forceinline__ bool tc_wait_slow(const TcWait &w, uint32_t bar, uint32_t parity, uint32_t tag,
                                          uint32_t tile, uint32_t kb) {
    const uint64_t t0 = tc_globaltimer();
    uint32_t spins = 0;
    for (;;) {
        if (tc_mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0u) {
            if (*w.abort_flag) return false;
            if (tc_globaltimer() - t0 > w.timeout_ns) {
                *w.abort_flag = 1u;
                if (atomicCAS(w.status, SGEMM_STATUS_OK, SGEMM_STATUS_TIMEOUT) == SGEMM_STATUS_OK) {
                    w.status[1] = tag;
                    w.status[2] = tile;
                    w.status[3] = kb;
                    w.status[4] = blockIdx.x;
                    w.status[5] = parity;
                }
                __threadfence();
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool tc_wait(const TcWait &w, uint32_t bar, uint32_t parity, uint32_t tag,
                                        uint32_t tile, uint32_t kb) {
    if (tc_mbar_try_wait(bar, parity)) return true;
    return tc_wait_slow(w, bar, parity, tag, tile, kb);
}

// ------------------------------------------------------------------------- chunked accumulation
// A launch unit's k-blocks are cut into accumulation chunks of `chunk` k-blocks, except that the first two chunks of
// a tile are twice as long: while the epilogue warps write the previous tile out (and read C) they drain nothing,
// and the issuer can run ahead by the two accumulator buffers only — two long chunks cover that time.
__device__ __forceinline__ uint32_t tc_chunk_span(uint32_t blocks_done, uint32_t chunk) {
    return blocks_done < 4u * chunk ? 2u * chunk : chunk;
}
__device__ __forceinline__ uint32_t tc_chunk_count(uint32_t blocks, uint32_t chunk) {
    return blocks <= 4u * chunk ? (blocks + 2u * chunk - 1u) / (2u * chunk) : 2u + (blocks - 4u * chunk + chunk - 1u) / chunk;
}

// ---------------------------------------------------------------------------------- descriptors
// 64-bit shared-memory matrix descriptor: start address [0,14) and the two byte offsets [16,30),
// [32,46) in 16-byte units, descriptor version 1 at [46,48), swizzle mode at [61,64)
// (2 = 128-byte swizzle of 16-byte units, 1 = 128-byte swizzle of 32-byte units).
#define TC_LAYOUT_SW128 2ull
#define TC_LAYOUT_SW64 4ull
#define TC_LAYOUT_SW128_32B 1ull
#define TC_LAYOUT_KMAJOR (TC_KROW_BYTES == 128 ? TC_LAYOUT_SW128 : TC_LAYOUT_SW64)
#define TC_LAYOUT_MNMAJOR (TC_ELEM_BYTES == 4 ? TC_LAYOUT_SW128_32B : TC_LAYOUT_SW128)   // 32-bit MN-major needs 32-byte swizzle units
#define TC_KMAJOR_SBO (8 * TC_KROW_BYTES)      // 8 rows of a K-major tile
#define TC_KMAJOR_OFF(kk, sub_bytes) (((kk) / (TC_KSPAN / TC_MMA_K)) * (sub_bytes) + ((kk) % (TC_KSPAN / TC_MMA_K)) * 32)
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                 uint64_t layout) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
           ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) | (layout << 61);
}
// 32-bit instruction descriptor of kind::tf32: FP32 accumulate [4,6)=1, A/B format TF32 [7,10) and
// [10,13) = 2, A/B major [15]/[16] (1 = MN-major), N>>3 at [17,23), M>>4 at [24,29).
#define TC_IDESC ((1u << 4) | (TC_AB_FORMAT << 7) | (TC_AB_FORMAT << 10) | ((TC_A_KMAJOR ? 0u : 1u) << 15) | ((TC_B_MNMAJOR ? 1u : 0u) << 16) | \
                  ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_UMMA_M >> 4) << 24))

// --------------------------------------------------------------------------------------- kernel
#if TC_CTA_GROUP == 2
#define TC_CLUSTER_ATTR __cluster_dims__(2, 1, 1)
#else
#define TC_CLUSTER_ATTR
#endif
extern "C" __global__ void TC_CLUSTER_ATTR __launch_bounds__(TC_THREADS, 1)
generated_gemm(const float *a, const float *b, const float *c, float *d,
               uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
               float alpha, float beta, int32_t num_wg_x, int32_t num_wg_y,
               float *ws, uint32_t *status, uint32_t split_k,
               uint32_t *wave_sync, uint32_t wave_sync_base, uint32_t acc_chunk,
               const __grid_constant__ TcTensorMap map_a_hi, const __grid_constant__ TcTensorMap map_a_lo,
               const __grid_constant__ TcTensorMap map_b_hi, const __grid_constant__ TcTensorMap map_b_lo) {
    (void)a; (void)b; (void)lda; (void)ldb;
    extern __shared__ uint8_t tc_smem_raw[];
    const uint32_t smem_base = (tc_smem_u32(tc_smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + TC_STAGES * TC_STAGE_BYTES;
    // barrier block: full[S] | empty[S] | ready[S] | tmem_full[2] | tmem_empty[2] | tmem base (u32) | abort (u32)
    const uint32_t bar_full = bar_base;
    const uint32_t bar_empty = bar_base + 8 * TC_STAGES;
    const uint32_t bar_ready = bar_base + 16 * TC_STAGES;   // in-kernel split only
    const uint32_t bar_tfull = bar_base + 24 * TC_STAGES;
    const uint32_t bar_tempty = bar_tfull + 16;
    uint8_t *generic_base = tc_smem_raw + (smem_base - tc_smem_u32(tc_smem_raw));
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(generic_base + TC_STAGES * TC_STAGE_BYTES + 24 * TC_STAGES + 32);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    static_assert(24 * TC_STAGES + 32 + 8 <= 256, "barrier block size");

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TcWait waiter{abort_flag, status, TC_TIMEOUT_NS};
#if TC_CTA_GROUP == 2
    uint32_t cta_rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
#else
    const uint32_t cta_rank = 0;
#endif
    const uint32_t unit0 = blockIdx.x / TC_CTA_GROUP, unit_stride = gridDim.x / TC_CTA_GROUP;

    const uint32_t tiles_mn = (uint32_t)num_wg_x * (uint32_t)num_wg_y;
    const uint32_t num_tiles = tiles_mn * split_k;
    const uint32_t kb_total = (k + TC_BK - 1) / TC_BK;
    const uint32_t kb_per = (kb_total + split_k - 1) / split_k;
    // k-blocks per tensor-core accumulation chain (0: the whole K range in one chain); kernels generated without the
    // register path (TC_ACC_CHUNK == 0) ignore the argument
    const uint32_t chunk_blocks = TC_ACC_CHUNK ? acc_chunk : 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            tc_mbar_init(bar_full + 8 * s, 1);
            tc_mbar_init(bar_empty + 8 * s, 1);
            tc_mbar_init(bar_ready + 8 * s, (TC_XFORM_WARPS ? TC_XFORM_WARPS : 1) * TC_CTA_GROUP);
        }
        for (int i = 0; i < 2; ++i) {
            tc_mbar_init(bar_tfull + 8 * i, 1);
            tc_mbar_init(bar_tempty + 8 * i, TC_EPI_WARPS * TC_CTA_GROUP);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_prefetch_map(&map_a_hi);
        tc_prefetch_map(&map_a_lo);
        tc_prefetch_map(&map_b_hi);
        tc_prefetch_map(&map_b_lo);
    }
    if (warp == 1) {
#if TC_CTA_GROUP == 2
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem_u32(tmem_slot)), "r"((uint32_t)TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
#else
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem_u32(tmem_slot)), "r"((uint32_t)TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
#endif
    }
    tc_fence_before();
#if TC_CTA_GROUP == 2
    tc_cluster_sync();   // the peer's barriers must be initialised before anything is signalled to them
#else
    __syncthreads();
#endif
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up (barriers, TMEM, tensor-map prefetch) is done: let the next kernel of the stream get scheduled, and do not
    // touch global memory before the previous one (the split pre-pass, or an earlier call's kernels) has completed
    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();

    // Stopwatch: one thread of a warp that has no other work (warp 2 of block 0) reads the SM's cycle counter and the
    // global nanosecond timer here and again at the end, and adds both differences to status[8..11] (two 64-bit sums
    // the host reads and clears).  cycles / ns is the SM clock this launch really ran at — the number a clock sampled
    // from outside only approximates for launches of a few milliseconds.
    const bool stopwatch = blockIdx.x == 0 && threadIdx.x == 64;
    uint64_t watch_clk = 0, watch_ns = 0;
    if (stopwatch) {
        watch_clk = (uint64_t)clock64();
        watch_ns = tc_globaltimer();
    }

    // Register hand-over between warp groups (each scheduler partition holds one warp of every group): the groups
    // without a running sum shrink to TC_REGS_SMALL registers per thread, the epilogue groups grow to TC_REGS_EPI.
    // The counts add up to no more than a partition owns (checked above), so a growing group never waits for more
    // registers than the shrinking ones release.  Each group executes its instruction at the top of its own branch.
#if TC_REG_HANDOVER
#define TC_SHRINK_REGS() asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TC_REGS_SMALL))
#define TC_GROW_REGS() asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TC_REGS_EPI))
#else
#define TC_SHRINK_REGS()
#define TC_GROW_REGS()
#endif

    if (warp < TC_FIRST_EPI_WARP) {
    TC_SHRINK_REGS();
    if (warp == 0) {
        // ------------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            // in a CTA pair every load reports to the leader's "full" barrier
            const uint32_t full_base = TC_CTA_GROUP == 2 ? tc_map_to_cta(bar_full, 0u) : bar_full;
            uint32_t round = 0;
            for (uint32_t tile = unit0; alive && tile < num_tiles; tile += unit_stride, ++round) {
                // Soft wave alignment: launch units that run side by side share operand panels through L2 only
                // while they stream K at about the same place, and units that fall behind fall further behind.
                // At every tile boundary the leader counts itself in and waits — for TC_WAVE_SYNC_NS at most, then
                // it simply goes on — until all units of this round have begun it.  Never an error, never a deadlock:
                // a unit that is not resident only costs the others the bounded wait.
                if (wave_sync != nullptr && cta_rank == 0) {
                    atomicAdd(wave_sync, 1u);
                    if (round > 0) {
                        const uint32_t target = wave_sync_base + min(num_tiles, (round + 1u) * unit_stride);
                        const uint64_t t0 = tc_globaltimer();
                        while ((int32_t)(*reinterpret_cast<volatile uint32_t *>(wave_sync) - target) < 0 &&
                               tc_globaltimer() - t0 < TC_WAVE_SYNC_NS) {
                        }
                    }
                }
                const uint32_t z = tile / tiles_mn;
                uint32_t tx, ty;
                sgemm_tile_raster(tile - z * tiles_mn, (uint32_t)num_wg_x, (uint32_t)num_wg_y, OPT_WGM, tx, ty);
                const int32_t m0 = (int32_t)(tx * TC_UMMA_M + cta_rank * TC_BM);
                const int32_t n0 = (int32_t)(ty * TC_BN + cta_rank * TC_BN_CTA);
                const uint32_t kb_begin = min(kb_total, z * kb_per), kb_end = min(kb_total, kb_begin + kb_per);
                for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
                    if (!tc_wait(waiter, bar_empty + 8 * stage, phase ^ 1u, 0x100u + stage, tile, kb)) { alive = false; break; }
                    const uint32_t full = full_base + 8 * stage;
                    const uint32_t sa_hi = smem_base + stage * TC_STAGE_BYTES;
                    const uint32_t sa_lo = sa_hi + TC_A_BYTES;                       // (3xTF32 only)
                    const uint32_t sb_hi = sa_hi + TC_OPERAND_TILES * TC_A_BYTES;
                    const uint32_t sb_lo = sb_hi + TC_B_BYTES;                       // (3xTF32 only)
                    const int32_t k0 = (int32_t)(kb * TC_BK);
#if TC_SPLIT_INKERNEL
                    // raw tiles only (hybrid: and A's lo tile), reported to this CTA's own "full" barrier; the transform warps
                    // make the lo tiles (hybrid: B's)
                    (void)sa_lo; (void)sb_lo; (void)full;
                    const uint32_t own_full = bar_full + 8 * stage;
                    tc_mbar_expect_tx(own_full, (TC_SPLIT_HYBRID ? 2 : 1) * TC_A_BYTES + TC_B_BYTES);
#if TC_A_KMAJOR
#pragma unroll
                    for (int sub = 0; sub < TC_KSUBS; ++sub) {
                        tc_tma_load_2d_local(sa_hi + sub * TC_A_SUB_BYTES, &map_a_hi, own_full, k0 + TC_KSPAN * sub, m0);
                        if (TC_SPLIT_HYBRID) tc_tma_load_2d_local(sa_lo + sub * TC_A_SUB_BYTES, &map_a_lo, own_full, k0 + TC_KSPAN * sub, m0);
                    }
#else
#pragma unroll
                    for (int ch = 0; ch < TC_BM / TC_MN_CHUNK; ++ch) {
                        tc_tma_load_2d_local(sa_hi + ch * TC_A_CHUNK_BYTES, &map_a_hi, own_full, m0 + TC_MN_CHUNK * ch, k0);
                        if (TC_SPLIT_HYBRID) tc_tma_load_2d_local(sa_lo + ch * TC_A_CHUNK_BYTES, &map_a_lo, own_full, m0 + TC_MN_CHUNK * ch, k0);
                    }
#endif
#if TC_B_MNMAJOR
#pragma unroll
                    for (int ch = 0; ch < TC_BN_CTA / TC_MN_CHUNK; ++ch)
                        tc_tma_load_2d_local(sb_hi + ch * TC_A_CHUNK_BYTES, &map_b_hi, own_full, n0 + TC_MN_CHUNK * ch, k0);
#else
#pragma unroll
                    for (int sub = 0; sub < TC_KSUBS; ++sub)
                        tc_tma_load_2d_local(sb_hi + sub * TC_B_SUB_BYTES, &map_b_hi, own_full, k0 + TC_KSPAN * sub, n0);
#endif
#else
                    if (cta_rank == 0) tc_mbar_expect_tx(bar_full + 8 * stage, TC_CTA_GROUP * TC_STAGE_BYTES);
#if TC_A_KMAJOR
#pragma unroll
                    for (int sub = 0; sub < TC_KSUBS; ++sub) {
                        tc_tma_load_2d(sa_hi + sub * TC_A_SUB_BYTES, &map_a_hi, full, k0 + TC_KSPAN * sub, m0);
                        if (TC_TERMS == 3) tc_tma_load_2d(sa_lo + sub * TC_A_SUB_BYTES, &map_a_lo, full, k0 + TC_KSPAN * sub, m0);
                    }
#else
#pragma unroll
                    for (int ch = 0; ch < TC_BM / TC_MN_CHUNK; ++ch) {
                        tc_tma_load_2d(sa_hi + ch * TC_A_CHUNK_BYTES, &map_a_hi, full, m0 + TC_MN_CHUNK * ch, k0);
                        if (TC_TERMS == 3) tc_tma_load_2d(sa_lo + ch * TC_A_CHUNK_BYTES, &map_a_lo, full, m0 + TC_MN_CHUNK * ch, k0);
                    }
#endif
#if TC_B_MNMAJOR
#pragma unroll
                    for (int ch = 0; ch < TC_BN_CTA / TC_MN_CHUNK; ++ch) {
                        tc_tma_load_2d(sb_hi + ch * TC_A_CHUNK_BYTES, &map_b_hi, full, n0 + TC_MN_CHUNK * ch, k0);
                        if (TC_TERMS == 3) tc_tma_load_2d(sb_lo + ch * TC_A_CHUNK_BYTES, &map_b_lo, full, n0 + TC_MN_CHUNK * ch, k0);
                    }
#else
#pragma unroll
                    for (int sub = 0; sub < TC_KSUBS; ++sub) {
                        tc_tma_load_2d(sb_hi + sub * TC_B_SUB_BYTES, &map_b_hi, full, k0 + TC_KSPAN * sub, n0);
                        if (TC_TERMS == 3) tc_tma_load_2d(sb_lo + sub * TC_B_SUB_BYTES, &map_b_lo, full, k0 + TC_KSPAN * sub, n0);
                    }
#endif
#endif  // TC_SPLIT_INKERNEL
                    if (++stage == TC_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------------- MMA issuer
        if (lane == 0 && cta_rank == 0) {
            uint32_t stage = 0, phase = 0, handover = 0;   // handover: accumulator buffers given to the epilogue so far
            bool alive = true;
            for (uint32_t tile = unit0; alive && tile < num_tiles; tile += unit_stride) {
                const uint32_t z = tile / tiles_mn;
                const uint32_t kb_begin = min(kb_total, z * kb_per), kb_end = min(kb_total, kb_begin + kb_per);
                if (kb_begin == kb_end) {  // empty K range: nothing to wait for, hand a buffer over
                    const uint32_t buf = handover & 1u, acc_phase = (handover >> 1) & 1u;
                    if (!tc_wait(waiter, bar_tempty + 8 * buf, acc_phase ^ 1u, 0x200u + buf, tile, 0)) { alive = false; break; }
                    tc_mbar_arrive(bar_tfull + 8 * buf);
                    if (TC_CTA_GROUP == 2) tc_mbar_arrive_cluster(tc_map_to_cta(bar_tfull + 8 * buf, 1u));
                    ++handover;
                    continue;
                }
                // With chunk_blocks != 0 the K range is accumulated in chunks: each chunk starts a fresh accumulator in the
                // other TMEM buffer and is handed to the epilogue warps, which add the chunks up in FP32 registers.
                for (uint32_t kb = kb_begin; alive && kb < kb_end;) {
                    const uint32_t buf = handover & 1u, acc_phase = (handover >> 1) & 1u;
                    if (!tc_wait(waiter, bar_tempty + 8 * buf, acc_phase ^ 1u, 0x200u + buf, tile, kb)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * TC_BN;
                    const uint32_t chunk_begin = kb;
                    const uint32_t chunk_end = chunk_blocks ? min(kb_end, kb + tc_chunk_span(kb - kb_begin, chunk_blocks)) : kb_end;
                    for (; kb < chunk_end; ++kb) {
                        // operands of this stage are complete: TMA bytes landed (and, with the in-kernel split, lo tiles written)
                        if (!tc_wait(waiter, (TC_SPLIT_INKERNEL ? bar_ready : bar_full) + 8 * stage, phase, 0x300u + stage, tile, kb)) { alive = false; break; }
                        tc_fence_after();
                        const uint32_t sa_hi = smem_base + stage * TC_STAGE_BYTES;
                        const uint32_t sa_lo = sa_hi + TC_A_BYTES;                       // (3xTF32 only)
                        const uint32_t sb_hi = sa_hi + TC_OPERAND_TILES * TC_A_BYTES;
                        const uint32_t sb_lo = sb_hi + TC_B_BYTES;                       // (3xTF32 only)
#pragma unroll
                        for (int kk = 0; kk < TC_BK / TC_MMA_K; ++kk) {
#if TC_A_KMAJOR
                            const uint32_t a_off = TC_KMAJOR_OFF(kk, TC_A_SUB_BYTES);
                            const uint64_t da_hi = tc_smem_desc(sa_hi + a_off, 16, TC_KMAJOR_SBO, TC_LAYOUT_KMAJOR);
                            const uint64_t da_lo = tc_smem_desc(sa_lo + a_off, 16, TC_KMAJOR_SBO, TC_LAYOUT_KMAJOR);
#else
                            const uint32_t a_off = kk * TC_MN_STEP;
                            const uint64_t da_hi = tc_smem_desc(sa_hi + a_off, TC_A_CHUNK_BYTES, TC_MN_SBO, TC_LAYOUT_MNMAJOR);
                            const uint64_t da_lo = tc_smem_desc(sa_lo + a_off, TC_A_CHUNK_BYTES, TC_MN_SBO, TC_LAYOUT_MNMAJOR);
#endif
#if TC_B_MNMAJOR
                            const uint32_t b_off = kk * TC_MN_STEP;
                            const uint64_t db_hi = tc_smem_desc(sb_hi + b_off, TC_A_CHUNK_BYTES, TC_MN_SBO, TC_LAYOUT_MNMAJOR);
                            const uint64_t db_lo = tc_smem_desc(sb_lo + b_off, TC_A_CHUNK_BYTES, TC_MN_SBO, TC_LAYOUT_MNMAJOR);
#else
                            const uint32_t b_off = TC_KMAJOR_OFF(kk, TC_B_SUB_BYTES);
                            const uint64_t db_hi = tc_smem_desc(sb_hi + b_off, 16, TC_KMAJOR_SBO, TC_LAYOUT_KMAJOR);
                            const uint64_t db_lo = tc_smem_desc(sb_lo + b_off, 16, TC_KMAJOR_SBO, TC_LAYOUT_KMAJOR);
#endif
                            const uint32_t first = (kb == chunk_begin && kk == 0) ? 0u : 1u;
#if TC_TERMS == 3
                            tc_mma_tf32(d_tmem, da_lo, db_hi, TC_IDESC, first);
                            tc_mma_tf32(d_tmem, da_hi, db_lo, TC_IDESC, 1u);
                            tc_mma_tf32(d_tmem, da_hi, db_hi, TC_IDESC, 1u);
#else
                            (void)da_lo; (void)db_lo;
                            tc_mma_tf32(d_tmem, da_hi, db_hi, TC_IDESC, first);
#endif
                        }
                        tc_commit(bar_empty + 8 * stage);
                        if (++stage == TC_STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (alive) tc_commit(bar_tfull + 8 * buf);
                    ++handover;
                }
            }
        }
    }
    } else if (warp >= TC_FIRST_EPI_WARP + TC_EPI_WARPS) {
        // ------------------------------------------------------------------- transform (in-kernel split)
        TC_SHRINK_REGS();
#if TC_SPLIT_INKERNEL
        const uint32_t t = threadIdx.x - 32 * (TC_FIRST_EPI_WARP + TC_EPI_WARPS);   // 0 .. 32*TC_XFORM_WARPS-1
        const uint32_t ready_base = TC_CTA_GROUP == 2 ? tc_map_to_cta(bar_ready, 0u) : bar_ready;
        uint32_t stage = 0, phase = 0;
        bool alive = true;
        for (uint32_t tile = unit0; alive && tile < num_tiles; tile += unit_stride) {
            const uint32_t z = tile / tiles_mn;
            const uint32_t kb_begin = min(kb_total, z * kb_per), kb_end = min(kb_total, kb_begin + kb_per);
            for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
                alive = __all_sync(0xffffffffu, tc_wait(waiter, bar_full + 8 * stage, phase, 0x500u + stage, tile, kb));
                if (!alive) break;
                // [A_hi | A_lo | B_hi | B_lo]: lo = hi - trunc_tf32(hi), same offset in the neighbouring tile
                const float4 *a_src = reinterpret_cast<const float4 *>(generic_base + stage * TC_STAGE_BYTES);
                float4 *a_dst = reinterpret_cast<float4 *>(generic_base + stage * TC_STAGE_BYTES + TC_A_BYTES);
                const float4 *b_src = reinterpret_cast<const float4 *>(generic_base + stage * TC_STAGE_BYTES + 2 * TC_A_BYTES);
                float4 *b_dst = reinterpret_cast<float4 *>(generic_base + stage * TC_STAGE_BYTES + 2 * TC_A_BYTES + TC_B_BYTES);
#if !TC_SPLIT_HYBRID
#pragma unroll 4
                for (uint32_t i = t; i < TC_A_BYTES / 16; i += 32 * TC_XFORM_WARPS) {
                    float4 v = a_src[i];
                    v.x = sgemm_tf32_lo(v.x); v.y = sgemm_tf32_lo(v.y); v.z = sgemm_tf32_lo(v.z); v.w = sgemm_tf32_lo(v.w);
                    a_dst[i] = v;
                }
#else
                (void)a_src; (void)a_dst;   // A's lo tile came from the pre-pass by TMA
#endif
#pragma unroll 4
                for (uint32_t i = t; i < TC_B_BYTES / 16; i += 32 * TC_XFORM_WARPS) {
                    float4 v = b_src[i];
                    v.x = sgemm_tf32_lo(v.x); v.y = sgemm_tf32_lo(v.y); v.z = sgemm_tf32_lo(v.z); v.w = sgemm_tf32_lo(v.w);
                    b_dst[i] = v;
                }
                // generic-proxy writes -> visible to the tensor core (async proxy), then hand the stage to the issuer
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if (TC_CTA_GROUP == 2) tc_mbar_arrive_cluster(ready_base + 8 * stage);
                    else tc_mbar_arrive(bar_ready + 8 * stage);
                }
                if (++stage == TC_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
#endif
    } else {
        // ---------------------------------------------------------------------------- epilogue
        TC_GROW_REGS();
        const uint32_t quarter = warp & 3u;  // TMEM lane quarter this warp may read
        const uint32_t cbase = ((warp - TC_FIRST_EPI_WARP) >> 2) * TC_EPI_COLS;  // first accumulator column of this warp's share
        uint32_t handover = 0;               // accumulator buffers taken from the MMA issuer so far
        bool alive = true;
        // the accumulator buffer is handed back to the leader's MMA thread
        const uint32_t tempty_base = TC_CTA_GROUP == 2 ? tc_map_to_cta(bar_tempty, 0u) : bar_tempty;
        for (uint32_t tile = unit0; alive && tile < num_tiles; tile += unit_stride) {
            const uint32_t z = tile / tiles_mn;
            uint32_t tx, ty;
            sgemm_tile_raster(tile - z * tiles_mn, (uint32_t)num_wg_x, (uint32_t)num_wg_y, OPT_WGM, tx, ty);
            const uint32_t kb_begin = min(kb_total, z * kb_per), kb_end = min(kb_total, kb_begin + kb_per);
            const bool empty_k = kb_begin == kb_end;
            const uint32_t row = tx * TC_UMMA_M + cta_rank * TC_BM + quarter * 32 + lane;
            const uint32_t col0 = ty * TC_BN;
            const bool partial = split_k > 1;
            float *out = partial ? ws + (uint64_t)z * m * n : d;
            const uint32_t ldo = partial ? m : ldd;
            const bool use_c = !partial && beta != 0.0f;
#if TC_ACC_CHUNK
            const uint32_t chunks = (empty_k || !chunk_blocks) ? 1u : tc_chunk_count(kb_end - kb_begin, chunk_blocks);
            {
                // ---- the tile's accumulation chunks are added up in a running sum held in registers, then the sum
                // is scaled, combined with C and stored.  (Why chunks: the tensor core adds into its accumulator with
                // truncation — toward zero, two guard bits — so a long chain of MMAs drifts toward zero in proportion
                // to its length.  The chain is cut every acc_chunk k-blocks; the partial sums are added here in FP32
                // with round-to-nearest, in chunk order, so results do not depend on timing.)  Every TMEM buffer goes
                // back to the issuer as soon as it is added, so the issuer runs two chunks ahead while this tile is
                // written out.
                if (use_c) {
                    // ask L2 for this warp's part of the C tile now: lane L covers columns L, L + 32, ... of the warp's
                    // share (first and last row: a warp's 128 bytes of a column may straddle two lines)
                    const uint32_t row_first = row - lane;
                    if (row_first < m) {
                        const uint32_t row_last = min(row_first + 31u, m - 1u);
#pragma unroll
                        for (int j = 0; j < TC_EPI_COLS / 32; ++j) {
                            const uint32_t col = col0 + cbase + j * 32 + lane;
                            if (col < n) {
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(c + row_first + (uint64_t)col * ldc));
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(c + row_last + (uint64_t)col * ldc));
                            }
                        }
                    }
                }
                // C is fetched TC_CW columns at a time, two pieces ahead of its use (three register buffers); the
                // first two pieces are requested before the main loop of the tile has even finished.  (C may be the
                // same buffer as D: every element is read before this same thread overwrites it.)
                float cv[3][TC_CW];
                auto fetch_cw = [&](int piece, float (&dst)[TC_CW]) {
                    if (use_c && row < m) {
#pragma unroll
                        for (int j = 0; j < TC_CW; ++j) {
                            const uint32_t col = col0 + cbase + piece * TC_CW + j;
                            dst[j] = col < n ? c[row + (uint64_t)col * ldc] : 0.0f;
                        }
                    }
                };
                fetch_cw(0, cv[0]);
                if (TC_EPI_COLS / TC_CW > 1) fetch_cw(1, cv[1]);
                // the running sum: two columns per 64-bit register pair, added with the packed FP32 add (one
                // instruction per two columns; each half is an ordinary round-to-nearest FP32 add)
                uint64_t sum2[TC_EPI_COLS / 2];
                for (uint32_t ch = 0; ch < chunks; ++ch, ++handover) {
                    const uint32_t buf = handover & 1u, acc_phase = (handover >> 1) & 1u;
                    alive = __all_sync(0xffffffffu, tc_wait(waiter, bar_tfull + 8 * buf, acc_phase, 0x400u + buf, tile, ch));
                    if (!alive) break;
                    tc_fence_after();
#pragma unroll
                    for (int cc = 0; cc < TC_EPI_COLS / 16; ++cc) {
                        uint32_t r[16];
                        tc_tmem_ld16(tmem_base + ((quarter * 32u) << 16) + buf * TC_BN + cbase + cc * 16, r);
                        tc_tmem_ld_wait();
                        if (ch == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                asm("mov.b64 %0, {%1, %2};" : "=l"(sum2[cc * 8 + j])
                                    : "r"(empty_k ? 0u : r[2 * j]), "r"(empty_k ? 0u : r[2 * j + 1]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                asm("{\n\t.reg .b64 t;\n\tmov.b64 t, {%1, %2};\n\tadd.rn.f32x2 %0, %0, t;\n\t}"
                                    : "+l"(sum2[cc * 8 + j]) : "r"(r[2 * j]), "r"(r[2 * j + 1]));
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (TC_CTA_GROUP == 2) tc_mbar_arrive_cluster(tempty_base + 8 * buf);
                        else tc_mbar_arrive(bar_tempty + 8 * buf);
                    }
                }
                if (!alive) break;
#pragma unroll
                for (int piece = 0; piece < TC_EPI_COLS / TC_CW; ++piece) {
                    if (piece + 2 < TC_EPI_COLS / TC_CW) fetch_cw(piece + 2, cv[(piece + 2) % 3]);
                    if (row < m) {
#pragma unroll
                        for (int j = 0; j < TC_CW; ++j) {
                            const uint32_t col = col0 + cbase + piece * TC_CW + j;
                            if (col < n) {
                                float lo, hi;
                                asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(sum2[(piece * TC_CW + j) / 2]));
                                float v = (j & 1) ? hi : lo;
                                if (!partial) {
                                    v *= alpha;
                                    if (use_c) v = fmaf(beta, cv[piece % 3][j], v);
                                }
                                out[row + (uint64_t)col * ldo] = v;
                            }
                        }
                    }
                }
            }
#else
            // one accumulator per tile: drained straight from TMEM
            const uint32_t buf = handover & 1u, acc_phase = (handover >> 1) & 1u;
            ++handover;
            // C is fetched one 32-column chunk ahead of its use, all 32 loads of a chunk in flight together; the
            // first chunk is requested before the accumulator is even complete, so its latency hides behind the
            // tile's main loop.  (C may be the same buffer as D: every element is read before this same thread
            // overwrites it, and no other thread touches it.)
            float cv[2][32];
            auto fetch_c = [&](int cc, float (&dst)[32]) {
                if (use_c && row < m) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t col = col0 + cbase + cc * 32 + j;
                        dst[j] = col < n ? c[row + (uint64_t)col * ldc] : 0.0f;
                    }
                }
            };
            fetch_c(0, cv[0]);
            alive = __all_sync(0xffffffffu, tc_wait(waiter, bar_tfull + 8 * buf, acc_phase, 0x400u + buf, tile, 0));
            if (!alive) break;
            tc_fence_after();
#pragma unroll
            for (int cc = 0; cc < TC_EPI_COLS / 32; ++cc) {
                uint32_t r[32];
                tc_tmem_ld32(tmem_base + ((quarter * 32u) << 16) + buf * TC_BN + cbase + cc * 32, r);
                if (cc + 1 < TC_EPI_COLS / 32) fetch_c(cc + 1, cv[(cc + 1) & 1]);
                tc_tmem_ld_wait();
                if (row < m) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t col = col0 + cbase + cc * 32 + j;
                        if (col < n) {
                            float v = empty_k ? 0.0f : __uint_as_float(r[j]);
                            if (!partial) {
                                v *= alpha;
                                if (use_c) v = fmaf(beta, cv[cc & 1][j], v);
                            }
                            out[row + (uint64_t)col * ldo] = v;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (TC_CTA_GROUP == 2) tc_mbar_arrive_cluster(tempty_base + 8 * buf);
                else tc_mbar_arrive(bar_tempty + 8 * buf);
            }
#endif  // TC_ACC_CHUNK
        }
    }

    // teardown: every thread gets here on both the normal and the abort path
    tc_fence_before();
#if TC_CTA_GROUP == 2
    tc_cluster_sync();   // neither CTA may release TMEM or exit while the other can still reach into it
#else
    __syncthreads();
#endif
    if (stopwatch) {   // all roles of this (persistent) block are done: the interval is the block's working life
        atomicAdd(reinterpret_cast<unsigned long long *>(status + SGEMM_STATUS_WORDS), (unsigned long long)((uint64_t)clock64() - watch_clk));
        atomicAdd(reinterpret_cast<unsigned long long *>(status + SGEMM_STATUS_WORDS + 2), (unsigned long long)(tc_globaltimer() - watch_ns));
    }
    if (warp == 1) {
        if (*abort_flag) {
            // give copies and MMAs that may still be in flight time to land before TMEM is released
            const uint64_t t0 = tc_globaltimer();
            while (tc_globaltimer() - t0 < 2000000ull) __nanosleep(1000);
        }
        tc_fence_after();
#if TC_CTA_GROUP == 2
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TC_TMEM_COLS) : "memory");
#else
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"((uint32_t)TC_TMEM_COLS) : "memory");
#endif
    }
}

// ==== end of the per-kernel section (the generator instantiates everything above once per tcgen05 kernel) ====

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA initialises an mbarrier that nothing will ever arrive on and
// waits on it with the kernel's own wait routine and a short limit.  The wait must run out, record the
// status words and return, the kernel must end normally and the context must stay usable — this is the
// failure path of generated_gemm exercised without a hung pipeline behind it.
// ---------------------------------------------------------------------------------------------
extern "C" __global__ void sgemm_wait_selftest(uint32_t *status, uint64_t timeout_ns, uint32_t tag) {
    __shared__ __align__(8) uint64_t barrier_storage;
    __shared__ uint32_t abort_flag;
    sgemm_grid_dependency_wait();
    if (threadIdx.x == 0) {
        tc_mbar_init(tc_smem_u32(&barrier_storage), 1);
        abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const TcWait waiter{&abort_flag, status, timeout_ns};
    // every thread waits; the first whose limit runs out reports, the others leave through the abort flag
    const bool completed = tc_wait(waiter, tc_smem_u32(&barrier_storage), 0u, tag, 0u, threadIdx.x);
    if (completed && threadIdx.x == 0) status[6] = 0xBAD0BAD0u;   // cannot happen: nobody arrives
    __syncthreads();
}
