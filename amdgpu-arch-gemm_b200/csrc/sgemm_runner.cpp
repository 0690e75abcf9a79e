// libsgemm_runner.so — CUDA-driver runner behind the C ABI of include/sgemm_runner.h.
//
// Replaces the host side of the reference's runner (runner/generator_runner.cpp:69-190: module load,
// TOML -> config, kernel-argument packing, launch) for sm_100a cubins produced by generator.compile().
// The CUDA driver is bound at run time with dlopen("libcuda.so.1"), so the library itself loads (and its
// host-only entry points work) on a machine without a GPU; every device entry point then fails loudly.
#include "sgemm_runner.h"
#include "sgemm_internal.hpp"
#include "sgemm_toml.hpp"

#include <cuda.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#define SGEMM_API extern "C" __attribute__((visibility("default")))

namespace {

// ------------------------------------------------------------------------------------ driver binding
#define SGEMM_STR2(x) #x
#define SGEMM_STR(x) SGEMM_STR2(x)
#define DRIVER_FUNCTIONS(X)                                                                              \
    X(cuInit) X(cuDeviceGet) X(cuDeviceGetCount) X(cuDeviceGetAttribute) X(cuDevicePrimaryCtxRetain)     \
    X(cuDevicePrimaryCtxRelease) X(cuCtxPushCurrent) X(cuCtxPopCurrent) X(cuModuleLoad) X(cuModuleUnload) \
    X(cuModuleGetFunction) X(cuFuncSetAttribute) X(cuFuncGetAttribute) X(cuLaunchKernel) X(cuLaunchKernelEx) X(cuTensorMapEncodeTiled) \
    X(cuMemAlloc) X(cuMemFree) X(cuMemcpyHtoDAsync) X(cuMemcpyDtoHAsync) X(cuMemcpyHtoD) X(cuMemcpyDtoH) \
    X(cuMemsetD8) X(cuStreamSynchronize) X(cuCtxSynchronize) X(cuEventCreate)        \
    X(cuEventRecord) X(cuEventSynchronize) X(cuEventElapsedTime) X(cuEventDestroy) X(cuGetErrorString)   \
    X(cuStreamCreate) X(cuStreamDestroy) X(cuStreamWaitEvent)                                            \
    X(cuGetErrorName)

struct Driver {
#define DECL(name) decltype(&name) name##_ = nullptr;
    DRIVER_FUNCTIONS(DECL)
#undef DECL
    bool ok = false;
    std::string error;
};

Driver &driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        void *lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) {
            const char *why = dlerror();  // one call: dlerror clears its message when read
            d.error = std::string("cannot load the CUDA driver: ") + (why ? why : "libcuda.so.1 not found");
            return;
        }
        // cuda.h renames some entry points with macros (cuMemAlloc -> cuMemAlloc_v2): SGEMM_STR expands them.
#define LOAD(name)                                                                   \
        d.name##_ = reinterpret_cast<decltype(&name)>(dlsym(lib, SGEMM_STR(name)));  \
        if (!d.name##_) { d.error = std::string("CUDA driver lacks ") + SGEMM_STR(name); return; }
        DRIVER_FUNCTIONS(LOAD)
#undef LOAD
        CUresult r = d.cuInit_(0);
        if (r != CUDA_SUCCESS) {
            d.error = "cuInit failed with code " + std::to_string((int)r);
            return;
        }
        d.ok = true;
    });
    return d;
}

thread_local std::string g_open_error;

constexpr int kStatusWords = 8;    // what a kernel that gave up reports
constexpr int kStatusAlloc = 16;   // ... followed by the tensor kernels' stopwatch: 64-bit sums of SM cycles and nanoseconds
constexpr uint32_t kCounterWords = 64;
constexpr int kVariantSimt = 0, kVariantTensor = 1;

struct TensorMapKey {
    const void *base = nullptr;
    uint64_t d0 = 0, d1 = 0, stride = 0;
    uint32_t b0 = 0, b1 = 0;
    int swizzle = 0;
    bool operator==(const TensorMapKey &o) const {
        return base == o.base && d0 == o.d0 && d1 == o.d1 && stride == o.stride && b0 == o.b0 && b1 == o.b1 &&
               swizzle == o.swizzle;
    }
};
struct CachedMap {
    TensorMapKey key;
    alignas(64) CUtensorMap map;
    bool valid = false;
};

}  // namespace

// What the host has to know about one tcgen05 kernel of the cubin.
struct TensorKernel {
    CUfunction fn = nullptr;
    uint32_t tile_m = 0, tile_n = 0, bk = 0;   // tile of one launch unit, k per stage
    uint32_t group = 1;                         // CTAs per launch unit (2 = CTA pair)
    uint32_t threads = 0, smem = 0;
    bool split_inkernel = false;                // lo tiles made in the kernel: no pre-pass, no lo copies
    bool split_hybrid = false;                  // ... only B's: A's lo copy still comes from the pre-pass
    bool a_packed = false;                      // A is read from K-major packed copies made by a pre-pass
    uint32_t acc_chain = 0;                     // k per accumulation chain the kernel was generated for (0: no register path)
};

struct sgemm_handle {
    sgemm_config cfg{};
    int device = 0;
    CUdevice cu_device = 0;
    CUcontext ctx = nullptr;
    CUmodule module = nullptr;
    uint32_t elem_bytes = 4;    // size of an element of A and B: 4 (FP32) or 2 (FP16 / BF16, tensor variant only)
    CUfunction fn_pack16 = nullptr, fn_repitch = nullptr, fn_narrow16 = nullptr;
    CUfunction fn_main = nullptr, fn_simt = nullptr, fn_split_lo = nullptr, fn_pack_a = nullptr,
               fn_reduce = nullptr, fn_fill = nullptr, fn_tile_map = nullptr, fn_wait_selftest = nullptr;
    int sm_count = 0;
    uint32_t tile_m = 0, tile_n = 0;
    TensorKernel tk_main, tk_skinny;   // tk_skinny.fn == NULL: the cubin has no companion kernel
    TensorKernel tk_wholek;            // twin of tk_main with whole-K accumulation (fn == NULL: none)
    TensorKernel tk_thin;              // the companion with 32-column tiles, for N of a few columns (fn == NULL: none)
    CUdeviceptr status = 0;
    CUdeviceptr counters = 0;   // device words shared by all launches of the handle: [0] = wave-alignment counter
    // workspace: owned (grow on demand) or lent
    CUdeviceptr ws_owned = 0;
    size_t ws_owned_bytes = 0;
    CUdeviceptr ws_lent = 0;
    size_t ws_lent_bytes = 0;
    // host-path staging
    CUdeviceptr stage[4] = {0, 0, 0, 0};
    size_t stage_bytes[4] = {0, 0, 0, 0};
    // host path, pipelined: upload / compute / download streams and the events that order column chunks across them
    CUstream pipe_streams[3] = {nullptr, nullptr, nullptr};
    std::vector<CUevent> pipe_events;
    bool reuse_a_lo = false;    // set by the pipelined host path: A's lo copy of the previous chunk call is still valid
    // options and facts
    int64_t force_variant = 0, split_k_opt = 0, simt_below_flops = (int64_t)1 << 27;
    int64_t skinny_below_intensity = 200;   // flop per byte of A and B below which the companion kernel is used
    bool repitch = true;        // FP32 tensor path: operands TMA cannot describe are copied to an aligned pitch first
    int64_t repitch_above_flops = (int64_t)1 << 31;   // ... in auto mode for problems of at least this many flops
    int64_t skinny_below_flops = (int64_t)1 << 33;   // ... and problems smaller than this many flops (no pre-pass launch)
    bool wave_sync = true;      // tensor kernel: soft alignment of the persistent CTAs at tile boundaries
    uint32_t wave_sync_base = 0;   // value of the alignment counter before the next launch (it only ever counts up)
    bool pipeline_host = true;  // sgemm_run_host overlaps uploads, GEMM and downloads over column chunks
    int64_t pipeline_chunks = 16;  // ... this many of them (fewer when N is small); 8192^3: 11.5 ms with 8, 11.1 with 16, 12.8 with 32
    bool pdl = true;            // launch with programmatic stream serialisation (see launch())
    int64_t acc_chain_opt = -1;   // -1: as generated, 0: whole K in one chain, else k per chain
    int64_t last_variant = 0, last_split_k = 1, last_grid = 0, launches = 0, last_acc_chain = 0, last_tile_n = 0, last_feed_tma = 0;
    CachedMap maps[4];
    // optional timing of the main GEMM kernel alone (events around it on the caller's stream)
    bool profile = false;
    std::vector<std::pair<CUevent, CUevent>> prof_events;
    size_t prof_used = 0;
    void *noalloc_scratch = nullptr;   // device address of the library's static scratch array in this handle's context
    sgemm_internal::CommState comm;    // communicator over the GPUs of a sharded SGEMM (see sgemm_multi.cpp)
    std::string error;
};

namespace {

int fail(sgemm_handle *h, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h) h->error = buf; else g_open_error = buf;
    return code;
}

std::string cu_text(CUresult r) {
    const char *name = nullptr, *text = nullptr;
    Driver &d = driver();
    if (d.ok) {
        d.cuGetErrorName_(r, &name);
        d.cuGetErrorString_(r, &text);
    }
    return std::string(name ? name : "CUDA_ERROR") + " (" + std::to_string((int)r) + "): " + (text ? text : "?");
}

#define CU_CHECK(h, call)                                                                         \
    do {                                                                                          \
        CUresult _r = (call);                                                                     \
        if (_r != CUDA_SUCCESS) return fail(h, SGEMM_ERR_CUDA, "%s -> %s", #call, cu_text(_r).c_str()); \
    } while (0)

struct CtxGuard {
    bool pushed = false;
    explicit CtxGuard(sgemm_handle *h) {
        if (h && h->ctx && driver().ok) pushed = driver().cuCtxPushCurrent_(h->ctx) == CUDA_SUCCESS;
    }
    ~CtxGuard() {
        if (pushed) {
            CUcontext c;
            driver().cuCtxPopCurrent_(&c);
        }
    }
};

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ------------------------------------------------------------------------------------ launch plan
struct Plan {
    int variant = kVariantSimt;   // which kernel
    uint32_t split_k = 1;
    uint32_t tiles_m = 0, tiles_n = 0;
    uint32_t grid_x = 0;
    size_t lo_a_off = 0, lo_b_off = 0, hi_a_off = 0, hi_b_off = 0, partial_off = 0;  // byte offsets into the workspace
    uint64_t span_a = 0, span_b = 0;                                    // floats walked by the split pre-pass
    uint32_t ldt = 0;                                                   // K-major packed A: leading dimension
    size_t ws_bytes = 0;
    const TensorKernel *tk = nullptr;   // the tcgen05 kernel chosen (tensor variant only)
    // FP32 operands TMA cannot describe where they lie: aligned copies in the workspace, and the pitch they get
    bool repitch_a = false, repitch_b = false;
    size_t rp_a_off = 0, rp_b_off = 0;
    uint32_t lda_eff = 0, ldb_eff = 0;  // leading dimensions the tensor kernel and its pre-pass see
    uint32_t acc_chain = 0;             // k per tensor-core accumulation chain (0: all of K in one chain)
    bool ffma_tma = false;              // FFMA variant: the TMA-fed kernel serves this call (else the register-fed one)
};

// FP32: can TMA read this operand where it lies?  (a packed K-major copy of A gets its own pitch and alignment)
bool operand_tma_ok(const void *base, uint32_t ld) { return (((uintptr_t)base & 15) == 0) && (ld % 4) == 0; }

bool tensor_eligible(const sgemm_handle *h, const void *a, const void *b, uint32_t lda, uint32_t ldb) {
    if (h->cfg.variant != kVariantTensor) return false;
    // TMA: 16-byte aligned bases and row pitches that are multiples of 16 bytes
    const uint32_t per16 = 16 / h->elem_bytes;   // elements per 16 bytes
    if (h->elem_bytes != 4) {
        // 16-bit operands are read by TMA where they lie, in either orientation; only an A that goes through a packed
        // K-major copy (a_major = "k") has a pitch and an alignment of its own
        if (!(h->cfg.a_kmajor && !h->cfg.trans_a) && (((uintptr_t)a & 15) || (lda % per16) != 0)) return false;
        if (((uintptr_t)b & 15) || (ldb % per16) != 0) return false;
        return true;
    }
    if (((uintptr_t)a & 15) || ((uintptr_t)b & 15)) return false;
    if ((ldb % per16) != 0) return false;
    if ((!h->cfg.a_kmajor || h->cfg.trans_a) && (lda % per16) != 0) return false;   // a packed copy gets its own pitch
    return true;
}

// slots: launch units the device runs at a time (SMs / CTAs per unit for the persistent tensor kernels, two blocks
// per SM for the FFMA kernel)
uint32_t pick_split_k(const sgemm_handle *h, uint32_t tiles, uint32_t k, uint32_t bk, uint32_t slots) {
    const uint32_t kb_total = (k + bk - 1) / bk;
    slots = std::max<uint32_t>(1, slots);
    uint32_t split = 1;
    if (h->split_k_opt > 0) {
        split = (uint32_t)h->split_k_opt;
    } else if (tiles * 2 <= slots && kb_total >= 16) {
        // too few tiles to fill the device: cut K so that the launch units still fit one wave (a CTA pair takes two
        // SMs), keeping at least 8 k-blocks per split so the partial-sum traffic stays small next to the operand
        // traffic
        split = std::min<uint32_t>({slots / tiles, kb_total / 8, 32u});
    }
    split = std::max<uint32_t>(1, std::min(split, std::max<uint32_t>(kb_total, 1)));
    // no empty splits: recompute from the per-split block count
    const uint32_t per = (std::max<uint32_t>(kb_total, 1) + split - 1) / split;
    return (std::max<uint32_t>(kb_total, 1) + per - 1) / per;
}

int make_plan(sgemm_handle *h, const void *a, const void *b, uint32_t m, uint32_t n, uint32_t k, uint32_t lda,
              uint32_t ldb, Plan *p) {
    bool eligible = tensor_eligible(h, a, b, lda, ldb);
    p->lda_eff = lda;
    p->ldb_eff = ldb;
    if (!eligible && h->repitch && h->cfg.variant == kVariantTensor && h->elem_bytes == 4 && h->force_variant != 2 &&
        (h->force_variant != 0 || 2.0 * m * n * k >= (double)h->repitch_above_flops)) {
        // the tensor path through aligned copies: one more pass over the offending operand, then everything as usual
        const bool a_needs = !(h->cfg.a_kmajor && !h->cfg.trans_a) && !operand_tma_ok(a, lda);
        p->repitch_a = a_needs;
        p->repitch_b = !operand_tma_ok(b, ldb);
        if (p->repitch_a) p->lda_eff = (uint32_t)round_up(h->cfg.trans_a ? k : m, 4);
        if (p->repitch_b) p->ldb_eff = (uint32_t)round_up(h->cfg.trans_b ? n : k, 4);
        eligible = true;
    }
    lda = p->lda_eff;   // from here on the plan is made for the operands the kernels will see
    ldb = p->ldb_eff;
    int variant;
    const TensorKernel *tk = &h->tk_main;
    if (h->elem_bytes != 4 && (!eligible || h->force_variant == 2 || h->force_variant == 3))
        return fail(h, SGEMM_ERR_UNSUPPORTED, "16-bit operands run on the tensor-core kernel only: %s",
                    eligible ? "no FFMA or companion kernel exists for them"
                             : "operands must be 16-byte aligned with leading dimensions that are multiples of 8");
    if (h->force_variant == 3) {
        if (!eligible || !h->tk_skinny.fn)
            return fail(h, SGEMM_ERR_UNSUPPORTED, "companion tensor kernel forced but %s",
                        h->tk_skinny.fn ? "the operands are not TMA-eligible" : "the cubin has none");
        variant = kVariantTensor;
        tk = (h->tk_thin.fn && n <= h->tk_thin.tile_n) ? &h->tk_thin : &h->tk_skinny;
    } else if (h->force_variant == 1) {
        if (!eligible)
            return fail(h, SGEMM_ERR_UNSUPPORTED,
                        "tensor variant forced but not usable: cubin variant %d, lda %u, ldb %u, bases %p %p "
                        "(needs a tcgen05 cubin, 16-byte aligned A/B and lda, ldb multiples of 4)",
                        h->cfg.variant, lda, ldb, a, b);
        variant = kVariantTensor;
    } else if (h->force_variant == 2) {
        variant = kVariantSimt;
    } else {
        const double flops = 2.0 * m * n * k;
        variant = (eligible && (flops >= (double)h->simt_below_flops || h->elem_bytes != 4)) ? kVariantTensor : kVariantSimt;
        // few flops per byte of A and B (a skinny M or N with a long K): the pre-pass, which reads both operands and
        // writes and re-reads their lo copies, would cost as much as the GEMM; the companion kernel (small tiles,
        // lo terms made in the kernel) has neither pre-pass nor copies
        const double intensity = flops / (4.0 * ((double)m * k + (double)k * n));
        // small problems too: the pre-pass is one more dependent launch in a call that lasts a few of them
        if (variant == kVariantTensor && h->tk_skinny.fn &&
            (intensity < (double)h->skinny_below_intensity || flops < (double)h->skinny_below_flops))
            tk = (h->tk_thin.fn && n <= h->tk_thin.tile_n) ? &h->tk_thin : &h->tk_skinny;   // a few columns: 32-column tiles
    }
    p->variant = variant;
    if (variant == kVariantTensor) {
        // accumulation chain: the kernel's own unless the caller chose one
        uint32_t chain = h->acc_chain_opt < 0 ? tk->acc_chain : (uint32_t)h->acc_chain_opt;
        if (chain && (!tk->acc_chain || chain % tk->bk))
            return fail(h, SGEMM_ERR_UNSUPPORTED, "acc_chain %u: %s", chain,
                        tk->acc_chain ? "not a multiple of the kernel's k-block" : "this kernel was generated without chunked accumulation");
        p->tiles_m = (m + tk->tile_m - 1) / tk->tile_m;
        p->tiles_n = (n + tk->tile_n - 1) / tk->tile_n;
        p->split_k = pick_split_k(h, p->tiles_m * p->tiles_n, k, tk->bk, (uint32_t)h->sm_count / std::max<uint32_t>(tk->group, 1));
        // a launch unit whose k range is one accumulation chunk (no chunking, or up to two chains: the first chunks
        // are double length) does not need the running sum: the main kernel's whole-K twin (same tiles, same split)
        // writes the accumulator out straight from TMEM
        const uint32_t kb_total = (k + tk->bk - 1) / tk->bk;
        const uint32_t k_per_unit = (kb_total + p->split_k - 1) / p->split_k * tk->bk;
        if (tk == &h->tk_main && h->tk_wholek.fn && (chain == 0 || k_per_unit <= 2 * chain)) {
            tk = &h->tk_wholek;
            chain = 0;
        }
        p->acc_chain = chain;
    }
    p->tk = variant == kVariantTensor ? tk : nullptr;
    size_t off = 0;
    if (variant != kVariantTensor) p->repitch_a = p->repitch_b = false;
    // (everything that belongs to A comes first: the pipelined host path reuses A's copies across column chunks of
    // different widths, so their offsets must not depend on N)
    if (p->repitch_a) { p->rp_a_off = off; off += round_up((size_t)lda * (h->cfg.trans_a ? m : k) * 4, 256); }
    if (variant == kVariantTensor) {
        // persistent grid: one CTA (or CTA pair) per SM (pair of SMs), never more launch units than tiles
        const uint64_t units = (uint64_t)p->tiles_m * p->tiles_n * p->split_k;
        const uint32_t group = tk->group;
        p->grid_x = group * (uint32_t)std::min<uint64_t>(units, (uint64_t)std::max(1, h->sm_count / (int)group));
        // floats between the first and the last element of an operand as stored (op(B) is K x N: stored K x N with
        // pitch ldb, or, transposed, N x K with pitch ldb)
        p->span_b = h->cfg.trans_b ? (uint64_t)ldb * (k - 1) + n : (uint64_t)ldb * (n - 1) + k;
        if (h->elem_bytes != 4) {
            // 16-bit operands: no lo copies; with a_major = "k" an untransposed A is read from a K-major packed copy
            p->span_a = p->span_b = 0;
            p->ldt = (uint32_t)round_up(k, 8);
            if (tk->a_packed && !h->cfg.trans_a) { p->hi_a_off = off; off += round_up((size_t)p->ldt * m * 2, 256); }
        } else if (tk->a_packed) {
            p->ldt = (uint32_t)round_up(k, 4);
            p->hi_a_off = off; off += round_up((size_t)p->ldt * m * 4, 256);
            p->lo_a_off = off; off += round_up((size_t)p->ldt * m * 4, 256);
            p->span_a = 0;
        } else if (!tk->split_inkernel || tk->split_hybrid) {
            p->span_a = h->cfg.trans_a ? (uint64_t)lda * (m - 1) + k : (uint64_t)lda * (k - 1) + m;
            p->lo_a_off = off; off += round_up(p->span_a * 4, 256);
        }
        if (p->repitch_b) { p->rp_b_off = off; off += round_up((size_t)ldb * (h->cfg.trans_b ? k : n) * 4, 256); }
        if (!tk->split_inkernel && h->elem_bytes == 4) { p->lo_b_off = off; off += round_up(p->span_b * 4, 256); }
    } else {
        // an FFMA cubin's own kernel, unless it is the TMA-fed one and TMA cannot describe these operands: then, as in
        // a tensor-variant cubin, the register-fed fallback kernel
        p->ffma_tma = h->cfg.variant == kVariantSimt && h->cfg.feed_tma && operand_tma_ok(a, lda) && operand_tma_ok(b, ldb);
        const bool own = h->cfg.variant == kVariantSimt && (!h->cfg.feed_tma || p->ffma_tma);
        const uint32_t tm = own ? h->tile_m : (uint32_t)h->cfg.fallback_tile[0];
        const uint32_t tn = own ? h->tile_n : (uint32_t)h->cfg.fallback_tile[1];
        const uint32_t bk = own ? (uint32_t)h->cfg.depth_k : (uint32_t)h->cfg.fallback_tile[2];
        p->tiles_m = (m + tm - 1) / tm;
        p->tiles_n = (n + tn - 1) / tn;
        // blocks the device holds at a time: two per SM of the register-fed kernel, one of the TMA-fed one
        p->split_k = pick_split_k(h, p->tiles_m * p->tiles_n, k, bk, (p->ffma_tma ? 1u : 2u) * (uint32_t)h->sm_count);
        p->grid_x = p->tiles_m * p->tiles_n;
    }
    if (p->split_k > 1) {
        p->partial_off = off;
        off += round_up((size_t)p->split_k * m * n * 4, 256);
    }
    p->ws_bytes = off;
    return SGEMM_OK;
}

int ensure_workspace(sgemm_handle *h, size_t bytes, CUdeviceptr *ws) {
    *ws = 0;
    if (bytes == 0) return SGEMM_OK;
    if (h->ws_lent) {
        if (bytes > h->ws_lent_bytes)
            return fail(h, SGEMM_ERR_WORKSPACE, "lent workspace holds %zu bytes, this call needs %zu",
                        h->ws_lent_bytes, bytes);
        *ws = h->ws_lent;
        return SGEMM_OK;
    }
    if (bytes > h->ws_owned_bytes) {
        Driver &d = driver();
        if (h->ws_owned) {
            CU_CHECK(h, d.cuCtxSynchronize_());  // kernels of earlier calls may still use the old block
            d.cuMemFree_(h->ws_owned);
            h->ws_owned = 0;
            h->ws_owned_bytes = 0;
        }
        const size_t want = round_up(bytes, (size_t)1 << 20);
        CUresult r = d.cuMemAlloc_(&h->ws_owned, want);
        if (r != CUDA_SUCCESS)
            return fail(h, SGEMM_ERR_WORKSPACE, "cuMemAlloc of %zu workspace bytes failed: %s", want, cu_text(r).c_str());
        h->ws_owned_bytes = want;
    }
    *ws = h->ws_owned;
    return SGEMM_OK;
}

// 2-D FP32 tensor map, dims {d0 (contiguous), d1}, box {b0, b1}.  `swizzle`: 128-byte swizzle of 16-byte units
// for K-major operand tiles, of 32-byte units for the MN-major A tile (the only shared-memory layout the
// tensor core accepts for 32-bit MN-major operands).
int encode_map(sgemm_handle *h, int slot, const void *base, uint64_t d0, uint64_t d1, uint64_t stride_bytes,
               uint32_t b0, uint32_t b1, CUtensorMapSwizzle swizzle, const CUtensorMap **out,
               CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_FLOAT32) {
    CachedMap &c = h->maps[slot];
    TensorMapKey key{base, d0, d1, stride_bytes, b0, b1, (int)swizzle * 16 + (int)dtype};
    if (!(c.valid && c.key == key)) {
        const cuuint64_t dims[2] = {d0, d1};
        const cuuint64_t strides[1] = {stride_bytes};
        const cuuint32_t box[2] = {b0, b1};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = driver().cuTensorMapEncodeTiled_(&c.map, dtype, 2,
                                                      const_cast<void *>(base), dims, strides, box, estr,
                                                      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(h, SGEMM_ERR_CUDA, "cuTensorMapEncodeTiled(base %p, dims %llu x %llu, pitch %llu, box %u x %u) -> %s",
                        base, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)stride_bytes,
                        b0, b1, cu_text(r).c_str());
        c.key = key;
        c.valid = true;
    }
    *out = &c.map;
    return SGEMM_OK;
}

int launch(sgemm_handle *h, CUfunction f, uint32_t gx, uint32_t gy, uint32_t gz, uint32_t bx, uint32_t by,
           uint32_t smem, CUstream s, void **params) {
    if (h->pdl) {
        // programmatic dependent launch: the kernel may be scheduled while its predecessor in the stream is still
        // running; every kernel of the cubin executes griddepcontrol.wait before it touches global memory, so
        // only launch latency and per-CTA set-up overlap with the predecessor, never data.
        CUlaunchAttribute attr;
        attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr.value.programmaticStreamSerializationAllowed = 1;
        CUlaunchConfig cfg;
        std::memset(&cfg, 0, sizeof cfg);
        cfg.gridDimX = gx; cfg.gridDimY = gy; cfg.gridDimZ = gz;
        cfg.blockDimX = bx; cfg.blockDimY = by; cfg.blockDimZ = 1;
        cfg.sharedMemBytes = smem;
        cfg.hStream = s;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        CU_CHECK(h, driver().cuLaunchKernelEx_(&cfg, f, params, nullptr));
    } else {
        CU_CHECK(h, driver().cuLaunchKernel_(f, gx, gy, gz, bx, by, 1, smem, s, params, nullptr));
    }
    ++h->launches;
    return SGEMM_OK;
}

// Launch the main GEMM kernel; with the "profile" option on, bracket it with an event pair so that its
// duration can be read back separately from the pre-pass and the reduction (sgemm_get_info "profile_*").
int launch_main(sgemm_handle *h, CUfunction f, uint32_t gx, uint32_t gz, uint32_t threads, uint32_t smem, CUstream s,
                void **params) {
    constexpr size_t kMaxPairs = 8192;
    if (!h->profile || h->prof_used >= kMaxPairs) return launch(h, f, gx, 1, gz, threads, 1, smem, s, params);
    Driver &d = driver();
    if (h->prof_used == h->prof_events.size()) {
        CUevent e0, e1;
        CU_CHECK(h, d.cuEventCreate_(&e0, CU_EVENT_DEFAULT));
        CU_CHECK(h, d.cuEventCreate_(&e1, CU_EVENT_DEFAULT));
        h->prof_events.emplace_back(e0, e1);
    }
    auto &pair = h->prof_events[h->prof_used];
    CU_CHECK(h, d.cuEventRecord_(pair.first, s));
    int rc = launch(h, f, gx, 1, gz, threads, 1, smem, s, params);
    if (rc) return rc;
    CU_CHECK(h, d.cuEventRecord_(pair.second, s));
    ++h->prof_used;
    return SGEMM_OK;
}

int check_problem(sgemm_handle *h, const void *a, const void *b, const void *c, const void *d, float beta,
                  uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    if (m && n && !d) return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "D is NULL");
    if (m && n && k && (!a || !b)) return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "A or B is NULL");
    if (m && n && beta != 0.0f && !c) return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "C is NULL but beta != 0");
    const uint32_t a_rows = h->cfg.trans_a ? k : m, b_rows = h->cfg.trans_b ? n : k;   // rows of A and B as stored
    if (lda < std::max(a_rows, 1u) || ldb < std::max(b_rows, 1u) || ldd < std::max(m, 1u) || (beta != 0.0f && ldc < std::max(m, 1u)))
        return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "leading dimension too small: lda %u ldb %u ldc %u ldd %u for M %u N %u K %u "
                    "(trans_a %d, trans_b %d)", lda, ldb, ldc, ldd, m, n, k, h->cfg.trans_a, h->cfg.trans_b);
    if ((uint64_t)m * n >= ((uint64_t)1 << 40)) return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "problem too large");
    return SGEMM_OK;
}

int launch_device(sgemm_handle *h, const float *dA, const float *dB, const float *dC, float *dD, float alpha,
                  float beta, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb, uint32_t ldc,
                  uint32_t ldd, CUstream stream) {
    int rc = check_problem(h, dA, dB, dC, dD, beta, m, n, k, lda, ldb, ldc, ldd);
    if (rc) return rc;
    if (m == 0 || n == 0) return SGEMM_OK;
    CUdeviceptr status = h->status;
    if (k == 0) {  // D = beta * C: the reduction kernel with zero partial products
        const float *ws0 = nullptr;
        uint32_t zero = 0;
        void *params[] = {&ws0, &dC, &dD, &m, &n, &ldc, &ldd, &alpha, &beta, &zero};
        const uint32_t blocks = (uint32_t)std::min<uint64_t>(((uint64_t)m * n + 255) / 256, (uint64_t)h->sm_count * 8);
        h->last_variant = 2; h->last_split_k = 1; h->last_grid = blocks;
        return launch(h, h->fn_reduce, blocks, 1, 1, 256, 1, 0, stream, params);
    }
    Plan p;
    rc = make_plan(h, dA, dB, m, n, k, lda, ldb, &p);
    if (rc) return rc;
    CUdeviceptr ws = 0;
    rc = ensure_workspace(h, p.ws_bytes, &ws);
    if (rc) return rc;
    float *partial = p.split_k > 1 ? reinterpret_cast<float *>(ws + p.partial_off) : nullptr;
    int32_t nwx = (int32_t)p.tiles_m, nwy = (int32_t)p.tiles_n;
    uint32_t split = p.split_k;
    uint32_t *status_ptr = reinterpret_cast<uint32_t *>(status);

    if (p.variant == kVariantTensor) {
        const TensorKernel &tk = *p.tk;
        if (p.repitch_a || p.repitch_b) {
            const uint32_t copy_blocks = (uint32_t)h->sm_count * 8;
            if (p.repitch_a && !h->reuse_a_lo) {
                float *dst = reinterpret_cast<float *>(ws + p.rp_a_off);
                uint32_t inner = h->cfg.trans_a ? k : m, outer = h->cfg.trans_a ? m : k;
                void *pr[] = {&dA, &lda, &inner, &outer, &dst, &p.lda_eff};
                if ((rc = launch(h, h->fn_repitch, copy_blocks, 1, 1, 256, 1, 0, stream, pr))) return rc;
            }
            if (p.repitch_b) {
                float *dst = reinterpret_cast<float *>(ws + p.rp_b_off);
                uint32_t inner = h->cfg.trans_b ? n : k, outer = h->cfg.trans_b ? k : n;
                void *pr[] = {&dB, &ldb, &inner, &outer, &dst, &p.ldb_eff};
                if ((rc = launch(h, h->fn_repitch, copy_blocks, 1, 1, 256, 1, 0, stream, pr))) return rc;
            }
            if (p.repitch_a) dA = reinterpret_cast<const float *>(ws + p.rp_a_off);
            if (p.repitch_b) dB = reinterpret_cast<const float *>(ws + p.rp_b_off);
            lda = p.lda_eff;
            ldb = p.ldb_eff;
        }
        float *lo_a = reinterpret_cast<float *>(ws + p.lo_a_off);
        float *lo_b = reinterpret_cast<float *>(ws + p.lo_b_off);
        // a CTA pair stages half of the tile's columns of B per CTA
        const uint32_t bk = tk.bk, bn = tk.tile_n / tk.group;
        // K-major tiles: rows of min(bk, 32) floats, 128-byte swizzle (64-byte for bk = 16)
        const uint32_t kspan = std::min<uint32_t>(bk, 32);
        const CUtensorMapSwizzle ksw = kspan == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
        const CUtensorMap *ma_hi, *ma_lo, *mb_hi, *mb_lo;
        const uint32_t blocks = (uint32_t)h->sm_count * 4;
        if (h->elem_bytes != 4) {
            // FP16 / BF16.  An operand stored K-contiguous (A transposed, B untransposed) is a K-major tile of 64 k per
            // 128-byte row (32 k and the 64-byte swizzle for depth_k = 32); one stored M- or N-contiguous is an MN-major
            // tile in chunks of 64 rows of M (columns of N), bk rows of 128 bytes each, 128-byte swizzle.  Either way TMA
            // reads it where it lies; only a_major = "k" goes through a packed K-major copy of A made here.
            const CUtensorMapDataType dt = h->cfg.a_type == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
            const uint32_t span16 = std::min<uint32_t>(bk, 64);
            const CUtensorMapSwizzle sw16 = span16 == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
            if (h->cfg.trans_a) {
                rc = encode_map(h, 0, dA, k, m, (uint64_t)lda * 2, span16, 128, sw16, &ma_hi, dt);
            } else if (tk.a_packed) {
                void *packed = reinterpret_cast<void *>(ws + p.hi_a_off);
                void *pp[] = {&dA, &lda, &m, &k, &packed, &p.ldt};
                if (!h->reuse_a_lo) {
                    rc = launch(h, h->fn_pack16, (m + 31) / 32, (k + 31) / 32, 1, 32, 8, 0, stream, pp);
                    if (rc) return rc;
                }
                rc = encode_map(h, 0, packed, k, m, (uint64_t)p.ldt * 2, span16, 128, sw16, &ma_hi, dt);
            } else {
                rc = encode_map(h, 0, dA, m, k, (uint64_t)lda * 2, 64, bk, CU_TENSOR_MAP_SWIZZLE_128B, &ma_hi, dt);
            }
            if (rc) return rc;
            if (h->cfg.trans_b) rc = encode_map(h, 2, dB, n, k, (uint64_t)ldb * 2, 64, bk, CU_TENSOR_MAP_SWIZZLE_128B, &mb_hi, dt);
            else rc = encode_map(h, 2, dB, k, n, (uint64_t)ldb * 2, span16, bn, sw16, &mb_hi, dt);
            if (rc) return rc;
            ma_lo = ma_hi;
            mb_lo = mb_hi;
        } else if (tk.a_packed) {
            float *hi_t = reinterpret_cast<float *>(ws + p.hi_a_off);
            void *pp[] = {&dA, &lda, &m, &k, &hi_t, &lo_a, &p.ldt};
            if (!h->reuse_a_lo) {
                rc = launch(h, h->fn_pack_a, (m + 31) / 32, (k + 31) / 32, 1, 32, 8, 0, stream, pp);
                if (rc) return rc;
            }
            const float *na = nullptr;
            uint64_t zero = 0;
            void *ps[] = {&na, &na, &zero, &dB, &lo_b, &p.span_b};
            rc = launch(h, h->fn_split_lo, blocks, 1, 1, 256, 1, 0, stream, ps);
            if (rc) return rc;
            if ((rc = encode_map(h, 0, hi_t, k, m, (uint64_t)p.ldt * 4, kspan, 128, ksw, &ma_hi))) return rc;
            if ((rc = encode_map(h, 1, lo_a, k, m, (uint64_t)p.ldt * 4, kspan, 128, ksw, &ma_lo))) return rc;
        } else if (tk.split_inkernel) {
            // no pre-pass and no lo copies: the kernel's transform warps make the lo tiles; the lo map slots get the hi maps
            if (h->cfg.trans_a) rc = encode_map(h, 0, dA, k, m, (uint64_t)lda * 4, kspan, 128, ksw, &ma_hi);
            else rc = encode_map(h, 0, dA, m, k, (uint64_t)lda * 4, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, &ma_hi);
            if (rc) return rc;
            ma_lo = ma_hi;
            if (tk.split_hybrid) {
                // ... except A's lo copy, which the pre-pass writes (B's span is empty for it) and TMA loads
                uint64_t span_a = h->reuse_a_lo ? 0 : p.span_a, none = 0;
                const float *nb = nullptr;
                float *nlo = nullptr;
                void *ps[] = {&dA, &lo_a, &span_a, &nb, &nlo, &none};
                if (span_a && (rc = launch(h, h->fn_split_lo, blocks, 1, 1, 256, 1, 0, stream, ps))) return rc;
                if (h->cfg.trans_a) rc = encode_map(h, 1, lo_a, k, m, (uint64_t)lda * 4, kspan, 128, ksw, &ma_lo);
                else rc = encode_map(h, 1, lo_a, m, k, (uint64_t)lda * 4, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, &ma_lo);
                if (rc) return rc;
            }
        } else if (h->cfg.trans_a) {
            // A is stored K-contiguous: it is the K-major operand as it lies, and so is its lo copy
            uint64_t span_a = h->reuse_a_lo ? 0 : p.span_a;
            void *ps[] = {&dA, &lo_a, &span_a, &dB, &lo_b, &p.span_b};
            rc = launch(h, h->fn_split_lo, blocks, 1, 1, 256, 1, 0, stream, ps);
            if (rc) return rc;
            if ((rc = encode_map(h, 0, dA, k, m, (uint64_t)lda * 4, kspan, 128, ksw, &ma_hi))) return rc;
            if ((rc = encode_map(h, 1, lo_a, k, m, (uint64_t)lda * 4, kspan, 128, ksw, &ma_lo))) return rc;
        } else {
            uint64_t span_a = h->reuse_a_lo ? 0 : p.span_a;   // same A as the previous chunk of a pipelined host call
            void *ps[] = {&dA, &lo_a, &span_a, &dB, &lo_b, &p.span_b};
            rc = launch(h, h->fn_split_lo, blocks, 1, 1, 256, 1, 0, stream, ps);
            if (rc) return rc;
            if ((rc = encode_map(h, 0, dA, m, k, (uint64_t)lda * 4, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, &ma_hi))) return rc;
            if ((rc = encode_map(h, 1, lo_a, m, k, (uint64_t)lda * 4, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, &ma_lo))) return rc;
        }
        if (h->elem_bytes != 4) {
            // (both maps were made above)
        } else if (h->cfg.trans_b) {
            // B is stored N-contiguous: an MN-major operand, staged in 32-column chunks like the untransposed A
            if ((rc = encode_map(h, 2, dB, n, k, (uint64_t)ldb * 4, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, &mb_hi))) return rc;
            if (tk.split_inkernel) mb_lo = mb_hi;
            else if ((rc = encode_map(h, 3, lo_b, n, k, (uint64_t)ldb * 4, 32, bk, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, &mb_lo))) return rc;
        } else {
            if ((rc = encode_map(h, 2, dB, k, n, (uint64_t)ldb * 4, kspan, bn, ksw, &mb_hi))) return rc;
            if (tk.split_inkernel) mb_lo = mb_hi;
            else if ((rc = encode_map(h, 3, lo_b, k, n, (uint64_t)ldb * 4, kspan, bn, ksw, &mb_lo))) return rc;
        }
        // the alignment counter only ever counts up: every launch unit adds one per tile
        uint32_t *wave_sync = h->wave_sync ? reinterpret_cast<uint32_t *>(h->counters) : nullptr;
        uint32_t wave_base = h->wave_sync_base;
        if (wave_sync) h->wave_sync_base += p.tiles_m * p.tiles_n * p.split_k;
        uint32_t acc_chunk = p.acc_chain / tk.bk;
        h->last_acc_chain = p.acc_chain;
        void *params[] = {&dA, &dB, &dC, &dD, &m, &n, &k, &lda, &ldb, &ldc, &ldd, &alpha, &beta, &nwx, &nwy,
                          &partial, &status_ptr, &split, &wave_sync, &wave_base, &acc_chunk,
                          const_cast<CUtensorMap *>(ma_hi), const_cast<CUtensorMap *>(ma_lo),
                          const_cast<CUtensorMap *>(mb_hi), const_cast<CUtensorMap *>(mb_lo)};
        rc = launch_main(h, tk.fn, p.grid_x, 1, tk.threads, tk.smem, stream, params);
        if (rc) return rc;
    } else if (p.ffma_tma) {
        // TMA-fed FFMA kernel: one box per operand and k-step, no swizzle.  A tile: BK rows of BM floats (row = one k);
        // B tile: BN rows of BK floats (row = one n), or, for a transposed B, BK rows of BN floats
        const uint32_t bm = h->tile_m, bn = h->tile_n, bk = (uint32_t)h->cfg.depth_k;
        const CUtensorMap *ma, *mb;
        if ((rc = encode_map(h, 0, dA, m, k, (uint64_t)lda * 4, bm, bk, CU_TENSOR_MAP_SWIZZLE_NONE, &ma))) return rc;
        if (h->cfg.trans_b) rc = encode_map(h, 2, dB, n, k, (uint64_t)ldb * 4, bn, bk, CU_TENSOR_MAP_SWIZZLE_NONE, &mb);
        else rc = encode_map(h, 2, dB, k, n, (uint64_t)ldb * 4, bk, bn, CU_TENSOR_MAP_SWIZZLE_NONE, &mb);
        if (rc) return rc;
        uint32_t *wave_sync = nullptr;
        uint32_t wave_base = 0;
        void *params[] = {&dA, &dB, &dC, &dD, &m, &n, &k, &lda, &ldb, &ldc, &ldd, &alpha, &beta, &nwx, &nwy,
                          &partial, &status_ptr, &split, &wave_sync, &wave_base,
                          const_cast<CUtensorMap *>(ma), const_cast<CUtensorMap *>(mb)};
        rc = launch_main(h, h->fn_main, p.grid_x, p.split_k, (uint32_t)h->cfg.num_threads, (uint32_t)h->cfg.dynamic_smem_bytes,
                         stream, params);
        if (rc) return rc;
    } else {
        const bool own = h->cfg.variant == kVariantSimt && !h->cfg.feed_tma;
        CUfunction f = own ? h->fn_main : h->fn_simt;
        const uint32_t threads = own ? (uint32_t)h->cfg.num_threads : (uint32_t)h->cfg.fallback_threads;
        uint32_t *wave_sync = nullptr;
        uint32_t wave_base = 0;
        void *params[] = {&dA, &dB, &dC, &dD, &m, &n, &k, &lda, &ldb, &ldc, &ldd, &alpha, &beta, &nwx, &nwy,
                          &partial, &status_ptr, &split, &wave_sync, &wave_base};
        rc = launch_main(h, f, p.grid_x, p.split_k, threads, 0, stream, params);
        if (rc) return rc;
    }
    if (p.split_k > 1) {
        const float *wsp = partial;
        void *params[] = {&wsp, &dC, &dD, &m, &n, &ldc, &ldd, &alpha, &beta, &split};
        // one thread per four rows on the kernel's vector path (M a multiple of 4), per element otherwise
        const uint64_t items = (m % 4 == 0) ? (uint64_t)m * n / 4 : (uint64_t)m * n;
        const uint32_t blocks = (uint32_t)std::min<uint64_t>((items + 255) / 256, (uint64_t)h->sm_count * 8);
        rc = launch(h, h->fn_reduce, blocks, 1, 1, 256, 1, 0, stream, params);
        if (rc) return rc;
    }
    h->last_variant = p.variant != kVariantTensor ? 2 : ((p.tk == &h->tk_skinny || p.tk == &h->tk_thin) ? 3 : 1);
    if (p.variant != kVariantTensor) h->last_acc_chain = 0;
    h->last_tile_n = p.variant == kVariantTensor ? p.tk->tile_n : 0;
    h->last_feed_tma = p.variant == kVariantTensor || p.ffma_tma;
    h->last_split_k = p.split_k;
    h->last_grid = p.grid_x;
    return SGEMM_OK;
}

int config_from_toml(const char *path, sgemm_config *c, std::string *err) {
    sgemm_toml::Table t;
    if (!sgemm_toml::parse_file(path, &t, err)) return SGEMM_ERR_TOML;
    std::memset(c, 0, sizeof *c);
    auto need_int = [&](const char *key, int32_t *dst) {
        int64_t v;
        if (!t.get_int(key, &v)) { *err = std::string("missing or non-integer key '") + key + "' in " + path; return false; }
        *dst = (int32_t)v;
        return true;
    };
    auto need_arr = [&](const char *key, int32_t *dst, size_t count) {
        std::vector<int64_t> v;
        if (!t.get_int_array(key, &v) || v.size() != count) {
            *err = std::string("missing key or wrong length for integer array '") + key + "' in " + path;
            return false;
        }
        for (size_t i = 0; i < count; ++i) dst[i] = (int32_t)v[i];
        return true;
    };
    auto need_bool = [&](const char *key, int32_t *dst) {
        bool v;
        if (!t.get_bool(key, &v)) { *err = std::string("missing or non-boolean key '") + key + "' in " + path; return false; }
        *dst = v ? 1 : 0;
        return true;
    };
    // the keys the reference's runner reads (runner/generator_runner.cpp:103-122) are all required
    if (!need_int("a_type", &c->a_type) || !need_int("b_type", &c->b_type) || !need_int("cd_type", &c->cd_type) ||
        !need_int("scalar_type", &c->scalar_type) || !need_arr("mfma", c->mfma, 4) ||
        !need_arr("wave_group", c->wave_group, 2) || !need_arr("wave_tiling", c->wave_tiling, 2) ||
        !need_int("depth_k", &c->depth_k) || !need_bool("trans_a", &c->trans_a) || !need_bool("trans_b", &c->trans_b) ||
        !need_int("wavefront_size", &c->wavefront_size) || !need_int("lds_usage_bytes", &c->lds_usage_bytes))
        return SGEMM_ERR_TOML;
    int64_t v;
    c->vmem_stage = t.get_int("vmem_stage", &v) ? (int32_t)v : 1;
    std::string s;
    c->variant = (t.get_string("variant", &s) && s == "tcgen05_3xtf32") ? kVariantTensor : kVariantSimt;
    c->num_threads = t.get_int("num_threads", &v) ? (int32_t)v : c->wave_group[0] * c->wave_group[1] * c->wavefront_size;
    c->dynamic_smem_bytes = t.get_int("dynamic_smem_bytes", &v) ? (int32_t)v : 0;
    c->stages = t.get_int("stages", &v) ? (int32_t)v : c->vmem_stage + 1;
    c->a_kmajor = (t.get_string("a_major", &s) && s == "k") ? 1 : 0;
    c->split_inkernel = !t.get_string("split", &s) ? 0 : s == "inkernel" ? 1 : s == "hybrid" ? 2 : 0;
    c->feed_tma = (c->variant == kVariantSimt && t.get_string("feed", &s) && s == "tma") ? 1 : 0;
    std::vector<int64_t> fb;
    if (t.get_int_array("fallback_tile", &fb) && fb.size() == 3)
        for (int i = 0; i < 3; ++i) c->fallback_tile[i] = (int32_t)fb[i];
    c->fallback_threads = t.get_int("fallback_threads", &v) ? (int32_t)v : 0;
    std::vector<int64_t> sk;
    if (t.get_int_array("skinny_tile", &sk) && sk.size() == 3)
        for (int i = 0; i < 3; ++i) c->skinny_tile[i] = (int32_t)sk[i];
    c->skinny_threads = t.get_int("skinny_threads", &v) ? (int32_t)v : 0;
    c->skinny_smem_bytes = t.get_int("skinny_smem_bytes", &v) ? (int32_t)v : 0;
    std::snprintf(c->skinny_entry, sizeof c->skinny_entry, "%s", t.get_string("skinny_entry", &s) ? s.c_str() : "");
    c->acc_chain = t.get_int("acc_chain", &v) ? (int32_t)v : 0;
    std::snprintf(c->wholek_entry, sizeof c->wholek_entry, "%s", t.get_string("wholek_entry", &s) ? s.c_str() : "");
    c->skinny_acc_chain = t.get_int("skinny_acc_chain", &v) ? (int32_t)v : 0;
    if (t.get_int_array("thin_tile", &sk) && sk.size() == 3)
        for (int i = 0; i < 3; ++i) c->thin_tile[i] = (int32_t)sk[i];
    c->thin_threads = t.get_int("thin_threads", &v) ? (int32_t)v : 0;
    c->thin_smem_bytes = t.get_int("thin_smem_bytes", &v) ? (int32_t)v : 0;
    c->thin_acc_chain = t.get_int("thin_acc_chain", &v) ? (int32_t)v : 0;
    std::snprintf(c->thin_entry, sizeof c->thin_entry, "%s", t.get_string("thin_entry", &s) ? s.c_str() : "");
    std::snprintf(c->entry, sizeof c->entry, "%s", t.get_string("entry", &s) ? s.c_str() : "generated_gemm");
    std::snprintf(c->fallback_entry, sizeof c->fallback_entry, "%s", t.get_string("fallback_entry", &s) ? s.c_str() : "");
    if ((c->variant == kVariantTensor || c->feed_tma) && (c->fallback_threads <= 0 || c->fallback_tile[0] <= 0 || !c->fallback_entry[0])) {
        *err = "a config whose main kernel is fed by TMA lacks the fallback_* keys";
        return SGEMM_ERR_TOML;
    }
    for (int i = 0; i < 2; ++i)
        if (c->mfma[i] <= 0 || c->wave_group[i] <= 0 || c->wave_tiling[i] <= 0) { *err = "non-positive tiling value"; return SGEMM_ERR_TOML; }
    if (c->depth_k <= 0 || c->num_threads <= 0) { *err = "non-positive depth_k or num_threads"; return SGEMM_ERR_TOML; }
    return SGEMM_OK;
}

}  // namespace

// =============================================================================================== ABI
SGEMM_API const char *sgemm_strerror(int code) {
    switch (code) {
        case SGEMM_OK: return "ok";
        case SGEMM_ERR_INVALID_ARGUMENT: return "invalid argument";
        case SGEMM_ERR_TOML: return "kernel config (TOML) unreadable or incomplete";
        case SGEMM_ERR_NO_DRIVER: return "CUDA driver not available";
        case SGEMM_ERR_CUDA: return "CUDA driver call failed";
        case SGEMM_ERR_MODULE: return "cubin could not be loaded or lacks an entry point";
        case SGEMM_ERR_UNSUPPORTED: return "request not supported by the loaded kernel";
        case SGEMM_ERR_WORKSPACE: return "workspace too small or allocation failed";
        case SGEMM_ERR_DEVICE_STATUS: return "a kernel gave up on a bounded wait";
        case SGEMM_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the allocation-free entry point has";
        case SGEMM_ERR_COMM: return "NCCL not available, communicator missing, or a collective failed";
        default: return "unknown error";
    }
}

SGEMM_API const char *sgemm_last_error(sgemm_handle *h) { return h ? h->error.c_str() : g_open_error.c_str(); }

SGEMM_API int sgemm_device_count(void) {
    Driver &d = driver();
    if (!d.ok) return 0;
    int n = 0;
    return d.cuDeviceGetCount_(&n) == CUDA_SUCCESS ? n : 0;
}

SGEMM_API int sgemm_config_parse(const char *toml_path, sgemm_config *out) {
    if (!toml_path || !out) return fail(nullptr, SGEMM_ERR_INVALID_ARGUMENT, "NULL argument");
    std::string err;
    int rc = config_from_toml(toml_path, out, &err);
    if (rc) return fail(nullptr, rc, "%s", err.c_str());
    return SGEMM_OK;
}

SGEMM_API int sgemm_config_tile(const sgemm_config *cfg, uint32_t *tile_m, uint32_t *tile_n) {
    if (!cfg || !tile_m || !tile_n) return SGEMM_ERR_INVALID_ARGUMENT;
    *tile_m = (uint32_t)(cfg->mfma[0] * cfg->wave_group[0] * cfg->wave_tiling[0]);
    *tile_n = (uint32_t)(cfg->mfma[1] * cfg->wave_group[1] * cfg->wave_tiling[1]);
    return SGEMM_OK;
}

SGEMM_API int sgemm_open(const char *cubin_path, const char *toml_path, int device, sgemm_handle **out) {
    if (!cubin_path || !toml_path || !out) return fail(nullptr, SGEMM_ERR_INVALID_ARGUMENT, "NULL argument");
    *out = nullptr;
    sgemm_config cfg;
    std::string err;
    int rc = config_from_toml(toml_path, &cfg, &err);
    if (rc) return fail(nullptr, rc, "%s", err.c_str());
    FILE *probe = std::fopen(cubin_path, "rb");
    if (!probe) return fail(nullptr, SGEMM_ERR_MODULE, "cannot open cubin '%s'", cubin_path);
    std::fclose(probe);
    Driver &d = driver();
    if (!d.ok) return fail(nullptr, SGEMM_ERR_NO_DRIVER, "%s", d.error.c_str());
    int count = 0;
    if (d.cuDeviceGetCount_(&count) != CUDA_SUCCESS || device < 0 || device >= count)
        return fail(nullptr, SGEMM_ERR_INVALID_ARGUMENT, "device %d not present (%d visible)", device, count);

    sgemm_handle *h = new sgemm_handle();
    h->cfg = cfg;
    h->device = device;
    // element types as the generator numbers them: 0 = FP32, 1 = FP16, 2 = BF16
    if (cfg.a_type != cfg.b_type || cfg.a_type < 0 || cfg.a_type > 2 || cfg.cd_type != 0 || cfg.scalar_type != 0 ||
        (cfg.a_type != 0 && cfg.variant != kVariantTensor)) {
        delete h;
        return fail(nullptr, SGEMM_ERR_UNSUPPORTED, "element types a %d b %d cd %d scalar %d are not served (FP32 everywhere, or "
                    "FP16/BF16 A and B with the tensor variant)", cfg.a_type, cfg.b_type, cfg.cd_type, cfg.scalar_type);
    }
    h->elem_bytes = cfg.a_type == 0 ? 4u : 2u;
    sgemm_config_tile(&cfg, &h->tile_m, &h->tile_n);
    auto bail = [&](int code) {
        g_open_error = h->error;
        sgemm_close(h);
        return code;
    };
    CUresult r;
    if ((r = d.cuDeviceGet_(&h->cu_device, device)) != CUDA_SUCCESS ||
        (r = d.cuDevicePrimaryCtxRetain_(&h->ctx, h->cu_device)) != CUDA_SUCCESS) {
        h->ctx = nullptr;
        fail(h, SGEMM_ERR_CUDA, "cannot retain the primary context of device %d: %s", device, cu_text(r).c_str());
        return bail(SGEMM_ERR_CUDA);
    }
    CtxGuard guard(h);
    d.cuDeviceGetAttribute_(&h->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, h->cu_device);
    int cc_major = 0;
    d.cuDeviceGetAttribute_(&cc_major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, h->cu_device);
    if ((r = d.cuModuleLoad_(&h->module, cubin_path)) != CUDA_SUCCESS) {
        h->module = nullptr;
        fail(h, SGEMM_ERR_MODULE, "cuModuleLoad('%s') on device %d (compute capability %d.x) -> %s", cubin_path,
             device, cc_major, cu_text(r).c_str());
        return bail(SGEMM_ERR_MODULE);
    }
    struct Want { CUfunction *f; const char *name; bool required; };
    const Want wants[] = {
        {&h->fn_main, cfg.entry, true},
        {&h->fn_simt, cfg.fallback_entry, cfg.variant == kVariantTensor || cfg.feed_tma != 0},
        {&h->fn_split_lo, "sgemm_split_lo", true},
        {&h->fn_pack_a, "sgemm_pack_a_kmajor", true},
        {&h->fn_pack16, "sgemm_pack16_kmajor", true},
        {&h->fn_repitch, "sgemm_repitch", true},
        {&h->fn_narrow16, "sgemm_narrow16", true},
        {&h->fn_reduce, "sgemm_splitk_reduce", true},
        {&h->fn_fill, "sgemm_fill_uniform", true},
        {&h->fn_tile_map, "sgemm_tile_map", true},
        {&h->fn_wait_selftest, "sgemm_wait_selftest", cfg.variant == kVariantTensor || cfg.feed_tma != 0},
    };
    for (const Want &w : wants) {
        if (!w.required) continue;   // entry points that only one variant's cubin contains stay NULL in the other's handle
        if ((r = d.cuModuleGetFunction_(w.f, h->module, w.name)) != CUDA_SUCCESS) {
            fail(h, SGEMM_ERR_MODULE, "entry point '%s' not found in '%s': %s", w.name, cubin_path, cu_text(r).c_str());
            return bail(SGEMM_ERR_MODULE);
        }
    }
    h->tk_main.fn = h->fn_main;
    h->tk_main.tile_m = h->tile_m; h->tk_main.tile_n = h->tile_n; h->tk_main.bk = (uint32_t)cfg.depth_k;
    h->tk_main.group = (uint32_t)std::max(1, cfg.wave_group[0]);
    h->tk_main.threads = (uint32_t)cfg.num_threads; h->tk_main.smem = (uint32_t)cfg.dynamic_smem_bytes;
    h->tk_main.split_inkernel = cfg.split_inkernel != 0; h->tk_main.a_packed = cfg.a_kmajor != 0;
    h->tk_main.split_hybrid = cfg.split_inkernel == 2;
    h->tk_main.acc_chain = (uint32_t)std::max(cfg.acc_chain, 0);
    if (cfg.variant == kVariantTensor && cfg.wholek_entry[0]) {
        h->tk_wholek = h->tk_main;
        h->tk_wholek.acc_chain = 0;
        if ((r = d.cuModuleGetFunction_(&h->tk_wholek.fn, h->module, cfg.wholek_entry)) != CUDA_SUCCESS ||
            (r = d.cuFuncSetAttribute_(h->tk_wholek.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)h->tk_main.smem)) != CUDA_SUCCESS) {
            fail(h, SGEMM_ERR_MODULE, "whole-K entry point '%s' unusable in '%s': %s", cfg.wholek_entry, cubin_path, cu_text(r).c_str());
            return bail(SGEMM_ERR_MODULE);
        }
    }
    if (cfg.variant == kVariantTensor && cfg.skinny_entry[0] && cfg.skinny_threads > 0 && cfg.skinny_tile[0] > 0) {
        // companion kernel for low-intensity shapes: one CTA per 128-row tile, lo tiles made in the kernel
        if ((r = d.cuModuleGetFunction_(&h->tk_skinny.fn, h->module, cfg.skinny_entry)) != CUDA_SUCCESS ||
            (r = d.cuFuncSetAttribute_(h->tk_skinny.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, cfg.skinny_smem_bytes)) != CUDA_SUCCESS) {
            fail(h, SGEMM_ERR_MODULE, "companion entry point '%s' unusable in '%s': %s", cfg.skinny_entry, cubin_path, cu_text(r).c_str());
            return bail(SGEMM_ERR_MODULE);
        }
        h->tk_skinny.tile_m = (uint32_t)cfg.skinny_tile[0]; h->tk_skinny.tile_n = (uint32_t)cfg.skinny_tile[1];
        h->tk_skinny.bk = (uint32_t)cfg.skinny_tile[2];
        h->tk_skinny.group = 1; h->tk_skinny.threads = (uint32_t)cfg.skinny_threads; h->tk_skinny.smem = (uint32_t)cfg.skinny_smem_bytes;
        h->tk_skinny.split_inkernel = true; h->tk_skinny.a_packed = false;
        h->tk_skinny.acc_chain = (uint32_t)std::max(cfg.skinny_acc_chain, 0);
    }
    if (cfg.variant == kVariantTensor && cfg.thin_entry[0] && cfg.thin_threads > 0 && cfg.thin_tile[0] > 0) {
        if ((r = d.cuModuleGetFunction_(&h->tk_thin.fn, h->module, cfg.thin_entry)) != CUDA_SUCCESS ||
            (r = d.cuFuncSetAttribute_(h->tk_thin.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, cfg.thin_smem_bytes)) != CUDA_SUCCESS) {
            fail(h, SGEMM_ERR_MODULE, "entry point '%s' unusable in '%s': %s", cfg.thin_entry, cubin_path, cu_text(r).c_str());
            return bail(SGEMM_ERR_MODULE);
        }
        h->tk_thin.tile_m = (uint32_t)cfg.thin_tile[0]; h->tk_thin.tile_n = (uint32_t)cfg.thin_tile[1];
        h->tk_thin.bk = (uint32_t)cfg.thin_tile[2];
        h->tk_thin.group = 1; h->tk_thin.threads = (uint32_t)cfg.thin_threads; h->tk_thin.smem = (uint32_t)cfg.thin_smem_bytes;
        h->tk_thin.split_inkernel = true; h->tk_thin.a_packed = false;
        h->tk_thin.acc_chain = (uint32_t)std::max(cfg.thin_acc_chain, 0);
    }
    if (cfg.dynamic_smem_bytes > 0 &&
        (r = d.cuFuncSetAttribute_(h->fn_main, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, cfg.dynamic_smem_bytes)) != CUDA_SUCCESS) {
        fail(h, SGEMM_ERR_CUDA, "cannot opt in to %d bytes of dynamic shared memory: %s", cfg.dynamic_smem_bytes, cu_text(r).c_str());
        return bail(SGEMM_ERR_CUDA);
    }
    // Kernels that hand registers from one warp group to another (setmaxnreg) size the shares from the launch
    // allocation __launch_bounds__ allows, and a growing warp waits without limit for registers the block was never
    // given: a cubin whose entry was compiled to a different register count must not be launched.  That is the TMA-fed
    // FFMA kernel with 256 or more consumers, and a tensor kernel with chunked accumulation and 8 epilogue warps.
    auto hands_over = [&](uint32_t threads, bool inkernel, uint32_t acc_chain) {
        if (cfg.variant != kVariantTensor) return cfg.feed_tma != 0 && threads >= 384;
        const uint32_t epilogue_warps = (threads - 128 - (inkernel ? 128 : 0)) / 32;
        return acc_chain > 0 && epilogue_warps == 8;
    };
    struct Entry { CUfunction fn; const char *name; uint32_t threads; bool inkernel; uint32_t acc_chain; };
    const Entry entries[] = {
        {h->tk_main.fn, cfg.entry, h->tk_main.threads, h->tk_main.split_inkernel, h->tk_main.acc_chain},
        {h->tk_skinny.fn, cfg.skinny_entry, h->tk_skinny.threads, true, h->tk_skinny.acc_chain},
        {h->tk_thin.fn, cfg.thin_entry, h->tk_thin.threads, true, h->tk_thin.acc_chain},
    };
    for (const Entry &e : entries) {
        if (!e.fn || e.threads < 256 || !hands_over(e.threads, e.inkernel, e.acc_chain)) continue;
        int regs = 0;
        const int expect = (512 / (int)(e.threads / 128)) / 8 * 8;
        if ((r = d.cuFuncGetAttribute_(&regs, CU_FUNC_ATTRIBUTE_NUM_REGS, e.fn)) != CUDA_SUCCESS || regs != expect) {
            fail(h, SGEMM_ERR_MODULE, "'%s' in '%s' uses %d registers per thread where its register hand-over assumes %d",
                 e.name, cubin_path, regs, expect);
            return bail(SGEMM_ERR_MODULE);
        }
    }
    if ((r = d.cuMemAlloc_(&h->status, kStatusAlloc * 4)) != CUDA_SUCCESS ||
        (r = d.cuMemsetD8_(h->status, 0, kStatusAlloc * 4)) != CUDA_SUCCESS ||
        (r = d.cuMemAlloc_(&h->counters, (size_t)kCounterWords * 4)) != CUDA_SUCCESS ||
        (r = d.cuMemsetD8_(h->counters, 0, (size_t)kCounterWords * 4)) != CUDA_SUCCESS) {
        fail(h, SGEMM_ERR_CUDA, "cannot allocate the status buffer: %s", cu_text(r).c_str());
        return bail(SGEMM_ERR_CUDA);
    }
    *out = h;
    return SGEMM_OK;
}

SGEMM_API int sgemm_close(sgemm_handle *h) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    Driver &d = driver();
    if (d.ok && h->ctx) {
        {
            CtxGuard guard(h);
            d.cuCtxSynchronize_();
            if (h->comm.comm) sgemm_internal::comm_release(h->comm.comm);
            h->comm = sgemm_internal::CommState{};
            for (auto &pr : h->prof_events) {
                d.cuEventDestroy_(pr.first);
                d.cuEventDestroy_(pr.second);
            }
            if (h->status) d.cuMemFree_(h->status);
            if (h->counters) d.cuMemFree_(h->counters);
            if (h->ws_owned) d.cuMemFree_(h->ws_owned);
            for (CUdeviceptr p : h->stage)
                if (p) d.cuMemFree_(p);
            for (CUevent e : h->pipe_events) d.cuEventDestroy_(e);
            for (CUstream st : h->pipe_streams)
                if (st) d.cuStreamDestroy_(st);
            if (h->module) d.cuModuleUnload_(h->module);
        }
        d.cuDevicePrimaryCtxRelease_(h->cu_device);
    }
    delete h;
    return SGEMM_OK;
}

SGEMM_API int sgemm_launch(sgemm_handle *h, const float *dA, const float *dB, const float *dC, float *dD,
                           float alpha, float beta, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb,
                           uint32_t ldc, uint32_t ldd, void *stream) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    CtxGuard guard(h);
    return launch_device(h, dA, dB, dC, dD, alpha, beta, m, n, k, lda, ldb, ldc, ldd, (CUstream)stream);
}

namespace {

// Upload A as stored (`outer` columns of pitch lda, `inner` elements each) into the staging buffer, ordered on `s`:
// all of it, or — sharded — only this rank's slice of the columns, after which the ranks complete each other's
// buffers over NVLink (an in-place all-gather of the slices; ragged slices as grouped broadcasts).  A replicated
// operand then crosses the host link once per box instead of once per GPU.
int upload_a(sgemm_handle *h, const float *hA, size_t bytes_a, uint32_t inner, uint32_t outer, uint32_t lda, CUstream s,
             bool sharded) {
    Driver &d = driver();
    if (!bytes_a) return SGEMM_OK;
    if (!sharded || h->comm.world <= 1) {
        CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[0], hA, bytes_a, s));
        return SGEMM_OK;
    }
    const int world = h->comm.world;
    const size_t eb = h->elem_bytes;
    std::vector<size_t> offsets((size_t)world), bytes((size_t)world);
    for (int r = 0; r < world; ++r) {
        const uint64_t o0 = (uint64_t)outer * r / world, o1 = (uint64_t)outer * (r + 1) / world;
        offsets[r] = (size_t)o0 * lda * eb;
        // whole columns of pitch lda, except that the buffer ends with the last element of the last column
        bytes[r] = o1 > o0 ? ((size_t)(o1 - o0 - 1) * lda + (o1 == outer ? inner : lda)) * eb : 0;
    }
    const int me = h->comm.rank;
    if (bytes[me])
        CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[0] + offsets[me], reinterpret_cast<const char *>(hA) + offsets[me], bytes[me], s));
    return sgemm_internal::comm_complete(h, reinterpret_cast<void *>(h->stage[0]), offsets.data(), bytes.data(), s);
}

int run_host_impl(sgemm_handle *h, const float *hA, const float *hB, const float *hC, float *hD,
                  float alpha, float beta, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb,
                  uint32_t ldc, uint32_t ldd, bool sharded);

}  // namespace

SGEMM_API int sgemm_run_host(sgemm_handle *h, const float *hA, const float *hB, const float *hC, float *hD,
                             float alpha, float beta, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb,
                             uint32_t ldc, uint32_t ldd) {
    return run_host_impl(h, hA, hB, hC, hD, alpha, beta, m, n, k, lda, ldb, ldc, ldd, false);
}

SGEMM_API int sgemm_run_host_sharded(sgemm_handle *h, const float *hA, const float *hB, const float *hC, float *hD,
                                     float alpha, float beta, uint32_t m, uint32_t n_local, uint32_t k, uint32_t lda,
                                     uint32_t ldb, uint32_t ldc, uint32_t ldd) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    if (!h->comm.comm) return fail(h, SGEMM_ERR_COMM, "no communicator on this handle: call sgemm_comm_init first");
    // every rank must take part in the exchange of A, also one whose shard is empty
    return run_host_impl(h, hA, hB, hC, hD, alpha, beta, m, n_local, k, lda, ldb, ldc, ldd, true);
}

namespace {

int run_host_impl(sgemm_handle *h, const float *hA, const float *hB, const float *hC, float *hD,
                  float alpha, float beta, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb,
                  uint32_t ldc, uint32_t ldd, bool sharded) {
    int rc = check_problem(h, hA, hB, hC, hD, beta, m, n, k, lda, ldb, ldc, ldd);
    if (rc) return rc;
    if (sharded && m && k && !hA) return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "A is NULL");
    if (m == 0 || (n == 0 && !sharded)) return SGEMM_OK;
    const uint32_t a_inner = h->cfg.trans_a ? k : m, a_outer = h->cfg.trans_a ? m : k;
    CtxGuard guard(h);
    Driver &d = driver();
    const bool use_c = beta != 0.0f;
    const size_t a_floats = h->cfg.trans_a ? (size_t)lda * (m - 1) + k : (size_t)lda * (k - 1) + m;
    const size_t b_floats = !n ? 0 : h->cfg.trans_b ? (size_t)ldb * (k - 1) + n : (size_t)ldb * (n - 1) + k;
    const size_t eb = h->elem_bytes;   // A and B elements; C and D are FP32
    const size_t bytes[4] = {k ? a_floats * eb : 0, k ? b_floats * eb : 0,
                             use_c && n ? ((size_t)ldc * (n - 1) + m) * 4 : 0, n ? ((size_t)ldd * (n - 1) + m) * 4 : 0};
    for (int i = 0; i < 4; ++i) {
        if (bytes[i] > h->stage_bytes[i]) {
            if (h->stage[i]) {
                CU_CHECK(h, d.cuCtxSynchronize_());
                d.cuMemFree_(h->stage[i]);
                h->stage[i] = 0;
                h->stage_bytes[i] = 0;
            }
            CUresult r = d.cuMemAlloc_(&h->stage[i], round_up(bytes[i], 256));
            if (r != CUDA_SUCCESS)
                return fail(h, SGEMM_ERR_CUDA, "cuMemAlloc of %zu staging bytes failed: %s", bytes[i], cu_text(r).c_str());
            h->stage_bytes[i] = round_up(bytes[i], 256);
        }
    }
    // Large problems are pipelined over column chunks on three streams — upload of B (and C) chunk j+1, GEMM of
    // chunk j and download of D chunk j-1 overlap — because the call is bound by the host link, not by the GPU.
    // Columns of D are independent and every chunk runs the same kernel in the same k order, so the result is
    // the one the single-launch path produces.
    const uint32_t chunk_unit = std::max<uint32_t>(h->tile_n, 256);
    // (a transposed B keeps a column chunk of op(B) scattered over all of its rows: no contiguous chunk to upload)
    if (h->pipeline_host && !h->cfg.trans_b && k > 0 && n >= 4 * chunk_unit && bytes[0] + bytes[1] + bytes[3] >= ((size_t)64 << 20)) {
        const uint32_t want = (uint32_t)h->pipeline_chunks;
        const uint32_t nc = (uint32_t)round_up((n + want - 1) / want, chunk_unit);
        const uint32_t chunks = (n + nc - 1) / nc;
        for (CUstream &st : h->pipe_streams)
            if (!st) CU_CHECK(h, d.cuStreamCreate_(&st, CU_STREAM_NON_BLOCKING));
        while (h->pipe_events.size() < 1 + 2 * (size_t)chunks) {
            CUevent e;
            CU_CHECK(h, d.cuEventCreate_(&e, CU_EVENT_DISABLE_TIMING));
            h->pipe_events.push_back(e);
        }
        CUstream s_in = h->pipe_streams[0], s_cmp = h->pipe_streams[1], s_out = h->pipe_streams[2];
        CUevent ev_a = h->pipe_events[0];
        // every chunk uses the kernel variant and the split-K factor the whole problem would get, so that each
        // element of D is summed in exactly the order of the single-launch path
        Plan whole;
        if ((rc = make_plan(h, reinterpret_cast<const void *>(h->stage[0]), reinterpret_cast<const void *>(h->stage[1]), m, n, k,
                            lda, ldb, &whole)))
            return rc;
        // Whatever happens inside the chunk loop — a failed copy, event or launch — the handle gets its options
        // back and all three streams are drained before this function returns: nothing of the call may still be
        // reading or writing the caller's host buffers afterwards.
        struct Restore {
            sgemm_handle *h;
            int64_t variant, split;
            CUstream streams[3];
            CUresult drained = CUDA_SUCCESS;
            bool done = false;
            void run() {
                if (done) return;
                done = true;
                for (CUstream st : streams) {
                    CUresult r = driver().cuStreamSynchronize_(st);
                    if (r != CUDA_SUCCESS && drained == CUDA_SUCCESS) drained = r;
                }
                h->force_variant = variant;
                h->split_k_opt = split;
                h->reuse_a_lo = false;
            }
            ~Restore() { run(); }
        } restore{h, h->force_variant, h->split_k_opt, {s_in, s_cmp, s_out}};
        h->force_variant = whole.variant != kVariantTensor ? 2 : ((whole.tk == &h->tk_skinny || whole.tk == &h->tk_thin) ? 3 : 1);
        h->split_k_opt = whole.split_k;
        if ((rc = upload_a(h, hA, bytes[0], a_inner, a_outer, lda, s_in, sharded))) return rc;
        CU_CHECK(h, d.cuEventRecord_(ev_a, s_in));
        CU_CHECK(h, d.cuStreamWaitEvent_(s_cmp, ev_a, 0));
        for (uint32_t j = 0; j < chunks; ++j) {
            const uint32_t n0 = j * nc, nw = std::min(nc, n - n0);
            CUevent ev_in = h->pipe_events[1 + 2 * j], ev_done = h->pipe_events[2 + 2 * j];
            const size_t off_b = (size_t)n0 * ldb * eb, off_c = (size_t)n0 * ldc * 4, off_d = (size_t)n0 * ldd * 4;
            const size_t by_b = ((size_t)ldb * (nw - 1) + k) * eb, by_c = ((size_t)ldc * (nw - 1) + m) * 4,
                         by_d = ((size_t)ldd * (nw - 1) + m) * 4;
            CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[1] + off_b, reinterpret_cast<const char *>(hB) + off_b, by_b, s_in));
            if (use_c)
                CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[2] + off_c, reinterpret_cast<const char *>(hC) + off_c, by_c, s_in));
            if (ldd != m)
                CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[3] + off_d, reinterpret_cast<const char *>(hD) + off_d, by_d, s_in));
            CU_CHECK(h, d.cuEventRecord_(ev_in, s_in));
            CU_CHECK(h, d.cuStreamWaitEvent_(s_cmp, ev_in, 0));
            h->reuse_a_lo = j > 0;
            rc = launch_device(h, reinterpret_cast<const float *>(h->stage[0]),
                               reinterpret_cast<const float *>(h->stage[1] + off_b),
                               use_c ? reinterpret_cast<const float *>(h->stage[2] + off_c) : nullptr,
                               reinterpret_cast<float *>(h->stage[3] + off_d), alpha, beta, m, nw, k, lda, ldb, ldc, ldd, s_cmp);
            h->reuse_a_lo = false;
            if (rc) return rc;
            CU_CHECK(h, d.cuEventRecord_(ev_done, s_cmp));
            CU_CHECK(h, d.cuStreamWaitEvent_(s_out, ev_done, 0));
            CU_CHECK(h, d.cuMemcpyDtoHAsync_(reinterpret_cast<char *>(hD) + off_d, h->stage[3] + off_d, by_d, s_out));
        }
        restore.run();
        if (restore.drained != CUDA_SUCCESS)
            return fail(h, SGEMM_ERR_CUDA, "pipelined host call failed: %s", cu_text(restore.drained).c_str());
        return SGEMM_OK;
    }
    CUstream s = nullptr;
    if ((rc = upload_a(h, hA, bytes[0], a_inner, a_outer, lda, s, sharded))) return rc;
    if (n == 0) {   // (sharded call of a rank without columns: it only takes part in the exchange of A)
        CU_CHECK(h, d.cuStreamSynchronize_(s));
        return SGEMM_OK;
    }
    if (bytes[1]) CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[1], hB, bytes[1], s));
    if (bytes[2]) CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[2], hC, bytes[2], s));
    if (ldd != m)  // keep the caller's padding rows of D: the kernel writes only rows < M of each column
        CU_CHECK(h, d.cuMemcpyHtoDAsync_(h->stage[3], hD, bytes[3], s));
    rc = launch_device(h, reinterpret_cast<const float *>(h->stage[0]), reinterpret_cast<const float *>(h->stage[1]),
                       use_c ? reinterpret_cast<const float *>(h->stage[2]) : nullptr,
                       reinterpret_cast<float *>(h->stage[3]), alpha, beta, m, n, k, lda, ldb, ldc, ldd, s);
    if (rc) return rc;
    CU_CHECK(h, d.cuMemcpyDtoHAsync_(hD, h->stage[3], bytes[3], s));
    CU_CHECK(h, d.cuStreamSynchronize_(s));
    return SGEMM_OK;
}

}  // namespace

SGEMM_API int sgemm_bench(sgemm_handle *h, const float *dA, const float *dB, const float *dC, float *dD, float alpha,
                          float beta, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb, uint32_t ldc,
                          uint32_t ldd, uint32_t warmup, uint32_t runs, void *stream, float *ms_mean) {
    if (!h || !ms_mean || runs == 0) return SGEMM_ERR_INVALID_ARGUMENT;
    CtxGuard guard(h);
    Driver &d = driver();
    CUstream s = (CUstream)stream;
    int rc;
    for (uint32_t i = 0; i < warmup; ++i)
        if ((rc = launch_device(h, dA, dB, dC, dD, alpha, beta, m, n, k, lda, ldb, ldc, ldd, s))) return rc;
    CU_CHECK(h, d.cuStreamSynchronize_(s));
    CUevent e0, e1;
    CU_CHECK(h, d.cuEventCreate_(&e0, CU_EVENT_DEFAULT));
    CU_CHECK(h, d.cuEventCreate_(&e1, CU_EVENT_DEFAULT));
    CU_CHECK(h, d.cuEventRecord_(e0, s));
    for (uint32_t i = 0; i < runs; ++i)
        if ((rc = launch_device(h, dA, dB, dC, dD, alpha, beta, m, n, k, lda, ldb, ldc, ldd, s))) return rc;
    CU_CHECK(h, d.cuEventRecord_(e1, s));
    CU_CHECK(h, d.cuEventSynchronize_(e1));
    float ms = 0.f;
    CU_CHECK(h, d.cuEventElapsedTime_(&ms, e0, e1));
    d.cuEventDestroy_(e0);
    d.cuEventDestroy_(e1);
    *ms_mean = ms / (float)runs;
    return SGEMM_OK;
}

SGEMM_API int sgemm_last_status(sgemm_handle *h, uint32_t status[8]) {
    if (!h || !status) return SGEMM_ERR_INVALID_ARGUMENT;
    CtxGuard guard(h);
    Driver &d = driver();
    CU_CHECK(h, d.cuCtxSynchronize_());
    CU_CHECK(h, d.cuMemcpyDtoH_(status, h->status, kStatusWords * 4));
    if (status[0] != 0) {
        CU_CHECK(h, d.cuMemsetD8_(h->status, 0, kStatusWords * 4));
        // a kernel that gave up may have left the alignment counter half-counted
        CU_CHECK(h, d.cuMemsetD8_(h->counters, 0, (size_t)kCounterWords * 4));
        h->wave_sync_base = 0;
        return fail(h, SGEMM_ERR_DEVICE_STATUS, "kernel gave up waiting: tag 0x%x tile %u k-block %u block %u parity %u",
                    status[1], status[2], status[3], status[4], status[5]);
    }
    return SGEMM_OK;
}

SGEMM_API int sgemm_wait_selftest(sgemm_handle *h, uint32_t timeout_ms, uint32_t tag) {
    if (!h || timeout_ms == 0 || timeout_ms > 1000) return SGEMM_ERR_INVALID_ARGUMENT;
    if (!h->fn_wait_selftest)
        return fail(h, SGEMM_ERR_UNSUPPORTED, "the loaded cubin has no kernel fed by TMA, hence no bounded waits to test");
    CtxGuard guard(h);
    uint32_t *status_ptr = reinterpret_cast<uint32_t *>(h->status);
    uint64_t timeout_ns = (uint64_t)timeout_ms * 1000000ull;
    void *params[] = {&status_ptr, &timeout_ns, &tag};
    return launch(h, h->fn_wait_selftest, 1, 1, 1, 64, 1, 0, nullptr, params);
}

SGEMM_API int sgemm_set_option(sgemm_handle *h, const char *key, int64_t value) {
    if (!h || !key) return SGEMM_ERR_INVALID_ARGUMENT;
    const std::string k(key);
    if (k == "force_variant" && value >= 0 && value <= 3) h->force_variant = value;
    else if (k == "skinny_below_intensity" && value >= 0) h->skinny_below_intensity = value;
    else if (k == "skinny_below_flops" && value >= 0) h->skinny_below_flops = value;
    else if (k == "repitch" && (value == 0 || value == 1)) h->repitch = value != 0;
    else if (k == "repitch_above_flops" && value >= 0) h->repitch_above_flops = value;
    else if (k == "split_k" && value >= 0 && value <= 1024) h->split_k_opt = value;
    else if (k == "simt_below_flops" && value >= 0) h->simt_below_flops = value;
    else if (k == "pdl" && (value == 0 || value == 1)) h->pdl = value != 0;
    else if (k == "pipeline_host" && (value == 0 || value == 1)) h->pipeline_host = value != 0;
    else if (k == "pipeline_chunks" && value >= 2 && value <= 64) h->pipeline_chunks = value;
    else if (k == "wave_sync" && (value == 0 || value == 1)) h->wave_sync = value != 0;
    else if (k == "profile" && (value == 0 || value == 1)) { h->profile = value != 0; h->prof_used = 0; }
    else if (k == "acc_chain" && value >= -1 && value <= (1 << 20)) h->acc_chain_opt = value;
    else return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "unknown option or value out of range: %s = %lld", key, (long long)value);
    return SGEMM_OK;
}

SGEMM_API int sgemm_get_info(sgemm_handle *h, const char *key, int64_t *value) {
    if (!h || !key || !value) return SGEMM_ERR_INVALID_ARGUMENT;
    const std::string k(key);
    if (k == "variant") *value = h->cfg.variant;
    else if (k == "last_variant") *value = h->last_variant;
    else if (k == "last_split_k") *value = h->last_split_k;
    else if (k == "last_acc_chain") *value = h->last_acc_chain;
    else if (k == "last_tile_n") *value = h->last_tile_n;
    else if (k == "last_feed_tma") *value = h->last_feed_tma;
    else if (k == "acc_chain") *value = h->tk_main.acc_chain;
    else if (k == "skinny_acc_chain") *value = h->tk_skinny.acc_chain;
    else if (k == "last_grid") *value = h->last_grid;
    else if (k == "launches") *value = h->launches;
    else if (k == "tile_m") *value = h->tile_m;
    else if (k == "tile_n") *value = h->tile_n;
    else if (k == "sm_count") *value = h->sm_count;
    else if (k == "comm_rank") *value = h->comm.comm ? h->comm.rank : -1;
    else if (k == "comm_world") *value = h->comm.comm ? h->comm.world : 0;
    else if (k == "workspace_bytes") *value = (int64_t)(h->ws_lent ? h->ws_lent_bytes : h->ws_owned_bytes);
    else if (k == "sm_khz_effective") {
        // SM clock the tensor-kernel launches since the last read really ran at: cycles / nanoseconds as counted by
        // block 0 of each launch (0: no such launch).  Synchronises; clears the two sums.
        CtxGuard guard(h);
        Driver &d = driver();
        uint64_t sums[2] = {0, 0};
        CU_CHECK(h, d.cuCtxSynchronize_());
        CU_CHECK(h, d.cuMemcpyDtoH_(sums, h->status + kStatusWords * 4, sizeof sums));
        CU_CHECK(h, d.cuMemsetD8_(h->status + kStatusWords * 4, 0, sizeof sums));
        *value = sums[1] ? (int64_t)((double)sums[0] / (double)sums[1] * 1e6) : 0;
    }
    else if (k == "profile_count") *value = (int64_t)h->prof_used;
    else if (k == "profile_main_ns") {  // total device time of the bracketed main-kernel launches; resets the tally
        CtxGuard guard(h);
        Driver &d = driver();
        double total_ms = 0.0;
        for (size_t i = 0; i < h->prof_used; ++i) {
            float ms = 0.f;
            CU_CHECK(h, d.cuEventSynchronize_(h->prof_events[i].second));
            CU_CHECK(h, d.cuEventElapsedTime_(&ms, h->prof_events[i].first, h->prof_events[i].second));
            total_ms += ms;
        }
        h->prof_used = 0;
        *value = (int64_t)(total_ms * 1e6);
    }
    else return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "unknown info key: %s", key);
    return SGEMM_OK;
}

SGEMM_API int sgemm_workspace_bytes_for(sgemm_handle *h, const void *dA, const void *dB, uint32_t m, uint32_t n,
                                        uint32_t k, uint32_t lda, uint32_t ldb, size_t *bytes) {
    if (!h || !bytes) return SGEMM_ERR_INVALID_ARGUMENT;
    *bytes = 0;
    if (m == 0 || n == 0 || k == 0) return SGEMM_OK;
    Plan p;
    int rc = make_plan(h, dA, dB, m, n, k, lda, ldb, &p);
    if (rc) return rc;
    *bytes = p.ws_bytes;
    return SGEMM_OK;
}

SGEMM_API int sgemm_workspace_bytes(sgemm_handle *h, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb,
                                    size_t *bytes) {
    // the operands' addresses are unknown here: NULL stands for bases that are 16-byte aligned (the common case)
    return sgemm_workspace_bytes_for(h, nullptr, nullptr, m, n, k, lda, ldb, bytes);
}

SGEMM_API int sgemm_set_workspace(sgemm_handle *h, void *dptr, size_t bytes) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    if (dptr && ((uintptr_t)dptr & 255)) return fail(h, SGEMM_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
    h->ws_lent = (CUdeviceptr)(uintptr_t)dptr;
    h->ws_lent_bytes = dptr ? bytes : 0;
    for (CachedMap &c : h->maps) c.valid = false;
    return SGEMM_OK;
}

SGEMM_API int sgemm_fill_uniform(sgemm_handle *h, float *dptr, uint64_t count, uint64_t first_index,
                                 uint64_t stream_id, void *stream) {
    if (!h || (!dptr && count)) return SGEMM_ERR_INVALID_ARGUMENT;
    if (count == 0) return SGEMM_OK;
    CtxGuard guard(h);
    void *params[] = {&dptr, &count, &first_index, &stream_id};
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((count + 255) / 256, (uint64_t)h->sm_count * 16);
    return launch(h, h->fn_fill, blocks, 1, 1, 256, 1, 0, (CUstream)stream, params);
}

SGEMM_API int sgemm_narrow16(sgemm_handle *h, const float *dsrc, void *ddst, uint64_t count, void *stream) {
    if (!h || ((!dsrc || !ddst) && count)) return SGEMM_ERR_INVALID_ARGUMENT;
    if (h->elem_bytes != 2)
        return fail(h, SGEMM_ERR_UNSUPPORTED, "sgemm_narrow16 converts to the operand type of a cubin for FP16 or BF16 operands; this one takes FP32");
    if (count == 0) return SGEMM_OK;
    CtxGuard guard(h);
    uint32_t kind = (uint32_t)h->cfg.a_type;   // 1 = FP16, 2 = BF16
    void *params[] = {&dsrc, &ddst, &count, &kind};
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((count + 255) / 256, (uint64_t)h->sm_count * 16);
    return launch(h, h->fn_narrow16, blocks, 1, 1, 256, 1, 0, (CUstream)stream, params);
}

SGEMM_API int sgemm_tile_map(sgemm_handle *h, int32_t *host_xy, uint32_t nx, uint32_t ny) {
    if (!h || !host_xy || nx == 0 || ny == 0 || (uint64_t)nx * ny > (1u << 24)) return SGEMM_ERR_INVALID_ARGUMENT;
    CtxGuard guard(h);
    Driver &d = driver();
    const size_t bytes = (size_t)nx * ny * 2 * sizeof(int32_t);
    CUdeviceptr buf = 0;
    CU_CHECK(h, d.cuMemAlloc_(&buf, bytes));
    int32_t *dp = reinterpret_cast<int32_t *>(buf);
    void *params[] = {&dp, &nx, &ny};
    int rc = launch(h, h->fn_tile_map, (nx * ny + 255) / 256, 1, 1, 256, 1, 0, nullptr, params);
    if (rc == SGEMM_OK) {
        CUresult r = d.cuMemcpyDtoH_(host_xy, buf, bytes);
        if (r != CUDA_SUCCESS) rc = fail(h, SGEMM_ERR_CUDA, "cuMemcpyDtoH -> %s", cu_text(r).c_str());
    }
    d.cuMemFree_(buf);
    return rc;
}

SGEMM_API int sgemm_dev_alloc(sgemm_handle *h, size_t bytes, void **dptr) {
    if (!h || !dptr) return SGEMM_ERR_INVALID_ARGUMENT;
    CtxGuard guard(h);
    CUdeviceptr p = 0;
    CU_CHECK(h, driver().cuMemAlloc_(&p, bytes ? bytes : 1));
    *dptr = reinterpret_cast<void *>(p);
    return SGEMM_OK;
}
SGEMM_API int sgemm_dev_free(sgemm_handle *h, void *dptr) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    if (!dptr) return SGEMM_OK;
    CtxGuard guard(h);
    CU_CHECK(h, driver().cuMemFree_((CUdeviceptr)(uintptr_t)dptr));
    return SGEMM_OK;
}
SGEMM_API int sgemm_dev_upload(sgemm_handle *h, void *dptr, const void *host, size_t bytes) {
    if (!h || ((!dptr || !host) && bytes)) return SGEMM_ERR_INVALID_ARGUMENT;
    if (!bytes) return SGEMM_OK;
    CtxGuard guard(h);
    CU_CHECK(h, driver().cuMemcpyHtoD_((CUdeviceptr)(uintptr_t)dptr, host, bytes));
    return SGEMM_OK;
}
SGEMM_API int sgemm_dev_download(sgemm_handle *h, void *host, const void *dptr, size_t bytes) {
    if (!h || ((!dptr || !host) && bytes)) return SGEMM_ERR_INVALID_ARGUMENT;
    if (!bytes) return SGEMM_OK;
    CtxGuard guard(h);
    CU_CHECK(h, driver().cuMemcpyDtoH_(host, (CUdeviceptr)(uintptr_t)dptr, bytes));
    return SGEMM_OK;
}
SGEMM_API int sgemm_dev_memset(sgemm_handle *h, void *dptr, int byte_value, size_t bytes) {
    if (!h || (!dptr && bytes)) return SGEMM_ERR_INVALID_ARGUMENT;
    if (!bytes) return SGEMM_OK;
    CtxGuard guard(h);
    CU_CHECK(h, driver().cuMemsetD8_((CUdeviceptr)(uintptr_t)dptr, (unsigned char)byte_value, bytes));
    return SGEMM_OK;
}
SGEMM_API int sgemm_dev_sync(sgemm_handle *h) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    CtxGuard guard(h);
    CU_CHECK(h, driver().cuCtxSynchronize_());
    return SGEMM_OK;
}

// ------------------------------------------------------------------ seam used by sgemm_noalloc.cu
namespace sgemm_internal {

int handle_device(const sgemm_handle *h) { return h ? h->device : -1; }

int set_error(sgemm_handle *h, int code, const char *message) { return fail(h, code, "%s", message); }

int scratch_bytes(sgemm_handle *h, const void *dA, const void *dB, uint32_t m, uint32_t n, uint32_t k, uint32_t lda,
                  uint32_t ldb, size_t *bytes) {
    return sgemm_workspace_bytes_for(h, dA, dB, m, n, k, lda, ldb, bytes);
}

int with_context(sgemm_handle *h, int (*fn)(void *), void *arg) {
    if (!h || !fn) return SGEMM_ERR_INVALID_ARGUMENT;
    CtxGuard guard(h);
    if (!guard.pushed) return fail(h, SGEMM_ERR_CUDA, "cannot make the handle's CUDA context current");
    return fn(arg);
}

void **noalloc_scratch_slot(sgemm_handle *h) { return h ? &h->noalloc_scratch : nullptr; }

CommState *comm_state(sgemm_handle *h) { return h ? &h->comm : nullptr; }

int launch_with_scratch(sgemm_handle *h, void *scratch, size_t scratch_bytes, const float *dA, const float *dB,
                        const float *dC, float *dD, float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                        uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, void *stream) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    // Borrow the lent-workspace slot for the duration of this call: with a lent block ensure_workspace never
    // allocates, it only checks the size.  Tensor maps that point into a workspace are re-encoded whenever
    // their base address changes, so switching blocks between calls is safe.
    const CUdeviceptr saved_ptr = h->ws_lent;
    const size_t saved_bytes = h->ws_lent_bytes;
    h->ws_lent = (CUdeviceptr)(uintptr_t)scratch;
    h->ws_lent_bytes = scratch_bytes;
    int rc;
    {
        CtxGuard guard(h);
        rc = launch_device(h, dA, dB, dC, dD, alpha, beta, m, n, k, lda, ldb, ldc, ldd, (CUstream)stream);
    }
    h->ws_lent = saved_ptr;
    h->ws_lent_bytes = saved_bytes;
    // the only workspace failure possible here is "the borrowed block is too small": say so in this entry point's terms
    if (rc == SGEMM_ERR_WORKSPACE) rc = SGEMM_ERR_SCRATCH_LIMIT;
    return rc;
}

}  // namespace sgemm_internal
