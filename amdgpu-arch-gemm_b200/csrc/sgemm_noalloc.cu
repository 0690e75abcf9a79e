// sgemm_launch_noalloc — SGEMM for callers that must not allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits — a latency-critical serving loop whose
// device-memory budget was fixed at start-up (an allocation there can fail, and it synchronises the
// device), a real-time path that cannot afford a driver call that blocks, or a process whose device memory
// is owned by another allocator (a framework's caching allocator, a memory pool with a hard cap), where a
// library quietly taking more memory would break the owner's accounting.  The
// ordinary sgemm_launch grows a handle-owned workspace with cuMemAlloc when a problem needs more scratch
// than it has; this entry point never does.  Its scratch — the 3xTF32 "lo" copies of A and B and the
// split-K partial products — lives in one fixed array in device memory that is part of this library's
// image: SGEMM_NOALLOC_SCRATCH_BYTES (32 MiB) on every GPU that loads the library, held until the
// process exits.  Problems whose scratch does not fit are refused with SGEMM_ERR_SCRATCH_LIMIT.
//
// What to know before using it:
//   * The first call on a handle looks up the array's device address (cudaGetSymbolAddress, made with the
//     handle's own context current; on the first handle of a device it also makes the CUDA runtime load
//     this library's device image on that GPU).  That one-time set-up is not a cudaMalloc, but it is work
//     the driver does outside any stream: make the first call on each handle before starting a stream
//     capture.  The thread's current device and context are left as they were.
//   * All calls on a device share the one array, and it keeps whatever the previous call left in it.
//     Nothing in it has to start from zero — every call first overwrites each byte it later reads — but
//     two calls whose kernels overlap in time on the same GPU (different streams, different handles,
//     different threads) would overwrite each other's scratch.  Order such calls on one stream, or use
//     sgemm_launch with separately lent workspaces for concurrent work.
//   * A, B, C and D are still the caller's buffers, as in sgemm_launch.
#include "sgemm_internal.hpp"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#define SGEMM_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t kScratchBytes = SGEMM_NOALLOC_SCRATCH_BYTES;

// The scratch itself.  On the host this name is only a handle for the runtime's symbol table, never an
// address a kernel could use; the device address is obtained below, once per handle, in the handle's context.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct Lookup {
    void *address = nullptr;
    cudaError_t error = cudaSuccess;
};

// Runs with the handle's context current (sgemm_internal::with_context): the runtime binds to whatever context
// is current on the thread, so no cudaSetDevice is needed — and none is made, because a caller that only uses
// this C ABI has no "current runtime device", and switching to one (and back to ordinal 0) would create a
// primary context on GPU 0 in every process of a multi-GPU job.
int lookup_scratch(void *arg) {
    Lookup *out = static_cast<Lookup *>(arg);
    out->error = cudaGetSymbolAddress(&out->address, g_noalloc_scratch);
    return SGEMM_OK;
}

std::mutex g_lock;   // serialises first calls; the cached address itself lives in the handle

// Device address of g_noalloc_scratch for the device (and context) of `h`, looked up on the handle's first
// allocation-free call.  The handle keeps its context alive, so the address stays valid as long as the handle.
int scratch_address(sgemm_handle *h, void **out) {
    void **slot = sgemm_internal::noalloc_scratch_slot(h);
    std::lock_guard<std::mutex> guard(g_lock);
    if (!*slot) {
        Lookup found;
        int rc = sgemm_internal::with_context(h, lookup_scratch, &found);
        if (rc) return rc;
        if (found.error != cudaSuccess || !found.address) {
            char msg[256];
            std::snprintf(msg, sizeof msg, "cudaGetSymbolAddress for the static scratch on device %d failed: %s",
                          sgemm_internal::handle_device(h), cudaGetErrorString(found.error));
            return sgemm_internal::set_error(h, SGEMM_ERR_CUDA, msg);
        }
        *slot = found.address;
    }
    *out = *slot;
    return SGEMM_OK;
}

}  // namespace

SGEMM_API size_t sgemm_noalloc_scratch_bytes(void) { return kScratchBytes; }

SGEMM_API int sgemm_launch_noalloc(sgemm_handle *h, const float *dA, const float *dB, const float *dC, float *dD,
                                   float alpha, float beta, uint32_t m, uint32_t n, uint32_t k, uint32_t lda,
                                   uint32_t ldb, uint32_t ldc, uint32_t ldd, void *stream) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    // size check first: nothing is touched on the device when the problem does not fit
    size_t need = 0;
    // (planned for the real operands: an unaligned base or an odd leading dimension adds an aligned copy to the need)
    int rc = sgemm_internal::scratch_bytes(h, dA, dB, m, n, k, lda, ldb, &need);
    if (rc) return rc;
    if (need > kScratchBytes) {
        char msg[256];
        std::snprintf(msg, sizeof msg,
                      "problem %u x %u x %u needs %zu bytes of scratch, the allocation-free entry point has %zu "
                      "(use sgemm_launch, or lend a workspace with sgemm_set_workspace)", m, n, k, need, kScratchBytes);
        return sgemm_internal::set_error(h, SGEMM_ERR_SCRATCH_LIMIT, msg);
    }
    void *scratch = nullptr;
    rc = scratch_address(h, &scratch);
    if (rc) return rc;
    return sgemm_internal::launch_with_scratch(h, scratch, kScratchBytes, dA, dB, dC, dD, alpha, beta, m, n, k, lda, ldb,
                                               ldc, ldd, stream);
}
