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
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, which also
//     makes the CUDA runtime load this library's device image on that GPU).  That one-time set-up is not a
//     cudaMalloc, but it is work the driver does outside any stream: make the first call on each device
//     before starting a stream capture.
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
constexpr int kMaxDevices = 64;

// The scratch itself.  On the host this name is only a handle for the runtime's symbol table, never an
// address a kernel could use; the device address is obtained below, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

std::mutex g_lock;
void *g_scratch_address[kMaxDevices] = {};

// Device address of g_noalloc_scratch on `device`, looked up on first use with that device current.
int scratch_address(sgemm_handle *h, int device, void **out) {
    std::lock_guard<std::mutex> guard(g_lock);
    if (device < 0 || device >= kMaxDevices)
        return sgemm_internal::set_error(h, SGEMM_ERR_INVALID_ARGUMENT, "device ordinal out of range for the static scratch table");
    if (!g_scratch_address[device]) {
        int previous = -1;
        cudaError_t e = cudaGetDevice(&previous);
        if (e == cudaSuccess) e = cudaSetDevice(device);
        void *ptr = nullptr;
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (previous >= 0 && previous != device) cudaSetDevice(previous);
        if (e != cudaSuccess || !ptr) {
            char msg[256];
            std::snprintf(msg, sizeof msg, "cudaGetSymbolAddress for the static scratch on device %d failed: %s", device,
                          cudaGetErrorString(e));
            return sgemm_internal::set_error(h, SGEMM_ERR_CUDA, msg);
        }
        g_scratch_address[device] = ptr;
    }
    *out = g_scratch_address[device];
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
    int rc = sgemm_internal::scratch_bytes(h, m, n, k, lda, ldb, &need);
    if (rc) return rc;
    if (need > kScratchBytes) {
        char msg[256];
        std::snprintf(msg, sizeof msg,
                      "problem %u x %u x %u needs %zu bytes of scratch, the allocation-free entry point has %zu "
                      "(use sgemm_launch, or lend a workspace with sgemm_set_workspace)", m, n, k, need, kScratchBytes);
        return sgemm_internal::set_error(h, SGEMM_ERR_SCRATCH_LIMIT, msg);
    }
    void *scratch = nullptr;
    rc = scratch_address(h, sgemm_internal::handle_device(h), &scratch);
    if (rc) return rc;
    return sgemm_internal::launch_with_scratch(h, scratch, kScratchBytes, dA, dB, dC, dD, alpha, beta, m, n, k, lda, ldb,
                                               ldc, ldd, stream);
}
