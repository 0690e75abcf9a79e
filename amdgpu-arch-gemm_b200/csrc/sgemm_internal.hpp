// Internal seam between the translation units of libsgemm_runner.so (not part of the C ABI).
#pragma once
#include "sgemm_runner.h"

#include <cstddef>
#include <cstdint>

namespace sgemm_internal {

// Device ordinal the handle was opened on.
int handle_device(const sgemm_handle *h);

// Record a failure message on the handle (what sgemm_last_error returns) and hand `code` back.
int set_error(sgemm_handle *h, int code, const char *message);

// Scratch bytes sgemm_launch would need for this problem under the handle's current options, planned for the
// operands the call will really get (a base TMA cannot read where it lies adds an aligned copy to the need).
int scratch_bytes(sgemm_handle *h, const void *dA, const void *dB, uint32_t m, uint32_t n, uint32_t k, uint32_t lda,
                  uint32_t ldb, size_t *bytes);

// Run `fn(arg)` with the handle's CUDA context current on this thread (pushed before, popped after), so that
// CUDA runtime calls made inside bind to the device the handle was opened on without cudaSetDevice.  Returns
// what `fn` returns, or SGEMM_ERR_CUDA when the context cannot be made current.
int with_context(sgemm_handle *h, int (*fn)(void *), void *arg);

// One pointer-sized slot per handle for sgemm_noalloc.cu: the device address of the library's static scratch
// array as resolved in the handle's context (NULL until the first allocation-free call on the handle).
void **noalloc_scratch_slot(sgemm_handle *h);

// The handle's communicator over the GPUs that share one sharded SGEMM (sgemm_multi.cpp owns the NCCL side):
// `comm` is an ncclComm_t, NULL until sgemm_comm_init / sgemm_comm_init_all.
struct CommState {
    void *comm = nullptr;
    int rank = 0;
    int world = 1;
};
CommState *comm_state(sgemm_handle *h);

// In-place exchange over the handle's communicator, ordered on `stream`: piece r — `bytes[r]` bytes at
// `base + offsets[r]` on every rank, valid on rank r — is copied to the same place on all other ranks.  Equal,
// back-to-back pieces go as one all-gather, ragged ones as grouped broadcasts.
int comm_complete(sgemm_handle *h, void *base, const size_t *offsets, const size_t *bytes, void *stream);

// Destroy an ncclComm_t stored in a CommState (no-op for NULL or without NCCL).
void comm_release(void *comm);

// sgemm_launch with the scratch taken from [scratch, scratch + scratch_bytes) for this one call only; the
// handle's own workspace settings are put back before returning.  Never allocates device memory; a need beyond
// `scratch_bytes` comes back as SGEMM_ERR_SCRATCH_LIMIT.
int launch_with_scratch(sgemm_handle *h, void *scratch, size_t scratch_bytes, const float *dA, const float *dB,
                        const float *dC, float *dD, float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                        uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, void *stream);

}  // namespace sgemm_internal
