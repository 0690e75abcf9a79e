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

// Scratch bytes sgemm_launch would need for this problem under the handle's current options.
int scratch_bytes(sgemm_handle *h, uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb, size_t *bytes);

// sgemm_launch with the scratch taken from [scratch, scratch + scratch_bytes) for this one call only; the
// handle's own workspace settings are put back before returning.  Never allocates device memory.
int launch_with_scratch(sgemm_handle *h, void *scratch, size_t scratch_bytes, const float *dA, const float *dB,
                        const float *dC, float *dD, float alpha, float beta, uint32_t m, uint32_t n, uint32_t k,
                        uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd, void *stream);

}  // namespace sgemm_internal
