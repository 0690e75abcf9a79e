// Multi-GPU part of libsgemm_runner.so: column shards of one SGEMM over the GPUs of a box, and the two places
// where the shards exchange data over NVLink — completing the replicated A from per-rank slices on the host-buffer
// path, and the optional all-gather of D's column shards.  The reference is single-GPU (its runner never selects a
// device, runner/generator_runner.cpp:192-324), so nothing here has a counterpart there.
//
// NCCL is bound at run time (dlopen of libnccl.so.2) like the CUDA driver: the library loads, and everything
// single-GPU works, on a machine without NCCL; the entry points below then fail with SGEMM_ERR_COMM.  Every
// ncclResult_t is checked and turned into that code with NCCL's own message.  Only NCCL's collectives touch peer
// memory: no kernel of this library and no TMA descriptor ever covers another GPU's memory.
#include "sgemm_internal.hpp"

#include <nccl.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#define SGEMM_API extern "C" __attribute__((visibility("default")))

namespace {

#define NCCL_FUNCTIONS(X)                                                                               \
    X(ncclGetUniqueId) X(ncclCommInitRank) X(ncclCommDestroy) X(ncclGetErrorString) X(ncclBroadcast)     \
    X(ncclAllGather) X(ncclGroupStart) X(ncclGroupEnd)

struct Nccl {
#define DECL(name) decltype(&name) name##_ = nullptr;
    NCCL_FUNCTIONS(DECL)
#undef DECL
    bool ok = false;
    std::string error;
};

Nccl &nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        // SGEMM_NCCL_LIBRARY names another library file (or, in tests, one that does not exist)
        const char *wanted = std::getenv("SGEMM_NCCL_LIBRARY");
        void *lib = dlopen(wanted && *wanted ? wanted : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib && !(wanted && *wanted)) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) {
            const char *why = dlerror();
            n.error = std::string("cannot load NCCL: ") + (why ? why : "libnccl.so.2 not found");
            return;
        }
#define LOAD(name)                                                                 \
        n.name##_ = reinterpret_cast<decltype(&name)>(dlsym(lib, #name));          \
        if (!n.name##_) { n.error = std::string("NCCL lacks ") + #name; return; }
        NCCL_FUNCTIONS(LOAD)
#undef LOAD
        n.ok = true;
    });
    return n;
}

int comm_fail(sgemm_handle *h, const char *what, ncclResult_t r) {
    char msg[384];
    std::snprintf(msg, sizeof msg, "%s -> NCCL error %d: %s", what, (int)r, nccl().ok ? nccl().ncclGetErrorString_(r) : "?");
    return sgemm_internal::set_error(h, SGEMM_ERR_COMM, msg);
}

#define NCCL_CHECK(h, call)                                      \
    do {                                                         \
        ncclResult_t _r = (call);                                \
        if (_r != ncclSuccess) return comm_fail(h, #call, _r);   \
    } while (0)

int need_nccl(sgemm_handle *h) {
    Nccl &n = nccl();
    if (!n.ok) return sgemm_internal::set_error(h, SGEMM_ERR_COMM, n.error.c_str());
    return SGEMM_OK;
}

// the rule of runner/shard.py: whole tiles of tile_n columns, as even as possible, earlier ranks take the extra tile
void shard_of(uint32_t n, uint32_t world, uint32_t rank, uint32_t tile_n, uint32_t *n0, uint32_t *n1) {
    const uint64_t tiles = ((uint64_t)n + tile_n - 1) / tile_n;
    const uint64_t base = tiles / world, extra = tiles % world;
    const uint64_t t0 = (uint64_t)rank * base + std::min<uint64_t>(rank, extra);
    const uint64_t t1 = t0 + base + (rank < extra ? 1 : 0);
    *n0 = (uint32_t)std::min<uint64_t>(t0 * tile_n, n);
    *n1 = (uint32_t)std::min<uint64_t>(t1 * tile_n, n);
}

struct InitArgs {
    sgemm_handle *h;
    ncclUniqueId id;
    int rank, world;
    ncclComm_t comm;
};

int init_rank(void *p) {   // runs with the handle's context current: NCCL binds the communicator to that device
    InitArgs *a = static_cast<InitArgs *>(p);
    NCCL_CHECK(a->h, nccl().ncclCommInitRank_(&a->comm, a->world, a->id, a->rank));
    return SGEMM_OK;
}

struct PieceArgs {
    sgemm_handle *h;
    ncclComm_t comm;
    int world;
    char *base;
    const size_t *offsets, *bytes;
    cudaStream_t stream;
};

int broadcast_pieces(void *p) {
    PieceArgs *a = static_cast<PieceArgs *>(p);
    Nccl &n = nccl();
    bool equal = true;
    for (int r = 0; r < a->world; ++r)
        equal = equal && a->bytes[r] == a->bytes[0] && a->offsets[r] == (size_t)r * a->bytes[0];
    if (equal && a->bytes[0] > 0) {
        // equal, back-to-back pieces: one in-place all-gather (piece r already lies at its place on rank r)
        const int me = sgemm_internal::comm_state(a->h)->rank;
        NCCL_CHECK(a->h, n.ncclAllGather_(a->base + a->offsets[me], a->base, a->bytes[0], ncclChar, a->comm, a->stream));
        return SGEMM_OK;
    }
    // ragged pieces: one in-place broadcast per piece, grouped into a single NCCL launch
    NCCL_CHECK(a->h, n.ncclGroupStart_());
    for (int r = 0; r < a->world; ++r) {
        if (!a->bytes[r]) continue;
        ncclResult_t res = n.ncclBroadcast_(a->base + a->offsets[r], a->base + a->offsets[r], a->bytes[r], ncclChar, r, a->comm, a->stream);
        if (res != ncclSuccess) {
            n.ncclGroupEnd_();
            return comm_fail(a->h, "ncclBroadcast", res);
        }
    }
    NCCL_CHECK(a->h, n.ncclGroupEnd_());
    return SGEMM_OK;
}

}  // namespace

namespace sgemm_internal {

int comm_complete(sgemm_handle *h, void *base, const size_t *offsets, const size_t *bytes, void *stream) {
    CommState *cs = comm_state(h);
    if (!cs || !cs->comm) return set_error(h, SGEMM_ERR_COMM, "no communicator on this handle: call sgemm_comm_init first");
    int rc = need_nccl(h);
    if (rc) return rc;
    PieceArgs a{h, static_cast<ncclComm_t>(cs->comm), cs->world, static_cast<char *>(base), offsets, bytes,
                static_cast<cudaStream_t>(stream)};
    return with_context(h, broadcast_pieces, &a);
}

void comm_release(void *comm) {
    if (comm && nccl().ok) nccl().ncclCommDestroy_(static_cast<ncclComm_t>(comm));
}

}  // namespace sgemm_internal

SGEMM_API int sgemm_shard_columns(uint32_t n, uint32_t world, uint32_t rank, uint32_t tile_n, uint32_t *n0, uint32_t *n1) {
    if (!n0 || !n1 || world == 0 || rank >= world || tile_n == 0) return SGEMM_ERR_INVALID_ARGUMENT;
    shard_of(n, world, rank, tile_n, n0, n1);
    return SGEMM_OK;
}

SGEMM_API int sgemm_comm_unique_id(uint8_t id[SGEMM_COMM_ID_BYTES]) {
    static_assert(SGEMM_COMM_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "the id is passed through as NCCL made it");
    if (!id) return SGEMM_ERR_INVALID_ARGUMENT;
    int rc = need_nccl(nullptr);
    if (rc) return rc;
    ncclUniqueId u;
    NCCL_CHECK(nullptr, nccl().ncclGetUniqueId_(&u));
    std::memcpy(id, u.internal, SGEMM_COMM_ID_BYTES);
    return SGEMM_OK;
}

SGEMM_API int sgemm_comm_init(sgemm_handle *h, const uint8_t id[SGEMM_COMM_ID_BYTES], int rank, int world) {
    if (!h || !id || world < 1 || rank < 0 || rank >= world) return SGEMM_ERR_INVALID_ARGUMENT;
    sgemm_internal::CommState *cs = sgemm_internal::comm_state(h);
    if (cs->comm) return sgemm_internal::set_error(h, SGEMM_ERR_INVALID_ARGUMENT, "the handle already has a communicator");
    int rc = need_nccl(h);
    if (rc) return rc;
    InitArgs a{h, {}, rank, world, nullptr};
    std::memcpy(a.id.internal, id, SGEMM_COMM_ID_BYTES);
    rc = sgemm_internal::with_context(h, init_rank, &a);
    if (rc) return rc;
    cs->comm = a.comm;
    cs->rank = rank;
    cs->world = world;
    return SGEMM_OK;
}

SGEMM_API int sgemm_comm_init_all(sgemm_handle *const *handles, int count) {
    if (!handles || count < 1) return SGEMM_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < count; ++i) {
        if (!handles[i]) return SGEMM_ERR_INVALID_ARGUMENT;
        if (sgemm_internal::comm_state(handles[i])->comm)
            return sgemm_internal::set_error(handles[i], SGEMM_ERR_INVALID_ARGUMENT, "the handle already has a communicator");
        for (int j = 0; j < i; ++j)
            if (sgemm_internal::handle_device(handles[i]) == sgemm_internal::handle_device(handles[j]))
                return sgemm_internal::set_error(handles[i], SGEMM_ERR_INVALID_ARGUMENT, "two handles of one communicator share a device");
    }
    int rc = need_nccl(handles[0]);
    if (rc) return rc;
    Nccl &n = nccl();
    ncclUniqueId u;
    NCCL_CHECK(handles[0], n.ncclGetUniqueId_(&u));
    // one thread makes all ranks: the per-rank initialisations must be grouped or they would wait for each other
    std::vector<InitArgs> args((size_t)count);
    NCCL_CHECK(handles[0], n.ncclGroupStart_());
    rc = SGEMM_OK;
    for (int i = 0; i < count && rc == SGEMM_OK; ++i) {
        args[i] = InitArgs{handles[i], u, i, count, nullptr};
        rc = sgemm_internal::with_context(handles[i], init_rank, &args[i]);
    }
    ncclResult_t end = n.ncclGroupEnd_();
    if (rc == SGEMM_OK && end != ncclSuccess) rc = comm_fail(handles[0], "ncclGroupEnd (communicator set-up)", end);
    if (rc) {
        for (InitArgs &a : args)
            if (a.comm) n.ncclCommDestroy_(a.comm);
        return rc;
    }
    for (int i = 0; i < count; ++i) {
        sgemm_internal::CommState *cs = sgemm_internal::comm_state(handles[i]);
        cs->comm = args[i].comm;
        cs->rank = i;
        cs->world = count;
    }
    return SGEMM_OK;
}

SGEMM_API int sgemm_comm_destroy(sgemm_handle *h) {
    if (!h) return SGEMM_ERR_INVALID_ARGUMENT;
    sgemm_internal::CommState *cs = sgemm_internal::comm_state(h);
    if (cs->comm) sgemm_internal::comm_release(cs->comm);
    cs->comm = nullptr;
    cs->rank = 0;
    cs->world = 1;
    return SGEMM_OK;
}

SGEMM_API int sgemm_allgather_columns(sgemm_handle *h, float *dD_full, uint32_t m, uint32_t n, uint32_t ldd,
                                      uint32_t tile_n, void *stream) {
    if (!h || !dD_full || ldd < std::max(m, 1u) || tile_n == 0) return SGEMM_ERR_INVALID_ARGUMENT;
    sgemm_internal::CommState *cs = sgemm_internal::comm_state(h);
    if (!cs->comm) return sgemm_internal::set_error(h, SGEMM_ERR_COMM, "no communicator on this handle: call sgemm_comm_init first");
    if (m == 0 || n == 0) return SGEMM_OK;
    std::vector<size_t> offsets((size_t)cs->world), bytes((size_t)cs->world);
    for (int r = 0; r < cs->world; ++r) {
        uint32_t n0, n1;
        shard_of(n, (uint32_t)cs->world, (uint32_t)r, tile_n, &n0, &n1);
        offsets[r] = (size_t)n0 * ldd * 4;
        // whole columns of pitch ldd, except that the matrix ends with the last element of its last column
        bytes[r] = n1 > n0 ? ((size_t)(n1 - n0 - 1) * ldd + (n1 == n ? m : ldd)) * 4 : 0;
    }
    return sgemm_internal::comm_complete(h, dD_full, offsets.data(), bytes.data(), stream);
}
