// GeneratorRunner <cubin> <toml> M N K warmup runs validate
//
// The reference's runner program (runner/generator_runner.cpp:192-324) rebuilt on the C ABI of
// libsgemm_runner.so: same eight positional arguments, same stdout blocks in the same order (the tuner
// reads the third line from the end, tuner/sgemm_tuner.py:115), exit status 0 or 255 on mismatches.
// Deliberate differences: arguments are checked before anything is opened, every CUDA error ends the run
// with a message and a non-zero status, inputs are seeded (SGEMM_SEED, default 0) instead of drawn from
// std::random_device, beta comes from SGEMM_BETA (default 1, the reference's hard-coded value), and the
// time of the single CPU validation run is reported as measured rather than divided by `runs`.  Cubins for FP16 or
// BF16 operands (an addition; the reference is FP32 only) are driven too: A and B are drawn in FP32, converted on
// the device, the CPU check runs on the converted values and the SIMT block is printed with zeros.
//
// Extra diagnostics go to stderr so the stdout contract stays intact; with SGEMM_JSON=<path> the measured block is
// also written to that file as one JSON object (shape, variant, split-K, ms, TFLOP/s, GiB/s figure, mismatches).
//
// Several GPUs (an addition; the reference never selects a device): SGEMM_NGPUS=g runs the M x N x K problem
// column-sharded over GPUs SGEMM_DEVICE .. SGEMM_DEVICE+g-1 of this box in this one process — one handle per GPU,
// A replicated, B, C and D column blocks cut by sgemm_shard_columns, every GPU timed by its own host thread with its
// own events, no collective on the compute path.  stdout keeps its shape with the aggregate figures (time = the
// slowest GPU's); stderr and the JSON add the per-GPU figures.  SGEMM_ALLGATHER=1 computes every shard in place in
// a full-size D on each GPU and afterwards all-gathers D over NVLink (NCCL, in place), timed and reported apart
// from the GEMM; validation then checks the gathered D of the last GPU.
#include "sgemm_runner.h"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <thread>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// CPU validation GEMM with the arithmetic of the reference's cpuGemm (runner/generator_runner.cpp:16-33):
// per element a k-ascending sum of separate multiply and add, then beta*c + alpha*acc.  Columns are spread
// over the host threads; the order of operations inside one element is unchanged.
void cpu_gemm(const float *a, const float *b, const float *c, float *d, float alpha, float beta, uint32_t m,
              uint32_t n, uint32_t k) {
#pragma omp parallel
    {
        std::vector<float> acc(m);
#pragma omp for schedule(dynamic, 4)
        for (int64_t j = 0; j < (int64_t)n; ++j) {
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (uint32_t l = 0; l < k; ++l) {
                const float bv = b[l + (size_t)j * k];
                const float *col = a + (size_t)l * m;
                for (uint32_t i = 0; i < m; ++i) acc[i] += col[i] * bv;
            }
            for (uint32_t i = 0; i < m; ++i) d[i + (size_t)j * m] = beta * c[i + (size_t)j * m] + alpha * acc[i];
        }
    }
}

double gflops(uint32_t m, uint32_t n, uint32_t k, float ms) { return 2.0 * m * n * k / ms * 1e-6; }  // :75-77
float mem_bw(size_t m, size_t n, size_t k, float ms) {                                              // :79-83
    return (m * k + n * k + 2 * m * n) * sizeof(float) / ms / 1024.f / 1024.f;
}

// FP16 (type 1) or BF16 (type 2) word -> FP32
float widen16(uint16_t w, int type) {
    uint32_t bits;
    if (type == 2) {
        bits = (uint32_t)w << 16;
    } else {
        const uint32_t sign = (uint32_t)(w & 0x8000u) << 16, exp = (w >> 10) & 0x1Fu, man = w & 0x3FFu;
        if (exp == 0) {
            if (man == 0) {
                bits = sign;
            } else {   // subnormal half: renormalise
                int e = -1;
                uint32_t mm = man;
                do { ++e; mm <<= 1; } while (!(mm & 0x400u));
                bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mm & 0x3FFu) << 13);
            }
        } else if (exp == 31) {
            bits = sign | 0x7F800000u | (man << 13);
        } else {
            bits = sign | ((exp + 112u) << 23) | (man << 13);
        }
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// One GPU's part of the problem: its handle, its column range and its device buffers.
struct Rank {
    sgemm_handle *h = nullptr;
    uint32_t n0 = 0, n1 = 0;
    void *da = nullptr, *db = nullptr, *dc = nullptr, *dd = nullptr;   // dd: the shard, or the full D with SGEMM_ALLGATHER
    void *da16 = nullptr, *db16 = nullptr;
    float ms = 0.f;
    double sm_mhz = 0.0;   // SM clock the measured tensor-kernel launches ran at, counted on the device (0: no such launch)
    int rc = 0;
    uint32_t width() const { return n1 - n0; }
};

std::vector<Rank> g_ranks;

int die(sgemm_handle *h, const char *what, int rc) {
    std::fprintf(stderr, "GeneratorRunner: %s failed: %s (%d): %s\n", what, sgemm_strerror(rc), rc, sgemm_last_error(h));
    for (Rank &r : g_ranks)
        if (r.h) sgemm_close(r.h);   // frees the module and the handle's own memory; the process exits right after
    g_ranks.clear();
    // distinct exit codes: 2 = set-up or CUDA failure, 3 = multi-GPU request that cannot be served, 4 = NCCL
    return rc == SGEMM_ERR_COMM ? 4 : 2;
}

// Run `work(rank)` for every GPU at the same time, one host thread per GPU; returns the first non-zero status.
template <class F>
int on_all_gpus(F work) {
    std::vector<std::thread> threads;
    for (Rank &r : g_ranks) threads.emplace_back([&r, &work] { r.rc = work(r); });
    for (std::thread &t : threads) t.join();
    for (Rank &r : g_ranks)
        if (r.rc) return r.rc;
    return 0;
}

}  // namespace

int main(int argc, char **argv) {
    if (argc <= 8) {
        std::fprintf(stderr, "usage: %s <cubin> <toml> M N K warmup runs validate\n", argv[0]);
        return -1;
    }
    const uint32_t m = (uint32_t)std::atoll(argv[3]), n = (uint32_t)std::atoll(argv[4]), k = (uint32_t)std::atoll(argv[5]);
    const uint32_t warmup = (uint32_t)std::atoi(argv[6]), runs = (uint32_t)std::atoi(argv[7]);
    const bool validate = std::atoi(argv[8]) != 0;
    if (!m || !n || !k || !runs) {
        std::fprintf(stderr, "GeneratorRunner: M, N, K and runs must be positive\n");
        return -1;
    }
    const char *env = std::getenv("SGEMM_SEED");
    const uint64_t seed = env ? std::strtoull(env, nullptr, 10) : 0;
    env = std::getenv("SGEMM_BETA");
    const float alpha = 1.0f, beta = env ? std::strtof(env, nullptr) : 1.0f;
    env = std::getenv("SGEMM_DEVICE");
    const int device = env ? std::atoi(env) : 0;
    env = std::getenv("SGEMM_NGPUS");
    const int ngpus = env ? std::atoi(env) : 1;
    env = std::getenv("SGEMM_ALLGATHER");
    const bool allgather = env && std::atoi(env) != 0;
    if (ngpus < 1 || device < 0) {
        std::fprintf(stderr, "GeneratorRunner: SGEMM_NGPUS must be at least 1 and SGEMM_DEVICE non-negative\n");
        return 3;
    }

    // kernels for FP16 / BF16 operands (a_type 1 / 2 in the TOML; the reference has FP32 only): A and B are drawn in
    // FP32 like everything else here and converted on the device; the CPU check runs on the converted values
    sgemm_config parsed;
    const bool half = sgemm_config_parse(argv[2], &parsed) == 0 && parsed.a_type != 0;
    if (half && (parsed.trans_a || parsed.trans_b)) {
        std::fprintf(stderr, "GeneratorRunner: %s describes a 16-bit kernel for transposed operands; this program drives the NN layout\n", argv[2]);
        return 2;
    }
    if (ngpus > 1 || allgather) {
        const int visible = sgemm_device_count();
        if (device + ngpus > visible) {
            std::fprintf(stderr, "GeneratorRunner: SGEMM_NGPUS=%d from device %d asks for more GPUs than the %d visible\n",
                         ngpus, device, visible);
            return 3;
        }
    }
    int rc = 0;
    g_ranks.resize((size_t)ngpus);
    for (int i = 0; i < ngpus; ++i)
        if ((rc = sgemm_open(argv[1], argv[2], device + i, &g_ranks[i].h))) return die(nullptr, "sgemm_open", rc);
    sgemm_handle *h = g_ranks[0].h;
    int64_t tile_n = 1;
    sgemm_get_info(h, "tile_n", &tile_n);
    for (int i = 0; i < ngpus; ++i)
        sgemm_shard_columns(n, (uint32_t)ngpus, (uint32_t)i, (uint32_t)tile_n, &g_ranks[i].n0, &g_ranks[i].n1);
    if (allgather) {
        std::vector<sgemm_handle *> handles;
        for (Rank &r : g_ranks) handles.push_back(r.h);
        if ((rc = sgemm_comm_init_all(handles.data(), ngpus))) return die(h, "communicator set-up", rc);
    }

    const size_t na = (size_t)m * k, nb = (size_t)k * n, nc = (size_t)m * n;
    // A, B, C ~ U[-1, 1): streams seed, seed+1, seed+2 of the index-hash generator, filled on the device; every GPU
    // holds all of A and the columns [n0, n1) of B and C, filled by GLOBAL element index (column j of B starts at j*K)
    rc = on_all_gpus([&](Rank &r) -> int {
        const size_t w = r.width();
        int e;
        if ((e = sgemm_dev_alloc(r.h, na * 4, &r.da)) || (e = sgemm_dev_alloc(r.h, std::max<size_t>(w * k, 1) * 4, &r.db)) ||
            (e = sgemm_dev_alloc(r.h, std::max<size_t>(w * m, 1) * 4, &r.dc)) ||
            (e = sgemm_dev_alloc(r.h, (allgather ? nc : std::max<size_t>(w * m, 1)) * 4, &r.dd)))
            return e;
        if ((e = sgemm_fill_uniform(r.h, (float *)r.da, na, 0, seed, nullptr)) ||
            (e = sgemm_fill_uniform(r.h, (float *)r.db, w * k, (uint64_t)r.n0 * k, seed + 1, nullptr)) ||
            (e = sgemm_fill_uniform(r.h, (float *)r.dc, w * m, (uint64_t)r.n0 * m, seed + 2, nullptr)) || (e = sgemm_dev_sync(r.h)))
            return e;
        if (half) {
            if ((e = sgemm_dev_alloc(r.h, na * 2, &r.da16)) || (e = sgemm_dev_alloc(r.h, std::max<size_t>(w * k, 1) * 2, &r.db16)))
                return e;
            if ((e = sgemm_narrow16(r.h, (const float *)r.da, r.da16, na, nullptr)) ||
                (e = sgemm_narrow16(r.h, (const float *)r.db, r.db16, w * k, nullptr)) || (e = sgemm_dev_sync(r.h)))
                return e;
        }
        return 0;
    });
    if (rc) return die(h, "device allocation and input fill", rc);

    std::vector<float> cpu_d;
    if (validate) {
        std::vector<float> ha(na), hb(nb), hc(nc);
        cpu_d.resize(nc);
        if (half) {   // the values the kernel multiplies: the 16-bit words, widened
            std::vector<uint16_t> wa(na), wb(nb);
            if ((rc = sgemm_dev_download(h, wa.data(), g_ranks[0].da16, na * 2))) return die(h, "input download", rc);
            for (Rank &r : g_ranks)
                if (r.width() && (rc = sgemm_dev_download(r.h, wb.data() + (size_t)r.n0 * k, r.db16, (size_t)r.width() * k * 2)))
                    return die(r.h, "input download", rc);
            for (size_t i = 0; i < na; ++i) ha[i] = widen16(wa[i], parsed.a_type);
            for (size_t i = 0; i < nb; ++i) hb[i] = widen16(wb[i], parsed.a_type);
        } else {
            if ((rc = sgemm_dev_download(h, ha.data(), g_ranks[0].da, na * 4))) return die(h, "input download", rc);
            for (Rank &r : g_ranks)
                if (r.width() && (rc = sgemm_dev_download(r.h, hb.data() + (size_t)r.n0 * k, r.db, (size_t)r.width() * k * 4)))
                    return die(r.h, "input download", rc);
        }
        for (Rank &r : g_ranks)
            if (r.width() && (rc = sgemm_dev_download(r.h, hc.data() + (size_t)r.n0 * m, r.dc, (size_t)r.width() * m * 4)))
                return die(r.h, "input download", rc);
        const auto t0 = std::chrono::steady_clock::now();
        cpu_gemm(ha.data(), hb.data(), hc.data(), cpu_d.data(), alpha, beta, m, n, k);
        const auto t1 = std::chrono::steady_clock::now();
        int threads = 1;
#ifdef _OPENMP
        threads = omp_get_max_threads();
#endif
        std::cout << "cpuGemm func: " << std::chrono::duration<float, std::milli>(t1 - t0).count() << " ms\n";
        std::fprintf(stderr, "cpuGemm ran on %d host thread(s)\n", threads);
    }

    // one timed run on every GPU at once (each on its own shard, its own default stream and events); the call's time
    // is the slowest GPU's
    auto bench_all = [&](int force_variant, float *ms_out) -> int {
        int e = on_all_gpus([&](Rank &r) -> int {
            r.ms = 0.f;
            if (!r.width()) return 0;
            int e2 = sgemm_set_option(r.h, "force_variant", force_variant);
            if (e2) return e2;
            const float *A = (const float *)(half ? r.da16 : r.da), *B = (const float *)(half ? r.db16 : r.db);
            float *D = (float *)r.dd + (allgather ? (size_t)r.n0 * m : 0);
            return sgemm_bench(r.h, A, B, (const float *)r.dc, D, alpha, beta, m, r.width(), k, m, k, m, m, warmup, runs, nullptr, &r.ms);
        });
        *ms_out = 0.f;
        for (Rank &r : g_ranks) *ms_out = std::max(*ms_out, r.ms);
        return e;
    };
    float ms = 0.f;
    int64_t info = 0;

    // comparison block: the FFMA SIMT kernel of the same cubin (the reference times a naive HIP kernel here); there
    // is none for 16-bit operands, the block is then printed with zeros so that the shape of the output stays
    if (half) {
        std::fprintf(stderr, "no FFMA comparison kernel for 16-bit operands: the SIMT block is empty\n");
        std::cout << "SIMT gemm: 0 ms\nGflops: 0\nGiB/s: 0\n";
    } else {
        if ((rc = bench_all(2, &ms))) return die(h, "SIMT comparison run", rc);
        std::cout << "SIMT gemm: " << ms << " ms\n"
                  << "Gflops: " << gflops(m, n, k, ms) << '\n'
                  << "GiB/s: " << mem_bw(m, n, k, ms) << '\n';
    }

    // measured block: the kernel the config asks for, chosen by the library (tensor path when eligible).
    // The label "ASM gemm" is the reference's and is kept for scripts that look for it.
    env = std::getenv("SGEMM_FORCE_VARIANT");
    for (Rank &r : g_ranks)
        if ((rc = sgemm_dev_memset(r.h, r.dd, 0, (allgather ? nc : std::max<size_t>((size_t)r.width() * m, 1)) * 4)))
            return die(r.h, "result reset", rc);
    int64_t khz = 0;
    for (Rank &r : g_ranks) sgemm_get_info(r.h, "sm_khz_effective", &khz);   // clears the device-side stopwatch
    if ((rc = bench_all(env ? std::atoi(env) : 0, &ms))) return die(h, "measured run", rc);
    for (Rank &r : g_ranks) {
        uint32_t status[8];
        if ((rc = sgemm_last_status(r.h, status))) return die(r.h, "device status check", rc);
        if (sgemm_get_info(r.h, "sm_khz_effective", &khz) == 0) r.sm_mhz = (double)khz * 1e-3;
    }
    int64_t variant = 0, split = 0, fed_by_tma = 0;
    sgemm_get_info(h, "last_variant", &variant);
    sgemm_get_info(h, "last_feed_tma", &fed_by_tma);
    sgemm_get_info(h, "last_split_k", &split);
    sgemm_get_info(h, "launches", &info);
    // 1 = the cubin's main tensor kernel, 3 = its companion for problems with few flops per input byte, 2 = SIMT
    const char *variant_text = half ? (parsed.a_type == 2 ? "tcgen05 BF16" : "tcgen05 FP16")
                               : variant == 1 ? "tcgen05 3xTF32" : variant == 3 ? "tcgen05 3xTF32 (companion)"
                               : fed_by_tma ? "SIMT FFMA (fed by TMA)" : "SIMT FFMA";
    const char *variant_key = half ? (parsed.a_type == 2 ? "tcgen05_bf16" : "tcgen05_fp16")
                              : variant == 1 ? "tcgen05_3xtf32" : variant == 3 ? "tcgen05_3xtf32_companion"
                              : fed_by_tma ? "simt_ffma_tma" : "simt_ffma";
    std::fprintf(stderr, "measured kernel: %s, split_k %lld, %.3f TFLOPS, %lld launches in total, SM clock counted on the device %.0f MHz\n",
                 variant_text, (long long)split, gflops(m, n, k, ms) * 1e-3, (long long)info, g_ranks[0].sm_mhz);
    std::string per_gpu_json = "[";
    if (ngpus > 1)
        std::fprintf(stderr, "%d GPUs, columns sharded in whole tiles of %lld: aggregate %.3f TFLOPS (time of the slowest GPU)\n",
                     ngpus, (long long)tile_n, gflops(m, n, k, ms) * 1e-3);
    for (int i = 0; i < ngpus; ++i) {
        const Rank &r = g_ranks[i];
        const double tf = r.ms > 0 ? gflops(m, r.width(), k, r.ms) * 1e-3 : 0.0;
        if (ngpus > 1)
            std::fprintf(stderr, "  GPU %d: columns [%u, %u), %.4f ms, %.3f TFLOPS, SM clock counted on the device %.0f MHz\n",
                         device + i, r.n0, r.n1, r.ms, tf, r.sm_mhz);
        char item[200];
        std::snprintf(item, sizeof item, "%s{\"device\": %d, \"n0\": %u, \"n1\": %u, \"ms\": %.6f, \"tflops\": %.4f, \"sm_mhz\": %.1f}",
                      i ? ", " : "", device + i, r.n0, r.n1, r.ms, tf, r.sm_mhz);
        per_gpu_json += item;
    }
    per_gpu_json += "]";

    // optional: all-gather of D over NVLink, in place in the full-size D of every GPU; reported apart from the GEMM
    double gather_ms = 0.0, gather_gbs = 0.0;
    if (allgather) {
        for (int pass = 0; pass < 2; ++pass) {   // the first pass pays NCCL's channel set-up
            const auto t0 = std::chrono::steady_clock::now();
            rc = on_all_gpus([&](Rank &r) -> int {
                int e = sgemm_allgather_columns(r.h, (float *)r.dd, m, n, m, (uint32_t)tile_n, nullptr);
                return e ? e : sgemm_dev_sync(r.h);
            });
            const auto t1 = std::chrono::steady_clock::now();
            if (rc) return die(h, "all-gather of D", rc);
            gather_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
        }
        size_t least = nc;
        for (Rank &r : g_ranks) least = std::min(least, (size_t)r.width() * m);
        gather_gbs = (double)(nc - least) * 4 / gather_ms * 1e-6;   // bytes the GPU with the smallest shard receives
        std::fprintf(stderr, "all-gather of D over %d GPUs: %.3f ms, %.1f GB/s received per GPU (not part of the GEMM time)\n",
                     ngpus, gather_ms, gather_gbs);
    }

    std::cout << "ASM gemm: " << ms << " ms\n"
              << "Gflops: " << gflops(m, n, k, ms) << '\n'
              << "GiB/s: " << mem_bw(m, n, k, ms) << '\n';

    size_t mismatches = 0;
    if (validate) {
        std::vector<float> gpu_d(nc);
        if (allgather) {   // every GPU holds all of D: check the last one's copy
            Rank &last = g_ranks.back();
            if ((rc = sgemm_dev_download(last.h, gpu_d.data(), last.dd, nc * 4))) return die(last.h, "result download", rc);
        } else {
            for (Rank &r : g_ranks)
                if (r.width() && (rc = sgemm_dev_download(r.h, gpu_d.data() + (size_t)r.n0 * m, r.dd, (size_t)r.width() * m * 4)))
                    return die(r.h, "result download", rc);
        }
        for (size_t i = 0; i < nc; ++i) {
            if (!(std::fabs(gpu_d[i] - cpu_d[i]) < 1e-3f)) {  // runner/Utils/Math.hpp:5-8 with delta 1e-3 (:295)
                if (mismatches < 10) {
                    std::cout << "gpu & cpu results mismatched at index: " << i << '\n';
                    std::cout << gpu_d[i] << " != " << cpu_d[i] << '\n';
                }
                ++mismatches;
            }
        }
        std::cout << "# of mismatches: " << mismatches << "/" << nc << '\n';
    }
    if (const char *json_path = std::getenv("SGEMM_JSON")) {
        if (FILE *f = std::fopen(json_path, "w")) {
            std::fprintf(f, "{\"m\": %u, \"n\": %u, \"k\": %u, \"alpha\": %g, \"beta\": %g, \"seed\": %llu, \"warmup\": %u, "
                            "\"runs\": %u, \"variant\": \"%s\", \"split_k\": %lld, \"ms\": %.6f, \"tflops\": %.4f, "
                            "\"gib_per_s\": %.3f, \"validated\": %s, \"mismatches\": %zu, \"ngpus\": %d, \"per_gpu\": %s, "
                            "\"allgather_ms\": %.4f, \"allgather_gb_per_s_per_gpu\": %.2f}\n",
                         m, n, k, alpha, beta, (unsigned long long)seed, warmup, runs, variant_key,
                         (long long)split, ms, gflops(m, n, k, ms) * 1e-3, mem_bw(m, n, k, ms), validate ? "true" : "false", mismatches,
                         ngpus, per_gpu_json.c_str(), gather_ms, gather_gbs);
            std::fclose(f);
        } else {
            std::fprintf(stderr, "GeneratorRunner: cannot write %s\n", json_path);
        }
    }
    for (Rank &r : g_ranks) {
        for (void *p : {r.da, r.db, r.dc, r.dd, r.da16, r.db16})
            if (p) sgemm_dev_free(r.h, p);
        sgemm_close(r.h);
    }
    g_ranks.clear();
    return mismatches ? -1 : 0;
}
