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
#include "sgemm_runner.h"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
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

int die(sgemm_handle *h, const char *what, int rc) {
    std::fprintf(stderr, "GeneratorRunner: %s failed: %s (%d): %s\n", what, sgemm_strerror(rc), rc, sgemm_last_error(h));
    if (h) sgemm_close(h);
    return 2;
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

    // kernels for FP16 / BF16 operands (a_type 1 / 2 in the TOML; the reference has FP32 only): A and B are drawn in
    // FP32 like everything else here and converted on the device; the CPU check runs on the converted values
    sgemm_config parsed;
    const bool half = sgemm_config_parse(argv[2], &parsed) == 0 && parsed.a_type != 0;
    if (half && (parsed.trans_a || parsed.trans_b)) {
        std::fprintf(stderr, "GeneratorRunner: %s describes a 16-bit kernel for transposed operands; this program drives the NN layout\n", argv[2]);
        return 2;
    }
    sgemm_handle *h = nullptr;
    int rc = sgemm_open(argv[1], argv[2], device, &h);
    if (rc) return die(nullptr, "sgemm_open", rc);

    const size_t na = (size_t)m * k, nb = (size_t)k * n, nc = (size_t)m * n;
    void *da = nullptr, *db = nullptr, *dc = nullptr, *dd = nullptr;
    if ((rc = sgemm_dev_alloc(h, na * 4, &da)) || (rc = sgemm_dev_alloc(h, nb * 4, &db)) ||
        (rc = sgemm_dev_alloc(h, nc * 4, &dc)) || (rc = sgemm_dev_alloc(h, nc * 4, &dd)))
        return die(h, "device allocation", rc);
    // A, B, C ~ U[-1, 1): streams seed, seed+1, seed+2 of the index-hash generator, filled on the device
    if ((rc = sgemm_fill_uniform(h, (float *)da, na, 0, seed, nullptr)) ||
        (rc = sgemm_fill_uniform(h, (float *)db, nb, 0, seed + 1, nullptr)) ||
        (rc = sgemm_fill_uniform(h, (float *)dc, nc, 0, seed + 2, nullptr)) || (rc = sgemm_dev_sync(h)))
        return die(h, "input fill", rc);

    void *da16 = nullptr, *db16 = nullptr;
    if (half) {
        if ((rc = sgemm_dev_alloc(h, na * 2, &da16)) || (rc = sgemm_dev_alloc(h, nb * 2, &db16)))
            return die(h, "device allocation", rc);
        if ((rc = sgemm_narrow16(h, (const float *)da, da16, na, nullptr)) ||
            (rc = sgemm_narrow16(h, (const float *)db, db16, nb, nullptr)) || (rc = sgemm_dev_sync(h)))
            return die(h, "operand conversion", rc);
    }

    std::vector<float> cpu_d;
    if (validate) {
        std::vector<float> ha(na), hb(nb), hc(nc);
        cpu_d.resize(nc);
        if (half) {   // the values the kernel multiplies: the 16-bit words, widened
            std::vector<uint16_t> wa(na), wb(nb);
            if ((rc = sgemm_dev_download(h, wa.data(), da16, na * 2)) || (rc = sgemm_dev_download(h, wb.data(), db16, nb * 2)))
                return die(h, "input download", rc);
            for (size_t i = 0; i < na; ++i) ha[i] = widen16(wa[i], parsed.a_type);
            for (size_t i = 0; i < nb; ++i) hb[i] = widen16(wb[i], parsed.a_type);
            if ((rc = sgemm_dev_download(h, hc.data(), dc, nc * 4))) return die(h, "input download", rc);
        } else if ((rc = sgemm_dev_download(h, ha.data(), da, na * 4)) || (rc = sgemm_dev_download(h, hb.data(), db, nb * 4)) ||
            (rc = sgemm_dev_download(h, hc.data(), dc, nc * 4)))
            return die(h, "input download", rc);
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

    const float *A = (const float *)(half ? da16 : da), *B = (const float *)(half ? db16 : db), *C = (const float *)dc;
    float *D = (float *)dd;
    float ms = 0.f;
    int64_t info = 0;

    // comparison block: the FFMA SIMT kernel of the same cubin (the reference times a naive HIP kernel here); there
    // is none for 16-bit operands, the block is then printed with zeros so that the shape of the output stays
    if (half) {
        std::fprintf(stderr, "no FFMA comparison kernel for 16-bit operands: the SIMT block is empty\n");
        std::cout << "SIMT gemm: 0 ms\nGflops: 0\nGiB/s: 0\n";
    } else {
        if ((rc = sgemm_set_option(h, "force_variant", 2)) ||
            (rc = sgemm_bench(h, A, B, C, D, alpha, beta, m, n, k, m, k, m, m, warmup, runs, nullptr, &ms)))
            return die(h, "SIMT comparison run", rc);
        std::cout << "SIMT gemm: " << ms << " ms\n"
                  << "Gflops: " << gflops(m, n, k, ms) << '\n'
                  << "GiB/s: " << mem_bw(m, n, k, ms) << '\n';
    }

    // measured block: the kernel the config asks for, chosen by the library (tensor path when eligible).
    // The label "ASM gemm" is the reference's and is kept for scripts that look for it.
    env = std::getenv("SGEMM_FORCE_VARIANT");
    if ((rc = sgemm_dev_memset(h, dd, 0, nc * 4)) || (rc = sgemm_set_option(h, "force_variant", env ? std::atoi(env) : 0)) ||
        (rc = sgemm_bench(h, A, B, C, D, alpha, beta, m, n, k, m, k, m, m, warmup, runs, nullptr, &ms)))
        return die(h, "measured run", rc);
    uint32_t status[8];
    if ((rc = sgemm_last_status(h, status))) return die(h, "device status check", rc);
    int64_t variant = 0, split = 0;
    sgemm_get_info(h, "last_variant", &variant);
    sgemm_get_info(h, "last_split_k", &split);
    sgemm_get_info(h, "launches", &info);
    // 1 = the cubin's main tensor kernel, 3 = its companion for problems with few flops per input byte, 2 = SIMT
    const char *variant_text = half ? (parsed.a_type == 2 ? "tcgen05 BF16" : "tcgen05 FP16")
                               : variant == 1 ? "tcgen05 3xTF32" : variant == 3 ? "tcgen05 3xTF32 (companion)" : "SIMT FFMA";
    const char *variant_key = variant == 1 ? "tcgen05_3xtf32" : variant == 3 ? "tcgen05_3xtf32_companion" : "simt_ffma";
    std::fprintf(stderr, "measured kernel: %s, split_k %lld, %.3f TFLOPS, %lld launches in total\n",
                 variant_text, (long long)split, gflops(m, n, k, ms) * 1e-3, (long long)info);
    std::cout << "ASM gemm: " << ms << " ms\n"
              << "Gflops: " << gflops(m, n, k, ms) << '\n'
              << "GiB/s: " << mem_bw(m, n, k, ms) << '\n';

    size_t mismatches = 0;
    if (validate) {
        std::vector<float> gpu_d(nc);
        if ((rc = sgemm_dev_download(h, gpu_d.data(), dd, nc * 4))) return die(h, "result download", rc);
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
                            "\"gib_per_s\": %.3f, \"validated\": %s, \"mismatches\": %zu}\n",
                         m, n, k, alpha, beta, (unsigned long long)seed, warmup, runs, variant_key,
                         (long long)split, ms, gflops(m, n, k, ms) * 1e-3, mem_bw(m, n, k, ms), validate ? "true" : "false", mismatches);
            std::fclose(f);
        } else {
            std::fprintf(stderr, "GeneratorRunner: cannot write %s\n", json_path);
        }
    }
    sgemm_dev_free(h, da);
    sgemm_dev_free(h, db);
    sgemm_dev_free(h, dc);
    sgemm_dev_free(h, dd);
    if (da16) sgemm_dev_free(h, da16);
    if (db16) sgemm_dev_free(h, db16);
    sgemm_close(h);
    return mismatches ? -1 : 0;
}
