// ---------------------------------------------------------------------------------------------
// Shared device code of every generated SGEMM translation unit (text-included by the generator,
// so that the emitted .cu is one self-contained file that nvcc turns into one cubin).
//
// Problem: column-major NN FP32 GEMM   D = alpha * A * B + beta * C
//   A is M x K, element (i,l) at a[i + l*lda]     B is K x N, element (l,j) at b[l + j*ldb]
//   C, D are M x N, element (i,j) at [i + j*ldc] / [i + j*ldd]
// (the kernel ABI and the math of the reference kernel: generator/generator.py:2603-2618 for the
//  fifteen arguments, runner/generator_runner.cpp:16-33 for the arithmetic).
// ---------------------------------------------------------------------------------------------
#include <stdint.h>

#ifndef OPT_WGM
#define OPT_WGM 1
#endif

// Device status words written by a kernel that gave up on a bounded wait.
//   status[0] = code (0 ok, 1 a bounded wait ran out)   status[1] = role/barrier tag
//   status[2] = tile index   status[3] = k-block   status[4] = block index   status[5] = parity waited for
// Behind them, status[8..9] and status[10..11] are two 64-bit sums kept by the tensor-core GEMM kernels: SM cycles and
// nanoseconds that block 0 of each launch ran for (their quotient is the SM clock the launches really had).
#define SGEMM_STATUS_WORDS 8
#define SGEMM_STATUS_OK 0u
#define SGEMM_STATUS_TIMEOUT 1u

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  The runner launches every kernel with "programmatic stream
// serialisation": a kernel's CTAs may become resident while the previous kernel of the stream is
// still running.  sgemm_grid_dependency_wait() blocks until that previous kernel has completed and
// its writes are visible; every kernel calls it before its first access to global memory (reads of
// what the predecessor wrote, and writes to what the predecessor may still read).  Because each
// kernel waits for its immediate predecessor, completion is transitive along the stream.
// sgemm_launch_dependents() lets the next kernel's CTAs be scheduled early.  Both are no-ops for a
// kernel launched the ordinary way.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void sgemm_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void sgemm_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Tile rasterisation ("wgm", the workgroup remap of generator/generator.py:1437-1464).
// wgm <= 1: no remap, z = x + y*nx (M index fastest), as the reference when wgm is 1.
// wgm  > 1: the linear id z walks groups of `wgm` tiles in M; inside a group the M index moves
// fastest, then the N index; groups follow each other along M:
//   x' = (z % wgm) + (z / wgm / ny) * wgm ,  y' = (z / wgm) % ny
// which is the reference's formula when nx is a multiple of wgm.  The last, narrower group (nx not
// a multiple of wgm) is walked with its own width so that every tile is visited exactly once.
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ void sgemm_tile_raster(uint32_t z, uint32_t nx, uint32_t ny,
                                                           uint32_t wgm, uint32_t &x, uint32_t &y) {
    if (wgm <= 1) {
        x = z % nx;
        y = z / nx;
        return;
    }
    const uint32_t group_tiles = wgm * ny;
    const uint32_t g = z / group_tiles;
    const uint32_t first_x = g * wgm;
    const uint32_t width = (nx - first_x) < wgm ? (nx - first_x) : wgm;
    const uint32_t r = z - g * group_tiles;
    x = first_x + r % width;
    y = r / width;
}

extern "C" __global__ void sgemm_tile_map(int32_t *xy, uint32_t nx, uint32_t ny) {
    sgemm_grid_dependency_wait();
    const uint32_t z = blockIdx.x * blockDim.x + threadIdx.x;
    if (z >= nx * ny) return;
    uint32_t x, y;
    sgemm_tile_raster(z, nx, ny, OPT_WGM, x, y);
    xy[2 * z] = (int32_t)x;
    xy[2 * z + 1] = (int32_t)y;
}

// ---------------------------------------------------------------------------------------------
// Seeded inputs: splitmix64 finaliser over (element index, stream), top 24 bits -> [-1, 1).
// Bit-identical to the host generator used by the tests, so that host and device fills agree.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float sgemm_uniform(uint64_t idx, uint64_t stream) {
    uint64_t x = idx + 0x9E3779B97F4A7C15ull * (stream + 1ull);
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return (float)(x >> 40) * 0x1p-23f - 1.0f;
}

extern "C" __global__ void sgemm_fill_uniform(float *dst, uint64_t count, uint64_t first_index,
                                              uint64_t stream) {
    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
        dst[i] = sgemm_uniform(first_index + i, stream);
}

// ---------------------------------------------------------------------------------------------
// Split pre-pass for the 3xTF32 path: lo = x - trunc_tf32(x).  The tensor core reads only the top
// 19 bits of each FP32 word (sign, 8 exponent, 10 mantissa bits), so the raw FP32 operand already
// acts as the "hi" term; the remainder is exact in FP32.  One launch covers A's and B's spans.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float sgemm_tf32_lo(float x) {
    return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
}

extern "C" __global__ void sgemm_split_lo(const float *__restrict__ src_a, float *__restrict__ lo_a,
                                          uint64_t count_a, const float *__restrict__ src_b,
                                          float *__restrict__ lo_b, uint64_t count_b) {
    sgemm_launch_dependents();   // the GEMM kernel may set itself up while this pass runs
    sgemm_grid_dependency_wait();
    // both spans are walked in float4 units; bases are 16-byte aligned (checked on the host)
    const uint64_t va = count_a >> 2, vb = count_b >> 2;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (uint64_t i = tid; i < va + vb; i += stride) {
        const bool is_a = i < va;
        const float4 *s = is_a ? reinterpret_cast<const float4 *>(src_a) + i
                               : reinterpret_cast<const float4 *>(src_b) + (i - va);
        float4 *o = is_a ? reinterpret_cast<float4 *>(lo_a) + i
                         : reinterpret_cast<float4 *>(lo_b) + (i - va);
        float4 v = __ldg(s);
        v.x = sgemm_tf32_lo(v.x);
        v.y = sgemm_tf32_lo(v.y);
        v.z = sgemm_tf32_lo(v.z);
        v.w = sgemm_tf32_lo(v.w);
        *o = v;
    }
    if (tid < (count_a & 3)) lo_a[(va << 2) + tid] = sgemm_tf32_lo(src_a[(va << 2) + tid]);
    if (tid < (count_b & 3)) lo_b[(vb << 2) + tid] = sgemm_tf32_lo(src_b[(vb << 2) + tid]);
}

// K-major packing of A for the tensor path's alternative operand layout: writes
//   hi_t[l + i*ldt] = a[i + l*lda]  and  lo_t[l + i*ldt] = lo(a[i + l*lda])   (32x32 smem transpose)
extern "C" __global__ void sgemm_pack_a_kmajor(const float *__restrict__ a, uint32_t lda, uint32_t m,
                                               uint32_t k, float *__restrict__ hi_t,
                                               float *__restrict__ lo_t, uint32_t ldt) {
    __shared__ float tile[32][33];
    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    const uint32_t i0 = blockIdx.x * 32, l0 = blockIdx.y * 32;
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        const uint32_t i = i0 + threadIdx.x, l = l0 + r;
        tile[r][threadIdx.x] = (i < m && l < k) ? a[i + (uint64_t)l * lda] : 0.0f;
    }
    __syncthreads();
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        const uint32_t i = i0 + r, l = l0 + threadIdx.x;
        if (i < m && l < k) {
            const float v = tile[threadIdx.x][r];
            hi_t[l + (uint64_t)i * ldt] = v;
            lo_t[l + (uint64_t)i * ldt] = sgemm_tf32_lo(v);
        }
    }
}

// Copy of an operand to an aligned pitch, for operands TMA cannot describe (a base that is not 16-byte aligned, a
// leading dimension that is not a multiple of 4): dst[i + j*ld_dst] = src[i + j*ld_src], i < inner, j < outer.
extern "C" __global__ void sgemm_repitch(const float *__restrict__ src, uint32_t ld_src, uint32_t inner, uint32_t outer,
                                         float *__restrict__ dst, uint32_t ld_dst) {
    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    const uint64_t total = (uint64_t)inner * outer;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const uint32_t i = (uint32_t)(e % inner), j = (uint32_t)(e / inner);
        dst[i + (uint64_t)j * ld_dst] = __ldg(src + i + (uint64_t)j * ld_src);
    }
}

// FP32 -> FP16 (kind 1) or BF16 (kind 2) words, round to nearest even: how callers that hold FP32 data (the runner
// program, the tuner) make operands for the kernels with 16-bit A and B.
extern "C" __global__ void sgemm_narrow16(const float *__restrict__ src, uint16_t *__restrict__ dst, uint64_t count,
                                          uint32_t kind) {
    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float x = __ldg(src + i);
        uint16_t w;
        if (kind == 1) asm("cvt.rn.f16.f32 %0, %1;" : "=h"(w) : "f"(x));
        else asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(w) : "f"(x));
        dst[i] = w;
    }
}

// The same packing for 16-bit operands (FP16 / BF16 words are copied as they are, there is no lo term):
//   out[l + i*ldt] = a[i + l*lda]
extern "C" __global__ void sgemm_pack16_kmajor(const uint16_t *__restrict__ a, uint32_t lda, uint32_t m, uint32_t k,
                                               uint16_t *__restrict__ out, uint32_t ldt) {
    __shared__ uint16_t tile[32][34];
    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    const uint32_t i0 = blockIdx.x * 32, l0 = blockIdx.y * 32;
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        const uint32_t i = i0 + threadIdx.x, l = l0 + r;
        tile[r][threadIdx.x] = (i < m && l < k) ? a[i + (uint64_t)l * lda] : (uint16_t)0;
    }
    __syncthreads();
    for (uint32_t r = threadIdx.y; r < 32; r += blockDim.y) {
        const uint32_t i = i0 + r, l = l0 + threadIdx.x;
        if (i < m && l < k) out[l + (uint64_t)i * ldt] = tile[threadIdx.x][r];
    }
}

// ---------------------------------------------------------------------------------------------
// Deterministic split-K second pass: D = alpha * (ws[0] + ws[1] + ... in fixed order) + beta * C.
// ws holds nsplit dense M x N partial products (leading dimension M).  nsplit = 0 gives
// D = beta * C, which is also how K = 0 is served.
// ---------------------------------------------------------------------------------------------
extern "C" __global__ void sgemm_splitk_reduce(const float *__restrict__ ws, const float *c, float *d,
                                               uint32_t m, uint32_t n, uint32_t ldc, uint32_t ldd,
                                               float alpha, float beta, uint32_t nsplit) {
    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    const uint64_t total = (uint64_t)m * n;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool use_c = beta != 0.0f;
    // fast path: four consecutive rows of one column per thread, 16-byte loads and stores
    const bool vec = (m % 4 == 0) && (ldd % 4 == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(ws) & 15) == 0) &&
                     (!use_c || ((ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0)));
    if (vec) {
        const uint32_t m4 = m / 4;
        const uint64_t total4 = total / 4;
        for (uint64_t e = tid; e < total4; e += stride) {
            const uint32_t i = (uint32_t)(e % m4) * 4, j = (uint32_t)(e / m4);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t s = 0; s < nsplit; ++s) {
                const float4 v = *reinterpret_cast<const float4 *>(ws + (uint64_t)s * total + e * 4);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            float4 r = make_float4(alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w);
            if (use_c) {
                const float4 cv = *reinterpret_cast<const float4 *>(c + i + (uint64_t)j * ldc);
                r.x = fmaf(beta, cv.x, r.x); r.y = fmaf(beta, cv.y, r.y);
                r.z = fmaf(beta, cv.z, r.z); r.w = fmaf(beta, cv.w, r.w);
            }
            *reinterpret_cast<float4 *>(d + i + (uint64_t)j * ldd) = r;
        }
        return;
    }
    for (uint64_t e = tid; e < total; e += stride) {
        const uint32_t i = (uint32_t)(e % m), j = (uint32_t)(e / m);
        float acc = 0.0f;
        for (uint32_t s = 0; s < nsplit; ++s) acc += ws[(uint64_t)s * total + e];
        float r = alpha * acc;
        if (use_c) r = fmaf(beta, c[i + (uint64_t)j * ldc], r);
        d[i + (uint64_t)j * ldd] = r;
    }
}
