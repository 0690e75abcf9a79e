// ---------------------------------------------------------------------------------------------
// Pure-FFMA SIMT SGEMM (strict FP32): the small / skinny / TMA-ineligible path and the fallback
// entry inside every tensor-core cubin.  One thread block computes a SIMT_BM x SIMT_BN tile of D,
// K is walked in steps of SIMT_BK through a double-buffered shared-memory ring; every thread owns
// a SIMT_TM x SIMT_TN register tile made of 4x4 sub-blocks strided over the block tile, so that
// shared-memory fragment reads are 16-byte and conflict-free.
//
// op(A), op(B): GEMM_TRANS_A / GEMM_TRANS_B select at compile time whether A (B) is stored transposed.
//
// Arbitrary M, N, K and leading dimensions: loads are 16-byte when base pointer and leading
// dimension allow it and the whole vector is in range, guarded scalars otherwise (zero fill).
//
// Generator-supplied macros: SIMT_ENTRY (kernel name), SIMT_BM, SIMT_BN, SIMT_BK, SIMT_TM,
// SIMT_TN, SIMT_PLR (0: read fragments just in time, 1: prefetch the next k-slice's fragments
// into registers while the current one is multiplied), OPT_WGM (tile rasterisation width).
//
// Launch: grid (tiles_m * tiles_n, 1, split_k), block SIMT_THREADS.  With split_k > 1 every z
// slice writes its raw partial product to ws[z][M x N] and sgemm_splitk_reduce finishes the job
// in a fixed order (no atomics: results are bit-reproducible).
// ---------------------------------------------------------------------------------------------
#define SIMT_TX (SIMT_BM / SIMT_TM)
#define SIMT_TY (SIMT_BN / SIMT_TN)
#define SIMT_THREADS (SIMT_TX * SIMT_TY)
#define SIMT_GM (SIMT_TM / 4)
#define SIMT_GN (SIMT_TN / 4)
#define SIMT_A_VEC ((SIMT_BM * SIMT_BK / 4 + SIMT_THREADS - 1) / SIMT_THREADS)
#define SIMT_B_VEC ((SIMT_BN * SIMT_BK / 4 + SIMT_THREADS - 1) / SIMT_THREADS)
#define SIMT_B_PAD 4

static_assert(SIMT_TM % 4 == 0 && SIMT_TN % 4 == 0, "thread tile is built from 4x4 blocks");
static_assert(SIMT_BM % SIMT_TM == 0 && SIMT_BN % SIMT_TN == 0, "block tile / thread tile");
static_assert(SIMT_BK % 4 == 0, "K step is loaded in 16-byte vectors");

#ifndef GEMM_TRANS_A
#define GEMM_TRANS_A 0   // 1: A is stored transposed (K x M column-major, element (i,l) at a[l + i*lda])
#endif
#ifndef GEMM_TRANS_B
#define GEMM_TRANS_B 0   // 1: B is stored transposed (N x K column-major, element (l,j) at b[j + l*ldb])
#endif

struct SimtSmem {
    float a[2][SIMT_BK][SIMT_BM + SIMT_B_PAD];  // k-major rows of the A tile
    float b[2][SIMT_BK][SIMT_BN + SIMT_B_PAD];  // k-major rows of the B tile
};

// Both operands end up in shared memory as [k][mn] rows.  An operand whose MN index is contiguous in global
// memory (A not transposed, B transposed) is loaded in 16-byte vectors along MN and stored as is; an operand
// whose K index is contiguous (B not transposed, A transposed) is loaded in vectors along K and transposed on
// the store.  MN = rows of the tile, ld = leading dimension, mn0 / mn_end = tile origin / matrix extent.
template <int TILE_MN>
struct SimtLoader {
    static constexpr int VEC = (TILE_MN * SIMT_BK / 4 + SIMT_THREADS - 1) / SIMT_THREADS;

    __device__ static __forceinline__ void load_mn_contiguous(float4 (&r)[VEC], const float *__restrict__ p0, uint32_t mn_end,
                                                              uint32_t ld, uint32_t mn0, uint32_t k0, uint32_t k_end, bool vec_ok) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const uint32_t id = threadIdx.x + v * SIMT_THREADS;
            const uint32_t i = mn0 + (id % (TILE_MN / 4)) * 4, l = k0 + id / (TILE_MN / 4);
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (id < TILE_MN * SIMT_BK / 4 && l < k_end) {
                const float *p = p0 + i + (uint64_t)l * ld;
                if (vec_ok && i + 3 < mn_end) {
                    x = __ldg(reinterpret_cast<const float4 *>(p));
                } else {
                    if (i + 0 < mn_end) x.x = __ldg(p + 0);
                    if (i + 1 < mn_end) x.y = __ldg(p + 1);
                    if (i + 2 < mn_end) x.z = __ldg(p + 2);
                    if (i + 3 < mn_end) x.w = __ldg(p + 3);
                }
            }
            r[v] = x;
        }
    }

    __device__ static __forceinline__ void load_k_contiguous(float4 (&r)[VEC], const float *__restrict__ p0, uint32_t mn_end,
                                                             uint32_t ld, uint32_t mn0, uint32_t k0, uint32_t k_end, bool vec_ok) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const uint32_t id = threadIdx.x + v * SIMT_THREADS;
            const uint32_t l = k0 + (id % (SIMT_BK / 4)) * 4, j = mn0 + id / (SIMT_BK / 4);
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (id < TILE_MN * SIMT_BK / 4 && j < mn_end) {
                const float *p = p0 + l + (uint64_t)j * ld;
                if (vec_ok && l + 3 < k_end) {
                    x = __ldg(reinterpret_cast<const float4 *>(p));
                } else {
                    if (l + 0 < k_end) x.x = __ldg(p + 0);
                    if (l + 1 < k_end) x.y = __ldg(p + 1);
                    if (l + 2 < k_end) x.z = __ldg(p + 2);
                    if (l + 3 < k_end) x.w = __ldg(p + 3);
                }
            }
            r[v] = x;
        }
    }

    __device__ static __forceinline__ void store_mn_contiguous(float (*rows)[TILE_MN + SIMT_B_PAD], const float4 (&r)[VEC]) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const uint32_t id = threadIdx.x + v * SIMT_THREADS;
            if (id < TILE_MN * SIMT_BK / 4)
                *reinterpret_cast<float4 *>(&rows[id / (TILE_MN / 4)][(id % (TILE_MN / 4)) * 4]) = r[v];
        }
    }

    __device__ static __forceinline__ void store_k_contiguous(float (*rows)[TILE_MN + SIMT_B_PAD], const float4 (&r)[VEC]) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const uint32_t id = threadIdx.x + v * SIMT_THREADS;
            if (id < TILE_MN * SIMT_BK / 4) {
                const uint32_t l = (id % (SIMT_BK / 4)) * 4, j = id / (SIMT_BK / 4);
                rows[l + 0][j] = r[v].x;
                rows[l + 1][j] = r[v].y;
                rows[l + 2][j] = r[v].z;
                rows[l + 3][j] = r[v].w;
            }
        }
    }
};

__device__ __forceinline__ void simt_load_a(float4 (&ra)[SIMT_A_VEC], const float *__restrict__ a,
                                            uint32_t m, uint32_t lda, uint32_t m0, uint32_t k0,
                                            uint32_t k_end, bool vec_ok) {
#if GEMM_TRANS_A
    SimtLoader<SIMT_BM>::load_k_contiguous(ra, a, m, lda, m0, k0, k_end, vec_ok);
#else
    SimtLoader<SIMT_BM>::load_mn_contiguous(ra, a, m, lda, m0, k0, k_end, vec_ok);
#endif
}

__device__ __forceinline__ void simt_load_b(float4 (&rb)[SIMT_B_VEC], const float *__restrict__ b,
                                            uint32_t n, uint32_t ldb, uint32_t n0, uint32_t k0,
                                            uint32_t k_end, bool vec_ok) {
#if GEMM_TRANS_B
    SimtLoader<SIMT_BN>::load_mn_contiguous(rb, b, n, ldb, n0, k0, k_end, vec_ok);
#else
    SimtLoader<SIMT_BN>::load_k_contiguous(rb, b, n, ldb, n0, k0, k_end, vec_ok);
#endif
}

__device__ __forceinline__ void simt_store_tiles(SimtSmem &s, int buf, const float4 (&ra)[SIMT_A_VEC],
                                                 const float4 (&rb)[SIMT_B_VEC]) {
#if GEMM_TRANS_A
    SimtLoader<SIMT_BM>::store_k_contiguous(s.a[buf], ra);
#else
    SimtLoader<SIMT_BM>::store_mn_contiguous(s.a[buf], ra);
#endif
#if GEMM_TRANS_B
    SimtLoader<SIMT_BN>::store_mn_contiguous(s.b[buf], rb);
#else
    SimtLoader<SIMT_BN>::store_k_contiguous(s.b[buf], rb);
#endif
}

__device__ __forceinline__ void simt_read_frag(const SimtSmem &s, int buf, int kk, uint32_t tx,
                                               uint32_t ty, float (&fa)[SIMT_TM], float (&fb)[SIMT_TN]) {
#pragma unroll
    for (int g = 0; g < SIMT_GM; ++g) {
        const float4 v = *reinterpret_cast<const float4 *>(&s.a[buf][kk][g * SIMT_TX * 4 + tx * 4]);
        fa[g * 4 + 0] = v.x; fa[g * 4 + 1] = v.y; fa[g * 4 + 2] = v.z; fa[g * 4 + 3] = v.w;
    }
#pragma unroll
    for (int g = 0; g < SIMT_GN; ++g) {
        const float4 v = *reinterpret_cast<const float4 *>(&s.b[buf][kk][g * SIMT_TY * 4 + ty * 4]);
        fb[g * 4 + 0] = v.x; fb[g * 4 + 1] = v.y; fb[g * 4 + 2] = v.z; fb[g * 4 + 3] = v.w;
    }
}

#ifndef SIMT_FMA2
#define SIMT_FMA2 1   // accumulate with the packed FP32 FMA of sm_100 (fma.rn.f32x2): same results, half the FMA instructions
#endif
#ifndef SGEMM_FFMA_SHARED
#define SGEMM_FFMA_SHARED
#ifndef FFMA_PACKED
#define FFMA_PACKED 1   // 0: two scalar FMAs in place of each packed one (the same arithmetic; for comparison)
#endif
// (shared by the register-fed kernel below and the TMA-fed kernel of sgemm_ffma_tma.cuh; emitted once per translation unit)
// acc2[j][i] (+)= {fa[2i], fa[2i+1]} * {fb[j], fb[j]}: one packed FMA per two rows of the thread tile
template <int TM, int TN>
__device__ __forceinline__ void ffma_outer_product2(uint64_t (&acc2)[TN][TM / 2], const float (&fa)[TM], const float (&fb)[TN]) {
    uint64_t a2[TM / 2];
#pragma unroll
    for (int i = 0; i < TM / 2; ++i) asm("mov.b64 %0, {%1, %2};" : "=l"(a2[i]) : "f"(fa[2 * i]), "f"(fa[2 * i + 1]));
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        uint64_t b2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(b2) : "f"(fb[j]));
#pragma unroll
        for (int i = 0; i < TM / 2; ++i) {
#if FFMA_PACKED
            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[j][i]) : "l"(a2[i]), "l"(b2));
#else
            float lo, hi;
            asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc2[j][i]));
            lo = fmaf(fa[2 * i], fb[j], lo);
            hi = fmaf(fa[2 * i + 1], fb[j], hi);
            asm("mov.b64 %0, {%1, %2};" : "=l"(acc2[j][i]) : "f"(lo), "f"(hi));
#endif
        }
    }
}

// Epilogue of one thread: d = alpha*acc + beta*c (C is not read when beta == 0), or, with split_k > 1, the raw partial
// product to this split's M x N slab of ws.  16-byte accesses where base and leading dimension allow, guarded scalars
// at the edges.
// The thread tile TM x TN is made of 4 x 4 blocks strided over the block tile: rows gi*TX*4 + tx*4 + (0..3), columns
// gj*TY*4 + ty*4 + (0..3).
template <int TM, int TN, int TX, int TY>
__device__ __forceinline__ void ffma_epilogue(const float (&acc)[TN][TM], const float *c, float *d, float *ws,
                                              uint32_t m, uint32_t n, uint32_t ldc, uint32_t ldd, float alpha, float beta,
                                              uint32_t split_k, uint32_t m0, uint32_t n0, uint32_t tx, uint32_t ty) {
    const bool partial = split_k > 1;
    float *out = partial ? ws + (uint64_t)blockIdx.z * m * n : d;
    const uint32_t ldo = partial ? m : ldd;
    const bool o_vec = ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && (ldo % 4 == 0);
    const bool c_vec = ((reinterpret_cast<uintptr_t>(c) & 15) == 0) && (ldc % 4 == 0);
#pragma unroll
    for (int gj = 0; gj < (TN / 4); ++gj) {
#pragma unroll
        for (int rj = 0; rj < 4; ++rj) {
            const uint32_t col = n0 + gj * TY * 4 + ty * 4 + rj;
            if (col >= n) continue;
#pragma unroll
            for (int gi = 0; gi < (TM / 4); ++gi) {
                const uint32_t row = m0 + gi * TX * 4 + tx * 4;
                if (row >= m) continue;
                float r[4];
#pragma unroll
                for (int ri = 0; ri < 4; ++ri) r[ri] = acc[gj * 4 + rj][gi * 4 + ri];
                if (!partial) {
#pragma unroll
                    for (int ri = 0; ri < 4; ++ri) r[ri] *= alpha;
                    if (beta != 0.0f) {
                        const float *cp = c + row + (uint64_t)col * ldc;
                        if (c_vec && row + 3 < m) {
                            const float4 cv = *reinterpret_cast<const float4 *>(cp);
                            r[0] = fmaf(beta, cv.x, r[0]); r[1] = fmaf(beta, cv.y, r[1]);
                            r[2] = fmaf(beta, cv.z, r[2]); r[3] = fmaf(beta, cv.w, r[3]);
                        } else {
#pragma unroll
                            for (int ri = 0; ri < 4; ++ri)
                                if (row + ri < m) r[ri] = fmaf(beta, cp[ri], r[ri]);
                        }
                    }
                }
                float *op = out + row + (uint64_t)col * ldo;
                if (o_vec && row + 3 < m) {
                    *reinterpret_cast<float4 *>(op) = make_float4(r[0], r[1], r[2], r[3]);
                } else {
#pragma unroll
                    for (int ri = 0; ri < 4; ++ri)
                        if (row + ri < m) op[ri] = r[ri];
                }
            }
        }
    }
}
#endif  // SGEMM_FFMA_SHARED

extern "C" __global__ void __launch_bounds__(SIMT_THREADS)
SIMT_ENTRY(const float *__restrict__ a, const float *__restrict__ b, const float *c, float *d,
           uint32_t m, uint32_t n, uint32_t k, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t ldd,
           float alpha, float beta, int32_t num_wg_x, int32_t num_wg_y,
           float *ws, uint32_t *status, uint32_t split_k,
           uint32_t *wave_sync, uint32_t wave_sync_base) {
    __shared__ __align__(16) SimtSmem s;
    (void)status;
    (void)wave_sync; (void)wave_sync_base;   // one tile per block: nothing to align

    sgemm_launch_dependents();
    sgemm_grid_dependency_wait();
    uint32_t tile_x, tile_y;
    sgemm_tile_raster(blockIdx.x, (uint32_t)num_wg_x, (uint32_t)num_wg_y, OPT_WGM, tile_x, tile_y);
    const uint32_t m0 = tile_x * SIMT_BM, n0 = tile_y * SIMT_BN;
    const uint32_t tx = threadIdx.x % SIMT_TX, ty = threadIdx.x / SIMT_TX;

    // K range of this split (whole SIMT_BK steps per split; the last split takes the tail)
    const uint32_t steps_total = (k + SIMT_BK - 1) / SIMT_BK;
    const uint32_t steps_per = (steps_total + split_k - 1) / split_k;
    const uint32_t k_begin = min(k, blockIdx.z * steps_per * SIMT_BK);
    const uint32_t k_end = min(k, k_begin + steps_per * SIMT_BK);
    const uint32_t steps = (k_end - k_begin + SIMT_BK - 1) / SIMT_BK;

    const bool a_vec = ((reinterpret_cast<uintptr_t>(a) & 15) == 0) && (lda % 4 == 0);
    const bool b_vec = ((reinterpret_cast<uintptr_t>(b) & 15) == 0) && (ldb % 4 == 0);

#if SIMT_FMA2
    // accumulators as pairs of rows in 64-bit registers, updated with the packed FP32 FMA (two IEEE fused
    // multiply-adds per instruction: the same arithmetic, half the issue slots)
    uint64_t acc2[SIMT_TN][SIMT_TM / 2];
#pragma unroll
    for (int j = 0; j < SIMT_TN; ++j)
#pragma unroll
        for (int i = 0; i < SIMT_TM / 2; ++i) acc2[j][i] = 0ull;
#else
    float acc[SIMT_TN][SIMT_TM];
#pragma unroll
    for (int j = 0; j < SIMT_TN; ++j)
#pragma unroll
        for (int i = 0; i < SIMT_TM; ++i) acc[j][i] = 0.0f;
#endif

    float4 ra[SIMT_A_VEC], rb[SIMT_B_VEC];
    if (steps > 0) {
        simt_load_a(ra, a, m, lda, m0, k_begin, k_end, a_vec);
        simt_load_b(rb, b, n, ldb, n0, k_begin, k_end, b_vec);
        simt_store_tiles(s, 0, ra, rb);
    }
    __syncthreads();

    for (uint32_t t = 0; t < steps; ++t) {
        const int buf = t & 1;
        const bool more = t + 1 < steps;
        if (more) {
            simt_load_a(ra, a, m, lda, m0, k_begin + (t + 1) * SIMT_BK, k_end, a_vec);
            simt_load_b(rb, b, n, ldb, n0, k_begin + (t + 1) * SIMT_BK, k_end, b_vec);
        }
#if SIMT_PLR
        float fa[2][SIMT_TM], fb[2][SIMT_TN];
        simt_read_frag(s, buf, 0, tx, ty, fa[0], fb[0]);
#pragma unroll
        for (int kk = 0; kk < SIMT_BK; ++kk) {
            if (kk + 1 < SIMT_BK) simt_read_frag(s, buf, kk + 1, tx, ty, fa[(kk + 1) & 1], fb[(kk + 1) & 1]);
#if SIMT_FMA2
            ffma_outer_product2<SIMT_TM, SIMT_TN>(acc2, fa[kk & 1], fb[kk & 1]);
#else
#pragma unroll
            for (int j = 0; j < SIMT_TN; ++j)
#pragma unroll
                for (int i = 0; i < SIMT_TM; ++i)
                    acc[j][i] = fmaf(fa[kk & 1][i], fb[kk & 1][j], acc[j][i]);
#endif
        }
#else
#pragma unroll
        for (int kk = 0; kk < SIMT_BK; ++kk) {
            float fa[SIMT_TM], fb[SIMT_TN];
            simt_read_frag(s, buf, kk, tx, ty, fa, fb);
#if SIMT_FMA2
            ffma_outer_product2<SIMT_TM, SIMT_TN>(acc2, fa, fb);
#else
#pragma unroll
            for (int j = 0; j < SIMT_TN; ++j)
#pragma unroll
                for (int i = 0; i < SIMT_TM; ++i) acc[j][i] = fmaf(fa[i], fb[j], acc[j][i]);
#endif
        }
#endif
        if (more) simt_store_tiles(s, buf ^ 1, ra, rb);
        __syncthreads();
    }

#if SIMT_FMA2
    float acc[SIMT_TN][SIMT_TM];
#pragma unroll
    for (int j = 0; j < SIMT_TN; ++j)
#pragma unroll
        for (int i = 0; i < SIMT_TM / 2; ++i)
            asm("mov.b64 {%0, %1}, %2;" : "=f"(acc[j][2 * i]), "=f"(acc[j][2 * i + 1]) : "l"(acc2[j][i]));
#endif
    ffma_epilogue<SIMT_TM, SIMT_TN, SIMT_TX, SIMT_TY>(acc, c, d, ws, m, n, ldc, ldd, alpha, beta, split_k, m0, n0, tx, ty);
}
