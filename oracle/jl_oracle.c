/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the projection that the
 * reference's fast_jl CUDA kernel computes.  The product never links, loads
 * or calls this file; only tests, the smoke check and the CPU-baseline leg of
 * the benchmark do, and only as the checker.
 *
 * What it restates (paths are relative to the reference checkout):
 *   - the per-stream seed         fast_jl/random.cuh:13-22
 *   - which stream / draw / bit defines matrix element P[f, n]
 *                                 fast_jl/random.cuh:24-60 (element order inside a
 *                                 16x32 factor tile), fast_jl/fast_jl_kernel.cuh:34-45
 *                                 (column owned by a thread), :60-87 (one tile per
 *                                 16 features, in feature order), :121-127 (feature
 *                                 tile size), fast_jl/fast_jl.cu:42 (tile clamp)
 *   - which input element meets which tile row      fast_jl/data_loading.cuh:24-55
 *   - the generator itself: XORWOW seeded as curand_init(seed, 0, 0) and the
 *     Box-Muller pairing of curand_normal, as defined in the CUDA toolkit's
 *     curand_kernel.h / curand_normal.h (third-party, CUDA 12.9; the reference
 *     pins no version).
 *
 * Pins: the XORWOW core is checked against known answers from NVIDIA's cuRAND
 * *host* generator (tests/test_oracle_rng.py); the element map is checked
 * against golden vectors produced by the compiled reference kernel on a B200
 * (tests/golden/fastjl_*.npz).  Gaussian entries go through the host libm
 * (logf, sinf, cosf) where the GPU uses its own logf / __sincosf, so for the
 * Gaussian matrix this oracle is expected to agree with the GPU to within one
 * fp16 unit in the last place on a small fraction of entries, not bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TBO_RADEMACHER 0
#define TBO_NORMAL 1

typedef struct {
    uint32_t v[5];
    uint32_t d;
} xw_state;

/* curand_init(seed, 0, 0) for a seed that fits 32 bits (the kernel's seed is a
 * uint32_t widened to 64 bits, so the high word is always zero). */
static void xw_seed(xw_state *s, uint32_t seed) {
    uint32_t s0 = seed ^ 0xaad26b49u;
    uint32_t s1 = 0u ^ 0xf7dcefddu;
    uint32_t t0 = 1099087573u * s0;
    uint32_t t1 = 2591861531u * s1;
    s->d = 6615241u + t1 + t0;
    s->v[0] = 123456789u + t0;
    s->v[1] = 362436069u ^ t0;
    s->v[2] = 521288629u + t1;
    s->v[3] = 88675123u ^ t1;
    s->v[4] = 5783321u + t0;
}

static inline uint32_t xw_next(xw_state *s) {
    uint32_t t = s->v[0] ^ (s->v[0] >> 2);
    s->v[0] = s->v[1];
    s->v[1] = s->v[2];
    s->v[2] = s->v[3];
    s->v[3] = s->v[4];
    s->v[4] = (s->v[4] ^ (s->v[4] << 4)) ^ (t ^ (t << 1));
    s->d += 362437u;
    return s->v[4] + s->d;
}

static inline float f16_round(float x) { return (float)(_Float16)x; }

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* The two normals curand_normal hands out for the draw pair (x, y): first
 * s*sin(v), then s*cos(v). */
static inline void box_muller(uint32_t x, uint32_t y, float *first, float *second) {
    const float inv = 2.3283064e-10f;
    const float inv2pi = 2.3283064e-10f * 6.2831855f;
    float u = fmaf((float)x, inv, inv / 2);
    float v = fmaf((float)y, inv2pi, inv2pi / 2);
    float s = sqrtf(-2.0f * logf(u));
    *first = sinf(v) * s;
    *second = cosf(v) * s;
}

static inline uint32_t stream_seed(uint32_t seed, uint32_t column, uint32_t tile) {
    return seed + 658105236u * column + 359124577u * tile;
}

/* Geometry shared by every entry point. */
typedef struct {
    uint64_t F;
    uint32_t N, tiles, fts;
} geom;

static int make_geom(geom *g, uint64_t F, uint32_t N, uint32_t tiles) {
    if (F == 0 || N == 0 || (N % 32) != 0 || tiles == 0) return -1;
    g->F = F;
    g->N = N;
    g->tiles = (F < (uint64_t)tiles) ? (uint32_t)F : tiles;
    g->fts = (uint32_t)((F - 1) / g->tiles + 1);
    return 0;
}

/* One 16x32 factor tile (16 consecutive features x one warp's 32 columns) from
 * the 32 streams of that warp, advancing each stream. out[k*32 + nl]. */
static void factor_tile(int ptype, xw_state st[32], float out[16 * 32]) {
    for (int L = 0; L < 32; L++) {
        int kpar = L >> 4;          /* this stream feeds rows k with k&1 == kpar */
        int c0 = 2 * (L & 15);      /* and the column pair (c0, c0+1)            */
        if (ptype == TBO_RADEMACHER) {
            uint32_t bits = xw_next(&st[L]);
            for (int x = 0; x < 8; x++) {
                int k = 2 * x + kpar;
                out[k * 32 + c0] = (bits & 1u) ? 1.0f : -1.0f;
                bits >>= 1;
                out[k * 32 + c0 + 1] = (bits & 1u) ? 1.0f : -1.0f;
                bits >>= 1;
            }
        } else {
            for (int x = 0; x < 8; x++) {
                int k = 2 * x + kpar;
                uint32_t a = xw_next(&st[L]);
                uint32_t b = xw_next(&st[L]);
                float n0, n1;
                box_muller(a, b, &n0, &n1);
                out[k * 32 + c0] = f16_round(n0);
                out[k * 32 + c0 + 1] = f16_round(n1);
            }
        }
    }
}

/* ---- exported: RNG core, for the known-answer tests ---------------------- */

void tbo_xorwow_draws(uint32_t seed, uint32_t n, uint32_t *out) {
    xw_state s;
    xw_seed(&s, seed);
    for (uint32_t i = 0; i < n; i++) out[i] = xw_next(&s);
}

void tbo_box_muller(uint32_t x, uint32_t y, float *out2) {
    box_muller(x, y, &out2[0], &out2[1]);
}

uint32_t tbo_feature_tile_size(uint64_t F, uint32_t tiles) {
    geom g;
    if (make_geom(&g, F, 32, tiles)) return 0;
    return g.fts;
}

/* ---- exported: rows of the virtual matrix -------------------------------- */

/* out[i*N + n] = P[feats[i], n].  Cost grows with the position of the feature
 * inside its tile (streams are sequential). */
int tbo_matrix_rows(int ptype, uint64_t F, uint32_t N, uint32_t seed, uint32_t tiles,
                    const uint64_t *feats, uint32_t nfeats, float *out) {
    geom g;
    if (make_geom(&g, F, N, tiles)) return -1;
    for (uint32_t i = 0; i < nfeats; i++) {
        uint64_t f = feats[i];
        if (f >= F) return -2;
        uint32_t by = (uint32_t)(f / g.fts);
        uint32_t t = (uint32_t)(f % g.fts);
        uint32_t r = t >> 4, k = t & 15;
#pragma omp parallel for schedule(static)
        for (uint32_t w = 0; w < N / 32; w++) {
            xw_state st[32];
            float tile[16 * 32];
            for (int L = 0; L < 32; L++) xw_seed(&st[L], stream_seed(seed, w * 32 + L, by));
            for (uint32_t rr = 0; rr <= r; rr++) factor_tile(ptype, st, tile);
            memcpy(out + (size_t)i * N + w * 32, tile + k * 32, 32 * sizeof(float));
        }
    }
    return 0;
}

/* ---- exported: the projection itself, accumulated in fp64 ---------------- */

/* dtype: 0 fp16, 1 bf16, 2 fp32, 3 fp64.  round_f16 != 0 rounds each input to
 * fp16 first, as the reference does for fp32 inputs (data_loading.cuh:10).
 * out[b*N + n] = sum_f G[b*ld + f] * P[f, n]. */
static void project_column_group(int ptype, const void *G, int dtype, uint64_t B, uint64_t F, uint64_t ld,
                                 const geom *g, uint32_t seed, int round_f16, uint32_t w, double *out,
                                 uint64_t out_ld, uint64_t out_col0) {
    /* the 32 output columns 32w .. 32w+31, written to out[b*out_ld + out_col0 + nl] */
    uint32_t ntiles_used = (uint32_t)((F - 1) / g->fts + 1);
    double *acc = (double *)calloc((size_t)B * 32, sizeof(double));
    float *gin = (float *)malloc(sizeof(float) * B * 16);
    float tile[16 * 32];
    xw_state st[32];
    for (uint32_t by = 0; by < ntiles_used; by++) {
        uint64_t f0 = (uint64_t)by * g->fts;
        uint64_t len = F - f0 < g->fts ? F - f0 : g->fts;
        for (int L = 0; L < 32; L++) xw_seed(&st[L], stream_seed(seed, w * 32 + L, by));
        for (uint64_t t0 = 0; t0 < len; t0 += 16) {
            factor_tile(ptype, st, tile);
            int kk = (int)(len - t0 < 16 ? len - t0 : 16);
            for (uint64_t b = 0; b < B; b++)
                for (int k = 0; k < kk; k++) {
                    size_t idx = (size_t)b * ld + f0 + t0 + k;
                    float x;
                    switch (dtype) {
                    case 0: x = (float)((const _Float16 *)G)[idx]; break;
                    case 1: x = bf16_to_f32(((const uint16_t *)G)[idx]); break;
                    case 2: x = ((const float *)G)[idx]; break;
                    default: x = 0; break;
                    }
                    if (dtype == 3) {
                        double xd = ((const double *)G)[idx];
                        gin[b * 16 + k] = 0;
                        /* fp64 inputs bypass the float staging below */
                        for (int nl = 0; nl < 32; nl++) acc[b * 32 + nl] += xd * (double)tile[k * 32 + nl];
                        continue;
                    }
                    if (round_f16) x = f16_round(x);
                    gin[b * 16 + k] = x;
                }
            if (dtype != 3)
                for (uint64_t b = 0; b < B; b++)
                    for (int k = 0; k < kk; k++) {
                        double x = (double)gin[b * 16 + k];
                        const float *row = tile + k * 32;
                        double *a = acc + b * 32;
                        for (int nl = 0; nl < 32; nl++) a[nl] += x * (double)row[nl];
                    }
        }
    }
    for (uint64_t b = 0; b < B; b++)
        for (int nl = 0; nl < 32; nl++) out[b * out_ld + out_col0 + nl] = acc[b * 32 + nl];
    free(acc);
    free(gin);
}

int tbo_project(int ptype, const void *G, int dtype, uint64_t B, uint64_t F, uint64_t ld,
                uint32_t N, uint32_t seed, uint32_t tiles, int round_f16, double *out) {
    geom g;
    if (make_geom(&g, F, N, tiles)) return -1;
    if (dtype < 0 || dtype > 3) return -3;
    memset(out, 0, sizeof(double) * B * N);
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t w = 0; w < N / 32; w++)
        project_column_group(ptype, G, dtype, B, F, ld, &g, seed, round_f16, w, out, N, (uint64_t)w * 32);
    return 0;
}

/* The same for some 32-column groups only (a column of the matrix does not depend on how many columns
 * there are): out[b*(32*ngroups) + 32*i + nl] = sum_f G[b*ld + f] * P[f, 32*groups[i] + nl].  Lets a test
 * check a few columns of a projection whose full oracle would take minutes. */
int tbo_project_column_groups(int ptype, const void *G, int dtype, uint64_t B, uint64_t F, uint64_t ld,
                              uint32_t seed, uint32_t tiles, int round_f16, const uint32_t *groups,
                              uint32_t ngroups, double *out) {
    geom g;
    if (ngroups == 0 || make_geom(&g, F, 32, tiles)) return -1;
    if (dtype < 0 || dtype > 3) return -3;
    memset(out, 0, sizeof(double) * B * 32 * ngroups);
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t i = 0; i < ngroups; i++)
        project_column_group(ptype, G, dtype, B, F, ld, &g, seed, round_f16, groups[i], out,
                             (uint64_t)32 * ngroups, (uint64_t)i * 32);
    return 0;
}
