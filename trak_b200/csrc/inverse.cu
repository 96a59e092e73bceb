// Regularised SPD inverse for the after-kernel:  A <- inv(A + lambda*I), optionally divided by
// the mean absolute entry (the reference's rescale, trak/score_computers.py:160-168).
//
// The reference calls torch.linalg.inv (LU).  A + lambda*I is symmetric positive definite, so this
// goes through Cholesky, all in fp32:
//   1. two-level right-looking Cholesky A = L L^T: 64-wide steps (panel solve and update as tiled
//      fp32 kernels) stay inside a 512-wide block column, and everything to the right of it gets
//      one rank-512 update per block column from the tensor cores (gemm.cu, symmetric, chunked
//      accumulation); the CTA that updates the first tile of the trailing block factors and inverts
//      it right away (it is the next diagonal block) while the other CTAs finish the update;
//   2. W = L^-1 bottom-up: the 64-wide diagonal blocks are inverted with the factorisation, then
//      neighbouring blocks of size s = 64, 128, ... are merged, W21 = -W22 (L21 W11): all pairs of
//      one size in two batched fp32 launches up to s = 512, tensor-core GEMMs (gemm.cu, chunked
//      accumulation) from s = 1024 on;
//   3. A^-1 = W^T W with the tensor-core GEMM of gemm.cu (symmetric mode, chunked accumulation);
//   4. mean |entry| with a fixed-order two-pass reduction, then the rescale.
// A non-positive pivot is recorded in the device status word (ST_NOT_SPD).
#include <algorithm>

#include "gemm.h"
#include "host_util.h"
#include "ptx.cuh"

namespace tb {

constexpr int NB = 64;      // panel width
constexpr int OUTER = 512;    // block column of the two-level Cholesky
constexpr int MERGE_TC_FROM = 1024;  // block size from which the merge products go to the tensor cores
constexpr int TS = 68;      // padded row length of a shared-memory tile (floats)

// acc[4][4] += sum_t At[t][ty*4 + i] * Bt[t][tx*4 + j]   (both tiles stored t-major)
__device__ __forceinline__ void tile_mma(const float (*At)[TS], const float (*Bt)[TS], int ty, int tx,
                                         float (&acc)[4][4]) {
#pragma unroll 8
    for (int t = 0; t < NB; ++t) {
        const float4 a = *reinterpret_cast<const float4*>(&At[t][ty * 4]);
        const float4 b = *reinterpret_cast<const float4*>(&Bt[t][tx * 4]);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
}

// dst[t][i] = src[i*ld + t]  (operand element (i, t) is row-major in global memory), zero outside
__device__ __forceinline__ void load_tile_T(float (*dst)[TS], const float* src, int64_t ld, int rows, int cols) {
    for (int e = threadIdx.x; e < NB * NB; e += blockDim.x) {
        const int i = e >> 6, t = e & 63;
        dst[t][i] = (i < rows && t < cols) ? src[(int64_t)i * ld + t] : 0.0f;
    }
}
// dst[t][c] = src[t*ld + c]
__device__ __forceinline__ void load_tile_N(float (*dst)[TS], const float* src, int64_t ld, int rows, int cols) {
    for (int e = threadIdx.x; e < NB * NB; e += blockDim.x) {
        const int t = e >> 6, c = e & 63;
        dst[t][c] = (t < rows && c < cols) ? src[(int64_t)t * ld + c] : 0.0f;
    }
}

__global__ void add_diag_kernel(float* A, int64_t lda, int k, float lambda) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < k) A[(int64_t)i * lda + i] += lambda;
}

// Factors the jb x jb diagonal block A = L L^T and inverts L in the same sweep; writes L back over the
// lower triangle and inv(L) (lower, zero above, zero-padded to 64 x 64) to dinv.  256 threads as a
// 16 x 16 grid, thread (ty, tx) keeping the 4 x 4 piece S[4 ty.., 4 tx..] of the block and the same piece
// of W (which starts as the identity and ends as inv(L): forward elimination of [L | I]) in registers.
// The block is walked four columns at a time, two barriers per step instead of two per column (a
// column-by-column sweep spent 1000 cycles per column, almost all of it waiting: 33 us per block):
//   1. the thread on the diagonal publishes its 4 x 4 piece D;
//   2. every thread of piece column q factors D = Ld Ld^T itself (a few dozen operations), turns its
//      piece into the matching rows of L (B Ld^-T) and publishes them; every thread of piece row q
//      applies Ld^-1 to its four rows of W, which makes them final, and publishes them;
//   3. the threads below apply the rank-four updates  S -= L_q L_q^T  (pieces right of column q)
//      and  W -= L_q W_q  (pieces up to column q; W_q is zero beyond).
// Rows and columns beyond jb are an identity block.  `buf` is 16 + 2 * 256 floats of shared memory.
struct Chol4 {
    float l10, l20, l30, l21, l31, l32;  // strictly lower part of Ld
    float r0, r1, r2, r3;                // reciprocals of its diagonal
    float d0, d1, d2, d3;                // its diagonal
    bool ok;
};
__device__ __forceinline__ float rsqrt_newton(float d) {
    float r = rsqrtf(d);
    return r * (1.5f - 0.5f * d * r * r);
}
__device__ __forceinline__ Chol4 chol4(const float* D) {  // D: 4 x 4 row-major, lower part used
    Chol4 c;
    c.ok = true;
    float p = D[0];
    c.ok = c.ok && p > 0.0f;
    c.r0 = rsqrt_newton(p);
    c.d0 = p * c.r0;
    c.l10 = D[4] * c.r0;
    c.l20 = D[8] * c.r0;
    c.l30 = D[12] * c.r0;
    p = fmaf(-c.l10, c.l10, D[5]);
    c.ok = c.ok && p > 0.0f;
    c.r1 = rsqrt_newton(p);
    c.d1 = p * c.r1;
    c.l21 = fmaf(-c.l20, c.l10, D[9]) * c.r1;
    c.l31 = fmaf(-c.l30, c.l10, D[13]) * c.r1;
    p = fmaf(-c.l21, c.l21, fmaf(-c.l20, c.l20, D[10]));
    c.ok = c.ok && p > 0.0f;
    c.r2 = rsqrt_newton(p);
    c.d2 = p * c.r2;
    c.l32 = fmaf(-c.l31, c.l21, fmaf(-c.l30, c.l20, D[14])) * c.r2;
    p = fmaf(-c.l32, c.l32, fmaf(-c.l31, c.l31, fmaf(-c.l30, c.l30, D[15])));
    c.ok = c.ok && p > 0.0f;
    c.r3 = rsqrt_newton(p);
    c.d3 = p * c.r3;
    return c;
}
// x <- Ld^-1 x for one column of four values (forward substitution)
__device__ __forceinline__ void solve4(const Chol4& c, float& x0, float& x1, float& x2, float& x3) {
    x0 = x0 * c.r0;
    x1 = fmaf(-c.l10, x0, x1) * c.r1;
    x2 = fmaf(-c.l21, x1, fmaf(-c.l20, x0, x2)) * c.r2;
    x3 = fmaf(-c.l32, x2, fmaf(-c.l31, x1, fmaf(-c.l30, x0, x3))) * c.r3;
}
__device__ void chol_block(float* A, int64_t lda, int jb, float* dinv, uint32_t* status, float* buf, int* bad) {
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    float* diagbuf = buf;                                                  // [4][4]
    float (*colbuf)[4] = reinterpret_cast<float(*)[4]>(buf + 16);          // [64][4]: rows of L_q
    float (*rowbuf)[NB] = reinterpret_cast<float(*)[NB]>(buf + 16 + 256);  // [4][64]: rows of W_q
    float sblk[4][4], wblk[4][4];
    if (tid == 0) *bad = 0;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = ty * 4 + a, j = tx * 4 + b;
            // the diagonal pieces hold both triangles (symmetric), the others only what lies below
            const bool in = i < jb && j < jb && (j <= i || tx == ty);
            sblk[a][b] = in ? A[(int64_t)(j <= i ? i : j) * lda + (j <= i ? j : i)] : (i == j ? 1.0f : 0.0f);
            wblk[a][b] = i == j ? 1.0f : 0.0f;
        }
    const int steps = (jb + 3) >> 2;
    for (int q = 0; q < steps; ++q) {
        if (ty == q && tx == q) {
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) diagbuf[a * 4 + b] = sblk[a][b];
        }
        __syncthreads();
        if (tx == q || ty == q) {
            const Chol4 c = chol4(diagbuf);
            if (ty == q && tx == q && !c.ok) *bad = 1;
            if (tx == q && ty >= q) {
                if (ty == q) {  // the diagonal piece becomes Ld
                    sblk[0][0] = c.d0;
                    sblk[1][0] = c.l10; sblk[1][1] = c.d1;
                    sblk[2][0] = c.l20; sblk[2][1] = c.l21; sblk[2][2] = c.d2;
                    sblk[3][0] = c.l30; sblk[3][1] = c.l31; sblk[3][2] = c.l32; sblk[3][3] = c.d3;
                    sblk[0][1] = sblk[0][2] = sblk[0][3] = sblk[1][2] = sblk[1][3] = sblk[2][3] = 0.0f;
                } else {        // rows of L below it: B Ld^-T, i.e. Ld^-1 applied along each row
#pragma unroll
                    for (int a = 0; a < 4; ++a) solve4(c, sblk[a][0], sblk[a][1], sblk[a][2], sblk[a][3]);
                }
#pragma unroll
                for (int a = 0; a < 4; ++a)
                    *reinterpret_cast<float4*>(colbuf[ty * 4 + a]) =
                        make_float4(sblk[a][0], sblk[a][1], sblk[a][2], sblk[a][3]);
            }
            if (ty == q) {      // four rows of W become final: Ld^-1 applied down each column
#pragma unroll
                for (int b = 0; b < 4; ++b) solve4(c, wblk[0][b], wblk[1][b], wblk[2][b], wblk[3][b]);
#pragma unroll
                for (int a = 0; a < 4; ++a)
                    *reinterpret_cast<float4*>(&rowbuf[a][tx * 4]) =
                        make_float4(wblk[a][0], wblk[a][1], wblk[a][2], wblk[a][3]);
            }
        }
        __syncthreads();
        if (ty > q) {
            float li[4][4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float4 v = *reinterpret_cast<const float4*>(colbuf[ty * 4 + a]);
                li[a][0] = v.x; li[a][1] = v.y; li[a][2] = v.z; li[a][3] = v.w;
            }
            if (tx > q && tx <= ty) {
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const float4 v = *reinterpret_cast<const float4*>(colbuf[tx * 4 + b]);
#pragma unroll
                    for (int a = 0; a < 4; ++a)
                        sblk[a][b] = fmaf(-li[a][3], v.w, fmaf(-li[a][2], v.z, fmaf(-li[a][1], v.y,
                                          fmaf(-li[a][0], v.x, sblk[a][b]))));
                }
            }
            if (tx <= q) {
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const float4 v = *reinterpret_cast<const float4*>(&rowbuf[cc][tx * 4]);
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        wblk[a][0] = fmaf(-li[a][cc], v.x, wblk[a][0]);
                        wblk[a][1] = fmaf(-li[a][cc], v.y, wblk[a][1]);
                        wblk[a][2] = fmaf(-li[a][cc], v.z, wblk[a][2]);
                        wblk[a][3] = fmaf(-li[a][cc], v.w, wblk[a][3]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = ty * 4 + a, j = tx * 4 + b;
            const bool in = i < jb && j <= i;
            if (in) A[(int64_t)i * lda + j] = sblk[a][b];
            dinv[i * NB + j] = in ? wblk[a][b] : 0.0f;
        }
    __syncthreads();
    if (tid == 0 && *bad) atomicCAS(status, 0u, (uint32_t)ST_NOT_SPD);
}

__global__ void __launch_bounds__(256) chol_diag_kernel(float* A, int64_t lda, int jb, float* dinv,
                                                        uint32_t* status) {
    __shared__ __align__(16) float buf[16 + 2 * 256];
    __shared__ int bad;
    chol_block(A, lda, jb, dinv, status, buf, &bad);
}

// MODE 0 (Cholesky panel):  X[i, c] <- sum_t X[i, t] * D[c, t]      (X * D^T, in place)
// MODE 1 (inverse, step 1): T[i, c] <- sum_t X[i, t] * D[t, c]      (X * D, to a separate buffer)
// X is r x jb (leading dimension ldx), D is the zero-padded 64 x 64 block; one CTA per 64 rows.
template <int MODE>
__global__ void __launch_bounds__(256) panel_kernel(float* X, int64_t ldx, int r, int jb, const float* D,
                                                    float* T, int64_t ldt) {
    __shared__ __align__(16) float At[NB][TS];
    __shared__ __align__(16) float Bt[NB][TS];
    const int i0 = blockIdx.x * NB;
    const int rows = min(NB, r - i0);
    load_tile_T(At, X + (int64_t)i0 * ldx, ldx, rows, jb);
    if (MODE == 0)
        load_tile_T(Bt, D, NB, NB, NB);  // Bt[t][c] = D[c][t]
    else
        load_tile_N(Bt, D, NB, NB, NB);  // Bt[t][c] = D[t][c]
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    tile_mma(At, Bt, ty, tx, acc);
    __syncthreads();  // everyone has read X before anyone overwrites it (MODE 0 is in place)
    float* out = MODE == 0 ? X : T;
    const int64_t ldo = MODE == 0 ? ldx : ldt;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ii = ty * 4 + i, c = tx * 4 + j;
            if (ii < rows && c < jb) out[(int64_t)(i0 + ii) * ldo + c] = acc[i][j];
        }
}

// Trailing update of a Cholesky step:  C[i, j] -= sum_t P[i, t] * P[j, t]  for the tiles on or below
// the diagonal in the first gridDim.x tile columns of the r x r trailing block; P is the r x jb panel
// (same leading dimension as C).  The CTA of tile (0, 0) then holds the next diagonal block in its
// final state and factors it on the spot (dinv_next = where its inverse goes), overlapping with the
// other CTAs' updates.
__global__ void __launch_bounds__(256) syrk_update_kernel(float* C, const float* P, int64_t ld, int r, int jb,
                                                          float* dinv_next, uint32_t* status) {
    if (blockIdx.x > blockIdx.y) return;  // tile column > tile row: upper part, not needed
    __shared__ __align__(16) float At[NB][TS];
    __shared__ __align__(16) float Bt[NB][TS];
    __shared__ int bad;
    const int i0 = blockIdx.y * NB, j0 = blockIdx.x * NB;
    const int rows = min(NB, r - i0), cols = min(NB, r - j0);
    load_tile_T(At, P + (int64_t)i0 * ld, ld, rows, jb);
    load_tile_T(Bt, P + (int64_t)j0 * ld, ld, cols, jb);
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    tile_mma(At, Bt, ty, tx, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ii = ty * 4 + i, jj = tx * 4 + j;
            if (ii < rows && jj < cols) C[(int64_t)(i0 + ii) * ld + j0 + jj] -= acc[i][j];
        }
    if (blockIdx.x == 0 && blockIdx.y == 0 && dinv_next != nullptr) {
        __syncthreads();  // the tile is complete in global memory and the operand tiles are free
        chol_block(C, ld, rows, dinv_next, status, &At[0][0], &bad);
    }
}

// Inverse of the triangular factor, bottom-up.  At block size s the matrix holds, in every aligned
// diagonal block of size s, the finished inverse W of that block of L (upper triangle zero).  Pair p
// joins the blocks at base = 2 s p:  W11 = [base, base + s),  W22 = the s2 = min(s, k - base - s)
// rows after it, and the block below W11 still holds L21.  The inverse of the joined block needs
//     W21 = - W22 (L21 W11),
// computed as T = L21 W11 (STEP 0, into Tbuf[row][0..s)) and W21 = -W22 T (STEP 1, over L21).
// One CTA per 64 x 64 tile of the result, blockIdx.z = pair; the triangles skip their zero tiles.
template <int STEP>
__global__ void __launch_bounds__(256) tri_merge_kernel(float* A, int64_t lda, int k, int s, float* Tbuf) {
    __shared__ __align__(16) float At[NB][TS];
    __shared__ __align__(16) float Bt[NB][TS];
    const int base = (int)blockIdx.z * 2 * s;
    const int s2 = min(s, k - base - s);
    const int i0 = blockIdx.y * NB, j0 = blockIdx.x * NB;
    if (s2 <= 0 || i0 >= s2) return;
    const int rows = min(NB, s2 - i0), cols = min(NB, s - j0);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    const float* L21 = A + (int64_t)(base + s) * lda + base;
    const float* W11 = A + (int64_t)base * lda + base;
    const float* W22 = A + (int64_t)(base + s) * lda + base + s;
    const float* T = Tbuf + (int64_t)(base + s) * s;
    // STEP 0: t runs over the columns of L21 / rows of W11, and W11[t, j] = 0 for t < j
    // STEP 1: t runs over the columns of W22 / rows of T,   and W22[i, t] = 0 for t > i
    const int t_first = STEP == 0 ? j0 : 0;
    const int t_end = STEP == 0 ? s : min(s2, i0 + NB);
    for (int t0 = t_first; t0 < t_end; t0 += NB) {
        const int tc = min(NB, t_end - t0);
        if (STEP == 0) {
            load_tile_T(At, L21 + (int64_t)i0 * lda + t0, lda, rows, tc);
            load_tile_N(Bt, W11 + (int64_t)t0 * lda + j0, lda, tc, cols);
        } else {
            load_tile_T(At, W22 + (int64_t)i0 * lda + t0, lda, rows, tc);
            load_tile_N(Bt, T + (int64_t)t0 * s + j0, s, tc, cols);
        }
        __syncthreads();
        tile_mma(At, Bt, ty, tx, acc);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ii = ty * 4 + i, jj = tx * 4 + j;
            if (ii < rows && jj < cols) {
                if (STEP == 0)
                    Tbuf[(int64_t)(base + s + i0 + ii) * s + j0 + jj] = acc[i][j];
                else
                    A[(int64_t)(base + s + i0 + ii) * lda + base + j0 + jj] = -acc[i][j];
            }
        }
}

// Every 64-wide diagonal block <- its inverse from the factorisation (lower, zero above); one CTA each.
__global__ void write_diag_inverse_kernel(float* A, int64_t lda, int k, const float* dinv) {
    const int j0 = blockIdx.x * NB, jb = min(NB, k - j0);
    const float* D = dinv + (size_t)blockIdx.x * NB * NB;
    for (int e = threadIdx.x; e < NB * NB; e += blockDim.x) {
        const int i = e >> 6, j = e & 63;
        if (i < jb && j < jb) A[(int64_t)(j0 + i) * lda + j0 + j] = D[e];
    }
}
// The three whole-matrix passes below walk rows per CTA and columns per thread (no index division), four
// columns at a time where the rows are 16-byte aligned.
__device__ __forceinline__ bool rows_are_vec4(const float* A, int64_t lda, int k) {
    return (k & 3) == 0 && (lda & 3) == 0 && (reinterpret_cast<uintptr_t>(A) & 15u) == 0;
}

__global__ void zero_upper_kernel(float* A, int64_t lda, int k) {
    for (int i = blockIdx.x; i < k; i += gridDim.x) {
        float* row = A + (int64_t)i * lda;
        for (int j = i + 1 + threadIdx.x; j < k; j += blockDim.x) row[j] = 0.0f;
    }
}

constexpr int RED_BLOCKS = 1024;
__global__ void __launch_bounds__(256) abs_partial_kernel(const float* A, int64_t lda, int k, double* partial) {
    __shared__ double sh[256];
    double s = 0.0;
    const bool vec = rows_are_vec4(A, lda, k);
    for (int i = blockIdx.x; i < k; i += RED_BLOCKS) {   // fixed assignment of entries to threads: same sum every run
        const float* row = A + (int64_t)i * lda;
        if (vec) {
            for (int j4 = threadIdx.x; j4 < (k >> 2); j4 += 256) {
                const float4 v = *reinterpret_cast<const float4*>(row + 4 * j4);
                s += (double)fabsf(v.x) + (double)fabsf(v.y) + (double)fabsf(v.z) + (double)fabsf(v.w);
            }
        } else {
            for (int j = threadIdx.x; j < k; j += 256) s += (double)fabsf(row[j]);
        }
    }
    sh[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
__global__ void __launch_bounds__(256) abs_final_kernel(const double* partial, int k, float* mean_out) {
    __shared__ double sh[256];
    double s = 0.0;
    for (int e = threadIdx.x; e < RED_BLOCKS; e += 256) s += partial[e];
    sh[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *mean_out = (float)(sh[0] / ((double)k * (double)k));
}
__global__ void scale_by_inverse_kernel(float* A, int64_t lda, int k, const float* mean) {
    const float inv = 1.0f / *mean;
    const bool vec = rows_are_vec4(A, lda, k);
    for (int i = blockIdx.x; i < k; i += gridDim.x) {
        float* row = A + (int64_t)i * lda;
        if (vec) {
            for (int j4 = threadIdx.x; j4 < (k >> 2); j4 += blockDim.x) {
                float4 v = *reinterpret_cast<float4*>(row + 4 * j4);
                v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
                *reinterpret_cast<float4*>(row + 4 * j4) = v;
            }
        } else {
            for (int j = threadIdx.x; j < k; j += blockDim.x) row[j] *= inv;
        }
    }
}

struct InvLayout {
    size_t dinv, partial, mean, scratch, total;
};
// Scratch of the merge at block size s (first block s rows, second block s2 rows): both packed
// operands of the larger product and T; all of it is free again before W^T W is packed.
static size_t merge_scratch_bytes(int64_t s, int64_t s2) {
    const size_t pa = std::max(packed_geometry(TB_F32, s2, s).bytes, packed_geometry(TB_F32, s2, s2).bytes);
    const size_t pb = packed_geometry(TB_F32, s, std::max(s, s2)).bytes;
    return pa + pb + align_up((size_t)s2 * s * sizeof(float), 1024);
}
static InvLayout inv_layout(int64_t k) {
    InvLayout l;
    const size_t nblk = (size_t)((k + NB - 1) / NB);
    size_t off = 0;
    l.dinv = off;
    off += align_up(nblk * NB * NB * sizeof(float), 256);
    l.partial = off;
    off += align_up(RED_BLOCKS * sizeof(double), 256);
    l.mean = off;
    off += 256;
    l.scratch = off;
    size_t need = packed_geometry(TB_F32, k, k).bytes;  // also covers the r x OUTER panels of the Cholesky
    for (int64_t s = NB; s < k; s *= 2) {
        if (s < MERGE_TC_FROM)
            need = std::max(need, align_up((size_t)k * s * sizeof(float), 1024));  // T of every pair
        else
            need = std::max(need, merge_scratch_bytes(s, std::min<int64_t>(s, k - s)));
    }
    off += need;
    l.total = off + 1024;
    return l;
}

}  // namespace tb

extern "C" {

size_t tb_spd_inverse_workspace_bytes(int64_t k) {
    if (k <= 0) return 0;
    return tb::inv_layout(k).total;
}

int tb_spd_inverse(int device, void* stream_, float* A, int64_t k, int64_t lda, float lambda,
                   int rescale_by_mean_abs, float* mean_abs_out, void* ws, size_t ws_bytes) {
    using namespace tb;
    if (k <= 0 || lda < k || k > 0x3fffffff) return TB_ERR_BAD_SHAPE;
    if (!A) return TB_ERR_BAD_ARG;
    if (!ws || ((uintptr_t)ws & 255u) != 0 || ws_bytes < tb_spd_inverse_workspace_bytes(k)) return TB_ERR_WORKSPACE;
    int sm_count = 0;
    int rc = select_device(device, &sm_count);
    if (rc != TB_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const InvLayout l = inv_layout(k);
    uint8_t* base = static_cast<uint8_t*>(ws);
    float* dinv = reinterpret_cast<float*>(base + l.dinv);
    double* partial = reinterpret_cast<double*>(base + l.partial);
    float* mean = reinterpret_cast<float*>(base + l.mean);
    uint8_t* scratch = base + l.scratch;
    const int K = (int)k;
    const int nblk = (K + NB - 1) / NB;

    if (lambda != 0.0f) add_diag_kernel<<<(K + 255) / 256, 256, 0, stream>>>(A, lda, K, lambda);

    // 1. Cholesky (lower triangle of A becomes L); dinv[b] = inverse of the b-th diagonal block of L.
    //    Two levels: inside a block column of OUTER columns the 64-wide steps update only that block
    //    column (fp32 tiles); what lies to its right gets one rank-OUTER update per block column from
    //    the tensor cores (symmetric chunked GEMM, alpha = -1, accumulating).  The first diagonal block
    //    of a block column is factored by its own launch, every other one inside the update that
    //    completes it.
    for (int o0 = 0; o0 < K; o0 += OUTER) {
        const int o1 = o0 + OUTER < K ? o0 + OUTER : K;  // end of this block column
        chol_diag_kernel<<<1, 256, 0, stream>>>(A + (int64_t)o0 * lda + o0, lda, o1 - o0 < NB ? o1 - o0 : NB,
                                                dinv + (size_t)(o0 / NB) * NB * NB, status_ptr(device));
        for (int j0 = o0; j0 < o1; j0 += NB) {
            const int b = j0 / NB, jb = K - j0 < NB ? K - j0 : NB, r = K - j0 - jb;
            if (r <= 0) break;
            float* A21 = A + (int64_t)(j0 + jb) * lda + j0;
            const int rt = (r + NB - 1) / NB;
            panel_kernel<0><<<rt, 256, 0, stream>>>(A21, lda, r, jb, dinv + (size_t)b * NB * NB, nullptr, 0);
            const int wt = (o1 - j0 - jb + NB - 1) / NB;  // tile columns left in the block column
            if (wt > 0)
                syrk_update_kernel<<<dim3(wt, rt), 256, 0, stream>>>(A + (int64_t)(j0 + jb) * lda + j0 + jb, A21, lda, r, jb,
                                                                      dinv + (size_t)(b + 1) * NB * NB, status_ptr(device));
        }
        const int64_t r = K - o1;
        if (r > 0) {
            // A22 -= L21 L21^T with L21 = the r x (o1 - o0) block below this block column's diagonal block
            const int64_t w = o1 - o0;
            uint16_t* packed = reinterpret_cast<uint16_t*>(scratch);
            const Packed g = packed_geometry(TB_F32, r, w);
            rc = launch_pack(A + (int64_t)o1 * lda + o0, TB_F32, false, (uint64_t)r, (uint64_t)w, (uint64_t)lda, packed, g,
                             sm_count, stream);
            if (rc != TB_OK) return rc;
            rc = launch_gemm(device, stream, packed, g, packed, g, TB_F32, r, r, A + (int64_t)o1 * lda + o1, lda, nullptr,
                             -1.0f, 1, 1, 1);
            if (rc != TB_OK) return rc;
        }
    }
    TB_CUDA(cudaGetLastError());

    // 2. W = L^-1: clear the upper triangle, put the inverted diagonal blocks in place, then merge
    //    neighbouring blocks of size 64, 128, ...
    zero_upper_kernel<<<sm_count * 8, 256, 0, stream>>>(A, lda, K);
    write_diag_inverse_kernel<<<nblk, 256, 0, stream>>>(A, lda, K, dinv);
    for (int64_t s = NB; s < k; s *= 2) {
        const int pairs = (int)((k + 2 * s - 1) / (2 * s));
        if (s < MERGE_TC_FROM) {
            float* Tbuf = reinterpret_cast<float*>(scratch);
            const dim3 grid((unsigned)(s / NB), (unsigned)(s / NB), (unsigned)pairs);
            tri_merge_kernel<0><<<grid, 256, 0, stream>>>(A, lda, K, (int)s, Tbuf);
            tri_merge_kernel<1><<<grid, 256, 0, stream>>>(A, lda, K, (int)s, Tbuf);
            continue;
        }
        for (int pr = 0; pr < pairs; ++pr) {
            const int64_t b0 = (int64_t)pr * 2 * s, s2 = std::min<int64_t>(s, k - b0 - s);
            if (s2 <= 0) continue;
            float* W11 = A + b0 * lda + b0;
            float* L21 = A + (b0 + s) * lda + b0;
            float* W22 = A + (b0 + s) * lda + b0 + s;
            const Packed g_l21 = packed_geometry(TB_F32, s2, s), g_w22 = packed_geometry(TB_F32, s2, s2);
            const Packed g_w11t = packed_geometry(TB_F32, s, s), g_tt = packed_geometry(TB_F32, s, s2);
            const size_t pa_bytes = std::max(g_l21.bytes, g_w22.bytes), pb_bytes = std::max(g_w11t.bytes, g_tt.bytes);
            uint16_t* pa = reinterpret_cast<uint16_t*>(scratch);
            uint16_t* pb = reinterpret_cast<uint16_t*>(scratch + pa_bytes);
            float* T = reinterpret_cast<float*>(scratch + pa_bytes + pb_bytes);
            // T[s2 x s] = L21 . W11 = L21 . (W11^T)^T
            rc = launch_pack(L21, TB_F32, false, (uint64_t)s2, (uint64_t)s, (uint64_t)lda, pa, g_l21, sm_count, stream);
            if (rc != TB_OK) return rc;
            rc = launch_pack(W11, TB_F32, true, (uint64_t)s, (uint64_t)s, (uint64_t)lda, pb, g_w11t, sm_count, stream);
            if (rc != TB_OK) return rc;
            rc = launch_gemm(device, stream, pa, g_l21, pb, g_w11t, TB_F32, s2, s, T, s, nullptr, 1.0f, 0, 0, 1);
            if (rc != TB_OK) return rc;
            // W21[s2 x s] = - W22 . T = - W22 . (T^T)^T, written over L21
            rc = launch_pack(W22, TB_F32, false, (uint64_t)s2, (uint64_t)s2, (uint64_t)lda, pa, g_w22, sm_count, stream);
            if (rc != TB_OK) return rc;
            rc = launch_pack(T, TB_F32, true, (uint64_t)s, (uint64_t)s2, (uint64_t)s, pb, g_tt, sm_count, stream);
            if (rc != TB_OK) return rc;
            rc = launch_gemm(device, stream, pa, g_w22, pb, g_tt, TB_F32, s2, s, L21, lda, nullptr, -1.0f, 0, 0, 1);
            if (rc != TB_OK) return rc;
        }
    }
    TB_CUDA(cudaGetLastError());

    // 3. A^-1 = W^T W (full symmetric result written over A; the operand was packed first)
    {
        uint16_t* packed = reinterpret_cast<uint16_t*>(scratch);
        const Packed g = packed_geometry(TB_F32, k, k);
        rc = launch_pack(A, TB_F32, true, (uint64_t)k, (uint64_t)k, (uint64_t)lda, packed, g, sm_count, stream);
        if (rc != TB_OK) return rc;
        rc = launch_gemm(device, stream, packed, g, packed, g, TB_F32, k, k, A, lda, nullptr, 1.0f, 0, 1, 1);
        if (rc != TB_OK) return rc;
    }

    // 4. mean |entry| and the reference's rescale
    if (rescale_by_mean_abs || mean_abs_out) {
        abs_partial_kernel<<<RED_BLOCKS, 256, 0, stream>>>(A, lda, K, partial);
        abs_final_kernel<<<1, 256, 0, stream>>>(partial, K, mean);
        if (mean_abs_out)
            TB_CUDA(cudaMemcpyAsync(mean_abs_out, mean, sizeof(float), cudaMemcpyDeviceToDevice, stream));
        if (rescale_by_mean_abs) scale_by_inverse_kernel<<<sm_count * 8, 256, 0, stream>>>(A, lda, K, mean);
    }
    TB_CUDA(cudaGetLastError());
    return TB_OK;
}

}  // extern "C"
