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
// 16 x 16 grid, each keeping a 4 x 4 piece of the block and of the inverse in registers.  Column c:
// the owners publish the current column c of the block and row c of the inverse in shared memory,
// one barrier, then every thread applies the rank-one updates
//     S[i][j] -= S[i][c] S[j][c] / pivot   (i, j > c),     W[i][:] -= S[i][c] W[c][:] / pivot   (i > c)
// (the second is forward elimination of [L | I]) with r = 1/sqrt(pivot) folded into both factors and
// the operands of rows and columns <= c replaced by zero, so the sixteen multiply-adds of a piece need
// no predicates.  Column c of the block and row c of the inverse are final after step c up to the
// factor r, which is kept per column and applied once at the end.  The buffers alternate between
// columns, so one barrier per column is enough.  Rows and columns beyond jb are an identity block.
// `buf` is 5 * 64 floats of shared memory, `bad` one shared int.
__device__ void chol_block(float* A, int64_t lda, int jb, float* dinv, uint32_t* status, float* buf, int* bad) {
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    float (*colbuf)[NB] = reinterpret_cast<float(*)[NB]>(buf);
    float (*rowbuf)[NB] = reinterpret_cast<float(*)[NB]>(buf + 2 * NB);
    float* rscale = buf + 4 * NB;
    float sblk[4][4], wblk[4][4];
    if (tid == 0) *bad = 0;
    if (tid < NB) rscale[tid] = 1.0f;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = ty * 4 + a, j = tx * 4 + b;
            sblk[a][b] = (i < jb && j <= i) ? A[(int64_t)i * lda + j] : (i == j ? 1.0f : 0.0f);
            wblk[a][b] = i == j ? 1.0f : 0.0f;
        }
    for (int c = 0; c < jb; ++c) {
        const int pb = c & 1, cq = c >> 2, cr = c & 3;
        if (tx == cq) {
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                float v = sblk[a][0];
                if (cr == 1) v = sblk[a][1];
                if (cr == 2) v = sblk[a][2];
                if (cr == 3) v = sblk[a][3];
                colbuf[pb][ty * 4 + a] = v;
            }
        }
        if (ty == cq) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                float v = wblk[0][b];
                if (cr == 1) v = wblk[1][b];
                if (cr == 2) v = wblk[2][b];
                if (cr == 3) v = wblk[3][b];
                rowbuf[pb][tx * 4 + b] = v;
            }
        }
        __syncthreads();
        const float d = colbuf[pb][c];
        // 1/sqrt(pivot): hardware estimate and one Newton step
        float r = rsqrtf(d);
        r = r * (1.5f - 0.5f * d * r * r);
        if (tid == 0) {
            if (!(d > 0.0f)) *bad = 1;
            rscale[c] = r;
        }
        if (ty * 4 + 3 <= c) continue;  // none of this thread's rows lies below row c
        float li[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) li[a] = ty * 4 + a > c ? colbuf[pb][ty * 4 + a] * r : 0.0f;
        if (tx * 4 + 3 > c) {  // columns beyond c: the block itself
            float lj[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) lj[b] = tx * 4 + b > c ? colbuf[pb][tx * 4 + b] * r : 0.0f;
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) sblk[a][b] = fmaf(-li[a], lj[b], sblk[a][b]);
        }
        if (tx * 4 <= c) {  // columns up to c: the inverse (its row c is zero beyond column c)
            float wr[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) wr[b] = rowbuf[pb][tx * 4 + b] * r;
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) wblk[a][b] = fmaf(-li[a], wr[b], wblk[a][b]);
        }
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int i = ty * 4 + a, j = tx * 4 + b;
            const bool in = i < jb && j <= i;
            if (in) A[(int64_t)i * lda + j] = sblk[a][b] * rscale[j];
            dinv[i * NB + j] = in ? wblk[a][b] * rscale[i] : 0.0f;
        }
    __syncthreads();
    if (tid == 0 && *bad) atomicCAS(status, 0u, (uint32_t)ST_NOT_SPD);
}

__global__ void __launch_bounds__(256) chol_diag_kernel(float* A, int64_t lda, int jb, float* dinv,
                                                        uint32_t* status) {
    __shared__ float buf[5 * NB];
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
__global__ void zero_upper_kernel(float* A, int64_t lda, int k) {
    const int64_t total = (int64_t)k * k;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(e / k), j = (int)(e % k);
        if (j > i) A[(int64_t)i * lda + j] = 0.0f;
    }
}

constexpr int RED_BLOCKS = 1024;
__global__ void __launch_bounds__(256) abs_partial_kernel(const float* A, int64_t lda, int k, double* partial) {
    __shared__ double sh[256];
    const int64_t total = (int64_t)k * k;
    double s = 0.0;
    for (int64_t e = blockIdx.x * 256ll + threadIdx.x; e < total; e += (int64_t)RED_BLOCKS * 256)
        s += fabs((double)A[(e / k) * lda + (e % k)]);
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
    const int64_t total = (int64_t)k * k;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x)
        A[(e / k) * lda + (e % k)] *= inv;
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
