// Regularised SPD inverse for the after-kernel:  A <- inv(A + lambda*I), optionally divided by
// the mean absolute entry (the reference's rescale, trak/score_computers.py:160-168).
//
// The reference calls torch.linalg.inv (LU).  A + lambda*I is symmetric positive definite, so this
// goes through Cholesky, all in fp32:
//   1. blocked right-looking Cholesky A = L L^T with 64-wide panels (diagonal block in one CTA,
//      panel solve and trailing update as tiled fp32 kernels);
//   2. W = L^-1, block column by block column from the last to the first;
//   3. A^-1 = W^T W with the tensor-core GEMM of gemm.cu (symmetric mode, bf16 hi/lo split);
//   4. mean |entry| with a fixed-order two-pass reduction, then the rescale.
// A non-positive pivot is recorded in the device status word (ST_NOT_SPD).
#include "gemm.h"
#include "host_util.h"
#include "ptx.cuh"

namespace tb {

constexpr int NB = 64;      // panel width
constexpr int TRTRI_SPLIT = 16;  // most parts the triangular-inverse product is split into
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

// Factor the jb x jb diagonal block (lower triangle) in shared memory, write L back, and write
// inv(L) (lower, zero above, zero-padded to 64 x 64) to dinv.
__global__ void __launch_bounds__(256) chol_diag_kernel(float* A, int64_t lda, int jb, float* dinv,
                                                        uint32_t* status) {
    __shared__ float S[NB][NB + 1];
    __shared__ float Winv[NB][NB + 1];
    __shared__ int bad;
    const int tid = threadIdx.x;
    if (tid == 0) bad = 0;
    for (int e = tid; e < NB * NB; e += 256) {
        const int i = e >> 6, j = e & 63;
        S[i][j] = (i < jb && j <= i) ? A[(int64_t)i * lda + j] : 0.0f;
        Winv[i][j] = 0.0f;
    }
    __syncthreads();
    for (int c = 0; c < jb; ++c) {
        if (tid == 0) {
            const float d = S[c][c];
            if (!(d > 0.0f)) bad = 1;
            S[c][c] = sqrtf(d);
        }
        __syncthreads();
        const float piv = S[c][c];
        for (int i = c + 1 + tid; i < jb; i += 256) S[i][c] /= piv;
        __syncthreads();
        const int m = jb - c - 1;  // trailing size
        for (int e = tid; e < m * m; e += 256) {
            const int i = c + 1 + e / m, j = c + 1 + e % m;
            if (j <= i) S[i][j] -= S[i][c] * S[j][c];
        }
        __syncthreads();
    }
    // inverse of the lower-triangular block by forward substitution: column c is handled by the four
    // lanes 4c..4c+3 of one warp, which split every dot product and combine with two shuffles
    {
        const int c = tid >> 2, part = tid & 3;
        if (part == 0 && c < jb) Winv[c][c] = 1.0f / S[c][c];
        __syncwarp();
        for (int i = 1; i < jb; ++i) {
            float s = 0.0f;
            if (c < i) {
                for (int t = c + part; t < i; t += 4) s = fmaf(S[i][t], Winv[t][c], s);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (part == 0 && c < i) Winv[i][c] = -s / S[i][i];
            __syncwarp();
        }
    }
    __syncthreads();
    for (int e = tid; e < NB * NB; e += 256) {
        const int i = e >> 6, j = e & 63;
        if (i < jb && j <= i) A[(int64_t)i * lda + j] = S[i][j];
        dinv[e] = Winv[i][j];
    }
    if (tid == 0 && bad) atomicCAS(status, 0u, (uint32_t)ST_NOT_SPD);
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

// Trailing update of the Cholesky step:  C[i, j] -= sum_t P[i, t] * P[j, t]  for tiles on or below the
// diagonal of the r x r trailing block; P is the r x jb panel (same leading dimension as C).
__global__ void __launch_bounds__(256) syrk_update_kernel(float* C, const float* P, int64_t ld, int r, int jb) {
    if (blockIdx.x > blockIdx.y) return;  // tile column > tile row: upper part, not needed
    __shared__ __align__(16) float At[NB][TS];
    __shared__ __align__(16) float Bt[NB][TS];
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
}

// Inverse, step 2:  W21[i, c] <- - sum_{t <= i} W22[i, t] * T[t, c]
// W22 is the already inverted lower-triangular trailing block (r x r), T is r x jb.  The sum over
// t is split: CTA (bi, sp) adds the tiles bt = sp, sp + nsplit, ... <= bi of block row bi into
// part[sp][i][c]; trtri_reduce_kernel then adds the parts in a fixed order and negates.
__global__ void __launch_bounds__(256) trtri_partial_kernel(const float* W22, int64_t ld, const float* T,
                                                            int64_t ldt, int r, int jb, float* part) {
    __shared__ __align__(16) float At[NB][TS];
    __shared__ __align__(16) float Bt[NB][TS];
    const int bi = blockIdx.x, i0 = bi * NB, sp = blockIdx.y, nsplit = gridDim.y;
    const int rows = min(NB, r - i0);
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    for (int bt = sp; bt <= bi; bt += nsplit) {
        const int t0 = bt * NB, tcols = min(NB, r - t0);
        load_tile_T(At, W22 + (int64_t)i0 * ld + t0, ld, rows, tcols);
        if (bt == bi) {  // diagonal tile of a lower-triangular matrix: drop what lies above the diagonal
            __syncthreads();
            for (int e = threadIdx.x; e < NB * NB; e += 256) {
                const int i = e >> 6, t = e & 63;
                if (t > i) At[t][i] = 0.0f;
            }
        }
        load_tile_N(Bt, T + (int64_t)t0 * ldt, ldt, tcols, jb);
        __syncthreads();
        tile_mma(At, Bt, ty, tx, acc);
        __syncthreads();
    }
    float* dst = part + ((size_t)sp * r + i0) * NB;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ii = ty * 4 + i, c = tx * 4 + j;
            if (ii < rows) dst[(size_t)ii * NB + c] = acc[i][j];
        }
}
__global__ void trtri_reduce_kernel(const float* part, int nsplit, int r, int jb, float* W21, int64_t ld) {
    const int total = r * NB;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int i = e >> 6, c = e & 63;
        if (c >= jb) continue;
        float s = 0.0f;
        for (int sp = 0; sp < nsplit; ++sp) s += part[((size_t)sp * r + i) * NB + c];
        W21[(int64_t)i * ld + c] = -s;
    }
}

// A[j0.., j0..] diagonal block <- dinv block (lower), and zero the strict upper triangle of the
// block row so that W is a clean lower-triangular matrix.
__global__ void write_diag_inverse_kernel(float* A, int64_t lda, int k, int j0, int jb, const float* dinv) {
    for (int e = threadIdx.x; e < NB * NB; e += blockDim.x) {
        const int i = e >> 6, j = e & 63;
        if (i < jb && j < jb) A[(int64_t)(j0 + i) * lda + j0 + j] = dinv[e];
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
    size_t dinv, tbuf, tpart, partial, mean, packed, total;
};
static InvLayout inv_layout(int64_t k) {
    InvLayout l;
    const size_t nblk = (size_t)((k + NB - 1) / NB);
    size_t off = 0;
    l.dinv = off;
    off += align_up(nblk * NB * NB * sizeof(float), 256);
    l.tbuf = off;
    off += align_up((size_t)k * NB * sizeof(float), 256);
    l.tpart = off;
    off += align_up((size_t)TRTRI_SPLIT * k * NB * sizeof(float), 256);
    l.partial = off;
    off += align_up(RED_BLOCKS * sizeof(double), 256);
    l.mean = off;
    off += 256;
    l.packed = off;
    off += packed_geometry(TB_F32, k, k).bytes;
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
    float* tbuf = reinterpret_cast<float*>(base + l.tbuf);
    float* tpart = reinterpret_cast<float*>(base + l.tpart);
    double* partial = reinterpret_cast<double*>(base + l.partial);
    float* mean = reinterpret_cast<float*>(base + l.mean);
    uint16_t* packed = reinterpret_cast<uint16_t*>(base + l.packed);
    const int K = (int)k;
    const int nblk = (K + NB - 1) / NB;

    if (lambda != 0.0f) add_diag_kernel<<<(K + 255) / 256, 256, 0, stream>>>(A, lda, K, lambda);

    // 1. Cholesky (lower triangle of A becomes L); dinv[b] = inverse of the b-th diagonal block of L
    for (int b = 0; b < nblk; ++b) {
        const int j0 = b * NB, jb = K - j0 < NB ? K - j0 : NB, r = K - j0 - jb;
        float* Ajj = A + (int64_t)j0 * lda + j0;
        chol_diag_kernel<<<1, 256, 0, stream>>>(Ajj, lda, jb, dinv + (size_t)b * NB * NB, status_ptr(device));
        if (r > 0) {
            float* A21 = A + (int64_t)(j0 + jb) * lda + j0;
            const int rt = (r + NB - 1) / NB;
            panel_kernel<0><<<rt, 256, 0, stream>>>(A21, lda, r, jb, dinv + (size_t)b * NB * NB, nullptr, 0);
            syrk_update_kernel<<<dim3(rt, rt), 256, 0, stream>>>(A + (int64_t)(j0 + jb) * lda + j0 + jb, A21, lda, r, jb);
        }
    }
    TB_CUDA(cudaGetLastError());

    // 2. W = L^-1, last block column first
    for (int b = nblk - 1; b >= 0; --b) {
        const int j0 = b * NB, jb = K - j0 < NB ? K - j0 : NB, r = K - j0 - jb;
        const float* D = dinv + (size_t)b * NB * NB;
        if (r > 0) {
            float* L21 = A + (int64_t)(j0 + jb) * lda + j0;
            const int rt = (r + NB - 1) / NB;
            panel_kernel<1><<<rt, 256, 0, stream>>>(L21, lda, r, jb, D, tbuf, NB);
            int nsplit = (2 * sm_count + rt - 1) / rt;  // about two CTAs per SM
            if (nsplit > TRTRI_SPLIT) nsplit = TRTRI_SPLIT;
            if (nsplit > rt) nsplit = rt;
            trtri_partial_kernel<<<dim3(rt, nsplit), 256, 0, stream>>>(A + (int64_t)(j0 + jb) * lda + j0 + jb, lda, tbuf,
                                                                         NB, r, jb, tpart);
            trtri_reduce_kernel<<<(r * NB + 255) / 256, 256, 0, stream>>>(tpart, nsplit, r, jb, L21, lda);
        }
        write_diag_inverse_kernel<<<1, 256, 0, stream>>>(A, lda, K, j0, jb, D);
    }
    zero_upper_kernel<<<sm_count * 8, 256, 0, stream>>>(A, lda, K);
    TB_CUDA(cudaGetLastError());

    // 3. A^-1 = W^T W (full symmetric result written over A; the operand was packed first)
    {
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
