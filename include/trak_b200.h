/*
 * trak_b200 -- C ABI of the B200 (sm_100a) implementation of TRAK's two
 * data-parallel hot paths: the Johnson-Lindenstrauss projection of per-example
 * gradients and the after-kernel scoring.
 *
 * Conventions
 *   - plain pointers and sizes only; every device pointer is memory of `device`
 *   - the library allocates nothing on the device: outputs and workspaces are
 *     the caller's, sized with the *_workspace_bytes queries
 *   - calls enqueue work on `stream` (a cudaStream_t passed as void*) and
 *     return without waiting; inputs, outputs and workspace must stay alive
 *     until that work has run
 *   - return value: TB_OK or a TB_ERR_* code; tb_strerror() names it
 *   - kernels never wait without a bound; a wait that runs out is recorded in a
 *     per-device status word that tb_device_status() reads (after a sync)
 *
 * Paths named in the comments are relative to the reference checkout
 * (MadryLab/trak).
 */
#ifndef TRAK_B200_H
#define TRAK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB_OK 0
#define TB_ERR_BAD_DTYPE 1      /* dtype not one of TB_F16 / TB_BF16 / TB_F32            */
#define TB_ERR_BAD_SHAPE 2      /* zero or negative extent, ld < F, B out of range ...    */
#define TB_ERR_BAD_PROJ_DIM 3   /* N is not a positive multiple of 512                    */
#define TB_ERR_BAD_ARG 4        /* null pointer, unknown proj_type, misaligned output ... */
#define TB_ERR_WORKSPACE 5      /* workspace missing, misaligned or too small             */
#define TB_ERR_CUDA 6           /* a CUDA runtime / driver call failed (see tb_last_cuda_error) */
#define TB_ERR_DEVICE_TIMEOUT 7 /* a bounded wait inside a kernel ran out                 */
#define TB_ERR_UNSUPPORTED 8    /* not a B200-class device, or size beyond a stated limit */
#define TB_ERR_SCRATCH_LIMIT 9  /* tb_project_static: the shape needs more than the built-in scratch */
#define TB_ERR_NOT_SPD 10       /* tb_spd_inverse met a non-positive pivot (reported by tb_device_status) */

#define TB_F16 0
#define TB_BF16 1
#define TB_F32 2

/* Values follow the reference's enum order (fast_jl/types.cuh:3-6). */
#define TB_RADEMACHER 0
#define TB_NORMAL 1

int tb_version(void);
const char *tb_strerror(int code);
/* Text of the last CUDA error this thread's calls ran into ("" if none). */
const char *tb_last_cuda_error(void);

/* Synchronises `device` and returns TB_OK, or TB_ERR_DEVICE_TIMEOUT if any
 * kernel of this library gave up a wait since the last call, or TB_ERR_NOT_SPD if
 * tb_spd_inverse met a non-positive pivot (the word is cleared by the call).
 * *detail, if not null, receives the raw status word. */
int tb_device_status(int device, uint32_t *detail);

/* Failure-path self-test (no counterpart in the reference): launches one CTA that waits, with the
 * same bounded wait the pipelines use, on a barrier nothing arrives at.  After `limit_ms`
 * (1..2000) the wait gives up and records the time-out; the next tb_device_status returns
 * TB_ERR_DEVICE_TIMEOUT and the device stays usable.  Nothing faults, traps or hangs. */
int tb_selftest_wait_timeout(int device, void *stream, uint32_t limit_ms);

/* ---- JL projection ---------------------------------------------------------
 * out[b, n] = alpha * sum_f grads[b, f] * P[f, n]   (+ out[b, n] if accumulate)
 *
 * P is the F x N matrix that the reference's fast_jl kernel defines for
 * (seed, num_feature_tiles, proj_type); it is regenerated on the fly, never
 * stored.  Replaces fast_jl<p_type, NUM_BATCHES>() (fast_jl/fast_jl.cu:29-79),
 * project<>() (fast_jl/fast_jl_kernel.cuh:107-132) and project_kernel
 * (fast_jl/fast_jl_kernel.cuh:24-105), i.e. all six pybind entry points
 * project_{rademacher,normal}_{8,16,32} (fast_jl/fast_jl.cu:81-110).
 *
 *   grads   [B, F] row-major with leading dimension ld (elements), dtype
 *           TB_F16 / TB_BF16 / TB_F32; fp32 is rounded to fp16 on the way in,
 *           as the reference does (fast_jl/data_loading.cuh:10)
 *   out     [B, N] fp32 with leading dimension ld_out, 16-byte aligned rows
 *   N       positive multiple of 512 (fast_jl/fast_jl_kernel.cuh:113)
 *   num_feature_tiles  part of the matrix definition (the reference passes the
 *           SM count, trak/projectors.py:370,409); clamped to F as in
 *           fast_jl/fast_jl.cu:42
 *   alpha, accumulate   extras: fold 1/sqrt(D) and sum parameter chunks
 *           without another pass (trak/traker.py:426, trak/projectors.py:490)
 *   ws      workspace of at least tb_project_workspace_bytes(...) bytes,
 *           256-byte aligned; any B is accepted (no 8/16/32 variants).  The
 *           batch is walked in passes that each regenerate the matrix once:
 *           up to 256 rows per pass for TB_RADEMACHER, up to 512 for
 *           TB_NORMAL (whose generation is what the projection costs), so
 *           one large call is much cheaper than many small ones
 */
size_t tb_project_workspace_bytes(int dtype, int64_t B, int64_t F, uint32_t N,
                                  uint32_t num_feature_tiles);

int tb_project(int device, void *stream, const void *grads, int dtype, int64_t B, int64_t F,
               int64_t ld, float *out, int64_t ld_out, uint32_t N, uint32_t seed,
               uint32_t num_feature_tiles, int proj_type, float alpha, int accumulate, void *ws,
               size_t ws_bytes);

/* The same projection fed straight from the per-parameter gradient tensors, so that no
 * [B, D] copy has to be assembled first (the reference concatenates them with
 * vectorize(), trak/utils.py:80-110, and ChunkedCudaProjector copies them into a staging
 * buffer, trak/projectors.py:501-502).  The gradient vector of sample b is the
 * concatenation, in table order, of segs[i].numel elements starting at
 * segs[i].ptr + b * segs[i].row_stride (elements of `dtype`, device memory, any alignment);
 * F is the sum of the numel.  The table itself is host memory and may be released when the
 * call returns.  Everything else as in tb_project. */
typedef struct tb_segment {
    const void *ptr;
    int64_t numel;
    int64_t row_stride;
} tb_segment;

size_t tb_project_segments_workspace_bytes(int dtype, int64_t B, int64_t F, uint32_t N,
                                           uint32_t num_feature_tiles, int32_t nsegs);

int tb_project_segments(int device, void *stream, const tb_segment *segs, int32_t nsegs, int dtype,
                        int64_t B, float *out, int64_t ld_out, uint32_t N, uint32_t seed,
                        uint32_t num_feature_tiles, int proj_type, float alpha, int accumulate,
                        void *ws, size_t ws_bytes);

/* ---- projection with a stored matrix -----------------------------------------------
 * No counterpart in the reference, which regenerates its matrix in every call because D x k
 * entries do not fit the GPUs it was written for.  On a B200 they can: the matrix of
 * (F, N, seed, num_feature_tiles, proj_type) takes tb_matrix_bytes(...) bytes (2 bytes per
 * entry, feature tiles padded to 64 features: 91.6 GB for F = 11,173,962, N = 4096), and
 * reading it from HBM is about three times faster than regenerating a Gaussian matrix.
 * For a projector that serves many batches with one seed (TRAKer.featurize over a train
 * set):
 *
 *   tb_matrix_generate  fills `matrix` (device memory of the caller, 256-byte aligned, at
 *                       least tb_matrix_bytes) with the very entries tb_project generates,
 *                       as 16-bit values of `elem_dtype`: TB_F16 for fp16 and fp32
 *                       gradients, TB_BF16 for bf16 gradients
 *   tb_project_cached   out = alpha * grads . P (+ out) with P read from `matrix`; same
 *                       arguments, workspace and result as tb_project (seed and proj_type
 *                       are properties of the stored matrix); rows are walked 256 at a
 *                       time, each pass reading the matrix once
 *
 * The Rademacher matrix is cheaper to regenerate than to read at 128 rows and more; the
 * stored form pays for the Gaussian matrix and for small Rademacher batches. */
size_t tb_matrix_bytes(int64_t F, uint32_t N, uint32_t num_feature_tiles);
int tb_matrix_generate(int device, void *stream, int64_t F, uint32_t N, uint32_t seed,
                       uint32_t num_feature_tiles, int proj_type, int elem_dtype, void *matrix,
                       size_t matrix_bytes);
int tb_project_cached(int device, void *stream, const void *grads, int dtype, int64_t B, int64_t F,
                      int64_t ld, float *out, int64_t ld_out, uint32_t N, uint32_t num_feature_tiles,
                      const void *matrix, size_t matrix_bytes, float alpha, int accumulate, void *ws,
                      size_t ws_bytes);
/* The same from the per-parameter gradient tensors (the table of tb_project_segments above). */
int tb_project_segments_cached(int device, void *stream, const tb_segment *segs, int32_t nsegs,
                               int dtype, int64_t B, float *out, int64_t ld_out, uint32_t N,
                               uint32_t num_feature_tiles, const void *matrix, size_t matrix_bytes,
                               float alpha, int accumulate, void *ws, size_t ws_bytes);

/* ---- after-kernel scoring -------------------------------------------------------
 * The three products and the inverse of the reference's BasicScoreComputer
 * (trak/score_computers.py:114-189).  Matrices are row-major; `dtype` is the type of
 * the inputs (TB_F16 / TB_BF16 / TB_F32), results are fp32.  fp32 inputs are scaled
 * per operand row by a power of two, split into fp16 hi + lo planes and multiplied
 * with three tensor-core passes: about 1e-5 relative error in tb_gemm_nt (one long
 * tensor-core accumulation, which truncates), about 3e-7 in tb_gram and inside
 * tb_spd_inverse (accumulated 64 k at a time and summed with rounded fp32 adds,
 * because an inverse multiplies the Gram's error by its condition number); 16-bit
 * inputs are used as they are.  Workspaces: 256-byte aligned, at least the size the
 * matching *_workspace_bytes query returns.
 *
 * tb_gram        G[k x k] (+)= X^T X for X [n x k]            get_xtx, :145-155
 *                (full symmetric G; call it per row block with accumulate = 1)
 * tb_spd_inverse A <- inv(A + lambda I) in place, fp32, through Cholesky; with
 *                rescale_by_mean_abs the result is divided by its mean absolute
 *                entry as in :160-168 (torch.linalg.inv + `/= abs().mean()` there).
 *                mean_abs_out (device pointer, nullable) receives that mean.  A
 *                matrix that is not positive definite is reported by
 *                tb_device_status as TB_ERR_NOT_SPD.
 * tb_gemm_nt     C[M x N] (+)= alpha * row_scale[m] * A[M x K] . B[N x K]^T
 *                get_x_xtx_inv's `block @ xtx_inv` (:170-176; the inverse is symmetric,
 *                so it is its own transpose) and get_scores' `features @ target_grads.T`
 *                (:187-189, trak/utils.py:128-133).  row_scale (device pointer,
 *                nullable, length M) fuses the out-to-loss weighting that the
 *                reference applies on the host afterwards (trak/traker.py:676-678);
 *                that is the reference's result for ONE checkpoint only -- for several,
 *                see tb_finalize_scores.
 */
size_t tb_gram_workspace_bytes(int dtype, int64_t n, int64_t k);
int tb_gram(int device, void *stream, const void *X, int dtype, int64_t n, int64_t k, int64_t ld,
            float *G, int64_t ldg, int accumulate, void *ws, size_t ws_bytes);

size_t tb_spd_inverse_workspace_bytes(int64_t k);
int tb_spd_inverse(int device, void *stream, float *A, int64_t k, int64_t lda, float lambda,
                   int rescale_by_mean_abs, float *mean_abs_out, void *ws, size_t ws_bytes);

size_t tb_gemm_nt_workspace_bytes(int dtype, int64_t M, int64_t N, int64_t K);
int tb_gemm_nt(int device, void *stream, const void *A, int64_t lda, const void *B, int64_t ldb,
               int dtype, int64_t M, int64_t N, int64_t K, float *C, int64_t ldc,
               const float *row_scale, float alpha, int accumulate, void *ws, size_t ws_bytes);

/* ---- finalize_scores epilogue ------------------------------------------------------
 * out[r, c] = (score_sum[r, c] / num_models) * (out_to_loss_sum[r] / num_models)
 *
 * The last step of TRAKer.finalize_scores (trak/traker.py:676-678), which the reference
 * runs with numpy on the host over the whole [n_train, n_targets] array: score_sum is the
 * sum over the checkpoints of features_m @ target_grads_m^T (accumulate them on the device
 * with tb_gemm_nt(..., accumulate = 1)), out_to_loss_sum [n] the sum of the checkpoints'
 * out-to-loss weights (trak/traker.py:667-670), num_models the number of checkpoints used.
 * `out` is fp32 (TB_F32) or fp16 (TB_F16), the dtype of the scores store
 * (trak/savers.py:434-451).  Note the difference from tb_gemm_nt's row_scale: that one
 * weights each checkpoint's product by that checkpoint's own weights (a sum of products),
 * which equals the reference's product of sums only for ONE checkpoint; with several
 * checkpoints accumulate unweighted and finish with this call. */
int tb_finalize_scores(int device, void *stream, const float *score_sum, int64_t ld_sum,
                       const float *out_to_loss_sum, int64_t n, int64_t m, float num_models,
                       void *out, int out_dtype, int64_t ld_out);

/* ---- projection without a caller-provided workspace ------------------------------
 * No counterpart in the reference.  Same arguments and result as tb_project, minus
 * `ws` / `ws_bytes`: the scratch lives in a fixed array inside the loaded library
 * (TB_PROJECT_STATIC_SCRATCH_BYTES on every GPU that loads it, held until the
 * process exits).  Meant for hosts that cannot allocate device memory themselves,
 * e.g. a plugin in a process whose device memory already belongs to another
 * component's pool, or a serving loop that must avoid the device-wide
 * synchronisation of cudaMalloc / cudaFree.  The call allocates nothing.
 *
 *   - shapes with tb_project_workspace_bytes(...) > TB_PROJECT_STATIC_SCRATCH_BYTES
 *     are refused with TB_ERR_SCRATCH_LIMIT
 *   - arguments are checked first, with tb_project's codes; a device that is not a
 *     B200-class GPU gives TB_ERR_UNSUPPORTED
 *   - the first call on a device looks up the array's device address (a one-time
 *     set-up per device); make that first call before starting any stream capture.
 *     Where the CUDA runtime loads modules lazily, that look-up can be the moment the
 *     driver sets the array's bytes aside on that GPU: it can then fail for lack of
 *     device memory (TB_ERR_CUDA, see tb_last_cuda_error); a later call tries again
 *   - all calls on a device share the one array: calls whose kernels may overlap on
 *     the GPU (different streams, different threads) race on it and must be
 *     serialised by the caller.  The array keeps the previous call's bytes; every
 *     byte a call reads it has written first, so no clearing is needed. */
#define TB_PROJECT_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

int tb_project_static(int device, void *stream, const void *grads, int dtype, int64_t B, int64_t F,
                      int64_t ld, float *out, int64_t ld_out, uint32_t N, uint32_t seed,
                      uint32_t num_feature_tiles, int proj_type, float alpha, int accumulate);

/* Exhaustive self-test of the Gaussian generator's square root (no counterpart in the reference).
 * The generator computes sqrtf(-2 logf(u)) with logf told its argument range and a shortened correctly
 * rounded square root that is only valid on the values that expression can take.  This entry point
 * evaluates both that and the plain sqrtf(-2 logf(u)) for the draws first .. first + count - 1 (within
 * [0, 2^32)) and writes the number of draws on which they differ in any bit to *mismatches_dev (device
 * memory, 8 bytes).  Zero over the whole
 * 32-bit range is what keeps the matrix bit-identical to the reference's. */
int tb_selftest_sqrt(int device, void *stream, uint64_t first, uint64_t count, uint64_t *mismatches_dev);

/* ---- measurement aid (no counterpart in the reference) -------------------------
 * Arms the calling thread: the next tb_project call records the two events
 * (cudaEvent_t passed as void*) on its stream immediately before and after its
 * projection kernel (of the last 128-row pass), so a benchmark can time that
 * kernel apart from the restaging and reduction launches around it.  The arming
 * is consumed by that call; pass NULLs to disarm. */
int tb_profile_events(void *before, void *after);

#ifdef __cplusplus
}
#endif
#endif /* TRAK_B200_H */
