// Tensor-core GEMM for the after-kernel scoring:  C[M x N] (+)= alpha * s[m] * A[M x K] . B[N x K]^T
//
// Used for the three products of the reference's BasicScoreComputer
// (trak/score_computers.py:145-189):  X^T X  (A = B = X^T, symmetric mode),
// X . inv  (inv is symmetric, so it is its own transpose) and  features . targets^T.
//
// fp32 inputs are not rounded to one tensor-core format.  A packing pass scales every operand
// row by the power of two that brings its largest magnitude into [2^14, 2^15) and splits the
// scaled value into fp16 hi + fp16 lo (hi = rn(x), lo = rn(x - hi): 22 to 23 mantissa bits for
// every element within 2^-18 of its row's maximum, an absolute floor of 2^-40 of that maximum
// below), the kernels accumulate  hi*hi + hi*lo + lo*hi  in fp32 -- three MMAs per k-step at the
// 16-bit rate, the dropped lo*lo term is under 2^-22 -- and the epilogue multiplies the two
// inverse scales back in (powers of two: exact).  The scales cost one more read of the operand
// (row maxima) before the packing pass.  What is left is the tensor core's own accumulation,
// which truncates instead of rounding: every MMA whose addends reach below the accumulator's
// last place pulls the sum towards zero, and a K-long contraction is a chain of 3K/16 such steps.
//  * X . inv and features . targets^T (gemm_nt_kernel) keep one accumulation over all of K:
//    about 1e-5 relative at K = 3000 ... 8192 (one TF32 pass would give 5e-4).  With bf16
//    instead of fp16 planes (16 mantissa bits) these two products cost 2.5 times the error in
//    the scores of an ill-conditioned problem and were 5 % faster.
//  * X^T X and W^T W (gemm_nt_chunked_kernel) feed or form an inverse, which multiplies a
//    relative error of the Gram by its condition number (measured: condition number 1000 turned
//    the 1e-5 into 2e-3 in the scores where plain fp32 arithmetic gives 3e-5).  There the tensor
//    core accumulates only 64 k at a time and the chunks are summed with rounded fp32 adds:
//    within 2x of cuBLAS fp32 at n = 5000 and closer to the exact Gram than cuBLAS fp32 at
//    n = 65,536 (5e-7 against 8e-6).
// fp16 and bf16 inputs are exact in one plane and take one MMA per k-step, unscaled.
//
// The packing pass also tiles the operands the way the pipeline consumes them:
// [128-row block][32-wide k block][plane][128 rows][32 k], so every TMA box is one
// contiguous 8 KB run, and it can transpose (for X^T X the operand is X^T).
//
// Kernel: one CTA per 256 x 256 tile of C.  Warp 0 issues TMA (64-byte swizzle boxes,
// never multicast), warp 1 issues tcgen05.mma (both operands from shared memory,
// M = 128, N = 256, two accumulators fill the 512 TMEM columns), warps 4-11 run the
// epilogue (tcgen05.ld, scale, optional accumulate, optional mirrored store for the
// symmetric product).  Every mbarrier wait is bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm.h"
#include "host_util.h"
#include "ptx.cuh"

namespace tb {

constexpr uint32_t GK = 32;                 // k per pipeline stage (one 64-byte swizzle row)
constexpr uint32_t GTILE_BYTES = 128 * GK * 2;  // one [128 x 32] 16-bit tile: 8 KB

struct GemmParams {
    float* C;
    const float* row_scale;  // nullable, length M
    const uint32_t* amax_a;  // fp32 inputs: bit pattern of max |.| of every packed row of A (else null)
    const uint32_t* amax_b;  // the same for B
    uint32_t* status;
    int64_t ldc;
    uint32_t M, N;
    uint32_t kblocks;        // K / 32 (padded)
    uint32_t stages;
    uint32_t idesc;
    float alpha;
    int accumulate;
    int symmetric;           // A and B are the same packed operand; only tiles on/above the
                             // diagonal are computed and every result is stored twice
};

// Power-of-two scale of a packed fp32 operand row whose largest magnitude has the bit pattern
// `amax_bits`: the biased exponent E is clamped to [16, 254] so that both 2^(141 - E) (brings
// the maximum into [2^14, 2^15), inside fp16's range) and its inverse are normal numbers.
__device__ __forceinline__ uint32_t scale_exponent(uint32_t amax_bits) {
    const uint32_t e = amax_bits >> 23;
    return e < 16u ? 16u : (e > 254u ? 254u : e);
}
__device__ __forceinline__ float row_scale_up(uint32_t amax_bits) {
    return __uint_as_float((268u - scale_exponent(amax_bits)) << 23);
}
__device__ __forceinline__ float row_scale_down(uint32_t amax_bits) {
    return __uint_as_float((scale_exponent(amax_bits) - 14u) << 23);
}

__device__ __forceinline__ void gemm_fail(uint32_t* status, volatile uint32_t* abort_flag, uint32_t code,
                                          uint32_t detail) {
    *abort_flag = 1u;
    if (atomicCAS(status, 0u, code) == 0u) {
        status[1] = blockIdx.x + gridDim.x * blockIdx.y;
        status[2] = detail;
    }
}


// Epilogue store of one warp's 32 x 128 block of results, which sits in the warp's shared-memory
// slab as slab[row][column] (row length SLAB_LD floats: odd, so rows and columns are both
// conflict-free).  C[m_first + row, n0 + column] is written as rows of 128 consecutive floats
// (a lane holding one row in registers would touch 32 rows per store instruction).  When
// accumulating, the loads of a group are all issued before its first store: a load behind a store
// to a possibly aliasing address would wait for it.  Symmetric products store only n >= m that way
// and write the same bits to C[n, m] for n > m (for a fixed column the lanes run along m: coalesced).
constexpr uint32_t SLAB_LD = 129;
constexpr uint32_t SLAB_FLOATS = 32u * SLAB_LD;
__device__ __forceinline__ void store_block_from_slab(const GemmParams& p, const float* slab, uint32_t m_first,
                                                      uint32_t n0, uint32_t lane) {
    const bool sym = p.symmetric != 0;
#pragma unroll 1
    for (uint32_t r0 = 0; r0 < 32u && m_first + r0 < p.M; r0 += 4u) {
        float v[4][4];
        bool on[4][4];
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
#pragma unroll
            for (uint32_t ch = 0; ch < 4; ++ch) {
                const uint32_t mr = m_first + r0 + u, n = n0 + ch * 32u + lane;
                on[u][ch] = mr < p.M && n < p.N && (!sym || n >= mr);
                v[u][ch] = (p.accumulate && on[u][ch]) ? p.C[(int64_t)mr * p.ldc + n] : 0.0f;
            }
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
#pragma unroll
            for (uint32_t ch = 0; ch < 4; ++ch)
                if (on[u][ch])
                    p.C[(int64_t)(m_first + r0 + u) * p.ldc + n0 + ch * 32u + lane] =
                        v[u][ch] + slab[(r0 + u) * SLAB_LD + ch * 32u + lane];
    }
    const uint32_t m = m_first + lane;
    if (sym && m < p.N) {
#pragma unroll 1
        for (uint32_t i0 = 0; i0 < 128u; i0 += 16u) {
            float old[16];
#pragma unroll
            for (uint32_t u = 0; u < 16; ++u) {
                const bool on = n0 + i0 + u < p.M && n0 + i0 + u > m;
                old[u] = (p.accumulate && on) ? p.C[(int64_t)(n0 + i0 + u) * p.ldc + m] : 0.0f;
            }
#pragma unroll
            for (uint32_t u = 0; u < 16; ++u)
                if (n0 + i0 + u < p.M && n0 + i0 + u > m)
                    p.C[(int64_t)(n0 + i0 + u) * p.ldc + m] = slab[lane * SLAB_LD + i0 + u] + old[u];
        }
    }
}

template <int NPL>
__global__ void __launch_bounds__(384, 1)
gemm_nt_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmParams p) {
    constexpr uint32_t MAXS = 8;
    constexpr uint32_t A_BYTES = 2 * NPL * GTILE_BYTES;  // two row blocks x planes
    constexpr uint32_t STAGE_BYTES = 2 * A_BYTES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[MAXS];
    __shared__ uint64_t bar_empty[MAXS];
    __shared__ uint64_t bar_acc;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_word;
    __shared__ float col_factor[256];  // inverse scale of every column of this tile (1 when unscaled)
    volatile uint32_t* abort_flag = &abort_word;

    // Tile order: CTAs are numbered so that the ~148 that run together cover a block of about
    // 12 x 12 tiles (12 row panels of A and 12 of B share L2) instead of a few rows of all columns.
    constexpr uint32_t GROUP_M = 12;
    const uint32_t tiles_n = gridDim.x, tiles_m = gridDim.y;
    const uint32_t id = blockIdx.y * tiles_n + blockIdx.x;
    const uint32_t width = GROUP_M * tiles_n;
    const uint32_t first_m = (id / width) * GROUP_M;
    const uint32_t gsize = min(tiles_m - first_m, GROUP_M);
    const uint32_t tile_m = first_m + (id % width) % gsize, tile_n = (id % width) / gsize;
    if (p.symmetric && tile_n < tile_m) return;  // whole CTA leaves before any barrier or TMEM use

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t S = p.stages;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        abort_word = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0 && lane == 0) {
        // ------------------------------- TMA producer -------------------------------
        prefetch_tmap(&map_a);
        prefetch_tmap(&map_b);
        uint32_t slot = 0, ph = 0;
        for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
            if (!mbar_wait(smem_u32(&bar_empty[slot]), ph ^ 1u, abort_flag)) {
                gemm_fail(p.status, abort_flag, ST_TIMEOUT_EMPTY, kb);
                break;
            }
            const uint32_t bar = smem_u32(&bar_full[slot]);
            const uint32_t sa = smem_base + slot * STAGE_BYTES, sb = sa + A_BYTES;
            mbar_expect_tx(bar, STAGE_BYTES);
            // packed row index of (row block rb, k block kb, plane pl): ((rb*kblocks + kb)*NPL + pl)*128
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t rb_a = tile_m * 2u + h, rb_b = tile_n * 2u + h;
#pragma unroll
                for (uint32_t pl = 0; pl < (uint32_t)NPL; ++pl) {
                    // A: [block h][plane]; B: [plane][block h] so that 256 rows of one plane are adjacent
                    tma_load_2d(sa + (h * NPL + pl) * GTILE_BYTES, &map_a, 0,
                                (int)(((rb_a * p.kblocks + kb) * NPL + pl) * 128u), bar);
                    tma_load_2d(sb + (pl * 2u + h) * GTILE_BYTES, &map_b, 0,
                                (int)(((rb_b * p.kblocks + kb) * NPL + pl) * 128u), bar);
                }
            }
            if (++slot == S) {
                slot = 0;
                ph ^= 1u;
            }
        }
    } else if (warp == 1) {
        // -------------------------------- MMA issuer --------------------------------
        // whole warp in the loop, one elected lane issues (descriptors stay in uniform registers)
        const bool leader = elect_one();
        uint32_t slot = 0, ph = 0;
        bool ok = true;
        for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
            const bool got = mbar_wait(smem_u32(&bar_full[slot]), ph, abort_flag);
            if (!__all_sync(0xffffffffu, got)) {
                if (leader) gemm_fail(p.status, abort_flag, ST_TIMEOUT_FULL_B, kb);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t sa = smem_base + slot * STAGE_BYTES, sb = sa + A_BYTES;
            const uint64_t b_hi = smem_desc_k_sw64(sb), b_lo = smem_desc_k_sw64(sb + 2u * GTILE_BYTES);
#pragma unroll
            for (uint32_t mb = 0; mb < 2; ++mb) {
                const uint32_t d = tmem_base + mb * 256u;
                const uint64_t a_hi = smem_desc_k_sw64(sa + (mb * NPL) * GTILE_BYTES);
                const uint64_t a_lo = smem_desc_k_sw64(sa + (mb * NPL + (NPL - 1)) * GTILE_BYTES);
                if (leader) {
#pragma unroll
                    for (uint32_t kk = 0; kk < 2; ++kk) {
                        const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
                        umma_f16_ss(d, a_hi + 2u * kk, b_hi + 2u * kk, p.idesc, acc);
                        if (NPL == 2) {
                            umma_f16_ss(d, a_hi + 2u * kk, b_lo + 2u * kk, p.idesc, 1u);
                            umma_f16_ss(d, a_lo + 2u * kk, b_hi + 2u * kk, p.idesc, 1u);
                        }
                    }
                }
            }
            if (leader) tc_commit(smem_u32(&bar_empty[slot]));
            if (++slot == S) {
                slot = 0;
                ph ^= 1u;
            }
        }
        if (ok && leader) tc_commit(smem_u32(&bar_acc));
    } else if (warp >= 4) {
        // --------------------------------- epilogue ---------------------------------
        const uint32_t q = warp & 3u, chalf = (warp - 4u) >> 2;  // TMEM lane quarter, column half
        {
            const uint32_t t = threadIdx.x - 128u, n = tile_n * 256u + t;
            col_factor[t] = (p.amax_b && n < p.N) ? row_scale_down(p.amax_b[n]) : 1.0f;
            asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight epilogue warps only
        }
        bool got = mbar_wait(smem_u32(&bar_acc), 0u, abort_flag);
        got = __all_sync(0xffffffffu, got);
        if (!got) {
            if (lane == 0) gemm_fail(p.status, abort_flag, ST_TIMEOUT_ACC, warp);
        } else {
            tc_fence_after();
            const uint32_t lane_base = (q * 32u) << 16;
            // The pipeline buffers are idle by now (the commit behind bar_acc covered every MMA and
            // every load has been consumed): each warp turns its 32 x 128 blocks around in its own slab.
            float* slab = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))) +
                          (size_t)(warp - 4u) * SLAB_FLOATS;
#pragma unroll 1
            for (uint32_t mb = 0; mb < 2; ++mb) {
                const uint32_t m_first = tile_m * 256u + mb * 128u + q * 32u, m = m_first + lane;
                const float rs = p.alpha * ((p.row_scale && m < p.M) ? p.row_scale[m] : 1.0f);
                const float fa = (p.amax_a && m < p.M) ? row_scale_down(p.amax_a[m]) : 1.0f;
#pragma unroll 1
                for (uint32_t cb = 0; cb < 8; cb += 2) {
                    const uint32_t c0 = chalf * 128u + cb * 16u;
                    uint32_t r0[16], r1[16];
                    tmem_ld_x16(tmem_base + lane_base + mb * 256u + c0, r0);
                    tmem_ld_x16(tmem_base + lane_base + mb * 256u + c0 + 16u, r1);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        slab[lane * SLAB_LD + cb * 16u + j] = ((__uint_as_float(r0[j]) * fa) * col_factor[c0 + j]) * rs;
                        slab[lane * SLAB_LD + cb * 16u + 16u + j] =
                            ((__uint_as_float(r1[j]) * fa) * col_factor[c0 + 16u + j]) * rs;
                    }
                }
                __syncwarp();
                store_block_from_slab(p, slab, m_first, tile_n * 256u + chalf * 128u, lane);
                __syncwarp();  // the slab is rewritten for the second row block
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(200000);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- chunked accumulation: the variant for products whose error gets amplified ---------------
// The tensor core adds into its fp32 accumulator by truncation, not rounding: every MMA whose
// addends reach below the accumulator's last place pulls the sum towards zero by up to one unit
// in the last place, and a K-long contraction is a chain of 3K/16 such steps (measured: 1e-5
// relative at K = 3000, 2e-3 in the scores once a Gram with condition number 1000 is inverted,
// where plain fp32 arithmetic gives 3e-5).  Here the chain is cut every 64 k: one CTA owns a
// 128 x 256 tile, TMEM holds two accumulator sets, the MMA warp fills one set with a 64-wide
// chunk -- per 32-k slot the hi*lo and lo*hi terms, then the two hi*hi MMAs, after which the
// slot goes back to the producer -- while the eight epilogue warps read the other set and add it,
// with ordinary rounded fp32 adds, to running sums they keep in registers (128 per thread).
// (Issuing all small terms of a chunk before its large ones halves the truncation that is left,
// a mean error of -2.3e-7 instead of -3.0e-7 on a Gram diagonal, but holds both slots until the
// chunk's end, and with only four slots the loads then arrive late: 12.6 against 11.5 ms.)
constexpr uint32_t CK_SLOTS = 4;
constexpr uint32_t CK_SLOT_BYTES = 6 * GTILE_BYTES;  // A: hi, lo; B: [plane][two row blocks]  (48 KB per 32 k)

__global__ void __launch_bounds__(384, 1)
gemm_nt_chunked_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[CK_SLOTS];
    __shared__ uint64_t bar_empty[CK_SLOTS];
    __shared__ uint64_t bar_acc_full[2];
    __shared__ uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_word;
    __shared__ float col_factor[256];
    volatile uint32_t* abort_flag = &abort_word;

    // same L2-friendly numbering as gemm_nt_kernel, with 128-row tiles
    constexpr uint32_t GROUP_M = 16;
    const uint32_t tiles_n = gridDim.x, tiles_m = gridDim.y;
    const uint32_t id = blockIdx.y * tiles_n + blockIdx.x;
    const uint32_t width = GROUP_M * tiles_n;
    const uint32_t first_m = (id / width) * GROUP_M;
    const uint32_t gsize = min(tiles_m - first_m, GROUP_M);
    const uint32_t tile_m = first_m + (id % width) % gsize, tile_n = (id % width) / gsize;
    // symmetric: a tile is needed when it holds some entry with n >= m
    if (p.symmetric && tile_n < (tile_m >> 1)) return;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t nchunks = (p.kblocks + 1u) >> 1;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < CK_SLOTS; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&bar_acc_full[s]), 1);
            mbar_init(smem_u32(&bar_acc_empty[s]), 8);  // one arrival per epilogue warp
        }
        abort_word = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    // Registers follow the work: the warpgroup of the two single-thread roles gives most of its
    // allocation back (168 -> 56 per thread), the two epilogue warpgroups take it (168 -> 224:
    // 128 running sums + 64 values in flight).  Each role's code sits wholly inside its branch,
    // which is what lets the compiler allocate past the launch bound there.
    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp == 0 && lane == 0) {
            // ------------------------------- TMA producer -------------------------------
            prefetch_tmap(&map_a);
            prefetch_tmap(&map_b);
            uint32_t slot = 0, ph = 0;
            for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
                if (!mbar_wait(smem_u32(&bar_empty[slot]), ph ^ 1u, abort_flag)) {
                    gemm_fail(p.status, abort_flag, ST_TIMEOUT_EMPTY, kb);
                    break;
                }
                const uint32_t bar = smem_u32(&bar_full[slot]);
                const uint32_t sa = smem_base + slot * CK_SLOT_BYTES, sb = sa + 2u * GTILE_BYTES;
                mbar_expect_tx(bar, CK_SLOT_BYTES);
#pragma unroll
                for (uint32_t pl = 0; pl < 2; ++pl) {
                    tma_load_2d(sa + pl * GTILE_BYTES, &map_a, 0, (int)(((tile_m * p.kblocks + kb) * 2u + pl) * 128u), bar);
#pragma unroll
                    for (uint32_t h = 0; h < 2; ++h)
                        tma_load_2d(sb + (pl * 2u + h) * GTILE_BYTES, &map_b, 0,
                                    (int)((((tile_n * 2u + h) * p.kblocks + kb) * 2u + pl) * 128u), bar);
                }
                if (++slot == CK_SLOTS) {
                    slot = 0;
                    ph ^= 1u;
                }
            }
        } else if (warp == 1) {
            // -------------------------------- MMA issuer --------------------------------
            // The whole warp runs the loop and one elected lane issues: with warp-uniform control flow the
            // descriptors and addresses stay in uniform registers, which the MMA and commit instructions
            // take directly (computed under a one-lane branch each would be moved there first).
            const bool leader = elect_one();
            uint32_t slot = 0, ph = 0;  // a chunk takes slots (slot, slot + 1); slot stays even, so no wrap inside one
            bool ok = true;
            for (uint32_t c = 0; c < nchunks && ok; ++c) {
                const uint32_t set = c & 1u, use = c >> 1;
                bool got = mbar_wait(smem_u32(&bar_acc_empty[set]), (use & 1u) ^ 1u, abort_flag);
                if (!__all_sync(0xffffffffu, got)) {
                    if (leader) gemm_fail(p.status, abort_flag, ST_TIMEOUT_ACC, 0x10000u + c);
                    break;
                }
                tc_fence_after();
                const uint32_t d = tmem_base + set * 256u;
                const uint32_t nkb = min(2u, p.kblocks - 2u * c);
                // per 32-k slot: its small terms first, then its large ones, and the slot is released
                for (uint32_t j = 0; j < nkb; ++j) {
                    got = mbar_wait(smem_u32(&bar_full[slot + j]), ph, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) {
                        if (leader) gemm_fail(p.status, abort_flag, ST_TIMEOUT_FULL_B, 2u * c + j);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + (slot + j) * CK_SLOT_BYTES, sb = sa + 2u * GTILE_BYTES;
                    const uint64_t a_hi = smem_desc_k_sw64(sa), a_lo = smem_desc_k_sw64(sa + GTILE_BYTES);
                    const uint64_t b_hi = smem_desc_k_sw64(sb), b_lo = smem_desc_k_sw64(sb + 2u * GTILE_BYTES);
                    if (leader) {
#pragma unroll
                        for (uint32_t kk = 0; kk < 2; ++kk) {
                            umma_f16_ss(d, a_hi + 2u * kk, b_lo + 2u * kk, p.idesc, (j > 0 || kk > 0) ? 1u : 0u);
                            umma_f16_ss(d, a_lo + 2u * kk, b_hi + 2u * kk, p.idesc, 1u);
                        }
#pragma unroll
                        for (uint32_t kk = 0; kk < 2; ++kk) umma_f16_ss(d, a_hi + 2u * kk, b_hi + 2u * kk, p.idesc, 1u);
                        tc_commit(smem_u32(&bar_empty[slot + j]));
                    }
                }
                if (!ok) break;
                if (leader) tc_commit(smem_u32(&bar_acc_full[set]));
                slot += nkb;
                if (slot >= CK_SLOTS) {
                    slot = 0;
                    ph ^= 1u;
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---------------------- running sums, then the epilogue ----------------------
        const uint32_t q = warp & 3u, chalf = (warp - 4u) >> 2;  // TMEM lane quarter, column half
        {
            const uint32_t t = threadIdx.x - 128u, n = tile_n * 256u + t;
            col_factor[t] = (p.amax_b && n < p.N) ? row_scale_down(p.amax_b[n]) : 1.0f;
            asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight epilogue warps only
        }
        const uint32_t lane_base = (q * 32u) << 16;
        float sum[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) sum[i] = 0.0f;
        bool ok = true;
#pragma unroll 1
        for (uint32_t c = 0; c < nchunks; ++c) {
            const uint32_t set = c & 1u, use = c >> 1;
            bool got = mbar_wait(smem_u32(&bar_acc_full[set]), use & 1u, abort_flag);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
                if (lane == 0) gemm_fail(p.status, abort_flag, ST_TIMEOUT_ACC, c);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t t0 = tmem_base + lane_base + set * 256u + chalf * 128u;
#pragma unroll
            for (uint32_t cb = 0; cb < 8; cb += 4) {  // four loads in flight per wait
                uint32_t r[4][16];
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) tmem_ld_x16(t0 + (cb + u) * 16u, r[u]);
                tmem_wait_ld();
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < 16; ++j) sum[(cb + u) * 16 + j] += __uint_as_float(r[u][j]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[set]));
        }
        if (ok) {
            const uint32_t m = tile_m * 128u + q * 32u + lane;
            const uint32_t n0 = tile_n * 256u + chalf * 128u;
            const float rs = p.alpha * ((p.row_scale && m < p.M) ? p.row_scale[m] : 1.0f);
            const float fa = (p.amax_a && m < p.M) ? row_scale_down(p.amax_a[m]) : 1.0f;
#pragma unroll
            for (int i = 0; i < 128; ++i) sum[i] = ((sum[i] * fa) * col_factor[chalf * 128u + i]) * rs;
            // The pipeline buffers are idle by now (the last commit covered every MMA and every load
            // has been consumed), so each warp turns its 32 x 128 block around in its own slab of them.
            float* slab = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))) +
                          (size_t)(warp - 4u) * SLAB_FLOATS;
#pragma unroll
            for (int i = 0; i < 128; ++i) slab[lane * SLAB_LD + i] = sum[i];
            __syncwarp();
            store_block_from_slab(p, slab, tile_m * 128u + q * 32u, n0, lane);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(200000);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- row maxima of fp32 operands (the scales of the packing pass) -------------------------
// amax[R] = bit pattern of max_k |operand[R][k]|  (non-negative floats order like their bits).
// Operand rows are source rows: one warp per row, lanes along k.
__global__ void amax_rows_kernel(const float* __restrict__ src, uint32_t* __restrict__ amax, uint64_t rows,
                                 uint64_t K, uint64_t ld) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t R = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; R < rows; R += warps) {
        const uint32_t* row = reinterpret_cast<const uint32_t*>(src + R * ld);
        uint32_t m = 0;
#pragma unroll 8
        for (uint64_t k = lane; k < K; k += 32u) m = max(m, row[k] & 0x7fffffffu);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) amax[R] = m;
    }
}
// Operand rows are source columns (the operand is the transpose): threads along the columns,
// blockIdx.y walks chunks of source rows; amax must be zero before the launch.
__global__ void amax_cols_kernel(const float* __restrict__ src, uint32_t* __restrict__ amax, uint64_t rows,
                                 uint64_t K, uint64_t ld, uint64_t chunk) {
    const uint64_t R = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (R >= rows) return;
    const uint64_t k0 = (uint64_t)blockIdx.y * chunk, k1 = min(K, k0 + chunk);
    const uint32_t* col = reinterpret_cast<const uint32_t*>(src) + R;
    uint32_t m = 0;
#pragma unroll 8
    for (uint64_t k = k0; k < k1; ++k) m = max(m, col[k * ld] & 0x7fffffffu);
    atomicMax(&amax[R], m);
}

// ---- packing ---------------------------------------------------------------------------
// packed[((rb*kblocks + kb)*NPL + pl)*128 + r][kk]  (16-bit), r < 128, kk < 32:
//   operand row  R = rb*128 + r,  k = kb*32 + kk;
//   value = src[R*ld + k]  (TRANS = false)  or  src[k*ld + R]  (TRANS = true: the operand is the
//   transpose of the row-major source), zero outside [rows x K].
// In: float (NPL = 2: the value times its row's power-of-two scale, as fp16 hi / lo planes) or a
// 16-bit type copied as is (NPL = 1).
template <typename In, int NPL, bool TRANS>
__global__ void pack_kernel(const In* __restrict__ src, uint16_t* __restrict__ packed,
                            const uint32_t* __restrict__ amax, uint64_t rows,
                            uint64_t K, uint64_t ld, uint32_t rowblocks, uint32_t kblocks) {
    // one thread = 8 consecutive k of one operand row (a 16-byte store per plane)
    const uint64_t total = (uint64_t)rowblocks * kblocks * 128u * 4u;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t r, oct;
        uint64_t rest;
        if (TRANS) {  // lanes run along operand rows = consecutive source columns
            r = (uint32_t)(i & 127u);
            oct = (uint32_t)((i >> 7) & 3u);
        } else {      // lanes run along k = consecutive source columns
            oct = (uint32_t)(i & 3u);
            r = (uint32_t)((i >> 2) & 127u);
        }
        rest = i >> 9;
        // consecutive CTAs take neighbouring pieces of the same source rows: along k when the operand
        // rows are source rows, along the operand rows when they are source columns
        uint32_t kb;
        uint64_t rb;
        if (rest <= 0xffffffffull) {  // 32-bit divisions whenever the piece number fits (it nearly always does)
            const uint32_t r32 = (uint32_t)rest, d = TRANS ? rowblocks : kblocks, q = r32 / d, m = r32 - q * d;
            kb = TRANS ? q : m;
            rb = TRANS ? m : q;
        } else {
            kb = TRANS ? (uint32_t)(rest / rowblocks) : (uint32_t)(rest % kblocks);
            rb = TRANS ? rest % rowblocks : rest / kblocks;
        }
        const uint64_t R = rb * 128u + r, k0 = (uint64_t)kb * 32u + oct * 8u;
        uint16_t hi[8], lo[8];
        float up = 1.0f;
        if constexpr (sizeof(In) == 4) up = R < rows ? row_scale_up(amax[R]) : 1.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            hi[e] = 0;
            lo[e] = 0;
            if (R < rows && k0 + e < K) {
                const In x = TRANS ? src[(k0 + e) * ld + R] : src[R * ld + k0 + e];
                if constexpr (sizeof(In) == 4) {
                    const float xs = x * up;  // exact: a power of two, |xs| < 2^15
                    const __half h = __float2half_rn(xs);
                    const __half l = __float2half_rn(xs - __half2float(h));  // the difference is exact
                    hi[e] = __half_as_ushort(h);
                    lo[e] = __half_as_ushort(l);
                } else {
                    hi[e] = *reinterpret_cast<const uint16_t*>(&x);
                }
            }
        }
        uint16_t* dst = packed + ((((rb * kblocks + kb) * NPL) * 128u + r) * 32u + oct * 8u);
        uint4 o;
        o.x = hi[0] | ((uint32_t)hi[1] << 16);
        o.y = hi[2] | ((uint32_t)hi[3] << 16);
        o.z = hi[4] | ((uint32_t)hi[5] << 16);
        o.w = hi[6] | ((uint32_t)hi[7] << 16);
        *reinterpret_cast<uint4*>(dst) = o;
        if (NPL == 2) {
            o.x = lo[0] | ((uint32_t)lo[1] << 16);
            o.y = lo[2] | ((uint32_t)lo[3] << 16);
            o.z = lo[4] | ((uint32_t)lo[5] << 16);
            o.w = lo[6] | ((uint32_t)lo[7] << 16);
            *reinterpret_cast<uint4*>(dst + 128u * 32u) = o;
        }
    }
}

// The transposed fp32 case through shared memory: one CTA step = one [128 operand rows x 32 k]
// tile, i.e. 32 source rows x 128 source columns.  Reads are 512-byte runs of source rows, and
// after the transpose in shared memory each plane of the tile leaves as one contiguous 8 KB run
// (the generic kernel's transposed stores are 16-byte pieces 64 bytes apart).
__global__ void __launch_bounds__(256) pack_trans_f32_kernel(const float* __restrict__ src, uint16_t* __restrict__ packed,
                                                             const uint32_t* __restrict__ amax, uint64_t rows, uint64_t K,
                                                             uint64_t ld, uint32_t rowblocks, uint32_t kblocks) {
    constexpr int LDS = 34;  // padded row of a plane tile, in 16-bit elements (17 words: conflict-free)
    __shared__ __align__(16) uint16_t tile[2][128][LDS];
    const uint32_t c = threadIdx.x & 127u, half = threadIdx.x >> 7;
    const uint64_t ntiles = (uint64_t)rowblocks * kblocks;
    for (uint64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const uint64_t rb = t % rowblocks, kb = t / rowblocks;  // neighbouring CTAs: neighbouring runs of the same source rows
        const uint64_t R = rb * 128u + c;
        const float up = R < rows ? row_scale_up(amax[R]) : 1.0f;
#pragma unroll 4
        for (uint32_t pass = 0; pass < 16; ++pass) {
            const uint32_t kk = pass * 2u + half;
            const uint64_t k = kb * 32u + kk;
            float x = 0.0f;
            if (R < rows && k < K) x = src[k * ld + R];
            const float xs = x * up;
            const __half h = __float2half_rn(xs);
            const __half l = __float2half_rn(xs - __half2float(h));
            tile[0][c][kk] = __half_as_ushort(h);
            tile[1][c][kk] = __half_as_ushort(l);
        }
        __syncthreads();
        uint16_t* dst = packed + (rb * kblocks + kb) * 2u * 128u * 32u;
#pragma unroll
        for (uint32_t it = 0; it < 4; ++it) {
            const uint32_t q = it * 256u + threadIdx.x;       // 16-byte piece: plane, row, eighth
            const uint32_t pl = q >> 9, r = (q >> 2) & 127u, oct = q & 3u;
            const uint32_t* w = reinterpret_cast<const uint32_t*>(&tile[pl][r][oct * 8u]);
            uint4 o;
            o.x = w[0];
            o.y = w[1];
            o.z = w[2];
            o.w = w[3];
            *reinterpret_cast<uint4*>(dst + (size_t)q * 8u) = o;
        }
        __syncthreads();
    }
}

// ---- host side -----------------------------------------------------------------------------
Packed packed_geometry(int dtype, int64_t rows, int64_t K) {
    Packed g;
    g.scaled = dtype == TB_F32;
    g.rowblocks = (uint32_t)((rows + 127) / 128);
    g.kblocks = (uint32_t)((K + 31) / 32);
    g.npl = dtype == TB_F32 ? 2u : 1u;
    g.data_bytes = align_up((size_t)g.rowblocks * g.kblocks * g.npl * GTILE_BYTES, 1024);
    // scaled operands carry the row maxima behind the tiles
    g.bytes = g.data_bytes + (g.scaled ? align_up((size_t)g.rowblocks * 128u * sizeof(uint32_t), 1024) : 0);
    return g;
}

int launch_pack(const void* src, int dtype, bool trans, uint64_t rows, uint64_t K, uint64_t ld,
                       uint16_t* packed, const Packed& g, int sm_count, cudaStream_t stream) {
    const uint64_t total = (uint64_t)g.rowblocks * g.kblocks * 512u;
    uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count * 32;
    if (blocks > cap) blocks = cap;
    const uint32_t nb = (uint32_t)blocks;
    if (dtype == TB_F32) {
        const float* s = static_cast<const float*>(src);
        uint32_t* amax = packed_amax(packed, g);
        if (trans) {
            TB_CUDA(cudaMemsetAsync(amax, 0, (size_t)g.rowblocks * 128u * sizeof(uint32_t), stream));
            const uint32_t bx = (uint32_t)((rows + 255) / 256);
            uint64_t by = ((uint64_t)sm_count * 16 + bx - 1) / bx;  // about 16 CTAs per SM in all
            if (by > (K + 63) / 64) by = (K + 63) / 64;
            if (by > 65535) by = 65535;
            const uint64_t chunk = (K + by - 1) / by;
            amax_cols_kernel<<<dim3(bx, (uint32_t)((K + chunk - 1) / chunk)), 256, 0, stream>>>(s, amax, rows, K, ld, chunk);
            uint64_t tb = (uint64_t)g.rowblocks * g.kblocks;
            if (tb > (uint64_t)sm_count * 16) tb = (uint64_t)sm_count * 16;
            pack_trans_f32_kernel<<<(uint32_t)tb, 256, 0, stream>>>(s, packed, amax, rows, K, ld, g.rowblocks, g.kblocks);
        } else {
            uint64_t ab = (rows + 7) / 8;  // eight warps (rows) per CTA
            if (ab > cap) ab = cap;
            amax_rows_kernel<<<(uint32_t)ab, 256, 0, stream>>>(s, amax, rows, K, ld);
            pack_kernel<float, 2, false><<<nb, 256, 0, stream>>>(s, packed, amax, rows, K, ld, g.rowblocks, g.kblocks);
        }
    } else {
        const uint16_t* s = static_cast<const uint16_t*>(src);
        if (trans)
            pack_kernel<uint16_t, 1, true><<<nb, 256, 0, stream>>>(s, packed, nullptr, rows, K, ld, g.rowblocks, g.kblocks);
        else
            pack_kernel<uint16_t, 1, false><<<nb, 256, 0, stream>>>(s, packed, nullptr, rows, K, ld, g.rowblocks, g.kblocks);
    }
    TB_CUDA(cudaGetLastError());
    return TB_OK;
}

// element format of the planes: fp16 for fp16 inputs and for scaled fp32 operands, else bf16
static bool planes_are_fp16(const Packed& g, int dtype) { return dtype == TB_F16 || g.scaled; }

static int packed_tmap(CUtensorMap* map, const uint16_t* packed, const Packed& g, int dtype) {
    const uint64_t dims[2] = {GK, (uint64_t)g.rowblocks * g.kblocks * g.npl * 128u};
    const uint64_t strides[1] = {GK * 2u};
    const uint32_t box[2] = {GK, 128};
    return encode_tmap(map, planes_are_fp16(g, dtype) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                       2, packed, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

// C[M x N] (+)= alpha * row_scale[m] * Apacked . Bpacked^T
int launch_gemm(int device, cudaStream_t stream, const uint16_t* pa, const Packed& ga,
                       const uint16_t* pb, const Packed& gb, int dtype, int64_t M, int64_t N, float* C,
                       int64_t ldc, const float* row_scale, float alpha, int accumulate, int symmetric,
                       int chunked) {
    CUtensorMap map_a, map_b;
    int rc = packed_tmap(&map_a, pa, ga, dtype);
    if (rc != TB_OK) return rc;
    rc = packed_tmap(&map_b, pb, gb, dtype);
    if (rc != TB_OK) return rc;
    GemmParams p;
    p.C = C;
    p.row_scale = row_scale;
    if (ga.scaled != gb.scaled || (chunked && !ga.scaled)) return TB_ERR_BAD_ARG;
    p.amax_a = ga.scaled ? packed_amax(pa, ga) : nullptr;
    p.amax_b = gb.scaled ? packed_amax(pb, gb) : nullptr;
    p.status = status_ptr(device);
    p.ldc = ldc;
    p.M = (uint32_t)M;
    p.N = (uint32_t)N;
    p.kblocks = ga.kblocks;
    p.idesc = idesc_f16(planes_are_fp16(ga, dtype) ? 0u : 1u, 256);
    p.alpha = alpha;
    p.accumulate = accumulate;
    p.symmetric = symmetric;
    if (chunked && ga.npl == 2) {
        const size_t smem = (size_t)CK_SLOTS * CK_SLOT_BYTES + 1024u;
        dim3 grid((uint32_t)((N + 255) / 256), (uint32_t)((M + 127) / 128), 1);
        TB_CUDA(cudaFuncSetAttribute(gemm_nt_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        gemm_nt_chunked_kernel<<<grid, 384, smem, stream>>>(map_a, map_b, p);
        TB_CUDA(cudaGetLastError());
        return TB_OK;
    }
    const uint32_t stage_bytes = 4u * ga.npl * GTILE_BYTES;
    p.stages = (200u * 1024u) / stage_bytes;
    if (p.stages > 8) p.stages = 8;
    const size_t smem = (size_t)p.stages * stage_bytes + 1024u;
    dim3 grid((uint32_t)((N + 255) / 256), (uint32_t)((M + 255) / 256), 1);
    if (ga.npl == 2) {
        auto kern = gemm_nt_kernel<2>;
        TB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, 384, smem, stream>>>(map_a, map_b, p);
    } else {
        auto kern = gemm_nt_kernel<1>;
        TB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, 384, smem, stream>>>(map_a, map_b, p);
    }
    TB_CUDA(cudaGetLastError());
    return TB_OK;
}

}  // namespace tb

extern "C" {

size_t tb_gemm_nt_workspace_bytes(int dtype, int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return tb::packed_geometry(dtype, M, K).bytes + tb::packed_geometry(dtype, N, K).bytes + 1024;
}

int tb_gemm_nt(int device, void* stream_, const void* A, int64_t lda, const void* B, int64_t ldb, int dtype,
               int64_t M, int64_t N, int64_t K, float* C, int64_t ldc, const float* row_scale, float alpha,
               int accumulate, void* ws, size_t ws_bytes) {
    using namespace tb;
    if (dtype != TB_F16 && dtype != TB_BF16 && dtype != TB_F32) return TB_ERR_BAD_DTYPE;
    if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < K || ldc < N || M > 0x7fffffff || N > 0x7fffffff)
        return TB_ERR_BAD_SHAPE;
    if (!A || !B || !C) return TB_ERR_BAD_ARG;
    if (!ws || ((uintptr_t)ws & 255u) != 0 || ws_bytes < tb_gemm_nt_workspace_bytes(dtype, M, N, K))
        return TB_ERR_WORKSPACE;
    int sm_count = 0;
    int rc = select_device(device, &sm_count);
    if (rc != TB_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const Packed ga = packed_geometry(dtype, M, K), gb = packed_geometry(dtype, N, K);
    if ((uint64_t)ga.rowblocks * ga.kblocks * ga.npl * 128u > 0x7fffffffull ||
        (uint64_t)gb.rowblocks * gb.kblocks * gb.npl * 128u > 0x7fffffffull)
        return TB_ERR_UNSUPPORTED;
    uint16_t* pa = static_cast<uint16_t*>(ws);
    uint16_t* pb = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(ws) + ga.bytes);
    rc = launch_pack(A, dtype, false, M, K, lda, pa, ga, sm_count, stream);
    if (rc != TB_OK) return rc;
    rc = launch_pack(B, dtype, false, N, K, ldb, pb, gb, sm_count, stream);
    if (rc != TB_OK) return rc;
    return launch_gemm(device, stream, pa, ga, pb, gb, dtype, M, N, C, ldc, row_scale, alpha, accumulate, 0, 0);
}

size_t tb_gram_workspace_bytes(int dtype, int64_t n, int64_t k) {
    if (n <= 0 || k <= 0) return 0;
    return tb::packed_geometry(dtype, k, n).bytes + 1024;
}

int tb_gram(int device, void* stream_, const void* X, int dtype, int64_t n, int64_t k, int64_t ld, float* G,
            int64_t ldg, int accumulate, void* ws, size_t ws_bytes) {
    using namespace tb;
    if (dtype != TB_F16 && dtype != TB_BF16 && dtype != TB_F32) return TB_ERR_BAD_DTYPE;
    if (n <= 0 || k <= 0 || ld < k || ldg < k || k > 0x7fffffff) return TB_ERR_BAD_SHAPE;
    if (!X || !G) return TB_ERR_BAD_ARG;
    if (!ws || ((uintptr_t)ws & 255u) != 0 || ws_bytes < tb_gram_workspace_bytes(dtype, n, k))
        return TB_ERR_WORKSPACE;
    int sm_count = 0;
    int rc = select_device(device, &sm_count);
    if (rc != TB_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // the operand is X^T: k operand rows, contraction over the n rows of X
    const Packed g = packed_geometry(dtype, k, n);
    if ((uint64_t)g.rowblocks * g.kblocks * g.npl * 128u > 0x7fffffffull) return TB_ERR_UNSUPPORTED;
    uint16_t* px = static_cast<uint16_t*>(ws);
    rc = launch_pack(X, dtype, true, k, n, ld, px, g, sm_count, stream);
    if (rc != TB_OK) return rc;
    // the Gram feeds an inverse, which amplifies its error by the condition number: chunked accumulation
    return launch_gemm(device, stream, px, g, px, g, dtype, k, k, G, ldg, nullptr, 1.0f, accumulate, 1,
                       dtype == TB_F32 ? 1 : 0);
}

}  // extern "C"
