// Projection with a materialised matrix.
//
// The reference never stores its projection matrix -- D x k entries do not fit the GPUs it was written for -- and
// regenerates it in every call.  On a B200 the Gaussian matrix of the CIFAR ResNet-18 configuration (11.17M x 4096
// fp16 = 91.6 GB) fits in HBM next to the gradients, and streaming it from HBM (14 ms at the measured 6.45 TB/s)
// is three times faster than regenerating it (43 ms of XORWOW + Box-Muller instruction issue).  A projector that is
// used for many batches with one seed -- TRAKer.featurize over a whole train set -- can therefore generate the
// matrix once (materialize_kernel: the very generator of project_kernel, writing to global memory) and project
// every batch with a plain tcgen05 GEMM whose two operands both arrive by TMA (project_cached_kernel).  The matrix
// is the same, bit for bit.
//
// Layout of the stored matrix: one [128 columns x 64 features] 16-bit tile of P^T (row = output column in the
// lane order of project_kernel, 128 bytes per row) per (column tile, feature tile, 64-feature stage), tiles in
// that order; a tile is exactly one TMA box of the K-major 128-byte-swizzle operand.
//
// Included by project.cu after the generator, ProjParams and fail().
#pragma once

namespace tb {

constexpr uint32_t CACHED_A_BYTES = 128u * STAGE_K * 2u;  // one stored tile: 16 KB
constexpr uint32_t CACHED_MAX_STAGES = 8;

// grid (N / 128, feature tiles), 128 threads: thread = one output column = one XORWOW stream of that tile
template <int PTYPE, bool BF16>
__global__ void __launch_bounds__(128) materialize_kernel(uint16_t* __restrict__ matrix, uint32_t seed, uint32_t tiles,
                                                          uint32_t nst) {
    const uint32_t q = threadIdx.x >> 5, lane = threadIdx.x & 31u, h = lane >> 4;
    const uint32_t stream_col = blockIdx.x * 128u + q * 32u + lane;
    const uint32_t by = blockIdx.y;
    const uint32_t sel_lo = h ? 0x1054u : 0x5410u;
    const uint32_t sel_hi = h ? 0x3276u : 0x7632u;
    Xw st;
    xw_seed(st, seed + 658105236u * stream_col + 359124577u * by);
    uint4* row = reinterpret_cast<uint4*>(matrix + ((size_t)(blockIdx.x * tiles + by) * nst) * (CACHED_A_BYTES / 2u)) +
                 threadIdx.x * 8u;  // this column's 128-byte row of the tile's first stage
    for (uint32_t s = 0; s < nst; ++s) {
        constexpr int CHUNK_UNROLL = PTYPE == TB_NORMAL ? 1 : 4;
#pragma unroll CHUNK_UNROLL
        for (uint32_t c = 0; c < 4; ++c) {
            uint32_t w[8];
            if (PTYPE == TB_RADEMACHER)
                gen_rademacher<BF16>(st, h, w);
            else
                gen_normal<BF16>(st, h, sel_lo, sel_hi, w);
            row[2u * c] = make_uint4(w[0], w[1], w[2], w[3]);
            row[2u * c + 1u] = make_uint4(w[4], w[5], w[6], w[7]);
        }
        row += CACHED_A_BYTES / 16u;
    }
}

// One CTA = 128 output columns x up to 256 rows x a bundle of feature tiles.  Warp 0 issues TMA (a stored matrix
// tile and the matching gradient box per 64 features, never multicast), warp 1 the MMAs, warps 2-5 read the
// accumulators out.  Both operands come from shared memory; the kernel is bound by the HBM stream of the matrix.
// The accumulation chains (ProjParams::epoch) alternate between two accumulators of 256 TMEM columns, so the MMA
// warp starts the next chain while the epilogue warps add the finished one to the partial.
__global__ void __launch_bounds__(192, 1)
project_cached_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const ProjParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[CACHED_MAX_STAGES];
    __shared__ uint64_t bar_empty[CACHED_MAX_STAGES];
    __shared__ uint64_t bar_acc[2];
    __shared__ uint64_t bar_drained[2];
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t S = p.stages;
    const uint32_t b_bytes = p.Bpad * 128u, stage_bytes = CACHED_A_BYTES + b_bytes;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t ct = blockIdx.x;
    const uint32_t tile0 = blockIdx.y * p.tiles_per_bundle;
    const uint32_t ntile = min(p.tiles_per_bundle, p.tiles - tile0);
    const uint32_t nblocks = ntile * p.nst;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (uint32_t a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_acc[a]), 1);
            mbar_init(smem_u32(&bar_drained[a]), 128u);
        }
        abort_word = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot), 512u);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        const bool leader = elect_one();
        if (leader) {
            prefetch_tmap(&tmap_a);
            prefetch_tmap(&tmap_b);
        }
        uint32_t slot = 0, ph = 0;
        for (uint32_t it = 0; it < nblocks; ++it) {
            bool got = mbar_wait(smem_u32(&bar_empty[slot]), ph ^ 1u, abort_flag);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
                if (leader) fail(p.status, abort_flag, ST_TIMEOUT_EMPTY, 0x8000u | it);
                break;
            }
            if (leader) {
                const uint32_t z = tile0 * p.nst + it;  // (feature tile, stage) of this block, stages in order
                const uint32_t bar = smem_u32(&bar_full[slot]);
                const uint32_t dst = smem_base + slot * stage_bytes;
                mbar_expect_tx(bar, stage_bytes);
                tma_load_3d(dst, &tmap_a, 0, 0, (int)(ct * p.tiles * p.nst + z), bar);
                tma_load_2d(dst + CACHED_A_BYTES, &tmap_b, 0, (int)(z * p.Bpad), bar);
            }
            if (++slot == S) {
                slot = 0;
                ph ^= 1u;
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer -------------------------------
        const bool leader = elect_one();
        bool ok = true;
        uint32_t slot = 0, ph = 0, started = 0, epoch_no = 0, until = p.epoch;
        for (uint32_t it = 0; it < nblocks; ++it) {
            bool got = mbar_wait(smem_u32(&bar_full[slot]), ph, abort_flag);
            if (!__all_sync(0xffffffffu, got)) {
                if (leader) fail(p.status, abort_flag, ST_TIMEOUT_FULL_B, it);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t sa = smem_base + slot * stage_bytes;
            const uint64_t a_desc = smem_desc_k_sw128(sa), b_desc = smem_desc_k_sw128(sa + CACHED_A_BYTES);
            if (leader) {
#pragma unroll
                for (uint32_t k = 0; k < 4; ++k)  // 16 features further: 32 bytes inside the swizzle row
                    umma_f16_ss(tmem_base + (epoch_no & 1u) * 256u, a_desc + 2u * k, b_desc + 2u * k, p.idesc,
                                started | (k > 0 ? 1u : 0u));
                tc_commit(smem_u32(&bar_empty[slot]));
            }
            started = 1u;
            if (++slot == S) {
                slot = 0;
                ph ^= 1u;
            }
            if (--until == 0 && it + 1 < nblocks) {
                // end of an accumulation chain (see ProjParams::epoch): hand this accumulator to the epilogue warps
                // and go on in the other one, once its chain before last has been read out
                until = p.epoch;
                if (leader) tc_commit(smem_u32(&bar_acc[epoch_no & 1u]));
                started = 0;
                ++epoch_no;
                if (epoch_no >= 2u) {
                    got = mbar_wait(smem_u32(&bar_drained[epoch_no & 1u]), ((epoch_no >> 1) - 1u) & 1u, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) {
                        if (leader) fail(p.status, abort_flag, ST_TIMEOUT_ACC, 0x8000u | it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                }
            }
        }
        if (ok && leader) tc_commit(smem_u32(&bar_acc[epoch_no & 1u]));
    } else {
        // --------------------------------- epilogue ---------------------------------
        const uint32_t q = warp & 3u, h = lane >> 4;   // a warp reaches the TMEM lanes 32 (warp % 4) ...
        const uint32_t n_out = ct * 128u + q * 32u + 2u * (lane & 15u) + h;  // lane order of the generator
        float* dst = p.partials + (size_t)blockIdx.y * p.B * p.N + n_out;
        const uint32_t lane_base = (q * 32u) << 16;
        const uint32_t drains = (nblocks + p.epoch - 1u) / p.epoch;
        for (uint32_t e = 0; e < drains; ++e) {
            bool got = mbar_wait(smem_u32(&bar_acc[e & 1u]), (e >> 1) & 1u, abort_flag);
            got = __all_sync(0xffffffffu, got);
            if (!got) {
                if (lane == 0) fail(p.status, abort_flag, ST_TIMEOUT_ACC, warp);
                break;
            }
            tc_fence_after();
            // chain 0 stores, the later chains add in the L2 (see drain_accumulators)
            for (uint32_t cb = 0; cb < p.Bpad / 8u; ++cb) {
                uint32_t r[8];
                tmem_ld_x8(tmem_base + lane_base + (e & 1u) * 256u + cb * 8u, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t b = cb * 8u + j;
                    if (b < p.B) {
                        if (e == 0)
                            __stcg(dst + (size_t)b * p.N, __uint_as_float(r[j]));
                        else
                            red_add_f32(dst + (size_t)b * p.N, __uint_as_float(r[j]));
                    }
                }
            }
            if (e + 2 < drains) {  // the chain after next accumulates here again
                tc_fence_before();
                mbar_arrive(smem_u32(&bar_drained[e & 1u]));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(200000);  // let copies and MMAs already in flight land
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512u);
    }
}

}  // namespace tb
