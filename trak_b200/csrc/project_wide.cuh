// Wide-batch variant of the projection kernel: one generated slice of P^T serves up to 512 rows.
//
// The matrix costs the same to generate whatever the batch, and the Gaussian generator
// (XORWOW + Box-Muller, fast_jl/random.cuh:50-60) is what bounds the projection, so the way to a
// high tensor-core rate is to amortise every generated element over as many rows as the SM can
// accumulate.  All 512 TMEM columns are accumulators here (128 output columns x up to 512 rows,
// two N = Bpad/2 MMAs per 16 features), which leaves no tensor memory for the generated operand:
// the generator threads write their slice into shared memory in the K-major 64-byte-swizzle
// layout (one thread = one output column = one 64-byte row of the operand) and hand it over with
// fence.proxy.async + an mbarrier; both MMA operands then come from shared memory.
//
//   * WIDE_NG generator groups of four warps, one CTA per SM; group g walks feature tiles
//     g, g + WIDE_NG, ... of the CTA's bundle, 32 features per slot, two slots per group; most bundles
//     hold WIDE_NG tiles, the last ones fewer so that the grid's last wave fills the SMs
//   * the gradient stream is ONE ring shared by all groups: the MMA warp consumes blocks in a
//     fixed round-robin order (which also fixes the summation order), and the TMA warp loads the
//     [Bpad x 32] boxes in that same order, so the ring holds the next few blocks whoever owns them
//   * the gradients are restaged with 32 features per stage, every box one contiguous run
//
// Included by project.cu after the generator and the ProjParams definitions.
#pragma once

namespace tb {

constexpr uint32_t WIDE_NG = 7;                        // 28 generator warps + TMA + MMA = 960 threads
constexpr uint32_t WIDE_SA = 2;                        // operand slots per generator group
constexpr uint32_t WIDE_K = 32;                        // features per slot and per gradient stage
constexpr uint32_t WIDE_A_BYTES = 128u * WIDE_K * 2u;  // one slot: 128 columns x 32 features, 8 KB
constexpr uint32_t WIDE_A_RING = WIDE_NG * WIDE_SA * WIDE_A_BYTES;
constexpr uint32_t WIDE_MAX_STAGES = 6;                // deepest gradient ring
constexpr uint32_t WIDE_MAX_ROWS = 512;                // rows per launch (all 512 TMEM columns)

template <int PTYPE, bool BF16>
__global__ void __launch_bounds__((4 * WIDE_NG + 2) * 32, 1)
project_wide_kernel(const __grid_constant__ CUtensorMap tmap, const ProjParams p) {
    constexpr uint32_t NG = WIDE_NG, SA = WIDE_SA;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full_a[NG][SA];
    __shared__ uint64_t bar_empty_a[NG][SA];
    __shared__ uint64_t bar_full_b[WIDE_MAX_STAGES];
    __shared__ uint64_t bar_empty_b[WIDE_MAX_STAGES];
    __shared__ uint64_t bar_acc;
    __shared__ uint64_t bar_drained;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t SB = p.stages;
    const uint32_t half_rows = p.Bpad / 2u;            // rows per MMA (N of the instruction)
    const uint32_t stage_bytes = p.Bpad * (WIDE_K * 2u);
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_ring = smem_base + WIDE_A_RING;

    const uint32_t col0 = blockIdx.x * 128u;
    // the first bundles_a bundles hold tiles_per_bundle tiles each, the ones behind them tiles_per_bundle_b
    const bool big = blockIdx.y < p.bundles_a;
    const uint32_t tpb = big ? p.tiles_per_bundle : p.tiles_per_bundle_b;
    const uint32_t tile0 = big ? blockIdx.y * p.tiles_per_bundle
                               : p.bundles_a * p.tiles_per_bundle + (blockIdx.y - p.bundles_a) * p.tiles_per_bundle_b;
    const uint32_t ntile = min(tpb, p.tiles - tile0);

    if (threadIdx.x == 0) {
        for (uint32_t g = 0; g < NG; ++g)
            for (uint32_t s = 0; s < SA; ++s) {
                mbar_init(smem_u32(&bar_full_a[g][s]), 128u);
                mbar_init(smem_u32(&bar_empty_a[g][s]), 1);
            }
        for (uint32_t s = 0; s < SB; ++s) {
            mbar_init(smem_u32(&bar_full_b[s]), 1);
            mbar_init(smem_u32(&bar_empty_b[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        mbar_init(smem_u32(&bar_drained), 4u * NG * 32u);
        abort_word = 0;
        fence_mbar_init();
    }
    if (warp == 4 * NG + 1) {
        tmem_alloc(smem_u32(&tmem_slot), 512u);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp < 4 * NG) {
        // ------------------------- generators, then epilogue -------------------------
        const uint32_t g = warp >> 2, q = warp & 3u;
        const uint32_t h = lane >> 4;
        const uint32_t m = q * 32u + lane;                 // operand row = TMEM lane of the results
        const uint32_t stream_col = col0 + m;
        const uint32_t sel_lo = h ? 0x1054u : 0x5410u;
        const uint32_t sel_hi = h ? 0x3276u : 0x7632u;
        const uint32_t row_addr = smem_base + g * (SA * WIDE_A_BYTES) + m * 64u;
        const uint32_t sw = (m >> 1) & 3u;                 // 64-byte swizzle of this row
        bool ok = true;
        uint32_t slot = 0, ph = 0;
        for (uint32_t ti = g; ti < ntile && ok; ti += NG) {
            const uint32_t by = tile0 + ti;
            Xw st;
            xw_seed(st, p.seed + 658105236u * stream_col + 359124577u * by);
            // a chain of the accumulators ends every p.epoch stages and at the end of the tile
            for (uint32_t s0 = 0; s0 < p.nst && ok; s0 += p.epoch) {
                const uint32_t s1 = min(s0 + p.epoch, p.nst);
                for (uint32_t s = s0; s < s1; ++s) {
                    bool got = mbar_wait(smem_u32(&bar_empty_a[g][slot]), ph ^ 1u, abort_flag);
                    got = __all_sync(0xffffffffu, got);
                    if (!got) {
                        if (lane == 0) fail(p.status, abort_flag, ST_TIMEOUT_EMPTY, (g << 16) | s);
                        ok = false;
                        break;
                    }
                    const uint32_t dst = row_addr + slot * WIDE_A_BYTES;
                    // one copy of the (long) Gaussian chunk body keeps the loop in the instruction cache
                    constexpr int CHUNK_UNROLL = PTYPE == TB_NORMAL ? 1 : 2;
#pragma unroll CHUNK_UNROLL
                    for (uint32_t c = 0; c < 2; ++c) {
                        uint32_t w[8];
                        if (PTYPE == TB_RADEMACHER)
                            gen_rademacher<BF16>(st, h, w);
                        else
                            gen_normal<BF16>(st, h, sel_lo, sel_hi, w);
                        // features 16c .. 16c+15 of this column: 16-byte pieces 2c and 2c + 1 of the row
                        st_shared_v4(dst + (((2u * c) ^ sw) << 4), w[0], w[1], w[2], w[3]);
                        st_shared_v4(dst + (((2u * c + 1u) ^ sw) << 4), w[4], w[5], w[6], w[7]);
                    }
                    fence_proxy_async_smem();
                    mbar_arrive(smem_u32(&bar_full_a[g][slot]));
                    if (++slot == SA) {
                        slot = 0;
                        ph ^= 1u;
                    }
                }
                if (!ok) break;
                const uint32_t tl = (ti - g) / NG;  // tiles this group has finished
                ok = drain_accumulators<NG, 4u>(p, smem_u32(&bar_acc), smem_u32(&bar_drained), &tmem_slot,
                                                tl * p.drains_per_tile + s0 / p.epoch,
                                                !(s1 == p.nst && tl + 1u == (ntile + NG - 1) / NG), abort_flag);
            }
        }
        // the drains of the tiles that group 0 still runs after this group's tiles are done
        {
            const uint32_t drains = ((ntile + NG - 1) / NG) * p.drains_per_tile;
            uint32_t d = (ntile > g ? (ntile - g + NG - 1) / NG : 0u) * p.drains_per_tile;
            for (; ok && d < drains; ++d)
                ok = drain_accumulators<NG, 4u>(p, smem_u32(&bar_acc), smem_u32(&bar_drained), &tmem_slot, d,
                                                d + 1u < drains, abort_flag);
        }
    } else {
        // blocks (32 features x 128 columns x all rows) each group contributes
        uint32_t cnt[NG];
#pragma unroll
        for (uint32_t g = 0; g < NG; ++g) cnt[g] = ntile > g ? ((ntile - g + NG - 1) / NG) * p.nst : 0u;
        const uint32_t maxcnt = cnt[0];
        if (warp == 4 * NG) {
            // ------------------------------ TMA producer ------------------------------
            const bool leader = elect_one();
            if (leader) prefetch_tmap(&tmap);
            bool ok = true;
            uint32_t slot = 0, ph = 0, s = 0, trow = 0;
            for (uint32_t it = 0; it < maxcnt && ok; ++it) {
#pragma unroll
                for (uint32_t g = 0; g < NG; ++g) {
                    if (it >= cnt[g]) continue;
                    bool got = mbar_wait(smem_u32(&bar_empty_b[slot]), ph ^ 1u, abort_flag);
                    got = __all_sync(0xffffffffu, got);
                    if (!got) {
                        if (leader) fail(p.status, abort_flag, ST_TIMEOUT_EMPTY, 0x8000u | (g << 16) | s);
                        ok = false;
                        break;
                    }
                    if (leader) {
                        const uint32_t bar = smem_u32(&bar_full_b[slot]);
                        const uint32_t dst = b_ring + slot * stage_bytes;
                        const int z = (int)((tile0 + g + trow) * p.nst + s);
                        mbar_expect_tx(bar, stage_bytes);
                        tma_load_3d(dst, &tmap, 0, 0, z, bar);
                        tma_load_3d(dst + half_rows * (WIDE_K * 2u), &tmap, 0, (int)half_rows, z, bar);
                    }
                    if (++slot == SB) {
                        slot = 0;
                        ph ^= 1u;
                    }
                }
                if (++s == p.nst) {
                    s = 0;
                    trow += NG;
                }
            }
        } else {
            // ------------------------------- MMA issuer -------------------------------
            // whole warp in the loop, one elected lane issues (operands stay in uniform registers)
            const bool leader = elect_one();
            bool ok = true;
            uint32_t started = 0, epoch_no = 0;
            uint32_t chain_end = min(p.epoch, p.nst);  // stages of every group until the current chain ends
            uint32_t aslot = 0, aph = 0, bslot = 0, bph = 0;
            for (uint32_t it = 0; it < maxcnt && ok; ++it) {
#pragma unroll
                for (uint32_t g = 0; g < NG; ++g) {
                    if (it >= cnt[g]) continue;
                    bool got = mbar_wait(smem_u32(&bar_full_b[bslot]), bph, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) {
                        if (leader) fail(p.status, abort_flag, ST_TIMEOUT_FULL_B, (g << 16) | it);
                        ok = false;
                        break;
                    }
                    got = mbar_wait(smem_u32(&bar_full_a[g][aslot]), aph, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) {
                        if (leader) fail(p.status, abort_flag, ST_TIMEOUT_FULL_A, (g << 16) | it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t a_desc = smem_desc_k_sw64(smem_base + (g * SA + aslot) * WIDE_A_BYTES);
                    const uint32_t sb = b_ring + bslot * stage_bytes;
                    const uint64_t b_lo = smem_desc_k_sw64(sb);
                    const uint64_t b_hi = smem_desc_k_sw64(sb + half_rows * (WIDE_K * 2u));
                    if (leader) {
#pragma unroll
                        for (uint32_t k = 0; k < 2; ++k) {
                            // 16 features further: 32 bytes inside the swizzle row
                            const uint32_t acc = started | (k > 0 ? 1u : 0u);
                            umma_f16_ss(tmem_base, a_desc + 2u * k, b_lo + 2u * k, p.idesc, acc);
                            umma_f16_ss(tmem_base + half_rows, a_desc + 2u * k, b_hi + 2u * k, p.idesc, acc);
                        }
                        tc_commit(smem_u32(&bar_empty_a[g][aslot]));
                        tc_commit(smem_u32(&bar_empty_b[bslot]));
                    }
                    started = 1u;
                    if (++bslot == SB) {
                        bslot = 0;
                        bph ^= 1u;
                    }
                }
                if (++aslot == SA) {
                    aslot = 0;
                    aph ^= 1u;
                }
                if (it + 1 == chain_end && ok && it + 1 < maxcnt) {
                    // end of an accumulation chain (every p.epoch stages of a feature tile and at its end): hand the
                    // accumulators to the generator warps, start afresh
                    chain_end += min(p.epoch, p.nst - chain_end % p.nst);
                    if (leader) tc_commit(smem_u32(&bar_acc));
                    const bool got = mbar_wait(smem_u32(&bar_drained), epoch_no & 1u, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) {
                        if (leader) fail(p.status, abort_flag, ST_TIMEOUT_ACC, 0x8000u | it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    started = 0;
                    ++epoch_no;
                }
            }
            if (ok && leader) tc_commit(smem_u32(&bar_acc));
        }
    }

    // ---------------------------------- teardown ----------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(200000);  // let copies and MMAs already in flight land
    if (warp == 4 * NG + 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512u);
    }
}

}  // namespace tb
