// Two-CTA (cta_group::2) variant of the segmented GEMM: a cluster of two CTAs on neighbouring SMs
// computes one 256 x bn tile.  Included by seg_gemm_kernels.cuh (inside namespace sq, after the helpers).
//
// Why: with one CTA per tile every SM reads a whole B tile from shared memory for each MMA and
// fills it by TMA; operand reads plus fills need ~190 bytes/clk of shared-memory bandwidth at full
// tensor rate.  In a pair each CTA stages and reads only HALF of the B tile (bn/2 rows) next to its
// own 128 rows of A, one tcgen05.mma.cta_group::2 instruction drives both tensor cores, and the
// requirement drops to ~128 bytes/clk.
//
// Differences from the one-CTA kernel:
//   * CTA r of the pair owns rows [m0 + 128 r, +128) of the tile and B rows [n0 + r bn/2, +bn/2).
//   * TMA loads carry .cta_group::2 and signal the LEADER's (rank 0) "full" barrier; only the leader
//     arms it, with the byte count of both CTAs.  No multicast is used anywhere.
//   * Only the leader's warp 1 issues MMAs.  tcgen05.commit is issued twice, once on the local and
//     once on the peer's barrier, so both CTAs see "stage empty" and "accumulator full".
//   * Epilogue warps of both CTAs drain their own tensor memory and arrive (cluster scope) on the
//     leader's "accumulator empty" barrier (count 16); W4A8 expansion warps of both CTAs arrive on
//     the leader's "converted" barrier (count 8), their packed bytes land on a CTA-local barrier.
//   * The cluster is synchronised after barrier initialisation and before exit.
// All waits stay bounded exactly as in the one-CTA kernel.
#pragma once

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}
// Bounded wait on a barrier that the other CTA of the pair also arrives at (see mbar_arrive_cluster for the semantics).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, long long limit) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((it & 1023u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                atomicCAS(&g_wait_status, 0ull, (static_cast<unsigned long long>(blockIdx.x) << 8) | static_cast<unsigned>(code));
                *abort_flag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_3d_2sm(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_2sm(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one arrival on the barrier at `cluster_addr` (own or peer CTA) once all MMAs issued so far are done
__device__ __forceinline__ void umma_commit_2sm(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
template <int KIND>
__device__ __forceinline__ void umma_2sm(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == SQ_GEMM_W8A8_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// KSUB = 128-byte K sub-tiles per pipeline stage: with 2 a stage carries 8 MMAs, which halves the
// per-MMA share of the barrier wait / commit cost of the issuing thread.
template <int KIND, bool DUAL, int KSUB>
struct Cfg2 {
    static constexpr bool kW4 = KIND == SQ_GEMM_W4A8;
    static constexpr uint32_t kBHalfBytes = 128 * BK;        // up to 128 rows of B per CTA and sub-tile
    static constexpr uint32_t kBpHalfBytes = 128 * BK / 2;   // packed int4 staging per sub-tile
    // W4A8: packed int4 lands in the upper half of each B sub-tile buffer and is expanded in place
    static constexpr uint32_t kStageBytes = KSUB * (kABytes * (DUAL ? 2 : 1) + kBHalfBytes);
    static constexpr int kStagesRaw = (192 * 1024) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kThreads = kW4 ? 512 : 384;
    static constexpr uint32_t kTabBytes = kTabBytesAll;
    static constexpr uint32_t kSmemBytes = 1024 + kStages * kStageBytes + kTabBytes + kStoreStageBytes + 256;
};

template <int KIND, bool DUAL, int KSUB>
__global__ void __launch_bounds__(Cfg2<KIND, DUAL, KSUB>::kThreads, 1)
seg_gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_an,
                 const __grid_constant__ CUtensorMap map_w, const __grid_constant__ OutMaps map_y,
                const __grid_constant__ GemmParams p) {
    using C = Cfg2<KIND, DUAL, KSUB>;
    constexpr int kStages = C::kStages;
    constexpr bool kW4 = C::kW4;
    constexpr int BKS = BK * KSUB;   // K covered by one stage

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[8], bar_empty[8], bar_cvt[8], bar_bp[8], bar_tmem_full[2], bar_tmem_empty[2], bar_tab_full[kTabSlots], bar_tab_empty[kTabSlots];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* tab = smem_gen + kStages * C::kStageBytes;   // kTabSlots scale-table slots

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();      // 0 = leader
    const uint32_t peer = rank ^ 1u;
    const int hb = p.bn >> 1;                     // B rows / accumulator-column share of one CTA

    // stage layout: A[KSUB] | A_neg[KSUB] | B[KSUB] (W4A8: packed bytes arrive in the upper half of each B sub-tile)
    auto stage_a = [&](int st, int j) { return smem_base + st * C::kStageBytes + j * kABytes; };
    auto stage_an = [&](int st, int j) { return smem_base + st * C::kStageBytes + (KSUB + j) * kABytes; };
    auto stage_b = [&](int st, int j) { return smem_base + st * C::kStageBytes + KSUB * kABytes * (DUAL ? 2 : 1) + j * C::kBHalfBytes; };
    auto stage_bp = [&](int st, int j) { return stage_b(st, j) + C::kBHalfBytes / 2; };

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(smem_u32(&bar_full[i]), 1);
            mbar_init(smem_u32(&bar_empty[i]), 1);
            mbar_init(smem_u32(&bar_cvt[i]), 8);
            mbar_init(smem_u32(&bar_bp[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bar_tmem_full[i]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[i]), 2 * (kEpiThreads / 32));
        }
        for (int i = 0; i < kTabSlots; ++i) {
            mbar_init(smem_u32(&bar_tab_full[i]), 2);                  // the two builder warps of this CTA
            mbar_init(smem_u32(&bar_tab_empty[i]), kEpiThreads / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&map_a);
        if (DUAL) prefetch_tmap(&map_an);
        prefetch_tmap(&map_w);
    }
    if (warp == 1) {
        tmem_alloc_2sm(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish_2sm();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before anything can signal them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    if (p.all_magic) {   // both CTAs fill their own tensor memory before the leader's first MMA may write either
        if (warp >= 4 && warp < 12) tmem_fill_magic(tmem_base, warp);
        tc_fence_before();
        __syncthreads();
        cluster_sync_all();
        tc_fence_after();
    }

    const int tiles_per_batch = p.tiles_m * p.tiles_n;   // tiles_m counts 256-row tiles here
    const long long first_tile = cluster_id_x();
    const long long tile_step = cluster_count_x();

    if (warp < 4) {
        reg_dec<kW4 ? SQ_W4_CTRL : kCtrlRegs>();
        if (warp == 0) {
            // ===== TMA producer (both CTAs) =====
            int trace_it = 0; (void)trace_it;
            int st = 0;
            uint32_t ph = 0;
            bool ok = true;
            const uint32_t tx_sub = 2u * kABytes * (DUAL ? 2 : 1) + (kW4 ? 0u : static_cast<uint32_t>(p.bn) * BK);   // both CTAs, one sub-tile
            // one elected lane runs the whole loop: waits, issue and commits are single-thread work, and a warp that walks the
            // loop together pays a divergence / reconvergence round trip at every lane-0 block (~150-200 cycles per stage)
            if (lane == 0) {
                for (long long tile = first_tile; ok && tile < p.total_tiles; tile += tile_step) {
                    const int b = static_cast<int>(tile / tiles_per_batch);
                    const int rem = static_cast<int>(tile - static_cast<long long>(b) * tiles_per_batch);
                    const int m0 = (rem / p.tiles_n) * BM2 + static_cast<int>(rank) * BM;
                    const int n0 = (rem % p.tiles_n) * p.bn + static_cast<int>(rank) * hb;
                    const int ab = p.a_batched ? b : 0;
                    for (int s = 0; ok && s < p.num_segs; ++s) {
                        const int k_beg = p.seg_bounds[s], k_end = p.seg_bounds[s + 1];
                        const int wb = p.w_seg_as_batch ? s : (p.w_batched ? b : 0);
                        const int wk_off = p.w_seg_as_batch ? k_beg : 0;
                        for (int k = k_beg; k < k_end; k += BKS) {
                            if (!mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1u, abort_flag, kWaitEmpty, p.wait_cycles)) { ok = false; break; }
                            {
                                SQ_STAMP(0, 2 * trace_it);
                                const int left = k_end - k;
                                const int nsub = left >= BKS ? KSUB : (left + BK - 1) / BK;   // sub-tiles that hold data
                                const uint32_t full_leader = map_to_rank(smem_u32(&bar_full[st]), 0);
                                if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bar_full[st]), tx_sub * nsub);
                                const uint32_t bp = smem_u32(&bar_bp[st]);
                                if (kW4) mbar_arrive_expect_tx(bp, static_cast<uint32_t>(hb) * (BK / 2) * nsub);
    #pragma unroll
                                for (int j = 0; j < KSUB; ++j) {
                                    if (j >= nsub) break;
                                    const int kj = k + j * BK;
                                    tma_load_3d_2sm(stage_a(st, j), &map_a, kj, m0, ab, full_leader);
                                    if (DUAL) tma_load_3d_2sm(stage_an(st, j), &map_an, kj, m0, ab, full_leader);
                                    if (kW4) tma_load_3d(stage_bp(st, j), &map_w, (kj - wk_off) >> 1, n0, wb, bp);
                                    else tma_load_3d_2sm(stage_b(st, j), &map_w, kj - wk_off, n0, wb, full_leader);
                                }
                            }
                            SQ_STAMP(0, 2 * trace_it + 1);
                            ++trace_it;
                            if (++st == kStages) { st = 0; ph ^= 1u; }
                        }
                    }
                }
            }
            __syncwarp();
        } else if (warp == 1 && rank == 0) {
            // ===== MMA issuer (leader CTA only) =====
            const uint32_t idesc = (make_idesc<KIND>() & ~(0x1Fu << 24)) | (static_cast<uint32_t>(BM2 >> 4) << 24) |
                                   (static_cast<uint32_t>(p.bn >> 3) << 17);
            const bool one_buf = DUAL && !p.dual_db;
            int st = 0;
            uint32_t ph = 0;
            uint32_t au = 0;
            uint32_t cur_buf = 0;
            int trace_mma = 0; (void)trace_mma;
            bool ok = true;
            // one elected lane runs the whole loop: waits, issue and commits are single-thread work, and a warp that walks the
            // loop together pays a divergence / reconvergence round trip at every lane-0 block (~150-200 cycles per stage)
            if (lane == 0) {
                for (long long tile = first_tile; ok && tile < p.total_tiles; tile += tile_step) {
                    for (int s = 0; ok && s < p.num_segs; ++s) {
                        const int k_beg = p.seg_bounds[s], k_end = p.seg_bounds[s + 1];
                        int u_end = k_beg;
                        uint32_t accumulate = p.all_magic ? 1u : 0u;
                        uint32_t d_pos = 0, d_neg = 0;
                        for (int kb = k_beg; ok && kb < k_end; kb += BKS) {
                            if (!mbar_wait(smem_u32(&bar_full[st]), ph, abort_flag, kWaitFull, p.wait_cycles)) { ok = false; break; }
                            if (kW4) {
                                if (!mbar_wait_cluster(smem_u32(&bar_cvt[st]), ph, abort_flag, kWaitCvt, p.wait_cycles)) { ok = false; break; }
                            }
                            tc_fence_after();
                            SQ_STAMP(1, 3 * trace_mma);
                            // sub-tile j of an operand starts (tile bytes >> 4) descriptor units after sub-tile j-1
                            const uint32_t a_lo = smem_desc_lo(stage_a(st, 0));
                            const uint32_t an_lo = smem_desc_lo(stage_an(st, 0));
                            const uint32_t b_lo = smem_desc_lo(stage_b(st, 0));
                            const int kmax = (k_end - kb) < BKS ? (k_end - kb) : BKS;
                            if (kb == u_end) {
                                // the stage opens a new unit: hand the finished TMEM buffer to both CTAs' epilogues and take the
                                // other one, once, before any MMA of the stage
                                if (kb != k_beg) {
                                    umma_commit_2sm(map_to_rank(smem_u32(&bar_tmem_full[cur_buf]), 0));
                                    umma_commit_2sm(map_to_rank(smem_u32(&bar_tmem_full[cur_buf]), 1));
                                }
                                const uint32_t buf = one_buf ? 0u : (au & 1u);
                                const uint32_t tph = one_buf ? (au & 1u) : ((au >> 1) & 1u);
                                if (!mbar_wait_cluster(smem_u32(&bar_tmem_empty[buf]), tph ^ 1u, abort_flag, kWaitTmemEmpty, p.wait_cycles)) { ok = false; break; }
                                tc_fence_after();
                                cur_buf = buf;
                                d_pos = tmem_base + buf * BN;
                                d_neg = tmem_base + (p.dual_db ? buf * BN + 128 : BN);
                                accumulate = p.all_magic ? 1u : 0u;
                                u_end = unit_end(p, s, kb);
                                ++au;
                            }
                            if (kb + kmax <= u_end) {
                                {
    #pragma unroll
                                    for (int i = 0; i < BKS / UMMA_K; ++i) {
                                        if (i * UMMA_K < kmax) {
                                            constexpr int kPerSub = BK / UMMA_K;
                                            const uint32_t ao = (i / kPerSub) * (kABytes >> 4) + 2 * (i % kPerSub);
                                            const uint32_t bo = (i / kPerSub) * (C::kBHalfBytes >> 4) + 2 * (i % kPerSub);
                                            const uint64_t db = smem_desc(b_lo + bo);
                                            const uint32_t accf = i == 0 ? accumulate : 1u;
                                            umma_2sm<KIND>(d_pos, smem_desc(a_lo + ao), db, idesc, accf);
                                            if (DUAL) umma_2sm<KIND>(d_neg, smem_desc(an_lo + ao), db, idesc, accf);
                                        }
                                    }
                                }
                                accumulate = 1;
                            } else {
                                // a unit ends inside this stage
                                for (int kk = 0; kk < kmax; kk += UMMA_K) {
                                    const int k = kb + kk;
                                    if (k == u_end) {
                                        {
                                            umma_commit_2sm(map_to_rank(smem_u32(&bar_tmem_full[cur_buf]), 0));
                                            umma_commit_2sm(map_to_rank(smem_u32(&bar_tmem_full[cur_buf]), 1));
                                        }
                                        const uint32_t buf = one_buf ? 0u : (au & 1u);
                                        const uint32_t tph = one_buf ? (au & 1u) : ((au >> 1) & 1u);
                                        if (!mbar_wait_cluster(smem_u32(&bar_tmem_empty[buf]), tph ^ 1u, abort_flag, kWaitTmemEmpty, p.wait_cycles)) { ok = false; break; }
                                        tc_fence_after();
                                        cur_buf = buf;
                                        d_pos = tmem_base + buf * BN;
                                        d_neg = tmem_base + (p.dual_db ? buf * BN + 128 : BN);
                                        accumulate = p.all_magic ? 1u : 0u;
                                        u_end = unit_end(p, s, k);
                                        ++au;
                                    }
                                    {
                                        const uint32_t sub = static_cast<uint32_t>(kk) / BK, within = (static_cast<uint32_t>(kk) % BK) >> 4;
                                        const uint64_t db = smem_desc(b_lo + sub * (C::kBHalfBytes >> 4) + within);
                                        umma_2sm<KIND>(d_pos, smem_desc(a_lo + sub * (kABytes >> 4) + within), db, idesc, accumulate);
                                        if (DUAL) umma_2sm<KIND>(d_neg, smem_desc(an_lo + sub * (kABytes >> 4) + within), db, idesc, accumulate);
                                    }
                                    accumulate = 1;
                                }
                                if (!ok) break;
                            }
                            SQ_STAMP(1, 3 * trace_mma + 1);
                            {   // stage free in both CTAs once these MMAs have read it
                                umma_commit_2sm(map_to_rank(smem_u32(&bar_empty[st]), 0));
                                umma_commit_2sm(map_to_rank(smem_u32(&bar_empty[st]), 1));
                            }
                            SQ_STAMP(1, 3 * trace_mma + 2);
                            ++trace_mma;
                            if (++st == kStages) { st = 0; ph ^= 1u; }
                        }
                        if (ok) {
                            umma_commit_2sm(map_to_rank(smem_u32(&bar_tmem_full[cur_buf]), 0));
                            umma_commit_2sm(map_to_rank(smem_u32(&bar_tmem_full[cur_buf]), 1));
                        }
                    }
                }
            }
            __syncwarp();
        } else if (warp >= 2) {
            // ===== warps 2-3 (both CTAs): per-unit scale tables for this CTA's epilogue =====
            table_builder<KIND, DUAL, true>(p, tab, smem_u32(&bar_tab_full[0]), smem_u32(&bar_tab_empty[0]), abort_flag, first_tile,
                                            tile_step, static_cast<int>(rank));
        }
    } else if (warp < 12) {
        // ===== epilogue (both CTAs): same as the one-CTA kernel on this CTA's 128 rows =====
        reg_inc<kW4 ? kEpiRegsW4 : kEpiRegs>();
        epilogue_role<KIND, DUAL, true>(p, &map_y, tmem_base, tab, smem_u32(&bar_tmem_full[0]), map_to_rank(smem_u32(&bar_tmem_empty[0]), 0),
                                        smem_u32(&bar_tab_full[0]), smem_u32(&bar_tab_empty[0]), abort_flag, first_tile, tile_step,
                                        static_cast<int>(rank), warp, lane,
                                        smem_gen + kStages * C::kStageBytes + C::kTabBytes + (warp - 4) * 2048);
        if (lane == 0) bulk_wait_all();   // this warp's TMA stores have reached memory before the CTA exits
    } else {
        // ===== int4 -> int8 expansion of this CTA's half of the weight tile (W4A8, both CTAs) =====
        if constexpr (kW4) {
            reg_dec<SQ_W4_CVT>();
            const int ct = threadIdx.x - 384;
            int st = 0;
            uint32_t ph = 0;
            uint32_t it = 0; (void)it;   // stage counter of the trace stamps
            bool ok = true;
            for (long long tile = first_tile; ok && tile < p.total_tiles; tile += tile_step) {
                for (int s = 0; ok && s < p.num_segs; ++s) {
                    const int k_beg = p.seg_bounds[s], k_end = p.seg_bounds[s + 1];
                    for (int kb = k_beg; kb < k_end; kb += BKS, ++it) {
                        SQ_CVT(0);
                        if (!mbar_wait(smem_u32(&bar_bp[st]), ph, abort_flag, kWaitFullCvt, p.wait_cycles)) { ok = false; break; }
                        SQ_CVT(1);
                        const int left = k_end - kb;
                        const int nsub = left >= BKS ? KSUB : (left + BK - 1) / BK;
                        // packed bytes sit in the upper half of the buffer they expand into: pull every chunk into
                        // registers, meet the other expansion warps on a hardware barrier, then write
                        uint4 pk[KSUB][4];
#pragma unroll
                        for (int jsub = 0; jsub < KSUB; ++jsub) {
                            if (jsub < nsub) {
                                const uint8_t* src = smem_gen + (stage_bp(st, jsub) - smem_base);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int c = ct + i * 128;
                                    if (c < hb * 4) pk[jsub][i] = *reinterpret_cast<const uint4*>(src + (c >> 2) * 64 + (c & 3) * 16);
                                }
                            }
                        }
                        SQ_CVT(2);
                        asm volatile("bar.sync 1, 128;" ::: "memory");   // see the one-CTA kernel: all four warps passed the same phase of bar_bp
                        SQ_CVT(3);
#pragma unroll
                        for (int jsub = 0; jsub < KSUB; ++jsub) {
                            if (jsub >= nsub) break;
                            uint8_t* dst = smem_gen + (stage_b(st, jsub) - smem_base);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int c = ct + i * 128;
                                if (c >= hb * 4) break;
                                const int row = c >> 2, qd = c & 3;
                                const uint32_t in[4] = {pk[jsub][i].x, pk[jsub][i].y, pk[jsub][i].z, pk[jsub][i].w};
                                uint32_t out[8];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const uint32_t lo = (in[j] << 4) & 0xF0F0F0F0u;
                                    const uint32_t hi = in[j] & 0xF0F0F0F0u;
                                    out[2 * j] = __byte_perm(lo, hi, 0x5140);
                                    out[2 * j + 1] = __byte_perm(lo, hi, 0x7362);
                                }
                                uint8_t* drow = dst + row * 128;
                                const int c0 = (2 * qd) ^ (row & 7), c1 = (2 * qd + 1) ^ (row & 7);
                                *reinterpret_cast<uint4*>(drow + c0 * 16) = make_uint4(out[0], out[1], out[2], out[3]);
                                *reinterpret_cast<uint4*>(drow + c1 * 16) = make_uint4(out[4], out[5], out[6], out[7]);
                            }
                        }
                        SQ_CVT(4);
                        fence_proxy_async_smem();
                        SQ_CVT(5);
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&bar_cvt[st]), 0));
                        SQ_CVT(6);
                        if (++st == kStages) { st = 0; ph ^= 1u; }
                    }
                }
            }
        }
    }

    // ---- teardown: nobody leaves while the peer may still signal this CTA's barriers
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_2sm(tmem_base, kTmemCols);
    }
    (void)peer;
}

// Launch on as many CTA pairs as can be resident.  Returns SQ_ERR_UNSUPPORTED if the device cannot
// host a pair of this kernel (the caller then uses the one-CTA kernel).
template <int KIND, bool DUAL, int KSUB>
static int launch_2cta_k(const CUtensorMap& ma, const CUtensorMap& man, const CUtensorMap& mw, const OutMaps& my, const GemmParams& p, cudaStream_t st) {
    using C = Cfg2<KIND, DUAL, KSUB>;
    static_assert(C::kStages >= 2 && C::kStages <= 8, "stage count");
    static int max_clusters[64] = {};
    int dev = 0;
    SQ_CUDA_OK(cudaGetDevice(&dev));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (dev >= 64 || max_clusters[dev] == 0) {
        SQ_CUDA_OK(cudaFuncSetAttribute(seg_gemm2_kernel<KIND, DUAL, KSUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        cfg.gridDim = dim3(kNumSMs, 1, 1);
        int n = 0;
        SQ_CUDA_OK(cudaOccupancyMaxActiveClusters(&n, seg_gemm2_kernel<KIND, DUAL, KSUB>, &cfg));
        if (n < 1) {
            set_error("sq_gemm: no CTA pair of the two-CTA kernel fits on this device");
            return SQ_ERR_UNSUPPORTED;
        }
        if (dev < 64) max_clusters[dev] = n;
        else max_clusters[0] = n;
    }
    const int resident = dev < 64 ? max_clusters[dev] : max_clusters[0];
    const long long clusters = p.total_tiles < resident ? p.total_tiles : resident;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
    SQ_CUDA_OK(cudaLaunchKernelEx(&cfg, seg_gemm2_kernel<KIND, DUAL, KSUB>, ma, man, mw, my, p));
    return SQ_OK;
}

// 256-byte K stages wherever two of them fit in shared memory (all but W4A8 + DualScale).
// SEGQUANT_B200_KSUB=1 / sq_set_gemm_schedule(ksub=1) forces 128-byte stages (tuning aid).
template <int KIND, bool DUAL>
static int launch_2cta(const CUtensorMap& ma, const CUtensorMap& man, const CUtensorMap& mw, const OutMaps& my, const GemmParams& p, cudaStream_t st) {
    constexpr bool can2 = Cfg2<KIND, DUAL, 2>::kStagesRaw >= 2;
    bool want2 = can2;
    if (p.short_units) want2 = false;   // a unit per stage: 256-byte stages would put a unit boundary inside every stage
    if (forced_ksub() != 0) want2 = can2 && forced_ksub() != 1;
    if constexpr (can2) {
        if (want2) return launch_2cta_k<KIND, DUAL, 2>(ma, man, mw, my, p, st);
    }
    return launch_2cta_k<KIND, DUAL, 1>(ma, man, mw, my, p, st);
}
