// De-quantising epilogue shared by the one-CTA and the two-CTA segmented GEMM kernels.
// Included by seg_gemm.cu inside namespace sq, after store_output().
//
// One call handles one output tile for one epilogue warp: for every accumulation unit of the tile (a
// K-segment, or a weight group inside a segment) it waits for the unit's accumulator in tensor memory,
// converts it to fp32, multiplies by the unit's reciprocal scales 1 / (s_x * s_w[n]) and adds it to the
// thread's fp32 row (128 columns at most); after the last unit it adds the bias, casts and stores.
//
// What keeps the drain of a unit short, which matters when units are short (many segments, or
// group-wise weight scales where a unit is a single 128-byte K stage):
//   * The scale table of unit u+1 is built while unit u is drained: the scales of u+2 are already in
//     registers (global loads issued one unit ahead), the table has four slots, and a warp waits for
//     table u only after every warp has published it one unit earlier, so nobody stalls on a global
//     load or on the table barrier between two units of a tile.
//   * Tensor-memory loads are software-pipelined: the load of chunk i+1 is in flight while chunk i is
//     converted and accumulated.
//   * The table is read with 128-bit shared loads (same address in all lanes: a broadcast).
//   * int32 -> fp32 uses the magic-number trick (one integer add, one float subtract, both full-rate)
//     instead of the quarter-rate conversion instruction whenever the unit is short enough for every
//     accumulator to lie in [-2^22, 2^22): K_unit * 128 * 128 < 2^22, i.e. K_unit <= 224.  Both forms
//     are exact, so results do not depend on which one ran.
#pragma once

constexpr int kMagicMaxUnitK = 224;

// tcgen05.wait::ld that also "touches" the destination registers of the load it completes, so the
// compiler cannot schedule a use of them above the wait.
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

template <int KIND, bool MAGIC>
__device__ __forceinline__ float acc_to_float(uint32_t v) {
    if constexpr (KIND == SQ_GEMM_W8A8_F8) return __uint_as_float(v);
    else if constexpr (MAGIC) return __uint_as_float(v + 0x4B400000u) - 12582912.0f;   // exact for v in [-2^22, 2^22)
    else return static_cast<float>(static_cast<int32_t>(v));
}

// Position of an accumulation unit inside a tile: segment s, first K index k.  s == num_segs: past the end.
struct UnitPos {
    int s, k;
};
__device__ __forceinline__ void unit_next(const GemmParams& p, UnitPos& u) {
    const int e = unit_end(p, u.s, u.k);
    if (e < p.seg_bounds[u.s + 1]) {
        u.k = e;
    } else {
        ++u.s;
        u.k = e;   // segments are contiguous: the next one starts where this one ends
    }
}

// Raw scales of one unit as this thread needs them: the weight scale of the table column it builds
// (column n0 + epi_tid) and the activation scales -- of the segment, or with per-token scales of the
// thread's own row (the table then holds 1 / s_w only).
template <bool DUAL>
__device__ __forceinline__ void load_unit_scales(const GemmParams& p, const UnitPos& u, int b, long long n, bool col_ok, int m,
                                                 bool row_ok, bool per_token, float& sw, float& sx, float& sxn) {
    sw = 1.0f;
    sx = 1.0f;
    sxn = 1.0f;
    if (u.s >= p.num_segs) return;
    const int g = p.group_size > 0 ? u.k / p.group_size : 0;
    if (col_ok) sw = load_sw(p, b * p.sw_bs + u.s * p.sw_ss + g * p.sw_gs + n * p.sw_cs);
    const long long off = b * p.sx_bs + u.s * p.sx_ss + (per_token ? m * p.sx_rs : 0);
    if (!per_token || row_ok) {
        sx = __ldg(p.sx + off);
        if (DUAL) sxn = __ldg(p.sx_neg + off);
    }
}

template <int KIND, bool DUAL>
__device__ __forceinline__ void write_table(float* rtab, uint32_t slot, int epi_tid, float sw, float sx, float sxn, bool col_ok,
                                            bool per_token) {
    float r = 0.0f, rn = 0.0f;
    if (col_ok) {
        r = 1.0f / ((per_token ? 1.0f : sx) * sw);
        if (DUAL) rn = 1.0f / ((per_token ? 1.0f : sxn) * sw);
        if (KIND == SQ_GEMM_W4A8) { r *= 0.0625f; rn *= 0.0625f; }   // int4 weights are expanded as 16*w
    }
    rtab[(slot * 2 + 0) * BN + epi_tid] = r;
    if (DUAL) rtab[(slot * 2 + 1) * BN + epi_tid] = rn;
}

// acc[0 .. 16 nch) += float(accumulator columns) * table, for one unit.  The TMEM load of the next
// 16-column chunk is issued before the current one is consumed.  rt_pos / t_pos address the positive
// side; the negative side sits BN floats / neg_cols TMEM columns further.
template <int KIND, bool DUAL, bool MAGIC>
__device__ __forceinline__ void drain_unit(const GemmParams& p, float (&acc)[128], uint32_t t_pos, const float* rt_pos, int nch,
                                           bool per_token, float rxm, float rxnm, int b, int unit_in_tile, int m, bool row_ok,
                                           int ncol0) {
    constexpr int SIDES = DUAL ? 2 : 1;
    const int nld = nch * SIDES;
    const uint32_t neg_cols = p.dual_db ? 128u : static_cast<uint32_t>(BN);
    uint32_t va[16], vb[16];
    tmem_ld_x16(t_pos, va);
    tmem_ld_wait_on(va);
#pragma unroll
    for (int i = 0; i < 8 * SIDES; ++i) {
        if (i >= nld) break;
        const int ch = DUAL ? (i >> 1) : i;
        const bool neg = DUAL && (i & 1);
        uint32_t (&cur)[16] = (i & 1) ? vb : va;
        uint32_t (&nxt)[16] = (i & 1) ? va : vb;
        if (i + 1 < nld) {
            const int chn = DUAL ? ((i + 1) >> 1) : (i + 1);
            tmem_ld_x16(t_pos + ((DUAL && ((i + 1) & 1)) ? neg_cols : 0u) + chn * 16, nxt);
        }
        const float4* rt4 = reinterpret_cast<const float4*>(rt_pos + (neg ? BN : 0) + ch * 16);
        const float rx = neg ? rxnm : rxm;
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            const float4 r4 = rt4[j4];
            float r0 = r4.x, r1 = r4.y, r2 = r4.z, r3 = r4.w;
            if (per_token) { r0 *= rx; r1 *= rx; r2 *= rx; r3 *= rx; }
            acc[ch * 16 + 4 * j4 + 0] = fmaf(acc_to_float<KIND, MAGIC>(cur[4 * j4 + 0]), r0, acc[ch * 16 + 4 * j4 + 0]);
            acc[ch * 16 + 4 * j4 + 1] = fmaf(acc_to_float<KIND, MAGIC>(cur[4 * j4 + 1]), r1, acc[ch * 16 + 4 * j4 + 1]);
            acc[ch * 16 + 4 * j4 + 2] = fmaf(acc_to_float<KIND, MAGIC>(cur[4 * j4 + 2]), r2, acc[ch * 16 + 4 * j4 + 2]);
            acc[ch * 16 + 4 * j4 + 3] = fmaf(acc_to_float<KIND, MAGIC>(cur[4 * j4 + 3]), r3, acc[ch * 16 + 4 * j4 + 3]);
        }
        if (p.acc_dump != nullptr && row_ok) {
            // raw accumulators for the parity tests: [batch][unit][side][M][N] int32
            const long long u = static_cast<long long>(b) * p.units + unit_in_tile;
            int32_t* d = static_cast<int32_t*>(p.acc_dump) + (u * SIDES + (neg ? 1 : 0)) * p.M * p.N + static_cast<long long>(m) * p.N + ncol0;
#pragma unroll   // static indices only: a dynamic index would move the accumulator registers to local memory
            for (int j = 0; j < 16; ++j)
                if (ncol0 + ch * 16 + j < p.N)
                    d[ch * 16 + j] = KIND == SQ_GEMM_W4A8 ? (static_cast<int32_t>(cur[j]) >> 4) : static_cast<int32_t>(cur[j]);
        }
        if (i + 1 < nld) tmem_ld_wait_on(nxt);
    }
}

// One tile for one epilogue warp.  `bar_tmem_empty` is the address arrivals go to: the CTA's own
// barrier array, or (PAIR) the cluster address of the leader's.  Returns false after a wait gave up.
template <int KIND, bool DUAL, bool PAIR>
__device__ __forceinline__ bool epilogue_tile(const GemmParams& p, const CUtensorMap* map_y, uint32_t tmem_base, float* rtab,
                                              uint32_t bar_tmem_full, uint32_t bar_tmem_empty, uint32_t bar_epi,
                                              volatile int* abort_flag, uint32_t& au, int b, int m0, int n0, int warp, int lane,
                                              uint8_t* stage) {
    const int epi_tid = threadIdx.x - 128;       // 0..255
    const int q = warp & 3;                      // TMEM lane quarter of this warp
    const int h = (warp - 4) >> 2;               // column half
    const bool per_token = p.sx_rs != 0;
    const bool one_buf = DUAL && !p.dual_db;
    const int hcols = p.bn >> 1;                 // columns per warpgroup: 64, 96 or 128
    const int nch = hcols >> 4;                  // 16-column chunks per thread
    const int m = m0 + q * 32 + lane;
    const bool row_ok = m < p.M;
    const long long n_tab = n0 + epi_tid;
    const bool col_ok = n_tab < p.N && epi_tid < p.bn;

    float acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) acc[i] = 0.0f;

    // table of the first unit (its latency is exposed once per tile), then look one unit further ahead
    UnitPos wr = {0, 0};
    float sw_n, sx_n, sxn_n;          // raw scales of the unit `wr` points at
    float sx_c, sxn_c;                // per-token scales of the unit being drained
    load_unit_scales<DUAL>(p, wr, b, n_tab, col_ok, m, row_ok, per_token, sw_n, sx_n, sxn_n);
    write_table<KIND, DUAL>(rtab, au & (kTabSlots - 1), epi_tid, sw_n, sx_n, sxn_n, col_ok, per_token);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_epi);
    sx_c = sx_n;
    sxn_c = sxn_n;
    unit_next(p, wr);
    load_unit_scales<DUAL>(p, wr, b, n_tab, col_ok, m, row_ok, per_token, sw_n, sx_n, sxn_n);

    UnitPos rd = {0, 0};
    int unit_in_tile = 0;
    while (rd.s < p.num_segs) {
        const int ke = unit_end(p, rd.s, rd.k);
        SQ_EPI(0);
        // table of this unit: published by every warp one unit ago (or just above for the first unit)
        if (!mbar_wait(bar_epi, au & 1u, abort_flag, kWaitEpi)) return false;
        SQ_EPI(1);
        float rxm = 1.0f, rxnm = 1.0f;
        if (per_token) {
            rxm = 1.0f / sx_c;
            if (DUAL) rxnm = 1.0f / sxn_c;
        }
        // publish the next unit's table and start the loads of the one after it
        if (wr.s < p.num_segs) {
            write_table<KIND, DUAL>(rtab, (au + 1) & (kTabSlots - 1), epi_tid, sw_n, sx_n, sxn_n, col_ok, per_token);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_epi);
            SQ_EPI(2);
            sx_c = sx_n;
            sxn_c = sxn_n;
            unit_next(p, wr);
            load_unit_scales<DUAL>(p, wr, b, n_tab, col_ok, m, row_ok, per_token, sw_n, sx_n, sxn_n);
        }
        SQ_EPI(3);
        const uint32_t buf = one_buf ? 0u : (au & 1u);
        const uint32_t tph = one_buf ? (au & 1u) : ((au >> 1) & 1u);
        if (!mbar_wait(bar_tmem_full + buf * 8, tph, abort_flag, kWaitTmemFull)) return false;
        SQ_EPI(4);
        tc_fence_after();
        if (threadIdx.x == 128) SQ_STAMP(2, 2 * au);
        const uint32_t t_pos = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + h * hcols;
        const float* rt_pos = rtab + ((au & (kTabSlots - 1)) * 2) * BN + h * hcols;
        if (KIND != SQ_GEMM_W8A8_F8 && ke - rd.k <= kMagicMaxUnitK)
            drain_unit<KIND, DUAL, true>(p, acc, t_pos, rt_pos, nch, per_token, rxm, rxnm, b, unit_in_tile, m, row_ok, n0 + h * hcols);
        else
            drain_unit<KIND, DUAL, false>(p, acc, t_pos, rt_pos, nch, per_token, rxm, rxnm, b, unit_in_tile, m, row_ok, n0 + h * hcols);
        // buffer drained: give it back to the MMA warp
        SQ_EPI(5);
        tc_fence_before();
        __syncwarp();
        SQ_EPI(6);
        if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(bar_tmem_empty + buf * 8);
            else mbar_arrive(bar_tmem_empty + buf * 8);
        }
        if (threadIdx.x == 128) SQ_STAMP(2, 2 * au + 1);
        SQ_EPI(7);
        ++au;
        ++unit_in_tile;
        unit_next(p, rd);
    }
    // ---- bias, cast, store
    store_output(p, map_y, acc, nch, b, m, m0 + q * 32, row_ok, n0 + h * hcols, stage, lane);
    return true;
}
