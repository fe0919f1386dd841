// De-quantising epilogue shared by the one-CTA and the two-CTA segmented GEMM kernels.
// Included by seg_gemm_kernels.cuh inside namespace sq, after store_output().
//
// Two roles live here.
//
// table_builder (warps 2 and 3 of the control warpgroup, 64 threads): walks the accumulation units of
// every tile this CTA owns (a unit = a K-segment, or a weight group inside a segment) and, up to
// kTabSlots units ahead of the epilogue, fills a shared-memory slot per unit with
//   r[n]   = 1 / (s_x * s_w[n])   for the tile's bn columns, positive and (DualScale) negative side,
//   rx[m]  = 1 / s_x[m]           for the tile's 128 rows when activation scales are per token
//                                 (r[n] is then 1 / s_w[n]),
//   bias[n]                       as fp32, in the slot of the tile's last unit.
// Global loads of the next unit's scales are issued before the current unit is written, so the
// builder's own period is a few hundred cycles.  Slots cycle through "full" / "empty" mbarriers.
//
// epilogue_tile (warps 4-11): for every unit waits for the slot and for the accumulator in tensor
// memory, and adds float(acc) * r[n] (* rx[m]) into the thread's fp32 row (128 columns at most); after
// the last unit it adds the bias, casts and stores.  Nothing but the drain is on its critical path:
// no cursor arithmetic, no global loads, no divisions.  Tensor-memory loads are software-pipelined
// (the next chunk is in flight while the current one is converted), the table is read with 128-bit
// broadcast loads, the fp32 math uses the packed two-wide instructions, and int32 -> fp32 uses one
// float subtract (full rate, packed) instead of the quarter-rate conversion when every unit of the launch has
// K_unit <= 224, which guarantees |acc| < 2^22: tensor memory is then pre-filled with the bit pattern of 1.5 * 2^23
// (kMagicBits), so an accumulator read as a float is 12582912 + sum.  All forms are exact, so results do not depend on
// which ran.
#pragma once

constexpr int kMagicMaxUnitK = 224;

// ---- slot layout (bytes): r_pos[BN] | r_neg[BN] | rx_pos[128] | rx_neg[128] | bias[BN] (last unit of a tile only)
constexpr uint32_t kSlotRNeg = BN * 4;
constexpr uint32_t kSlotRx = 2 * BN * 4;
constexpr uint32_t kSlotRxNeg = kSlotRx + BM * 4;
constexpr uint32_t kSlotBias = kSlotRx + 2 * BM * 4;
static_assert(kSlotBias + BN * 4 <= kTabSlotBytes, "table slot too small");

// tcgen05.wait::ld that also "touches" the destination registers of the load it completes, so the
// compiler cannot schedule a use of them above the wait.
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 SQ_TMEM_CLOBBER);
}
// Tile index -> batch, first row of THIS CTA's 128 rows, first column of the tile.
template <bool PAIR>
__device__ __forceinline__ void tile_coords(const GemmParams& p, long long tile, int rank, int& b, int& m0, int& n0) {
    const int tiles_per_batch = p.tiles_m * p.tiles_n;
    b = static_cast<int>(tile / tiles_per_batch);
    const int rem = static_cast<int>(tile - static_cast<long long>(b) * tiles_per_batch);
    m0 = PAIR ? (rem / p.tiles_n) * (2 * BM) + rank * BM : (rem / p.tiles_n) * BM;
    n0 = (rem % p.tiles_n) * p.bn;
}

// ---------------------------------------------------------------------------------------------
// Scale-table builder: 64 threads (warps 2 and 3).
// ---------------------------------------------------------------------------------------------
// Every address formed here is in bounds even for columns / rows outside the problem (the index is
// clamped to a valid one and the value replaced afterwards), and the optional pointers (bias, per-token
// scales) are only dereferenced inside a block guarded by a warp-uniform test, through plain loads: a
// load the compiler is free to speculate (a read-only intrinsic under a select) must never see a null
// or out-of-range address.
//
// The builder must keep up with units that are a single K stage long (weight-scale groups of 128: a new table
// every ~540 cycles of MMA work), so its loop carries as little as possible: only the four weight scales of the NEXT
// unit are prefetched into registers (their loads are strided by the group count and miss the small L1 that is left
// beside 227 KB of shared memory) together with the segment's activation scale; bias and
// per-token scales, needed once per tile or only by per-token layers, are loaded where they are written.  Holding a
// full second copy of every field in registers spilled to local memory under the control warps' small register
// allowance, and those local round trips made the builder, not the drain, the slowest stage of the pipeline.
template <bool DUAL>
__device__ __forceinline__ void builder_load_sw(const GemmParams& p, float (&sw)[4], float& sx, float& sxn, int t, int b, int n0, int s,
                                                int g, bool per_token) {
    sx = 1.0f;
    sxn = 1.0f;
    if (!per_token) {      // one uniform load each; fetched a unit ahead like the weight scales (an L1 miss here costs an L2 round trip)
        sx = p.sx[b * p.sx_bs + s * p.sx_ss];
        if (DUAL) sxn = p.sx_neg[b * p.sx_bs + s * p.sx_ss];
    }
    const long long sw_base = b * p.sw_bs + s * p.sw_ss + g * p.sw_gs;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = t + 64 * i;
        const bool valid = c < p.bn && n0 + c < p.N;
        const long long n = valid ? n0 + c : n0;          // n0 < N always
        const float w = load_sw(p, sw_base + n * p.sw_cs);
        sw[i] = valid ? w : 1.0f;
    }
}

template <int KIND, bool DUAL, bool PAIR>
__device__ __forceinline__ void table_builder(const GemmParams& p, uint8_t* tab, uint32_t bar_tab_full, uint32_t bar_tab_empty,
                                              volatile int* abort_flag, long long first_tile, long long tile_step, int rank) {
    const int t = threadIdx.x - 64;   // 0..63
    const int lane = threadIdx.x & 31;
    const bool per_token = p.sx_rs != 0;
    uint32_t au = 0;
    float sw_cur[4], sw_nxt[4], sx, sxn, sx_nxt = 1.0f, sxn_nxt = 1.0f;
    for (long long tile = first_tile; tile < p.total_tiles; tile += tile_step) {
        int b, m0, n0;
        tile_coords<PAIR>(p, tile, rank, b, m0, n0);
        int s = 0, g = 0;   // unit cursor: segment and weight group (segments and groups are walked, never divided)
        builder_load_sw<DUAL>(p, sw_cur, sx, sxn, t, b, n0, s, g, per_token);
        for (int u = 0; u < p.units; ++u, ++au) {
            const int seg_end = p.seg_bounds[s + 1];
            const int grp_end = p.group_size > 0 ? (g + 1) * p.group_size : seg_end;
            const int ke = grp_end < seg_end ? grp_end : seg_end;
            const int s2 = ke == seg_end ? s + 1 : s;
            const int g2 = (p.group_size > 0 && ke == grp_end) ? g + 1 : g;
            if (u + 1 < p.units) builder_load_sw<DUAL>(p, sw_nxt, sx_nxt, sxn_nxt, t, b, n0, s2, g2, per_token);

            const uint32_t slot = au & (kTabSlots - 1);
            const uint32_t par = (au / kTabSlots) & 1u;
#ifdef SQ_TRACE_EPI
            if (threadIdx.x == 64 && blockIdx.x == 0 && au < 500) g_trace[8 * au + 5] = clock64();
#endif
            if (!mbar_wait(bar_tab_empty + slot * 8, par ^ 1u, abort_flag, kWaitTabEmpty, p.wait_cycles)) return;
#ifdef SQ_TRACE_EPI
            if (threadIdx.x == 64 && blockIdx.x == 0 && au < 500) g_trace[8 * au + 6] = clock64();
#endif
            uint8_t* sl = tab + slot * kTabSlotBytes;
            const long long sx_base = b * p.sx_bs + s * p.sx_ss;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = t + 64 * i;
                // correctly rounded reciprocal of the scale product (the value 1.0f / x has, without the division's slow path)
                float r = __frcp_rn(sx * sw_cur[i]);
                float rn = DUAL ? __frcp_rn(sxn * sw_cur[i]) : 0.0f;
                if (KIND == SQ_GEMM_W4A8) { r *= 0.0625f; rn *= 0.0625f; }   // int4 weights are expanded as 16*w
                reinterpret_cast<float*>(sl)[c] = r;
                if (DUAL) reinterpret_cast<float*>(sl + kSlotRNeg)[c] = rn;
            }
            if (p.bias != nullptr && u + 1 == p.units) {     // warp-uniform: the tile's bias, as fp32, rides in its last unit's slot
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = t + 64 * i;
                    const bool valid = c < p.bn && n0 + c < p.N;
                    const long long idx = b * p.bias_bs + (valid ? n0 + c : n0);
                    float v;
                    if (p.bias_dtype == SQ_F32) v = static_cast<const float*>(p.bias)[idx];
                    else if (p.bias_dtype == SQ_F16) v = __half2float(static_cast<const __half*>(p.bias)[idx]);
                    else v = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[idx]);
                    reinterpret_cast<float*>(sl + kSlotBias)[c] = valid ? v : 0.0f;
                }
            }
            if (per_token) {                                 // warp-uniform
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const long long mm = m0 + t + 64 * j;
                    const bool valid = mm < p.M;
                    const long long m = valid ? mm : 0;      // row 0 always exists
                    const float a = p.sx[sx_base + m * p.sx_rs];
                    reinterpret_cast<float*>(sl + kSlotRx)[t + 64 * j] = valid ? __frcp_rn(a) : 1.0f;
                    if (DUAL) {
                        const float an = p.sx_neg[sx_base + m * p.sx_rs];
                        reinterpret_cast<float*>(sl + kSlotRxNeg)[t + 64 * j] = valid ? __frcp_rn(an) : 1.0f;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tab_full + slot * 8);
#ifdef SQ_TRACE_EPI
            if (threadIdx.x == 64 && blockIdx.x == 0 && au < 500) g_trace[8 * au + 7] = clock64();
#endif
#pragma unroll
            for (int i = 0; i < 4; ++i) sw_cur[i] = sw_nxt[i];
            sx = sx_nxt;
            sxn = sxn_nxt;
            s = s2;
            g = g2;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Drain
// ---------------------------------------------------------------------------------------------
// 16 columns: acc += float(v) * r (* rx).  Packed two-wide fp32 instructions (fma / add / mul .f32x2)
// halve the issue slots and the instruction bytes of the drain, whose straight-line code is otherwise
// limited by instruction fetch.  Each component is rounded exactly like the scalar instruction.
template <int KIND, bool MAGIC, bool PER_TOKEN>
__device__ __forceinline__ void fma16(float* acc, const uint32_t (&v)[16], const float* rt, float rx) {
    const float4* rt4 = reinterpret_cast<const float4*>(rt);
    const float2 rx2 = make_float2(rx, rx);
    const float2 unmagic = make_float2(-12582912.0f, -12582912.0f);
#pragma unroll
    for (int j4 = 0; j4 < 4; ++j4) {
        const float4 r4 = rt4[j4];
#pragma unroll
        for (int hp = 0; hp < 2; ++hp) {
            const int j = 4 * j4 + 2 * hp;
            float2 r = hp ? make_float2(r4.z, r4.w) : make_float2(r4.x, r4.y);
            if (PER_TOKEN) r = __fmul2_rn(r, rx2);
            float2 f;
            if constexpr (KIND == SQ_GEMM_W8A8_F8) {
                f = make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
            } else if constexpr (MAGIC) {   // the accumulator started from kMagicBits: its bits ARE the float 12582912 + sum
#ifdef SQ_DRAIN_SCALAR
                f = make_float2(__uint_as_float(v[j]) - 12582912.0f, __uint_as_float(v[j + 1]) - 12582912.0f);
#else
                f = __fadd2_rn(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), unmagic);
#endif
            } else {
                f = make_float2(static_cast<float>(static_cast<int32_t>(v[j])), static_cast<float>(static_cast<int32_t>(v[j + 1])));
            }
#ifdef SQ_DRAIN_SCALAR
            acc[j] = fmaf(f.x, r.x, acc[j]);
            acc[j + 1] = fmaf(f.y, r.y, acc[j + 1]);
#else
            const float2 a = __ffma2_rn(f, r, make_float2(acc[j], acc[j + 1]));
            acc[j] = a.x;
            acc[j + 1] = a.y;
#endif
        }
    }
}

template <int KIND>
__device__ __forceinline__ void dump16(const GemmParams& p, const uint32_t (&v)[16], int b, int unit_in_tile, int sides, int side, int m,
                                       int ncol) {
    // raw accumulators for the parity tests: [batch][unit][side][M][N] int32
    const long long u = static_cast<long long>(b) * p.units + unit_in_tile;
    int32_t* d = static_cast<int32_t*>(p.acc_dump) + (u * sides + side) * p.M * p.N + static_cast<long long>(m) * p.N + ncol;
#pragma unroll   // static indices only: a dynamic index would move the accumulator registers to local memory
    for (int j = 0; j < 16; ++j)
        if (ncol + j < p.N) d[j] = KIND == SQ_GEMM_W4A8 ? (static_cast<int32_t>(v[j]) >> 4) : static_cast<int32_t>(v[j]);
}

// Drain of one unit: the tensor-memory load of the next batch of 16-column chunks is in flight while the current
// one is consumed.  rt_pos / t_pos address the positive side; the negative side sits BN floats /
// neg_cols TMEM columns further.  The variant (MAGIC, PER_TOKEN, DUMP) is chosen once per unit so the
// code that runs is one contiguous block.
// Chunks (of 16 columns) fetched per tensor-memory round trip, and whether the next batch is in flight while the
// current one is consumed (tcgen05.wait::ld waits for ALL loads the thread has issued, so more bytes in flight means a
// bigger batch).  Measured on layers whose units are one K stage long (weight-scale groups of 128), INT8 and W4A8:
// batches of 32 or 64 columns are not faster than 16 (409 us vs 431 / 435 us at 4608 x 9216 x 3072), and 64-column
// batches spill in the W4A8 epilogue, which has 200 registers instead of 224 -- the round trip is not what bounds the drain.
#ifndef SQ_DRAIN_NB
#define SQ_DRAIN_NB 1
#endif
#ifndef SQ_DRAIN_DB
#define SQ_DRAIN_DB 1
#endif

// Orders every later use of the 16 registers after the statements above it (an empty volatile asm that "writes" them).
__device__ __forceinline__ void touch16(uint32_t (&r)[16]) {
    asm volatile(""
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 SQ_TMEM_CLOBBER);
}

template <int KIND, bool DUAL, bool MAGIC, bool PER_TOKEN, bool DUMP>
__device__ __forceinline__ void drain_unit(const GemmParams& p, float (&acc)[128], uint32_t t_pos, const float* rt_pos, int hcols,
                                           float rxm, float rxnm, int b, int unit_in_tile, int m, bool row_ok, int ncol0) {
    constexpr int SIDES = DUAL ? 2 : 1;
    constexpr int NB = SQ_DRAIN_NB;                   // chunks per batch
    constexpr bool DB = SQ_DRAIN_DB != 0;             // double-buffered batches
    const int nld = (hcols >> 4) * SIDES;             // 16-column chunks per unit, sides interleaved
    const uint32_t neg_cols = p.dual_db ? 128u : static_cast<uint32_t>(BN);
    uint32_t buf[DB ? 2 : 1][NB][16];
    MagicRegs mg;
    if constexpr (MAGIC) magic_regs_init(mg);
    auto chunk_addr = [&](int i) {
        return t_pos + static_cast<uint32_t>((i / SIDES) * 16) + ((DUAL && (i & 1)) ? neg_cols : 0u);
    };
    auto load_batch = [&](int i0, uint32_t (&dst)[NB][16]) {
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (i0 + j < nld) tmem_ld_x16(chunk_addr(i0 + j), dst[j]);
    };
    auto wait_batch = [&](uint32_t (&dst)[NB][16]) {
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < NB; ++j) touch16(dst[j]);
    };
    load_batch(0, buf[0]);
    wait_batch(buf[0]);
#pragma unroll
    for (int i0 = 0; i0 < 8 * SIDES; i0 += NB) {
        if (i0 >= nld) break;
        uint32_t (&cur)[NB][16] = buf[DB ? ((i0 / NB) & 1) : 0];
        uint32_t (&nxt)[NB][16] = buf[DB ? (((i0 / NB) & 1) ^ 1) : 0];
        if (DB && i0 + NB < nld) load_batch(i0 + NB, nxt);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int i = i0 + j;
            if (i < nld) {
                const int c0 = (i / SIDES) * 16;
                const bool neg = DUAL && (i & 1);
                if constexpr (MAGIC)   // chunk i is in registers: put the magic pattern back for the unit that accumulates here next
                    tmem_st_x16(chunk_addr(i), mg);
                fma16<KIND, MAGIC, PER_TOKEN>(&acc[c0], cur[j], rt_pos + (neg ? BN : 0) + c0, neg ? rxnm : rxm);
                if (DUMP && row_ok) dump16<KIND>(p, cur[j], b, unit_in_tile, SIDES, neg ? 1 : 0, m, ncol0 + c0);
            }
        }
        if (i0 + NB < nld) {
            if (!DB) load_batch(i0 + NB, nxt);
            wait_batch(nxt);
        }
    }
    if constexpr (MAGIC) tmem_st_wait();   // the refill has landed before the buffer is handed back to the MMA warp
}

// One tile for one epilogue warp.  `bar_tmem_empty` is the address arrivals go to: the CTA's own
// barrier array, or (PAIR) the cluster address of the leader's.  Returns false after a wait gave up.
template <int KIND, bool DUAL, bool PAIR, bool MAGIC, bool PER_TOKEN, bool DUMP, bool PEERS>
__device__ __forceinline__ bool epilogue_tile(const GemmParams& p, const OutMaps* map_y, uint32_t tmem_base, const uint8_t* tab,
                                              uint32_t bar_tmem_full, uint32_t bar_tmem_empty, uint32_t bar_tab_full,
                                              uint32_t bar_tab_empty, volatile int* abort_flag, uint32_t& au, int b, int m0, int n0,
                                              int warp, int lane, uint8_t* stage) {
    const int q = warp & 3;                      // TMEM lane quarter of this warp
    const int h = (warp - 4) >> 2;               // column half
    const bool one_buf = DUAL && !p.dual_db;
    const int hcols = p.bn >> 1;                 // columns per warpgroup: 64, 96 or 128
    const int m = m0 + q * 32 + lane;
    const bool row_ok = m < p.M;

    float acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) acc[i] = 0.0f;

    for (int u = 0; u < p.units; ++u) {
        const uint32_t slot = au & (kTabSlots - 1);
        if (!mbar_wait(bar_tab_full + slot * 8, (au / kTabSlots) & 1u, abort_flag, kWaitTabFull, p.wait_cycles)) return false;
        const uint8_t* sl = tab + slot * kTabSlotBytes;
        float rxm = 1.0f, rxnm = 1.0f;
        if (PER_TOKEN && p.sx_rs != 0) {
            rxm = reinterpret_cast<const float*>(sl + kSlotRx)[q * 32 + lane];
            if (DUAL) rxnm = reinterpret_cast<const float*>(sl + kSlotRxNeg)[q * 32 + lane];
        }
        const uint32_t buf = one_buf ? 0u : (au & 1u);
        const uint32_t tph = one_buf ? (au & 1u) : ((au >> 1) & 1u);
        if (!mbar_wait(bar_tmem_full + buf * 8, tph, abort_flag, kWaitTmemFull, p.wait_cycles)) return false;
        tc_fence_after();
        if (threadIdx.x == 128) SQ_STAMP(2, 2 * au);
        SQ_EPI(0);
        const uint32_t t_pos = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + h * hcols;
        const float* rt_pos = reinterpret_cast<const float*>(sl) + h * hcols;
#ifdef SQ_TRACE_EPI
        {   // latency of one extra tensor-memory load + wait, measured in place
            uint32_t tmp[16];
            SQ_EPI(1);
            tmem_ld_x16(t_pos, tmp);
            tmem_ld_wait_on(tmp);
            SQ_EPI(2);
            asm volatile("" ::"r"(tmp[0]), "r"(tmp[15]));
        }
#endif
        // every lane runs the drain (its tensor-memory loads are warp-collective); rows past M only skip the dump stores
        drain_unit<KIND, DUAL, MAGIC, PER_TOKEN, DUMP>(p, acc, t_pos, rt_pos, hcols, rxm, rxnm, b, u, m, row_ok, n0 + h * hcols);
        // accumulator and table slot consumed: hand both back
        SQ_EPI(3);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(bar_tmem_empty + buf * 8);
            else mbar_arrive(bar_tmem_empty + buf * 8);
            if (u + 1 < p.units) mbar_arrive(bar_tab_empty + slot * 8);   // the last slot also holds the bias: released below
        }
        if (threadIdx.x == 128) SQ_STAMP(2, 2 * au + 1);
        SQ_EPI(4);
        ++au;
    }
    // ---- bias, cast, store
    const uint32_t last_slot = (au - 1) & (kTabSlots - 1);
    store_output<PEERS>(p, map_y, acc, hcols >> 4, b, m, m0 + q * 32, row_ok, n0 + h * hcols, stage, lane,
                 reinterpret_cast<const float*>(tab + last_slot * kTabSlotBytes + kSlotBias) + h * hcols);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_tab_empty + last_slot * 8);
    return true;
}

// All tiles of this CTA for one epilogue warp, with ONE drain variant.
template <int KIND, bool DUAL, bool PAIR, bool MAGIC, bool PER_TOKEN, bool DUMP, bool PEERS>
__device__ __forceinline__ void epilogue_tiles(const GemmParams& p, const OutMaps* map_y, uint32_t tmem_base, const uint8_t* tab,
                                               uint32_t bar_tmem_full, uint32_t bar_tmem_empty, uint32_t bar_tab_full,
                                               uint32_t bar_tab_empty, volatile int* abort_flag, long long first_tile,
                                               long long tile_step, int rank, int warp, int lane, uint8_t* stage) {
    uint32_t au = 0;
    for (long long tile = first_tile; tile < p.total_tiles; tile += tile_step) {
        int b, m0, n0;
        tile_coords<PAIR>(p, tile, rank, b, m0, n0);
        if (!epilogue_tile<KIND, DUAL, PAIR, MAGIC, PER_TOKEN, DUMP, PEERS>(p, map_y, tmem_base, tab, bar_tmem_full, bar_tmem_empty, bar_tab_full,
                                                                     bar_tab_empty, abort_flag, au, b, m0, n0, warp, lane, stage))
            break;
    }
}

// The epilogue role.  The drain variant is picked once per launch and each variant is its own copy of
// the tile loop: what runs is then one compact, contiguous block of code.  With the choice made per
// unit inside one loop the variants' blocks interleaved, the drain overflowed the instruction cache
// and ran 2x slower (measured: "no instruction" was the top stall reason).
//   PEERS      fused all-gather (tiles also go to peer GPUs' buffers): generic arithmetic,
//   DUMP       parity tests (raw accumulators are also written): generic arithmetic,
//   PER_TOKEN  per-row activation scales multiply the table entry,
//   MAGIC      every unit of the launch is short enough for the magic-number int->float conversion.
template <int KIND, bool DUAL, bool PAIR>
__device__ __forceinline__ void epilogue_role(const GemmParams& p, const OutMaps* map_y, uint32_t tmem_base, const uint8_t* tab,
                                              uint32_t bar_tmem_full, uint32_t bar_tmem_empty, uint32_t bar_tab_full,
                                              uint32_t bar_tab_empty, volatile int* abort_flag, long long first_tile,
                                              long long tile_step, int rank, int warp, int lane, uint8_t* stage) {
#define SQ_EPI_RUN(MAGIC, PT, DUMP, PEERS)                                                                                        \
    epilogue_tiles<KIND, DUAL, PAIR, MAGIC, PT, DUMP, PEERS>(p, map_y, tmem_base, tab, bar_tmem_full, bar_tmem_empty, bar_tab_full, \
                                                             bar_tab_empty, abort_flag, first_tile, tile_step, rank, warp, lane, stage)
    constexpr bool kInt = KIND != SQ_GEMM_W8A8_F8;
    if (p.n_peers > 0) {
        SQ_EPI_RUN(false, true, false, true);      // fused all-gather: one generic variant (exact arithmetic, see DUMP)
    } else if (p.acc_dump != nullptr) {
        SQ_EPI_RUN(false, true, true, false);
    } else if (p.sx_rs != 0) {
        if (kInt && p.all_magic) SQ_EPI_RUN(kInt, true, false, false);
        else SQ_EPI_RUN(false, true, false, false);
    } else {
        if (kInt && p.all_magic) SQ_EPI_RUN(kInt, false, false, false);
        else SQ_EPI_RUN(false, false, false, false);
    }
#undef SQ_EPI_RUN
}
