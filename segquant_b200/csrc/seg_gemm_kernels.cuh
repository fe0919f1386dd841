// Segmented quantised GEMM with fused de-quantise epilogue for sm_100a.
//
//   TMA (cp.async.bulk.tensor, no multicast) -> 128B-swizzled shared memory -> tcgen05.mma
//   (kind::i8 / kind::f8f6f4, 128 x bn x 32 per CTA or 256 x bn x 32 per CTA pair) -> int32 / fp32
//   accumulators in tensor memory -> tcgen05.ld -> per-unit scale, running fp32 sum in registers, bias,
//   cast, TMA store.
//
// It replaces the CUTLASS mma.sync GemmUniversal of segquant/src/real_quant/real_gemm.cu:208-305,
// the fp32 scratch it writes, real_dequantize_{,dual_}scaled_kernel of
// segquant/src/real_quant/dequantizer.cuh:35-73 and the torch-side segment sum / bias add of
// segquant/layers/SegmentLinear.py:238-241.
//
// Persistent kernel, one CTA per SM, warp roles:
//   warp 0      : TMA producer (one lane)
//   warp 1      : allocates tensor memory, issues tcgen05.mma (one lane)
//   warps 2-3   : build the epilogue's per-unit scale tables (and stage the bias) in shared memory
//   warps 4-11  : epilogue, two warpgroups; warpgroup h owns half of the tile's columns,
//                 warp w reads TMEM lanes 32*(w%4) .. +31 (one output row per thread)
//   warps 12-15 : (W4A8 only) expand packed int4 weights to int8 in shared memory, in place
//
// K is cut into accumulation units (activation segments x weight-scale groups).  A unit's
// products are accumulated exactly in tensor memory; at a unit boundary the MMA warp switches to
// the other TMEM buffer while the epilogue drains the finished one into fp32 registers, so integer
// sums never cross a scale boundary.  With DualScale the positive and the negative activation
// tile share the weight tile: two MMAs per K step into the two TMEM buffers.
//
// Every wait in this file is bounded: when one runs out the kernel records a code in the device
// status word, raises a CTA-wide abort flag and every role leaves its loop.
//
// This header holds all device code.  It is compiled once per (KIND, DUAL) by seg_gemm_tu_*.cu, which
// define SQ_TU_KIND and SQ_TU_DUAL before including it.
#pragma once
#include <cstdlib>

#include "seg_gemm_params.cuh"

namespace sq {

// Written (first writer wins) when a bounded wait gives up: (block index << 8) | WaitCode.
// One copy per translation unit and device; read and cleared through tu_read_status().
static __device__ unsigned long long g_wait_status = 0ull;

// Timeline instrumentation, compiled in only with -DSQ_TRACE (never in the product library):
// clock64() stamps of block 0's producer (role 0), MMA issuer (role 1) and first epilogue thread (role 2).
#ifdef SQ_TRACE
static __device__ long long g_trace[3 * 4096];
#define SQ_STAMP(role, idx) do { if (blockIdx.x == 0 && (idx) < 4096) g_trace[(role) * 4096 + (idx)] = clock64(); } while (0)
#else
#define SQ_STAMP(role, idx) do { } while (0)
#endif
#ifdef SQ_TRACE_EPI   // eight stamps per accumulation unit of block 0's first epilogue thread, in role 0's slots
#undef SQ_STAMP
#define SQ_STAMP(role, idx) do { if ((role) != 0 && blockIdx.x == 0 && (idx) < 4096) g_trace[(role) * 4096 + (idx)] = clock64(); } while (0)
#define SQ_EPI(slot) do { if (threadIdx.x == 128 && blockIdx.x == 0 && au < 500) g_trace[8 * au + (slot)] = clock64(); } while (0)
#else
#define SQ_EPI(slot) do { } while (0)
#endif
#ifdef SQ_TRACE_CVT   // eight stamps per stage of block 0's first int4-expansion thread, in role 0's slots
#undef SQ_STAMP
#define SQ_STAMP(role, idx) do { if ((role) != 0 && blockIdx.x == 0 && (idx) < 4096) g_trace[(role) * 4096 + (idx)] = clock64(); } while (0)
#define SQ_CVT(slot) do { if (threadIdx.x == 384 && blockIdx.x == 0 && it < 500) g_trace[8 * it + (slot)] = clock64(); } while (0)
#else
#define SQ_CVT(slot) do { } while (0)
#endif
#ifdef SQ_TRACE_FINE
#define SQ_FINE(slot) do { if (lane == 0 && blockIdx.x == 0 && trace_mma < 500) g_trace[2 * 4096 + 8 * trace_mma + (slot)] = clock64(); } while (0)
#else
#define SQ_FINE(slot) do { } while (0)
#endif

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrival on a barrier of this CTA or of the other CTA of the pair (cluster address).  Default semantics (release at CTA
// scope): what the waiter consumes is tensor memory, ordered by the tcgen05 fences on both sides, or shared memory written
// for the async proxy, ordered by the writer's fence.proxy.async; a cluster-scope release here was measured at 1100-1900
// cycles per arrival (it was the longest step of the int4 expansion warps and of every accumulator hand-back of a pair).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// The same test with a suspend-time hint (nanoseconds): the thread may sleep in hardware until the phase completes instead
// of returning early to poll again.  Used by the MMA issuer of the one-CTA kernel with 8-bit weights: that kernel runs at
// its shared-memory roofline, every poll of a barrier is one more shared-memory access, and with the hint its K = 1536
// layers are 4-6 % faster when run back to back (8192 x 6144 x 1536: 71.2 -> 67.9 us; inside the MMDiT step, among other
// kernels, the difference is within noise).  Measured and left alone: the same hint on the producer's,
// table builders' and epilogue's waits (no change), on the int4 expansion path (3 % slower) and on the pair kernel's
// issuer (1 % slower on the headline layer).
__device__ __forceinline__ uint32_t mbar_try_wait_relaxed(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(20000)
        : "memory");
    return done;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: gives up after `limit` SM cycles (GemmParams::wait_cycles, 4e9 = about 2 s unless the host changed
// it), or as soon as another role has raised the abort flag.  (Backing off with nanosleep was measured: no gain for the epilogue, slower hand-offs.)  The timeout uses the SM-local cycle counter: reading %globaltimer costs microseconds.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, long long limit,
                                          bool relaxed = false) {
    if (relaxed ? mbar_try_wait_relaxed(bar, parity) : mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    for (uint32_t it = 1;; ++it) {
        if (relaxed ? mbar_try_wait_relaxed(bar, parity) : mbar_try_wait(bar, parity)) return true;
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

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// tcgen05.commit: the mbarrier gets one arrival when every tcgen05.mma issued so far by this
// thread has finished reading shared memory and writing tensor memory.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int KIND>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == SQ_GEMM_W8A8_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Tensor-memory loads / stores / waits are volatile (kept in program order among themselves and with the barrier
// operations) but do not clobber "memory": they touch nothing the compiler can see, and a memory clobber would pin the
// epilogue's shared-memory table reads between them instead of letting them be issued early.
#ifndef SQ_TMEM_CLOBBER
#define SQ_TMEM_CLOBBER
#endif
// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        SQ_TMEM_CLOBBER);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" :: SQ_TMEM_CLOBBER); }
// 32 lanes x 8 consecutive 32-bit columns (thread t writes lane base + t) from 8 registers.  The refill of the magic
// pattern passes the SAME eight registers every time (MagicRegs): a store needs its sources in one consecutive block,
// and values the compiler cannot see through stay in the block they were first put in, so no copies are made per store.
struct MagicRegs {
    uint32_t r[8];
};
__device__ __forceinline__ void magic_regs_init(MagicRegs& m) {
#pragma unroll
    for (int i = 0; i < 8; ++i) asm volatile("mov.b32 %0, 0x4B400000;" : "=r"(m.r[i]));
}
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const MagicRegs& m) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(m.r[0]), "r"(m.r[1]), "r"(m.r[2]), "r"(m.r[3]), "r"(m.r[4]), "r"(m.r[5]), "r"(m.r[6]), "r"(m.r[7])
        SQ_TMEM_CLOBBER);
}
// 16 columns
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const MagicRegs& m) {
    tmem_st_x8(taddr, m);
    tmem_st_x8(taddr + 8u, m);
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" :: SQ_TMEM_CLOBBER); }

// Bit pattern of 1.5 * 2^23.  An int32 accumulator that STARTS at this value and then collects a sum n with
// |n| < 2^22 holds, read as a float, exactly 12582912 + n: the epilogue gets float(n) with one subtraction instead of
// an integer add plus a subtraction (or a quarter-rate conversion).  Used when every accumulation unit of the launch is
// short (GemmParams::all_magic): the epilogue warps fill tensor memory with the pattern before the first tile and put it
// back after every chunk they drain, and the MMA warp always accumulates onto what it finds.
constexpr uint32_t kMagicBits = 0x4B400000u;

// Epilogue warp `warp` (4..11) fills its lane quarter of one half of tensor memory (256 columns) with the magic pattern.
__device__ __forceinline__ void tmem_fill_magic(uint32_t tmem_base, int warp) {
    const uint32_t lane_q = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t col0 = static_cast<uint32_t>((warp - 4) >> 2) * 256u;
    MagicRegs mg;
    magic_regs_init(mg);
#pragma unroll
    for (int c = 0; c < 16; ++c) tmem_st_x16(tmem_base + lane_q + col0 + c * 16, mg);
    tmem_st_wait();
}

template <uint32_t N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <uint32_t N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA SWIZZLE_128B writes).  Low word: start address >> 4 (14 bits) and the
// leading-dimension offset (unused for swizzled K-major layouts, set to 1).  High word: 8-row groups
// are 1024 bytes apart (SBO = 64), descriptor version 1 = Blackwell (bit 46), layout type 2 =
// SWIZZLE_128B (bits 61-63).  Stepping K by one MMA (32 bytes) adds 2 to the low word.
constexpr uint32_t kSmemDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t addr) { return ((addr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ uint64_t smem_desc(uint32_t lo) { return (static_cast<uint64_t>(kSmemDescHi) << 32) | lo; }

// Instruction descriptor: dense, no negate, both operands K-major, D = 128 x bn.
template <int KIND>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
    uint32_t d = 0;
    if (KIND == SQ_GEMM_W8A8_F8) {
        d |= 1u << 4;   // D format F32
        d |= 0u << 7;   // A = E4M3
        d |= 0u << 10;  // B = E4M3
    } else {
        d |= 2u << 4;   // D format S32
        d |= 1u << 7;   // A = signed 8-bit
        d |= 1u << 10;  // B = signed 8-bit
    }
    d |= static_cast<uint32_t>(BM >> 4) << 24;   // the N field (bits 17-22) is added at run time: bn >> 3
    return d;
}

// ---------------------------------------------------------------------------------------------
// Kernel configuration
// ---------------------------------------------------------------------------------------------
template <int KIND, bool DUAL>
struct Cfg {
    static constexpr bool kW4 = KIND == SQ_GEMM_W4A8;
    // W4A8: the packed int4 tile lands in the upper half of the operand buffer and is expanded in place (no extra staging)
    static constexpr uint32_t kStageBytes = kABytes * (DUAL ? 2 : 1) + kBBytes;
    static constexpr int kStages = (192 * 1024) / kStageBytes;
    static constexpr int kThreads = kW4 ? 512 : 384;
    static constexpr uint32_t kTxBytes = kABytes * (DUAL ? 2 : 1) + (kW4 ? kBPackedBytes : kBBytes);
    // dynamic shared memory: 1 KB alignment slack + stages + scale tables + output staging
    static constexpr uint32_t kTabBytes = kTabBytesAll;
    static constexpr uint32_t kSmemBytes = 1024 + kStages * kStageBytes + kTabBytes + kStoreStageBytes + 256;
};

struct UnitCursor {
    int s, k, k_end, g;
};

__device__ __forceinline__ int unit_end(const GemmParams& p, int s, int k) {
    int e = p.seg_bounds[s + 1];
    if (p.group_size > 0) {
        const int ge = (k / p.group_size + 1) * p.group_size;
        e = ge < e ? ge : e;
    }
    return e;
}

__device__ __forceinline__ float load_sw(const GemmParams& p, long long idx) {
    if (p.sw_is_bf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.sw)[idx]);
    return static_cast<const float*>(p.sw)[idx];
}

template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* dst, const float (&v)[16], int valid, bool vec_ok) {
    if (vec_ok && valid >= 16) {
        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    OutT lo = from_float<OutT>(v[8 * i + 2 * j]);
                    OutT hi = from_float<OutT>(v[8 * i + 2 * j + 1]);
                    w[j] = static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&lo)) |
                           (static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&hi)) << 16);
                }
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (i < valid) dst[i] = from_float<OutT>(v[i]);
    }
}

__device__ __forceinline__ float load_bias(const void* bias, int dtype, long long idx) {
    if (dtype == SQ_F32) return __ldg(static_cast<const float*>(bias) + idx);
    if (dtype == SQ_F16) return __half2float(__ldg(static_cast<const __half*>(bias) + idx));
    return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(bias) + idx));
}

// TMA store of a [rows x 16 columns] box from shared memory; out-of-range rows / columns are clipped.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }


// Fused all-gather: the same 16 output columns of row m go to every peer GPU's [M, *] buffer with plain
// 128-bit stores (peer memory mapped into this process; N is a multiple of 8 / 4 elements and every row
// offset is 16-byte aligned, checked on the host, so a 16-column chunk is either whole or absent).
__device__ __forceinline__ void store_peers(const GemmParams& p, const float (&o)[16], long long m, long long nc) {
    const int esz = p.out_dtype == SQ_F32 ? 4 : 2;
    int valid = static_cast<int>(p.N - nc);
    valid = valid > 16 ? 16 : valid;
    if (valid <= 0) return;
    for (int j = 0; j < p.n_peers; ++j) {
        uint8_t* dst = static_cast<uint8_t*>(p.peer_y[j]) + (m * p.peer_rs + p.peer_co + nc) * esz;
        if (p.out_dtype == SQ_F32) store_row_chunk<float>(reinterpret_cast<float*>(dst), o, valid, true);
        else if (p.out_dtype == SQ_F16) store_row_chunk<__half>(reinterpret_cast<__half*>(dst), o, valid, true);
        else store_row_chunk<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(dst), o, valid, true);
    }
}

// 16 output columns of row `r` of a box with 128-byte rows laid out with the 128-byte swizzle (16-byte piece index XOR
// row % 8: what a SWIZZLE_128B tensor map expects, and free of bank conflicts for lanes writing one row each).
// `piece0` = index of the first 16-byte piece of these columns inside the row (0, 2, 4, 6 / 0, 4).
template <typename OutT>
__device__ __forceinline__ void store_row_chunk_swz(uint8_t* box, int r, int piece0, const float (&v)[16]) {
    uint8_t* row = box + r * 128;
    const int x = r & 7;
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<float4*>(row + (((piece0 + i) ^ x) << 4)) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                OutT lo = from_float<OutT>(v[8 * i + 2 * j]);
                OutT hi = from_float<OutT>(v[8 * i + 2 * j + 1]);
                w[j] = static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&lo)) |
                       (static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&hi)) << 16);
            }
            *reinterpret_cast<uint4*>(row + (((piece0 + i) ^ x) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

// Fused all-gather with wide boxes.  Per 128 bytes of output row (CPB 16-column chunks: 64 columns of a 16-bit type, 32
// of fp32) the warp's 2 KB staging area is filled twice - rows 0-15 by lanes 0-15, then rows 16-31 by lanes 16-31 - and
// each time one TMA store per destination (this GPU's matrix and every peer's) moves [16 rows x 128 bytes]: whole
// 128-byte lines on NVLink instead of the 32-byte row pieces of a 16-column box.  The host only asks for this with tile
// widths whose per-warp column count is a multiple of the box (bn 128 / 256), so a box never reaches into the columns
// of the neighbouring warp; columns past N and rows past M are clipped by the tensor map.
template <int CPB>
__device__ __forceinline__ void store_output_wide(const GemmParams& p, const OutMaps* map_y, const float (&acc)[128], int nch,
                                                  int m_warp, long long ncol0, uint8_t* stage, int lane, const float* bias_s) {
    if (m_warp >= p.M) return;                       // nothing of this warp's 32 rows exists (warp-uniform)
    const int esz = CPB == 4 ? 2 : 4;
    const uint32_t stage_u32 = smem_u32(stage);
    const int row16 = lane & 15;
#pragma unroll
    for (int g = 0; g < 8 / CPB; ++g) {              // boxes along the warp's columns
        const int ch0 = g * CPB;
        const long long nc0 = ncol0 + ch0 * 16;
        if (ch0 >= nch || nc0 >= p.N) break;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (m_warp + 16 * half >= p.M) break;    // warp-uniform
            if (lane == 0) bulk_wait_read<0>();      // the staging area has been read by the previous box's stores
            __syncwarp();
            if ((lane >> 4) == half) {
#pragma unroll
                for (int cb = 0; cb < CPB; ++cb) {
                    const int ch = ch0 + cb;
                    if (ch < nch) {                  // chunks past N only fill bytes the tensor map clips
                        float o[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) o[j] = acc[ch * 16 + j];
                        if (p.bias != nullptr) {
#pragma unroll
                            for (int j4 = 0; j4 < 4; ++j4) {
                                const float4 bv = reinterpret_cast<const float4*>(bias_s + ch * 16)[j4];   // 0 beyond column N
                                o[4 * j4 + 0] += bv.x;
                                o[4 * j4 + 1] += bv.y;
                                o[4 * j4 + 2] += bv.z;
                                o[4 * j4 + 3] += bv.w;
                            }
                        }
                        if (CPB == 2) store_row_chunk_swz<float>(stage, row16, cb * 4, o);
                        else if (p.out_dtype == SQ_F16) store_row_chunk_swz<__half>(stage, row16, cb * 2, o);
                        else store_row_chunk_swz<__nv_bfloat16>(stage, row16, cb * 2, o);
                    }
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                const int c0 = static_cast<int>(nc0) * esz;   // the maps are byte-typed
                const int r0 = m_warp + 16 * half;
                tma_store_3d(&map_y->y, stage_u32, c0, r0, 0);
                for (int j = 0; j < p.n_peers; ++j) tma_store_3d(&map_y->peer[j], stage_u32, c0, r0, 0);
                bulk_commit();
            }
        }
    }
}

// Bias, cast and store of one thread's output row segment (up to 128 columns held in acc[]).
// bias_s: this thread's columns of the tile's bias in shared memory, as fp32 (written by the table builder).
// Aligned outputs go through shared memory and TMA stores (one [32 rows x 16 columns] box per warp and
// chunk; the LSU stays free for the MMA / producer warps, every DRAM sector is written whole);
// otherwise each thread writes its row directly.  `stage` is this warp's 2 KB staging area.
// PEERS: the launch also writes peer GPUs' buffers (fused all-gather); a compile-time switch, because even a skipped
// branch per chunk in this fully unrolled loop costs every launch about 1.5 % (measured).
template <bool PEERS>
__device__ __forceinline__ void store_output(const GemmParams& p, const OutMaps* map_y, const float (&acc)[128], int nch,
                                             long long b, long long m, int m_warp, bool row_ok, long long ncol0,
                                             uint8_t* stage, int lane, const float* bias_s) {
    const int esz = p.out_dtype == SQ_F32 ? 4 : 2;
    if constexpr (PEERS) {
        if (p.peer_wide) {
            if (esz == 2) store_output_wide<4>(p, map_y, acc, nch, m_warp, ncol0, stage, lane, bias_s);
            else store_output_wide<2>(p, map_y, acc, nch, m_warp, ncol0, stage, lane, bias_s);
            return;
        }
    }
    if (p.y_tma) {
        if (m_warp >= p.M) return;                           // nothing of this warp's 32 rows exists (warp-uniform)
        const uint32_t stage_u32 = smem_u32(stage);
        const uint32_t buf_bytes = 32u * 16u * esz;          // 1 KB (16-bit) or 2 KB (fp32)
        const bool two_bufs = esz == 2;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            const long long nc = ncol0 + ch * 16;
            if (ch >= nch || nc >= p.N) break;
            float o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = acc[ch * 16 + j];
            if (p.bias != nullptr) {
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                    const float4 bv = reinterpret_cast<const float4*>(bias_s + ch * 16)[j4];   // 0 beyond column N
                    o[4 * j4 + 0] += bv.x;
                    o[4 * j4 + 1] += bv.y;
                    o[4 * j4 + 2] += bv.z;
                    o[4 * j4 + 3] += bv.w;
                }
            }
            const uint32_t off = (two_bufs && (ch & 1)) ? buf_bytes : 0u;
            // the buffer about to be overwritten must have been read by its previous TMA store
            if (lane == 0) {
                if (two_bufs) bulk_wait_read<1>();
                else bulk_wait_read<0>();
            }
            __syncwarp();
            uint8_t* dst = stage + off + lane * 16 * esz;
            if (p.out_dtype == SQ_F32) store_row_chunk<float>(reinterpret_cast<float*>(dst), o, 16, true);
            else if (p.out_dtype == SQ_F16) store_row_chunk<__half>(reinterpret_cast<__half*>(dst), o, 16, true);
            else store_row_chunk<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(dst), o, 16, true);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(&map_y->y, stage_u32 + off, static_cast<int>(nc) * esz, m_warp, static_cast<int>(b));   // the map is byte-typed
                if constexpr (PEERS) {
                    if (p.peer_tma)   // fused all-gather: the same box goes to every peer GPU, asynchronously
                        for (int j = 0; j < p.n_peers; ++j)
                            tma_store_3d(&map_y->peer[j], stage_u32 + off, static_cast<int>(nc) * esz, m_warp, 0);
                }
                bulk_commit();
            }
            if constexpr (PEERS) {
                if (!p.peer_tma && row_ok) store_peers(p, o, m, nc);
            }
        }
        return;
    }
    if (!row_ok) return;
    uint8_t* yrow = static_cast<uint8_t*>(p.y) + (b * p.y_bs + m * p.y_rs + ncol0) * esz;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(yrow) & 15u) == 0;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
        const long long nc = ncol0 + ch * 16;
        int valid = static_cast<int>(p.N - nc);
        valid = valid > 16 ? 16 : valid;
        if (valid > 0 && ch < nch) {
            float o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = acc[ch * 16 + j];
            if (p.bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 16; ++j) o[j] += bias_s[ch * 16 + j];
            }
            if (p.out_dtype == SQ_F32) store_row_chunk<float>(reinterpret_cast<float*>(yrow) + ch * 16, o, valid, vec_ok);
            else if (p.out_dtype == SQ_F16) store_row_chunk<__half>(reinterpret_cast<__half*>(yrow) + ch * 16, o, valid, vec_ok);
            else store_row_chunk<__nv_bfloat16>(reinterpret_cast<__nv_bfloat16*>(yrow) + ch * 16, o, valid, vec_ok);
            if constexpr (PEERS) store_peers(p, o, m, nc);
        }
    }
}

#include "seg_gemm_epilogue.cuh"

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int KIND, bool DUAL>
__global__ void __launch_bounds__(Cfg<KIND, DUAL>::kThreads, 1)
seg_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_an,
                const __grid_constant__ CUtensorMap map_w, const __grid_constant__ OutMaps map_y,
                const __grid_constant__ GemmParams p) {
    using C = Cfg<KIND, DUAL>;
    constexpr int kStages = C::kStages;
    constexpr bool kW4 = C::kW4;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[8], bar_empty[8], bar_cvt[8], bar_tmem_full[2], bar_tmem_empty[2], bar_tab_full[kTabSlots], bar_tab_empty[kTabSlots];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* tab = smem_gen + kStages * C::kStageBytes;   // kTabSlots scale-table slots

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    auto stage_a = [&](int st) { return smem_base + st * C::kStageBytes; };
    auto stage_an = [&](int st) { return smem_base + st * C::kStageBytes + kABytes; };
    auto stage_b = [&](int st) { return smem_base + st * C::kStageBytes + kABytes * (DUAL ? 2 : 1); };
    auto stage_bp = [&](int st) { return smem_base + st * C::kStageBytes + kABytes * (DUAL ? 2 : 1) + kBBytes / 2; };   // upper half of B

    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(smem_u32(&bar_full[i]), 1);
            mbar_init(smem_u32(&bar_empty[i]), 1);
            mbar_init(smem_u32(&bar_cvt[i]), 4);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bar_tmem_full[i]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[i]), kEpiThreads / 32);
        }
        for (int i = 0; i < kTabSlots; ++i) {
            mbar_init(smem_u32(&bar_tab_full[i]), 2);                  // the two builder warps
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
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    if (p.all_magic) {   // warp-uniform: integer accumulators start from the magic pattern (see kMagicBits)
        if (warp >= 4 && warp < 12) tmem_fill_magic(tmem_base, warp);
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }

    const int tiles_per_batch = p.tiles_m * p.tiles_n;

    if (warp < 4) {
        // ------------------------------------------------------------------ producer / MMA warps
        // The producer and the MMA issuer are ONE thread each (lane 0 of their warps); the other lanes wait at the end.
        reg_dec<kW4 ? SQ_W4_CTRL : kCtrlRegs>();
        if (warp == 0) {
            // ===== TMA producer =====
            int trace_it = 0; (void)trace_it;
            int st = 0;
            uint32_t ph = 0;
            bool ok = true;
            // one elected lane runs the whole loop: waits, issue and commits are single-thread work, and a warp that walks the
            // loop together pays a divergence / reconvergence round trip at every lane-0 block (~150-200 cycles per stage)
            if (lane == 0) {
                for (long long tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                    const int b = static_cast<int>(tile / tiles_per_batch);
                    const int rem = static_cast<int>(tile - static_cast<long long>(b) * tiles_per_batch);
                    const int m0 = (rem / p.tiles_n) * BM;
                    const int n0 = (rem % p.tiles_n) * p.bn;
                    const int ab = p.a_batched ? b : 0;
                    for (int s = 0; ok && s < p.num_segs; ++s) {
                        const int k_beg = p.seg_bounds[s], k_end = p.seg_bounds[s + 1];
                        const int wb = p.w_seg_as_batch ? s : (p.w_batched ? b : 0);
                        const int wk_off = p.w_seg_as_batch ? k_beg : 0;
                        for (int k = k_beg; k < k_end; k += BK) {
                            if (!mbar_wait(smem_u32(&bar_empty[st]), ph ^ 1u, abort_flag, kWaitEmpty, p.wait_cycles)) { ok = false; break; }
                            {
                                SQ_STAMP(0, 2 * trace_it);
                                const uint32_t full = smem_u32(&bar_full[st]);
                                mbar_arrive_expect_tx(full, kABytes * (DUAL ? 2 : 1) + static_cast<uint32_t>(p.bn) * (kW4 ? BK / 2 : BK));
                                tma_load_3d(stage_a(st), &map_a, k, m0, ab, full);
                                if (DUAL) tma_load_3d(stage_an(st), &map_an, k, m0, ab, full);
                                if (kW4) tma_load_3d(stage_bp(st), &map_w, (k - wk_off) >> 1, n0, wb, full);
                                else tma_load_3d(stage_b(st), &map_w, k - wk_off, n0, wb, full);
                            }
                            SQ_STAMP(0, 2 * trace_it + 1);
                            ++trace_it;
                            if (++st == kStages) { st = 0; ph ^= 1u; }
                        }
                    }
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // ===== MMA issuer =====
            const uint32_t idesc = make_idesc<KIND>() | (static_cast<uint32_t>(p.bn >> 3) << 17);
            const bool one_buf = DUAL && !p.dual_db;   // DualScale with wide tiles: pos / neg fill all of TMEM
            int st = 0;
            uint32_t ph = 0;
            uint32_t au = 0;       // accumulation-unit counter (selects the TMEM buffer)
            uint32_t cur_buf = 0;  // buffer of the unit being accumulated
            int trace_mma = 0; (void)trace_mma;
            bool ok = true;
            // one elected lane runs the whole loop: waits, issue and commits are single-thread work, and a warp that walks the
            // loop together pays a divergence / reconvergence round trip at every lane-0 block (~150-200 cycles per stage)
            if (lane == 0) {
                for (long long tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                    for (int s = 0; ok && s < p.num_segs; ++s) {
                        const int k_beg = p.seg_bounds[s], k_end = p.seg_bounds[s + 1];
                        int u_end = k_beg;  // forces "new unit" at the first step of the segment
                        uint32_t accumulate = p.all_magic ? 1u : 0u;   // all_magic: the buffer holds the magic pattern, never garbage
                        uint32_t d_pos = 0, d_neg = 0;
                        for (int kb = k_beg; ok && kb < k_end; kb += BK) {
                            SQ_FINE(0);
                            if (!mbar_wait(smem_u32(&bar_full[st]), ph, abort_flag, kWaitFull, p.wait_cycles, !kW4)) { ok = false; break; }
                            if (kW4) {
                                if (!mbar_wait(smem_u32(&bar_cvt[st]), ph, abort_flag, kWaitCvt, p.wait_cycles)) { ok = false; break; }
                            }
                            SQ_FINE(1);
                            tc_fence_after();
                            SQ_FINE(2);
                            SQ_STAMP(1, 3 * trace_mma);
                            const uint32_t a_lo = smem_desc_lo(stage_a(st));
                            const uint32_t an_lo = smem_desc_lo(stage_an(st));
                            const uint32_t b_lo = smem_desc_lo(stage_b(st));
                            const int kmax = (k_end - kb) < BK ? (k_end - kb) : BK;
                            if (kb == u_end) {
                                // the stage opens a new unit (the common place for a boundary): hand the finished TMEM
                                // buffer to the epilogue and take the other one, once, before any MMA of the stage
                                if (kb != k_beg) umma_commit(smem_u32(&bar_tmem_full[cur_buf]));
                                const uint32_t buf = one_buf ? 0u : (au & 1u);
                                const uint32_t tph = one_buf ? (au & 1u) : ((au >> 1) & 1u);
                                if (!mbar_wait(smem_u32(&bar_tmem_empty[buf]), tph ^ 1u, abort_flag, kWaitTmemEmpty, p.wait_cycles, !kW4)) { ok = false; break; }
                                tc_fence_after();
                                cur_buf = buf;
                                d_pos = tmem_base + buf * BN;
                                d_neg = tmem_base + (p.dual_db ? buf * BN + 128 : BN);
                                accumulate = p.all_magic ? 1u : 0u;   // all_magic: the buffer holds the magic pattern, never garbage
                                u_end = unit_end(p, s, kb);
                                ++au;
                            }
                            if (kb + kmax <= u_end) {
                                // the whole stage lies inside the current unit: no checks between the MMAs
                                {
    #pragma unroll
                                    for (int i = 0; i < BK / UMMA_K; ++i) {
                                        if (i * UMMA_K < kmax) {
                                            const uint64_t db = smem_desc(b_lo + 2 * i);
                                            const uint32_t accf = i == 0 ? accumulate : 1u;
                                            umma<KIND>(d_pos, smem_desc(a_lo + 2 * i), db, idesc, accf);
                                            if (DUAL) umma<KIND>(d_neg, smem_desc(an_lo + 2 * i), db, idesc, accf);
                                            SQ_FINE(3 + i);
                                        }
                                    }
                                }
                                accumulate = 1;
                            } else {
                                // a unit ends inside this stage (segment bounds or groups that are not multiples of 128)
                                for (int kk = 0; kk < kmax; kk += UMMA_K) {
                                    const int k = kb + kk;
                                    if (k == u_end) {
                                        umma_commit(smem_u32(&bar_tmem_full[cur_buf]));
                                        const uint32_t buf = one_buf ? 0u : (au & 1u);
                                        const uint32_t tph = one_buf ? (au & 1u) : ((au >> 1) & 1u);
                                        if (!mbar_wait(smem_u32(&bar_tmem_empty[buf]), tph ^ 1u, abort_flag, kWaitTmemEmpty, p.wait_cycles, !kW4)) { ok = false; break; }
                                        tc_fence_after();
                                        cur_buf = buf;
                                        d_pos = tmem_base + buf * BN;
                                        d_neg = tmem_base + (p.dual_db ? buf * BN + 128 : BN);
                                        accumulate = p.all_magic ? 1u : 0u;   // all_magic: the buffer holds the magic pattern, never garbage
                                        u_end = unit_end(p, s, k);
                                        ++au;
                                    }
                                    {
                                        const uint64_t db = smem_desc(b_lo + (kk >> 4));
                                        umma<KIND>(d_pos, smem_desc(a_lo + (kk >> 4)), db, idesc, accumulate);
                                        if (DUAL) umma<KIND>(d_neg, smem_desc(an_lo + (kk >> 4)), db, idesc, accumulate);
                                    }
                                    accumulate = 1;
                                }
                                if (!ok) break;
                            }
                            SQ_STAMP(1, 3 * trace_mma + 1);
                            umma_commit(smem_u32(&bar_empty[st]));  // stage free once these MMAs have read it
                            SQ_STAMP(1, 3 * trace_mma + 2);
                            SQ_FINE(7);
                            ++trace_mma;
                            if (++st == kStages) { st = 0; ph ^= 1u; }
                        }
                        if (ok) umma_commit(smem_u32(&bar_tmem_full[cur_buf]));  // last unit of the segment
                    }
                }
            }
            __syncwarp();
        } else {
            // ===== warps 2-3: per-unit scale tables for the epilogue =====
            table_builder<KIND, DUAL, false>(p, tab, smem_u32(&bar_tab_full[0]), smem_u32(&bar_tab_empty[0]), abort_flag, blockIdx.x,
                                             gridDim.x, 0);
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------------ epilogue warps
        reg_inc<kW4 ? kEpiRegsW4 : kEpiRegs>();
        epilogue_role<KIND, DUAL, false>(p, &map_y, tmem_base, tab, smem_u32(&bar_tmem_full[0]), smem_u32(&bar_tmem_empty[0]),
                                         smem_u32(&bar_tab_full[0]), smem_u32(&bar_tab_empty[0]), abort_flag, blockIdx.x, gridDim.x, 0,
                                         warp, lane, smem_gen + kStages * C::kStageBytes + C::kTabBytes + (warp - 4) * 2048);
        if (lane == 0) bulk_wait_all();   // this warp's TMA stores have reached memory before the CTA exits
    } else {
        // ------------------------------------------------------------------ int4 -> int8 expansion warps (W4A8)
        if constexpr (kW4) {
            reg_dec<SQ_W4_CVT>();
            const int ct = threadIdx.x - 384;  // 0..127
            uint32_t it = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                for (int s = 0; ok && s < p.num_segs; ++s) {
                    const int k_beg = p.seg_bounds[s], k_end = p.seg_bounds[s + 1];
                    for (int kb = k_beg; kb < k_end; kb += BK, ++it) {
                        const int st = it % kStages;
                        const uint32_t ph = (it / kStages) & 1u;
                        SQ_CVT(0);
                        if (!mbar_wait(smem_u32(&bar_full[st]), ph, abort_flag, kWaitFullCvt, p.wait_cycles)) { ok = false; break; }
                        SQ_CVT(1);
                        const uint8_t* src = smem_gen + (stage_bp(st) - smem_base);
                        uint8_t* dst = smem_gen + (stage_b(st) - smem_base);
                        // The packed tile (bn rows x 64 bytes; 16-byte chunk = (row, quarter)) sits in the upper half of
                        // the 32 KB buffer it expands into.  Thread ct owns chunks (row0 + 32 i, qd), i = 0..7: the swizzle
                        // term (row % 8) and qd do not depend on i, so the destination offsets inside a row are constants.
                        // Rows < 128 expand into the lower half, which holds no packed bytes: done first, straight from
                        // shared memory.  Rows >= 128 overwrite the packed area: their chunks are pulled into registers
                        // up front, the four expansion warps meet on a barrier once everybody has read, and only
                        // then are they written.
                        const int row0 = ct >> 2, qd = ct & 3;
                        const int o0 = ((2 * qd) ^ (row0 & 7)) * 16, o1 = ((2 * qd + 1) ^ (row0 & 7)) * 16;
                        const uint8_t* srow = src + row0 * 64 + qd * 16;
                        uint8_t* drow = dst + row0 * 128;
                        auto expand_store = [&](const uint4& v, int i) {
                            const uint32_t in[4] = {v.x, v.y, v.z, v.w};
                            uint32_t out[8];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                // int8 value = 16 * int4 value: nibble moved to the top of its byte
                                const uint32_t lo = (in[j] << 4) & 0xF0F0F0F0u;  // even k
                                const uint32_t hi = in[j] & 0xF0F0F0F0u;         // odd k
                                out[2 * j] = __byte_perm(lo, hi, 0x5140);
                                out[2 * j + 1] = __byte_perm(lo, hi, 0x7362);
                            }
                            // 32 int8 = two 16-byte chunks of the 128-byte row, XOR-swizzled by (row % 8)
                            *reinterpret_cast<uint4*>(drow + i * 4096 + o0) = make_uint4(out[0], out[1], out[2], out[3]);
                            *reinterpret_cast<uint4*>(drow + i * 4096 + o1) = make_uint4(out[4], out[5], out[6], out[7]);
                        };
                        uint4 hi4[4], lo4[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (row0 + 32 * (i + 4) < p.bn) hi4[i] = *reinterpret_cast<const uint4*>(srow + (i + 4) * 2048);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (row0 + 32 * i < p.bn) lo4[i] = *reinterpret_cast<const uint4*>(srow + i * 2048);
                        SQ_CVT(2);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (row0 + 32 * i < p.bn) expand_store(lo4[i], i);
                        // Hardware barrier among the 128 expansion threads (an mbarrier round trip here cost ~200 cycles per
                        // stage, 6 % of the kernel).  It cannot be left waiting by a warp that gave up: all four warps have just
                        // passed the SAME phase of bar_full, which either completed (then each of them sees it completed: the phase
                        // cannot advance before all four have arrived on bar_cvt below) or did not (then none of them gets here).
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        SQ_CVT(3);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (row0 + 32 * (i + 4) < p.bn) expand_store(hi4[i], i + 4);
                        SQ_CVT(4);
                        fence_proxy_async_smem();  // generic-proxy writes -> visible to tcgen05.mma
                        SQ_CVT(5);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bar_cvt[st]));
                        SQ_CVT(6);
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag) {
        // give copies that may still be in flight time to land before shared memory is released
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

#include "seg_gemm_2cta.cuh"

template <int KIND, bool DUAL>
static int launch(const CUtensorMap& ma, const CUtensorMap& man, const CUtensorMap& mw, const OutMaps& my, const GemmParams& p, cudaStream_t st) {
    using C = Cfg<KIND, DUAL>;
    static_assert(C::kStages >= 2 && C::kStages <= 8, "stage count");
    static bool attr_set[64] = {};
    int dev = 0;
    SQ_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        SQ_CUDA_OK(cudaFuncSetAttribute(seg_gemm_kernel<KIND, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        attr_set[dev] = true;
    } else if (dev >= 64) {
        SQ_CUDA_OK(cudaFuncSetAttribute(seg_gemm_kernel<KIND, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    }
    const long long grid = p.total_tiles < kNumSMs ? p.total_tiles : kNumSMs;
    seg_gemm_kernel<KIND, DUAL><<<static_cast<int>(grid), C::kThreads, C::kSmemBytes, st>>>(ma, man, mw, my, p);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

// ---------------------------------------------------------------------------------------------
// This translation unit's entry points
// ---------------------------------------------------------------------------------------------
template <>
int launch_gemm<SQ_TU_KIND, SQ_TU_DUAL>(bool two_cta, const CUtensorMap& ma, const CUtensorMap& man, const CUtensorMap& mw,
                                        const OutMaps& my, const GemmParams& p, cudaStream_t st) {
    return two_cta ? launch_2cta<SQ_TU_KIND, SQ_TU_DUAL>(ma, man, mw, my, p, st) : launch<SQ_TU_KIND, SQ_TU_DUAL>(ma, man, mw, my, p, st);
}

// Stand-alone exercise of the bounded-wait / abort path the GEMM kernels rely on, for a test that must not make a
// GEMM kernel itself give up: one CTA, two warps.  Warp 0 waits (same mbar_wait helper, same status word) on a barrier
// nobody ever arrives at, so its wait runs out after `limit` cycles: it records (block << 8 | kWaitProbe), raises the
// CTA's abort flag and returns false.  Warp 1 waits on a second silent barrier with a 64 times longer limit and must
// leave early because it sees the abort flag.  Nothing traps and nothing spins without a bound.
// out[0] = abort flag at exit, out[1] / out[2] = what the two waits returned, out[3] = 1 if warp 1 left before its own limit.
static __global__ void wait_probe_kernel(long long limit, int* out) {
    __shared__ __align__(8) uint64_t bar[2];
    __shared__ int abort_flag_s;
    __shared__ int res[3];
    volatile int* abort_flag = &abort_flag_s;
    if (threadIdx.x == 0) {
        abort_flag_s = 0;
        mbar_init(smem_u32(&bar[0]), 1);
        mbar_init(smem_u32(&bar[1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    const long long t0 = clock64();
    const bool ok = warp == 0 ? mbar_wait(smem_u32(&bar[0]), 0u, abort_flag, kWaitProbe, limit)
                              : mbar_wait(smem_u32(&bar[1]), 0u, abort_flag, kWaitProbe + 1, 64 * limit);
    const long long waited = clock64() - t0;
    if ((threadIdx.x & 31) == 0) {
        res[warp] = ok ? 1 : 0;
        if (warp == 1) res[2] = waited < 32 * limit ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        out[0] = abort_flag_s;
        out[1] = res[0];
        out[2] = res[1];
        out[3] = res[2];
    }
}

template <>
int tu_wait_probe<SQ_TU_KIND, SQ_TU_DUAL>(long long limit_cycles, int* out_dev, cudaStream_t st) {
    wait_probe_kernel<<<1, 64, 0, st>>>(limit_cycles, out_dev);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

template <>
long long tu_read_status<SQ_TU_KIND, SQ_TU_DUAL>() {
    unsigned long long v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_status, sizeof(v)) != cudaSuccess) return SQ_ERR_CUDA;
    if (v != 0 && cudaMemcpyToSymbol(g_wait_status, &zero, sizeof(zero)) != cudaSuccess) return SQ_ERR_CUDA;
    return static_cast<long long>(v);
}

#ifdef SQ_TRACE
template <>
int tu_trace_read<SQ_TU_KIND, SQ_TU_DUAL>(long long* out, int n) {
    if (n > 3 * 4096) n = 3 * 4096;
    if (cudaMemcpyFromSymbol(out, g_trace, sizeof(long long) * n) != cudaSuccess) return SQ_ERR_CUDA;
    return n;
}
#endif

}  // namespace sq
