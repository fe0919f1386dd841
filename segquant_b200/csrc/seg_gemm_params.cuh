// Constants and the kernel parameter block shared by the host dispatch (seg_gemm.cu) and the kernel
// translation units (seg_gemm_tu_*.cu, which include seg_gemm_kernels.cuh).
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace sq {


constexpr int BM = 128;        // tile rows (TMEM lanes)
constexpr int BN = 256;        // widest tile (TMEM columns per buffer); the width in use is GemmParams::bn
constexpr int BK = 128;        // K elements per pipeline stage (= one 128-byte swizzle row)
constexpr int UMMA_K = 32;     // K per tcgen05.mma for 8-bit operands
constexpr int kTmemCols = 512;
constexpr int kEpiThreads = 256;

constexpr uint32_t kABytes = BM * BK;          // 16 KB
constexpr uint32_t kBBytes = BN * BK;          // 32 KB
constexpr uint32_t kBPackedBytes = BN * BK / 2;// 16 KB (int4 staging)
constexpr uint32_t kStoreStageBytes = 8 * 2048;  // output staging for TMA stores: 2 KB per epilogue warp
constexpr int kTabSlots = 4;                     // per-unit scale tables the builder warps may run ahead
constexpr uint32_t kTabSlotBytes = 4096;         // r[2][BN] + rx[2][BM] + bias[BN] floats, see seg_gemm_epilogue.cuh
constexpr uint32_t kTabBytesAll = kTabSlots * kTabSlotBytes;

// status-word codes (low byte = which wait, rest = block index)
enum WaitCode : int { kWaitProbe = 9, kWaitEmpty = 1, kWaitFull = 2, kWaitTmemEmpty = 3, kWaitTmemFull = 4, kWaitCvt = 5, kWaitFullCvt = 6, kWaitTabFull = 7, kWaitTabEmpty = 8 };

constexpr int BM2 = 256;  // tile rows of a CTA pair

// Register allowances (setmaxnreg) of the W4A8 kernels' control warps (producer, MMA issuer, table builders) and int4
// expansion warps; the eight epilogue warps take 200.  4 * control + 8 * 200 + 4 * expansion <= 2048.
// setmaxnreg moves registers inside the pool the CTA was LAUNCHED with (threads x the kernel's launch allowance, 168 for
// 384 threads and 128 for 512), not inside the SM's whole register file: a request beyond that pool is never granted and
// the warp waits for ever.  The static_asserts below keep every role split inside the pool.
#ifndef SQ_W4_CTRL
#define SQ_W4_CTRL 40
#endif
#ifndef SQ_W4_CVT
#define SQ_W4_CVT 72
#endif
constexpr int kCtrlRegs = 56, kEpiRegs = 224, kEpiRegsW4 = 200;
static_assert(4 * kCtrlRegs + 8 * kEpiRegs <= 12 * 168, "register split of the 384-thread kernels exceeds the launch pool");
static_assert(4 * SQ_W4_CTRL + 8 * kEpiRegsW4 + 4 * SQ_W4_CVT <= 16 * 128, "register split of the 512-thread kernels exceeds the launch pool");

struct GemmParams {
    long long M, N, K;
    int batch;
    int num_segs;
    int seg_bounds[SQ_MAX_SEGS + 1];
    int group_size;
    int w_seg_as_batch;
    int a_batched;
    int w_batched;   // 0: every problem of the batch uses the same weight matrix
    const float* sx;
    const float* sx_neg;
    long long sx_bs, sx_ss, sx_rs;
    const void* sw;
    int sw_is_bf16;
    long long sw_bs, sw_ss, sw_gs, sw_cs;
    const void* bias;
    int bias_dtype;
    long long bias_bs;
    void* y;
    int out_dtype;
    long long y_bs, y_rs;
    void* acc_dump;
    int units;
    int tiles_m, tiles_n;
    long long total_tiles;
    int y_tma;    // output goes through TMA stores (y base / strides are 16-byte aligned)
    int bn;       // tile width in use: 128, 192 or 256 (chosen on the host against wave quantisation)
    int n_peers;              // fused all-gather: further [M, *] outputs on peer GPUs
    int peer_tma;             // they are written by TMA stores (OutMaps::peer) rather than by the threads
    void* peer_y[SQ_MAX_PEERS];
    long long peer_rs, peer_co;
    int peer_wide;            // fused all-gather with [16 rows x 128 bytes] boxes (see store_output) instead of [32 rows x 16 columns]
    int short_units;  // every accumulation unit is one or two K stages long (weight-scale groups of 128 / 256): pairs use 128-byte K stages
    int all_magic;  // integer kind, every accumulation unit has K <= 224 (|sum| < 2^22), no dump / peer stores: accumulators start from kMagicBits
    int dual_db;  // DualScale with bn <= 128: four TMEM buffers (pos/neg x 2), epilogue overlaps the next tile
    long long wait_cycles;  // SM cycles after which a bounded wait gives up (default 4e9, about 2 s)
};

// Output descriptors: this rank's matrix and, for the fused all-gather, the same column range of every
// peer GPU's buffer (plain, non-multicast TMA stores; unused entries are copies of `y`).
struct OutMaps {
    CUtensorMap y;
    CUtensorMap peer[SQ_MAX_PEERS];
};

// One explicit specialisation per (KIND, DUAL), each in its own translation unit so the twelve-odd
// kernel instantiations compile in parallel.
template <int KIND, bool DUAL>
int launch_gemm(bool two_cta, const CUtensorMap& ma, const CUtensorMap& man, const CUtensorMap& mw, const OutMaps& my,
                const GemmParams& p, cudaStream_t st);
// Reads and clears the status word kernels of that translation unit write when a bounded wait gives up.
template <int KIND, bool DUAL>
long long tu_read_status();
// Launches the wait probe of that translation unit (see wait_probe_kernel in seg_gemm_kernels.cuh).
template <int KIND, bool DUAL>
int tu_wait_probe(long long limit_cycles, int* out_dev, cudaStream_t st);
int forced_ksub();      // seg_gemm.cu: process-wide schedule overrides (0 = automatic)
#ifdef SQ_TRACE
template <int KIND, bool DUAL>
int tu_trace_read(long long* out, int n);
#endif

}  // namespace sq
