// Column-block push to peer GPUs (the exchange step of a column-sharded layer, NVLink-bound).
//
// After a rank has computed its [rows, width] column block of the [rows, N] result -- in place, inside its own copy
// of the full matrix -- this kernel copies the block to the same position of every peer GPU's matrix (peer memory
// mapped into this process: CUDA IPC / symmetric memory).  It replaces an all-gather into a (ranks, rows, N/ranks)
// buffer followed by a permuting copy into [rows, N]: the data lands in its final layout, each byte crosses NVLink once
// per peer, and nothing is read back from a peer.  Every thread loads 16 bytes of the local block once (an L2 hit
// right after the GEMM) and issues one plain 16-byte store per peer; consecutive threads cover consecutive 16-byte
// chunks of a row, so a warp writes whole 512-byte row segments.  No multicast, no loads from peer memory, no waits:
// the caller orders the ranks (a stream-ordered barrier) before anyone reads its matrix.
// The reference has no multi-GPU code; no counterpart there.
#include "common.cuh"

namespace sq {

struct PushParams {
    const uint8_t* src;
    uint8_t* dst[SQ_MAX_PEERS];
    int n_peers;
    long long rows;
    long long chunks_per_row;        // width / 16 bytes
    long long src_row_stride;        // bytes
    long long dst_row_stride;        // bytes
};

template <int UNROLL>
__global__ void __launch_bounds__(256) peer_push_kernel(const __grid_constant__ PushParams p) {
    const long long total = p.rows * p.chunks_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * UNROLL) {
        uint4 v[UNROLL];
        long long off[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const long long i = i0 + u * stride;
            if (i < total) {
                const long long r = i / p.chunks_per_row, c = i - r * p.chunks_per_row;
                v[u] = *reinterpret_cast<const uint4*>(p.src + r * p.src_row_stride + c * 16);
                off[u] = r * p.dst_row_stride + c * 16;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (i0 + u * stride < total) {
                for (int j = 0; j < p.n_peers; ++j) *reinterpret_cast<uint4*>(p.dst[j] + off[u]) = v[u];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Stream-ordered barrier between the ranks of a sharded layer, one rank per GPU, over flag words in peer-mapped memory.
// Every rank owns an array of `world` 32-bit words (zero at start).  Call number `epoch` (1, 2, ... : the same on every
// rank, the calls are collective) stores `epoch` into word [rank] of every peer's array - after a system-scope fence, so
// everything this GPU wrote before the launch (its GEMM's or push kernel's stores into the peers' matrices) is visible
// to whoever sees the flag - and waits until its own words [j] have reached `epoch` for every peer j.  Epochs only
// grow, so the words are never reset and a late reader cannot miss one.  One small kernel instead of an all-reduce.
// The wait is bounded (the limit of every other wait of this library): when it runs out the kernel records
// (peer << 8 | kWaitPeerBarrier) in this file's status word, which sq_device_status() / sq_check_device() report, and
// returns.  Ranks must run on different GPUs: kernels that wait for one another cannot share one.
constexpr int kWaitPeerBarrier = 10;
static __device__ unsigned long long g_wait_status = 0ull;

struct BarrierParams {
    uint32_t* flags[SQ_MAX_PEERS + 1];   // every rank's array, own included
    int rank, world;
    uint32_t epoch;
    long long limit;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const __grid_constant__ BarrierParams p) {
    const int j = threadIdx.x;
    if (j >= p.world || j == p.rank) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[j] + p.rank), "r"(p.epoch) : "memory");
    const uint32_t* mine = p.flags[p.rank] + j;
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int32_t>(v - p.epoch) >= 0) break;
        if (clock64() - t0 > p.limit) {
            atomicCAS(&g_wait_status, 0ull, (static_cast<unsigned long long>(j) << 8) | static_cast<unsigned>(kWaitPeerBarrier));
            break;
        }
        __nanosleep(64);
    }
}

long long wait_limit_cycles();   // seg_gemm.cu

int peer_barrier(int rank, int world, void* const* flags, unsigned epoch, cudaStream_t st) {
    SQ_REQUIRE(world >= 1 && world <= SQ_MAX_PEERS + 1 && rank >= 0 && rank < world, SQ_ERR_INVALID_ARG,
               "sq_peer_barrier: rank %d / world %d out of range (at most %d ranks)", rank, world, SQ_MAX_PEERS + 1);
    if (world == 1) return SQ_OK;
    SQ_REQUIRE(flags != nullptr, SQ_ERR_INVALID_ARG, "sq_peer_barrier: flags is NULL");
    BarrierParams p;
    for (int j = 0; j <= SQ_MAX_PEERS; ++j) {
        p.flags[j] = j < world ? static_cast<uint32_t*>(flags[j]) : nullptr;
        if (j < world)
            SQ_REQUIRE(flags[j] != nullptr && reinterpret_cast<uintptr_t>(flags[j]) % 4 == 0, SQ_ERR_INVALID_ARG,
                       "sq_peer_barrier: flags[%d] is NULL or not 4-byte aligned", j);
    }
    p.rank = rank;
    p.world = world;
    p.epoch = epoch;
    p.limit = wait_limit_cycles();
    peer_barrier_kernel<<<1, 32, 0, st>>>(p);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

// reads and clears this file's status word (see read_device_status in seg_gemm.cu)
long long push_read_status() {
    unsigned long long v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_status, sizeof(v)) != cudaSuccess) return SQ_ERR_CUDA;
    if (v != 0 && cudaMemcpyToSymbol(g_wait_status, &zero, sizeof(zero)) != cudaSuccess) return SQ_ERR_CUDA;
    return static_cast<long long>(v);
}

int push_columns(const void* src, long long rows, long long width_bytes, long long src_row_stride, int n_peers,
                 void* const* peer_dst, long long dst_row_stride, cudaStream_t st) {
    SQ_REQUIRE(rows >= 0 && width_bytes >= 0, SQ_ERR_INVALID_ARG, "sq_push_columns: negative size");
    SQ_REQUIRE(n_peers >= 0 && n_peers <= SQ_MAX_PEERS, SQ_ERR_INVALID_ARG, "sq_push_columns: n_peers %d outside [0, %d]", n_peers, SQ_MAX_PEERS);
    if (rows == 0 || width_bytes == 0 || n_peers == 0) return SQ_OK;
    SQ_REQUIRE(src != nullptr && peer_dst != nullptr, SQ_ERR_INVALID_ARG, "sq_push_columns: NULL pointer");
    SQ_REQUIRE(width_bytes % 16 == 0 && src_row_stride % 16 == 0 && dst_row_stride % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0,
               SQ_ERR_ALIGNMENT, "sq_push_columns: block width, row strides and pointers must be multiples of 16 bytes");
    SQ_REQUIRE(src_row_stride >= width_bytes && dst_row_stride >= width_bytes, SQ_ERR_INVALID_ARG,
               "sq_push_columns: row stride smaller than the block width");
    PushParams p;
    p.src = static_cast<const uint8_t*>(src);
    p.n_peers = n_peers;
    for (int j = 0; j < SQ_MAX_PEERS; ++j) {
        p.dst[j] = j < n_peers ? static_cast<uint8_t*>(peer_dst[j]) : nullptr;
        if (j < n_peers)
            SQ_REQUIRE(peer_dst[j] != nullptr && reinterpret_cast<uintptr_t>(peer_dst[j]) % 16 == 0, SQ_ERR_INVALID_ARG,
                       "sq_push_columns: peer_dst[%d] is NULL or not 16-byte aligned", j);
    }
    p.rows = rows;
    p.chunks_per_row = width_bytes / 16;
    p.src_row_stride = src_row_stride;
    p.dst_row_stride = dst_row_stride;
    const long long total = rows * p.chunks_per_row;
    long long ctas = (total + 256 * 4 - 1) / (256 * 4);
    const long long cap = static_cast<long long>(kNumSMs) * 4;
    if (ctas > cap) ctas = cap;
    peer_push_kernel<4><<<static_cast<int>(ctas), 256, 0, st>>>(p);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

}  // namespace sq
