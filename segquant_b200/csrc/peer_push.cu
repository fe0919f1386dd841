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
