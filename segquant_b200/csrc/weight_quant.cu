// Weight quantise / int4 pack / int4 unpack kernels (HBM-bound, run once per layer).
//
// Replaces the weight overloads of real_quantize_scaled_kernel
// (segquant/src/real_quant/quantizer.cuh:55-68, :103-118) launched by
// real_quantized_quantize_weights<T> (segquant/src/real_quant/real_gemm.cu:538-638).
// Group-wise scales (scale_mode 2) have no counterpart there.
#include "common.cuh"

namespace sq {

struct WeightQuantParams {
    const void* w;
    const float* scale;
    void* out;
    long long N, K;
    float scale_scalar;
    int scale_mode;  // 0 scalar, 1 per row, 2 per (row, K-group)
    int group_size;
};

template <int OUT>
__device__ __forceinline__ void store16(void* out, long long elem_idx, const float (&v)[16]) {
    if constexpr (OUT == SQ_Q_INT4) {
        uint32_t w[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i >> 3] |= quant_int4(v[i]) << ((i & 7) * 4);  // element 2j -> low nibble
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(out) + (elem_idx >> 1)) = make_uint2(w[0], w[1]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if constexpr (OUT == SQ_Q_INT8)
                w[i] = quant_int8(v[4 * i]) | (quant_int8(v[4 * i + 1]) << 8) | (quant_int8(v[4 * i + 2]) << 16) |
                       (quant_int8(v[4 * i + 3]) << 24);
            else
                w[i] = quant_e4m3x2(v[4 * i], v[4 * i + 1]) | (quant_e4m3x2(v[4 * i + 2], v[4 * i + 3]) << 16);
        }
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(out) + elem_idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// K % 16 == 0: one warp per row, 16-element chunks per lane.
template <typename T, int OUT>
__global__ void __launch_bounds__(256) weight_quant_kernel(const __grid_constant__ WeightQuantParams p) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int kch = static_cast<int>(p.K >> 4);
    const T* __restrict__ w = static_cast<const T*>(p.w);
    const long long groups_per_row = p.scale_mode == 2 ? p.K / p.group_size : 0;
    for (long long row = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5); row < p.N;
         row += static_cast<long long>(gridDim.x) * warps_per_cta) {
        const T* wr = w + row * p.K;
        float sc = p.scale_scalar;
        if (p.scale_mode == 1) sc = __ldg(p.scale + row);
#pragma unroll 2
        for (int c = lane; c < kch; c += 32) {
            const int k = c << 4;
            if (p.scale_mode == 2) sc = __ldg(p.scale + row * groups_per_row + k / p.group_size);
            float v[16];
            load16<T>(wr + k, v);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] *= sc;
            store16<OUT>(p.out, row * p.K + k, v);
        }
    }
}

// Any K (the reference kernel accepts any numel): two flattened elements per thread.
template <typename T, int OUT>
__global__ void __launch_bounds__(256) weight_quant_scalar_kernel(const __grid_constant__ WeightQuantParams p) {
    const long long numel = p.N * p.K;
    const long long pairs = (numel + 1) / 2;
    const T* __restrict__ w = static_cast<const T*>(p.w);
    const long long groups_per_row = p.scale_mode == 2 ? p.K / p.group_size : 0;
    for (long long pr = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; pr < pairs;
         pr += static_cast<long long>(gridDim.x) * blockDim.x) {
        uint32_t q[2] = {0, 0};
        for (int j = 0; j < 2; ++j) {
            const long long idx = 2 * pr + j;
            if (idx >= numel) break;
            const long long row = idx / p.K;
            const long long k = idx - row * p.K;
            float sc = p.scale_scalar;
            if (p.scale_mode == 1) sc = p.scale[row];
            else if (p.scale_mode == 2) sc = p.scale[row * groups_per_row + k / p.group_size];
            const float v = to_float<T>(w[idx]) * sc;
            q[j] = OUT == SQ_Q_INT8 ? quant_int8(v) : OUT == SQ_Q_E4M3 ? quant_e4m3(v) : quant_int4(v);
            if constexpr (OUT != SQ_Q_INT4) static_cast<uint8_t*>(p.out)[idx] = static_cast<uint8_t>(q[j]);
        }
        if constexpr (OUT == SQ_Q_INT4) static_cast<uint8_t*>(p.out)[pr] = static_cast<uint8_t>(q[0] | (q[1] << 4));
    }
}

// int4 -> int8: every lane takes 8 packed bytes and writes 16 int8, so a warp reads 256 and writes 512
// contiguous bytes per instruction; four independent loads are in flight per lane.
__device__ __forceinline__ uint4 unpack8(uint2 pk) {
    const uint32_t src[2] = {pk.x, pk.y};
    uint32_t dst[4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        // low nibbles -> even elements, high nibbles -> odd elements; sign-extend 4 -> 8 bits
        const uint32_t lo = src[j] & 0x0F0F0F0Fu;
        const uint32_t hi = (src[j] >> 4) & 0x0F0F0F0Fu;
        const uint32_t lo_s = lo | ((lo & 0x08080808u) * 0x1Eu);
        const uint32_t hi_s = hi | ((hi & 0x08080808u) * 0x1Eu);
        dst[2 * j] = __byte_perm(lo_s, hi_s, 0x5140);
        dst[2 * j + 1] = __byte_perm(lo_s, hi_s, 0x7362);
    }
    return make_uint4(dst[0], dst[1], dst[2], dst[3]);
}

__global__ void __launch_bounds__(256) unpack_int4_kernel(const uint2* __restrict__ packed, uint4* __restrict__ out,
                                                          long long nvec) {
    constexpr int U = 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride * U) {
        uint2 pk[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i + u * stride < nvec) pk[u] = __ldg(packed + i + u * stride);
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i + u * stride < nvec) out[i + u * stride] = unpack8(pk[u]);
    }
}

__global__ void unpack_int4_tail_kernel(const uint8_t* __restrict__ packed, int8_t* __restrict__ out, long long first_byte,
                                        long long nbytes) {
    const long long i = first_byte + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= nbytes) return;
    const uint8_t b = packed[i];
    out[2 * i] = static_cast<int8_t>(static_cast<int8_t>(b << 4) >> 4);
    out[2 * i + 1] = static_cast<int8_t>(static_cast<int8_t>(b & 0xF0) >> 4);
}

template <typename T>
static void launch_weight(const WeightQuantParams& p, int out_kind, cudaStream_t st) {
    const bool vec = (p.K % 16 == 0) && (reinterpret_cast<uintptr_t>(p.w) % 16 == 0) &&
                     (reinterpret_cast<uintptr_t>(p.out) % 16 == 0) && (p.scale_mode != 2 || p.group_size % 16 == 0);
    if (vec) {
        long long ctas = (p.N + 7) / 8;
        if (ctas > kNumSMs * 8) ctas = kNumSMs * 8;
        const int grid = static_cast<int>(ctas < 1 ? 1 : ctas);
        if (out_kind == SQ_Q_INT8) weight_quant_kernel<T, SQ_Q_INT8><<<grid, 256, 0, st>>>(p);
        else if (out_kind == SQ_Q_E4M3) weight_quant_kernel<T, SQ_Q_E4M3><<<grid, 256, 0, st>>>(p);
        else weight_quant_kernel<T, SQ_Q_INT4><<<grid, 256, 0, st>>>(p);
    } else {
        long long ctas = ((p.N * p.K + 1) / 2 + 255) / 256;
        if (ctas > kNumSMs * 8) ctas = kNumSMs * 8;
        const int grid = static_cast<int>(ctas < 1 ? 1 : ctas);
        if (out_kind == SQ_Q_INT8) weight_quant_scalar_kernel<T, SQ_Q_INT8><<<grid, 256, 0, st>>>(p);
        else if (out_kind == SQ_Q_E4M3) weight_quant_scalar_kernel<T, SQ_Q_E4M3><<<grid, 256, 0, st>>>(p);
        else weight_quant_scalar_kernel<T, SQ_Q_INT4><<<grid, 256, 0, st>>>(p);
    }
}

int quantize_weight(const void* w, int w_dtype, long long N, long long K, int scale_mode, float scale_scalar,
                    const float* scale, int group_size, int out_kind, void* out, cudaStream_t st) {
    SQ_REQUIRE(w && out, SQ_ERR_INVALID_ARG, "sq_quantize_weight: w_dev / out_dev is NULL");
    SQ_REQUIRE(N >= 0 && K >= 0, SQ_ERR_INVALID_ARG, "sq_quantize_weight: negative size");
    SQ_REQUIRE(w_dtype == SQ_F32 || w_dtype == SQ_F16 || w_dtype == SQ_BF16, SQ_ERR_INVALID_ARG,
               "sq_quantize_weight: unknown w_dtype %d", w_dtype);
    SQ_REQUIRE(out_kind == SQ_Q_INT8 || out_kind == SQ_Q_E4M3 || out_kind == SQ_Q_INT4, SQ_ERR_INVALID_ARG,
               "sq_quantize_weight: unknown out_kind %d", out_kind);
    SQ_REQUIRE(scale_mode >= 0 && scale_mode <= 2, SQ_ERR_INVALID_ARG, "sq_quantize_weight: unknown scale_mode %d",
               scale_mode);
    SQ_REQUIRE(scale_mode == 0 || scale, SQ_ERR_INVALID_ARG, "sq_quantize_weight: scale_dev is NULL");
    if (scale_mode == 2)
        SQ_REQUIRE(group_size > 0 && K % group_size == 0, SQ_ERR_INVALID_ARG,
                   "sq_quantize_weight: group_size %d must divide K %lld", group_size, K);
    if (out_kind == SQ_Q_INT4)
        SQ_REQUIRE((N * K) % 2 == 0, SQ_ERR_ALIGNMENT,
                   "sq_quantize_weight: int4 needs an even number of elements (seg_utils.h:68-71)");
    if (N * K == 0) return SQ_OK;
    WeightQuantParams p{w, scale, out, N, K, scale_scalar, scale_mode, group_size};
    if (w_dtype == SQ_F32) launch_weight<float>(p, out_kind, st);
    else if (w_dtype == SQ_F16) launch_weight<__half>(p, out_kind, st);
    else launch_weight<__nv_bfloat16>(p, out_kind, st);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

int unpack_int4(const void* packed, void* out, long long numel, cudaStream_t st) {
    SQ_REQUIRE(packed && out, SQ_ERR_INVALID_ARG, "sq_unpack_int4: NULL pointer");
    SQ_REQUIRE(numel >= 0 && numel % 2 == 0, SQ_ERR_ALIGNMENT, "sq_unpack_int4: numel must be even and >= 0");
    if (numel == 0) return SQ_OK;
    const long long nbytes = numel / 2;
    long long nvec = 0;   // 8-byte input vectors (16 output bytes each)
    if (reinterpret_cast<uintptr_t>(packed) % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) nvec = nbytes / 8;
    if (nvec > 0) {
        long long ctas = (nvec + 4 * 256 - 1) / (4 * 256);
        if (ctas > kNumSMs * 8) ctas = kNumSMs * 8;
        unpack_int4_kernel<<<static_cast<int>(ctas), 256, 0, st>>>(static_cast<const uint2*>(packed),
                                                                  static_cast<uint4*>(out), nvec);
    }
    const long long tail = nbytes - nvec * 8;
    if (tail > 0)
        unpack_int4_tail_kernel<<<static_cast<int>((tail + 255) / 256), 256, 0, st>>>(
            static_cast<const uint8_t*>(packed), static_cast<int8_t*>(out), nvec * 8, nbytes);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

}  // namespace sq
