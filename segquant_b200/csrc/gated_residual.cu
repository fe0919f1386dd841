// Gated residual add of a DiT block: out[b, t, :] = x[b, t, :] + gate[b, :] * y[b, t, :]   (HBM-bound).
//
// The residual stream update after the attention output projection and after the MLP: y is the output of a
// quantised linear, gate a chunk of the adaLN modulation.  torch.addcmul with a gate broadcast over the tokens takes
// its strided-iterator path (scalar loads, ~2.5 TB/s); here one warp walks one row with 128-bit loads and stores and
// the gate row comes from L1/L2.  Arithmetic follows torch exactly (fp32 product rounded, then fp32 sum rounded, then
// one rounding to the 16-bit type), so the result is bit-identical to torch.addcmul.  No counterpart in the reference.
#include "common.cuh"

namespace sq {

struct GatedParams {
    const void* x;
    const void* gate;
    const void* y;
    void* out;
    long long batch, M, K;
    long long x_bs, x_rs, y_bs, y_rs, o_bs, o_rs, g_bs;   // elements
};

template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 unpack_pair<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float2 v);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float2 v) {
    const __nv_bfloat162 h = __float22bfloat162_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float2 v) {
    const __half2 h = __float22half2_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <typename T>
__device__ __forceinline__ uint32_t gated_pair(uint32_t x, uint32_t g, uint32_t y) {
    // separate multiply and add (no contraction into an fma): the two fp32 roundings of torch's a + b * c
    return pack_pair<T>(__fadd2_rn(unpack_pair<T>(x), __fmul2_rn(unpack_pair<T>(g), unpack_pair<T>(y))));
}

template <typename T>
__global__ void __launch_bounds__(256) gated_residual_kernel(const __grid_constant__ GatedParams p) {
    constexpr int U = 4;                           // 128-bit words in flight per lane and operand
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const long long rows = p.batch * p.M;
    const int words = static_cast<int>(p.K / 8);
    const T* x = static_cast<const T*>(p.x);
    const T* y = static_cast<const T*>(p.y);
    const T* gate = static_cast<const T*>(p.gate);
    T* out = static_cast<T*>(p.out);
    for (long long row = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5); row < rows;
         row += static_cast<long long>(gridDim.x) * warps_per_cta) {
        const long long b = row / p.M, r = row - b * p.M;
        const uint4* xr = reinterpret_cast<const uint4*>(x + b * p.x_bs + r * p.x_rs);
        const uint4* yr = reinterpret_cast<const uint4*>(y + b * p.y_bs + r * p.y_rs);
        const uint4* gr = reinterpret_cast<const uint4*>(gate + b * p.g_bs);
        uint4* orow = reinterpret_cast<uint4*>(out + b * p.o_bs + r * p.o_rs);
        for (int u0 = lane; u0 < words; u0 += 32 * U) {
            uint4 xv[U], yv[U];
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const int u = u0 + 32 * j;
                if (u < words) {
                    xv[j] = xr[u];                 // plain loads: out may alias x
                    yv[j] = __ldg(yr + u);
                }
            }
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const int u = u0 + 32 * j;
                if (u < words) {
                    const uint4 g = __ldg(gr + u);
                    orow[u] = make_uint4(gated_pair<T>(xv[j].x, g.x, yv[j].x), gated_pair<T>(xv[j].y, g.y, yv[j].y),
                                         gated_pair<T>(xv[j].z, g.z, yv[j].z), gated_pair<T>(xv[j].w, g.w, yv[j].w));
                }
            }
        }
    }
}

int gated_residual(const sq_gated_residual_args* a, cudaStream_t st) {
    SQ_REQUIRE(a != nullptr, SQ_ERR_INVALID_ARG, "sq_gated_residual: args is NULL");
    SQ_REQUIRE(a->batch >= 0 && a->M >= 0 && a->K >= 0, SQ_ERR_INVALID_ARG, "sq_gated_residual: negative size");
    if (a->batch * a->M * a->K == 0) return SQ_OK;
    SQ_REQUIRE(a->x_dev && a->gate_dev && a->y_dev && a->out_dev, SQ_ERR_INVALID_ARG, "sq_gated_residual: NULL pointer");
    SQ_REQUIRE(a->dtype == SQ_F16 || a->dtype == SQ_BF16, SQ_ERR_UNSUPPORTED, "sq_gated_residual: 16-bit tensors only (dtype %d)", a->dtype);
    SQ_REQUIRE(a->K % 8 == 0, SQ_ERR_ALIGNMENT, "sq_gated_residual: K (%lld) must be divisible by 8", static_cast<long long>(a->K));
    const long long strides[] = {a->x_batch_stride, a->x_row_stride, a->y_batch_stride, a->y_row_stride,
                                 a->out_batch_stride, a->out_row_stride, a->gate_batch_stride};
    for (long long s : strides) SQ_REQUIRE(s % 8 == 0, SQ_ERR_ALIGNMENT, "sq_gated_residual: strides must be multiples of 8 elements");
    const void* ptrs[] = {a->x_dev, a->gate_dev, a->y_dev, a->out_dev};
    for (const void* q : ptrs)
        SQ_REQUIRE(reinterpret_cast<uintptr_t>(q) % 16 == 0, SQ_ERR_ALIGNMENT, "sq_gated_residual: pointers must be 16-byte aligned");
    GatedParams p;
    p.x = a->x_dev; p.gate = a->gate_dev; p.y = a->y_dev; p.out = a->out_dev;
    p.batch = a->batch; p.M = a->M; p.K = a->K;
    p.x_bs = a->x_batch_stride; p.x_rs = a->x_row_stride; p.y_bs = a->y_batch_stride; p.y_rs = a->y_row_stride;
    p.o_bs = a->out_batch_stride; p.o_rs = a->out_row_stride; p.g_bs = a->gate_batch_stride;
    const long long rows = a->batch * a->M;
    long long ctas = (rows + 7) / 8;
    if (ctas > static_cast<long long>(kNumSMs) * 8) ctas = static_cast<long long>(kNumSMs) * 8;
    if (a->dtype == SQ_F16) gated_residual_kernel<__half><<<static_cast<int>(ctas), 256, 0, st>>>(p);
    else gated_residual_kernel<__nv_bfloat16><<<static_cast<int>(ctas), 256, 0, st>>>(p);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

}  // namespace sq
