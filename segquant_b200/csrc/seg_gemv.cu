// Skinny-M form of the segmented quantised GEMM (M <= 4 rows, e.g. the adaLN projections of a DiT
// block, whose input is one conditioning vector per sample): HBM-bound weight streaming on the CUDA
// cores instead of 128-row tensor-core tiles that would be 94 % padding and run on N / 128 SMs only.
//
// Same arithmetic as the tensor-core path (seg_gemm_kernels.cuh): per accumulation unit (K-segment x
// weight-scale group) the int8 products are summed exactly in int32 (dp4a), converted to fp32,
// multiplied by 1 / (s_x * s_w[n]) and added to the running fp32 sum; bias and cast at the end.  e4m3
// products are exact in fp32 and summed in fp32.
//
// One warp owns four output columns: every lane streams 16 bytes of each of the four weight rows per
// step (512 contiguous bytes per row and warp, twelve independent 128-bit loads in flight), the few
// activation rows sit in shared memory (both DualScale planes), partial sums are reduced with warp
// shuffles once per unit.  Algorithmic bytes: N * K (weights) + M * K * (1 | 2) + M * N * b_out.
#include <cuda_fp8.h>

#include <cstdlib>
#include <type_traits>

#include "seg_gemm_params.cuh"

namespace sq {

bool gemv_disabled();   // seg_gemm.cu: process-wide schedule overrides

constexpr int kGemvCols = 4;        // output columns per warp
constexpr int kGemvWarps = 8;       // warps per CTA
constexpr int kGemvSteps = 3;       // 512-byte steps of a weight row whose loads are in flight together
constexpr int kGemvMaxRows = 4;      // measured: at 8 rows the tensor-core path is faster again
constexpr long long kGemvMaxSmem = 96 * 1024;   // activation rows staged per CTA (both sides)

__device__ __forceinline__ float gemv_load_sw(const GemmParams& p, long long idx) {
    if (p.sw_is_bf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.sw)[idx]);
    return static_cast<const float*>(p.sw)[idx];
}

__device__ __forceinline__ void e4m3x4_to_float(uint32_t w, float (&f)[4]) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xFFFFu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

template <int KIND, bool DUAL, int MR>
__global__ void __launch_bounds__(kGemvWarps * 32) seg_gemv_kernel(const __grid_constant__ GemmParams p, const uint8_t* __restrict__ xq,
                                                                   const uint8_t* __restrict__ xq_neg, long long xq_rs,
                                                                   const uint8_t* __restrict__ wq, long long wq_rs) {
    extern __shared__ __align__(16) uint8_t xs[];          // [sides][MR][K] activation bytes (rows >= M are zero)
    constexpr int SIDES = DUAL ? 2 : 1;
    constexpr bool kF8 = KIND == SQ_GEMM_W8A8_F8;
    using Acc = typename std::conditional<kF8, float, int>::type;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = static_cast<int>(p.K);
    const int M = static_cast<int>(p.M);

    // stage the activation rows: 16-byte chunks, every thread of the CTA
    const int chunks_per_row = K >> 4;
    for (int c = threadIdx.x; c < SIDES * MR * chunks_per_row; c += blockDim.x) {
        const int side = c / (MR * chunks_per_row);
        const int rem = c - side * MR * chunks_per_row;
        const int m = rem / chunks_per_row, j = rem - m * chunks_per_row;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (m < M) v = *reinterpret_cast<const uint4*>((side ? xq_neg : xq) + m * xq_rs + j * 16);
        *reinterpret_cast<uint4*>(xs + (static_cast<size_t>(side * MR + m) * K) + j * 16) = v;
    }
    __syncthreads();

    const bool per_token = p.sx_rs != 0;
    const long long col_groups = (p.N + kGemvCols - 1) / kGemvCols;
    for (long long cg = static_cast<long long>(blockIdx.x) * kGemvWarps + warp; cg < col_groups;
         cg += static_cast<long long>(gridDim.x) * kGemvWarps) {
        const long long n0 = cg * kGemvCols;
        // clamp the row index of columns past N to a valid one: their results are simply not stored
        const uint8_t* wrow[kGemvCols];
#pragma unroll
        for (int c = 0; c < kGemvCols; ++c) wrow[c] = wq + (n0 + c < p.N ? n0 + c : p.N - 1) * wq_rs;

        float y[kGemvCols][MR];
#pragma unroll
        for (int c = 0; c < kGemvCols; ++c)
#pragma unroll
            for (int m = 0; m < MR; ++m) y[c][m] = 0.0f;

        int s = 0, k0 = 0, g = 0;
        for (int u = 0; u < p.units; ++u) {
            const int seg_end = p.seg_bounds[s + 1];
            const int grp_end = p.group_size > 0 ? (g + 1) * p.group_size : seg_end;
            const int k1 = grp_end < seg_end ? grp_end : seg_end;

            Acc acc[SIDES][kGemvCols][MR];
#pragma unroll
            for (int sd = 0; sd < SIDES; ++sd)
#pragma unroll
                for (int c = 0; c < kGemvCols; ++c)
#pragma unroll
                    for (int m = 0; m < MR; ++m) acc[sd][c][m] = 0;

            // kGemvSteps x 4 weight loads are issued before the first of them is consumed (12 independent 128-bit
            // loads per lane: a K = 1536 row is a single round trip to memory)
            for (int kb = k0 + (lane << 4); kb < k1; kb += 512 * kGemvSteps) {
                uint4 wv[kGemvSteps][kGemvCols];
#pragma unroll
                for (int t = 0; t < kGemvSteps; ++t)
#pragma unroll
                    for (int c = 0; c < kGemvCols; ++c)
                        if (kb + 512 * t < k1) wv[t][c] = __ldg(reinterpret_cast<const uint4*>(wrow[c] + kb + 512 * t));
#pragma unroll
                for (int t = 0; t < kGemvSteps; ++t) {
                    const int k = kb + 512 * t;
                    if (k < k1) {
#pragma unroll
                        for (int sd = 0; sd < SIDES; ++sd) {
#pragma unroll
                            for (int m = 0; m < MR; ++m) {
                                const uint4 xv = *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(sd * MR + m) * K + k);
                                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                                for (int c = 0; c < kGemvCols; ++c) {
                                    const uint32_t ww[4] = {wv[t][c].x, wv[t][c].y, wv[t][c].z, wv[t][c].w};
                                    if constexpr (kF8) {
#pragma unroll
                                        for (int q = 0; q < 4; ++q) {
                                            float xf[4], wf[4];
                                            e4m3x4_to_float(xw[q], xf);
                                            e4m3x4_to_float(ww[q], wf);
#pragma unroll
                                            for (int e = 0; e < 4; ++e) acc[sd][c][m] = fmaf(xf[e], wf[e], acc[sd][c][m]);
                                        }
                                    } else {
#pragma unroll
                                        for (int q = 0; q < 4; ++q)
                                            acc[sd][c][m] = __dp4a(static_cast<int>(xw[q]), static_cast<int>(ww[q]), acc[sd][c][m]);
                                    }
                                }
                            }
                        }
                    }
                }
            }
            // reduce over the warp, scale, add to the running fp32 sums (every lane ends with the same values)
#pragma unroll
            for (int c = 0; c < kGemvCols; ++c) {
                const long long n = n0 + c < p.N ? n0 + c : p.N - 1;
                const float swv = gemv_load_sw(p, s * p.sw_ss + g * p.sw_gs + n * p.sw_cs);
#pragma unroll
                for (int sd = 0; sd < SIDES; ++sd) {
                    const float* sxp = sd ? p.sx_neg : p.sx;
                    const float sxv = per_token ? 1.0f : sxp[s * p.sx_ss];
                    const float r = 1.0f / (sxv * swv);
#pragma unroll
                    for (int m = 0; m < MR; ++m) {
                        Acc a = acc[sd][c][m];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                        float rr = r;
                        if (per_token) rr *= 1.0f / sxp[s * p.sx_ss + (m < M ? m : 0) * p.sx_rs];
                        y[c][m] = fmaf(static_cast<float>(a), rr, y[c][m]);
                    }
                }
            }
            if (k1 == seg_end) ++s;
            if (p.group_size > 0 && k1 == grp_end) ++g;
            k0 = k1;
        }
        // bias, cast, store: lane c * MR + m writes y[c][m]
#pragma unroll
        for (int c = 0; c < kGemvCols; ++c) {
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                if (lane == c * MR + m && n0 + c < p.N && m < M) {
                    float v = y[c][m];
                    if (p.bias != nullptr) {
                        const long long bi = n0 + c;
                        if (p.bias_dtype == SQ_F32) v += static_cast<const float*>(p.bias)[bi];
                        else if (p.bias_dtype == SQ_F16) v += __half2float(static_cast<const __half*>(p.bias)[bi]);
                        else v += __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[bi]);
                    }
                    const long long oi = m * p.y_rs + n0 + c;
                    if (p.out_dtype == SQ_F32) static_cast<float*>(p.y)[oi] = v;
                    else if (p.out_dtype == SQ_F16) static_cast<__half*>(p.y)[oi] = __float2half_rn(v);
                    else static_cast<__nv_bfloat16*>(p.y)[oi] = __float2bfloat16_rn(v);
                }
            }
        }
    }
}

// True when the skinny path serves this problem (the caller has validated the arguments).
bool gemv_applies(const sq_gemm_args* a, bool dual) {
    if (a->kind == SQ_GEMM_W4A8 || a->batch != 1 || a->M > kGemvMaxRows || a->acc_dump_dev != nullptr || a->num_peer_outputs != 0 ||
        a->w_seg_as_batch)
        return false;
    if (gemv_disabled()) return false;   // SEGQUANT_B200_NO_GEMV=1 or sq_set_gemm_schedule(): tensor-core path only
    const int mr = a->M <= 2 ? 2 : 4;
    if (static_cast<long long>(mr) * a->K * (dual ? 2 : 1) > kGemvMaxSmem) return false;
    return (reinterpret_cast<uintptr_t>(a->xq_dev) % 16 == 0) && (a->xq_row_stride % 16 == 0) &&
           (reinterpret_cast<uintptr_t>(a->wq_dev) % 16 == 0) && (a->wq_row_stride % 16 == 0) &&
           (!dual || reinterpret_cast<uintptr_t>(a->xq_neg_dev) % 16 == 0);
}

template <int KIND, bool DUAL, int MR>
static int launch_gemv_mr(const GemmParams& p, const sq_gemm_args* a, cudaStream_t st) {
    const size_t smem = static_cast<size_t>(MR) * a->K * (DUAL ? 2 : 1);
    static bool attr_set[64] = {};
    int dev = 0;
    SQ_CUDA_OK(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && (dev >= 64 || !attr_set[dev])) {
        SQ_CUDA_OK(cudaFuncSetAttribute(seg_gemv_kernel<KIND, DUAL, MR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kGemvMaxSmem)));
        if (dev < 64) attr_set[dev] = true;
    }
    const long long col_groups = (a->N + kGemvCols - 1) / kGemvCols;
    long long ctas = (col_groups + kGemvWarps - 1) / kGemvWarps;
    if (ctas > kNumSMs * 8) ctas = kNumSMs * 8;
    seg_gemv_kernel<KIND, DUAL, MR><<<static_cast<int>(ctas), kGemvWarps * 32, smem, st>>>(
        p, static_cast<const uint8_t*>(a->xq_dev), static_cast<const uint8_t*>(a->xq_neg_dev), a->xq_row_stride,
        static_cast<const uint8_t*>(a->wq_dev), a->wq_row_stride);
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

template <int KIND, bool DUAL>
static int launch_gemv_kd(const GemmParams& p, const sq_gemm_args* a, cudaStream_t st) {
    if (a->M <= 2) return launch_gemv_mr<KIND, DUAL, 2>(p, a, st);
    return launch_gemv_mr<KIND, DUAL, 4>(p, a, st);
}

int launch_gemv(const GemmParams& p, const sq_gemm_args* a, bool dual, cudaStream_t st) {
    if (a->kind == SQ_GEMM_W8A8_I8)
        return dual ? launch_gemv_kd<SQ_GEMM_W8A8_I8, true>(p, a, st) : launch_gemv_kd<SQ_GEMM_W8A8_I8, false>(p, a, st);
    return dual ? launch_gemv_kd<SQ_GEMM_W8A8_F8, true>(p, a, st) : launch_gemv_kd<SQ_GEMM_W8A8_F8, false>(p, a, st);
}

}  // namespace sq
