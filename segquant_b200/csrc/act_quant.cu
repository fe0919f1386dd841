// Activation quantise kernels (HBM-bound).
//
// One pass over x: 128-bit loads, per-K-segment (or per-token) scale, int8 / e4m3 bytes out
// through 128-bit stores.  Replaces real_quantize_scaled_kernel / real_quantize_dual_scaled_kernel
// of segquant/src/real_quant/quantizer.cuh:159-206 (4 scalar elements per thread, a div/mod per
// element) and the `.contiguous()` segment copy in segquant/optimum/optimizer.py:105.
//
// Work split: one warp walks one row, one 128-bit load per lane and step, eight loads in flight per
// lane; the dynamic per-token kernel gives one warp to a (row, segment).
#include <type_traits>

#include "common.cuh"

namespace sq {

struct ActQuantParams {
    const void* x;
    const float* sx;
    const float* sx_neg;
    const float* smooth;
    uint8_t* xq;
    uint8_t* xq_neg;
    float* sx_out;      // dynamic only
    float* sx_neg_out;  // dynamic only
    long long batch, M, K;
    long long x_batch_stride, x_row_stride;
    long long sx_batch_stride, sx_seg_stride, sx_row_stride;
    long long xq_batch_stride, xq_row_stride;
    int num_segs;
    int uniform_seg;  // >0: every segment has this length
    int pre_act;      // SQ_ACT_*: activation applied to x before scaling (static kernel only)
    int seg_bounds[SQ_MAX_SEGS + 1];
};

__device__ __forceinline__ int find_segment(const ActQuantParams& p, int k) {
    if (p.uniform_seg > 0) return k / p.uniform_seg;
    int s = 0;
    while (s + 1 < p.num_segs && k >= p.seg_bounds[s + 1]) ++s;
    return s;
}

template <int OUT>
__device__ __forceinline__ uint4 pack16(const float (&v)[16]) {
    uint32_t w[4];
    if constexpr (OUT == SQ_Q_INT8) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = quant_int8(v[4 * i]) | (quant_int8(v[4 * i + 1]) << 8) | (quant_int8(v[4 * i + 2]) << 16) |
                   (quant_int8(v[4 * i + 3]) << 24);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            w[i] = quant_e4m3x2(v[4 * i], v[4 * i + 1]) | (quant_e4m3x2(v[4 * i + 2], v[4 * i + 3]) << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// DualScale (dynamic kernel): element >= 0 -> positive tensor, else the negative tensor
// (quantizer.cuh:178-206); the side an element does not belong to gets quantise(+0) = byte 0.
template <int OUT>
__device__ __forceinline__ void pack16_dual(const float (&x)[16], float sp, float sn, uint4& outp, uint4& outn) {
    float vp[16], vn[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const bool pos = x[i] >= 0.0f;
        vp[i] = pos ? x[i] * sp : 0.0f;
        vn[i] = pos ? 0.0f : x[i] * sn;
    }
    outp = pack16<OUT>(vp);
    outn = pack16<OUT>(vn);
}

// ---- static-scale kernel ---------------------------------------------------------------------
// Work unit = one 128-bit load = E elements (4 fp32 or 8 half/bf16).  One warp walks one row; lane l
// takes units l, l+32, ... so every load and store instruction of a warp is fully coalesced, and U
// independent loads per lane are issued before any of them is consumed.

// int8 bytes of four already scaled values: clamp, then round to nearest even by adding 1.5 * 2^23
// (the integer lands in the low mantissa bits; same result as rintf, without a float->int convert).
__device__ __forceinline__ uint32_t quant_int8x4(float a, float b, float c, float d) {
    constexpr float kMagic = 12582912.0f;
    const uint32_t ia = __float_as_uint(fminf(fmaxf(a, -128.0f), 127.0f) + kMagic);
    const uint32_t ib = __float_as_uint(fminf(fmaxf(b, -128.0f), 127.0f) + kMagic);
    const uint32_t ic = __float_as_uint(fminf(fmaxf(c, -128.0f), 127.0f) + kMagic);
    const uint32_t id = __float_as_uint(fminf(fmaxf(d, -128.0f), 127.0f) + kMagic);
    return __byte_perm(__byte_perm(ia, ib, 0x0040), __byte_perm(ic, id, 0x0040), 0x5410);
}

template <int OUT>
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d) {
    if constexpr (OUT == SQ_Q_INT8) return quant_int8x4(a, b, c, d);
    else return quant_e4m3x2(a, b) | (quant_e4m3x2(c, d) << 16);
}

template <typename T>
struct Unit;   // one 128-bit load, kept as raw words until it is consumed (4 registers per load in flight)
template <>
struct Unit<float> {
    static constexpr int E = 4;
    __device__ static __forceinline__ void unpack(const uint4& t, float (&v)[4]) {
        v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y); v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
    }
    __device__ static __forceinline__ uint4 pack(const float (&v)[4]) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
};
template <>
struct Unit<__half> {
    static constexpr int E = 8;
    __device__ static __forceinline__ void unpack(const uint4& t, float (&v)[8]) {
        const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __half22float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    }
    __device__ static __forceinline__ uint4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]); w[j] = *reinterpret_cast<const uint32_t*>(&h); }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <>
struct Unit<__nv_bfloat16> {
    static constexpr int E = 8;
    __device__ static __forceinline__ void unpack(const uint4& t, float (&v)[8]) {
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u); }
    }
    __device__ static __forceinline__ uint4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]); w[j] = *reinterpret_cast<const uint32_t*>(&h); }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// Activation functions fused in front of the quantiser (the layer after a GELU / SiLU is where the reference uses
// DualScale: segquant/pattern_detector.py:239-358).  Both are written as x * sigmoid(g(x)) = x / (1 + 2^(-log2(e) g(x))):
// tanh-GELU has g = 2 sqrt(2/pi) (x + 0.044715 x^3) since 0.5 (1 + tanh(u)) = sigmoid(2u), SiLU has g = x.  That form
// keeps the RELATIVE error small on the negative tail, where 0.5 x (1 + tanh(u)) cancels and where DualScale spends its
// second scale; ex2.approx / rcp.approx are good to 2^-22, far below the bf16 rounding the separate torch kernel
// applies.  Evaluated on pairs (f32x2) because the kernel is issue-bound once an activation is added.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <int PRE>
__device__ __forceinline__ void pre_activation2(float& a, float& b) {
    const float2 x = make_float2(a, b);
    float2 arg;                                    // -log2(e) * g(x)
    if constexpr (PRE == SQ_ACT_GELU_TANH) {
        constexpr float c0 = -2.0f * 1.4426950408889634f * 0.7978845608028654f;
        constexpr float c1 = c0 * 0.044715f;
        arg = __fmul2_rn(x, __ffma2_rn(__fmul2_rn(x, x), make_float2(c1, c1), make_float2(c0, c0)));
    } else {
        arg = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
    }
    const float2 den = __fadd2_rn(make_float2(ex2_approx(arg.x), ex2_approx(arg.y)), make_float2(1.0f, 1.0f));
    const float2 r = __fmul2_rn(x, make_float2(rcp_approx(den.x), rcp_approx(den.y)));
    a = r.x;
    b = r.y;
}

template <int OUT, bool DUAL, int E>
__device__ __forceinline__ void quant_store(const float (&x)[E], float sp, float sn, uint8_t* q, uint8_t* qn) {
    uint32_t wp[E / 4], wn[E / 4];
    if constexpr (!DUAL) {
#pragma unroll
        for (int i = 0; i < E / 4; ++i) wp[i] = quant4<OUT>(x[4 * i] * sp, x[4 * i + 1] * sp, x[4 * i + 2] * sp, x[4 * i + 3] * sp);
    } else {
        float vp[E], vn[E];
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const bool pos = x[i] >= 0.0f;
            vp[i] = pos ? x[i] * sp : 0.0f;
            vn[i] = pos ? 0.0f : x[i] * sn;
        }
#pragma unroll
        for (int i = 0; i < E / 4; ++i) {
            wp[i] = quant4<OUT>(vp[4 * i], vp[4 * i + 1], vp[4 * i + 2], vp[4 * i + 3]);
            wn[i] = quant4<OUT>(vn[4 * i], vn[4 * i + 1], vn[4 * i + 2], vn[4 * i + 3]);
        }
    }
    if constexpr (E == 8) {
        *reinterpret_cast<uint2*>(q) = make_uint2(wp[0], wp[1]);
        if constexpr (DUAL) *reinterpret_cast<uint2*>(qn) = make_uint2(wn[0], wn[1]);
    } else {
        *reinterpret_cast<uint32_t*>(q) = wp[0];
        if constexpr (DUAL) *reinterpret_cast<uint32_t*>(qn) = wn[0];
    }
}

constexpr int kPreSmooth = -1;   // PRE: 0 nothing, kPreSmooth = divide by the smoothing vector, SQ_ACT_* = that activation

template <typename T, int OUT, bool DUAL, int PRE>
__global__ void __launch_bounds__(256, 4) act_quant_kernel(const __grid_constant__ ActQuantParams p) {
    constexpr int E = Unit<T>::E;
    constexpr int U = 8;
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const long long rows = p.batch * p.M;
    const int units = static_cast<int>(p.K / E);
    const T* __restrict__ x = static_cast<const T*>(p.x);

    for (long long row = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5); row < rows;
         row += static_cast<long long>(gridDim.x) * warps_per_cta) {
        long long b = 0, r = row;
        if (p.batch > 1) { b = row / p.M; r = row - b * p.M; }
        const T* xr = x + b * p.x_batch_stride + r * p.x_row_stride;
        const float* sxr = p.sx + b * p.sx_batch_stride + r * p.sx_row_stride;
        const float* sxnr = DUAL ? p.sx_neg + b * p.sx_batch_stride + r * p.sx_row_stride : nullptr;
        uint8_t* qr = p.xq + b * p.xq_batch_stride + r * p.xq_row_stride;
        uint8_t* qnr = DUAL ? p.xq_neg + b * p.xq_batch_stride + r * p.xq_row_stride : nullptr;

        // segment cursor: this lane's k only grows, so the segment index only moves forward
        int s = 0;
        int next_bound = p.seg_bounds[1];
        float sc = __ldg(sxr);
        float scn = DUAL ? __ldg(sxnr) : 0.0f;

        for (int u0 = lane; u0 < units; u0 += 32 * U) {
            uint4 raw[U];
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const int u = u0 + 32 * j;
                if (u < units) raw[j] = __ldg(reinterpret_cast<const uint4*>(xr + u * E));
            }
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const int u = u0 + 32 * j;
                if (u >= units) break;
                const int k = u * E;
                float v[E];
                Unit<T>::unpack(raw[j], v);
                while (k >= next_bound) {
                    ++s;
                    next_bound = p.seg_bounds[s + 1];
                    sc = __ldg(sxr + s * p.sx_seg_stride);
                    if constexpr (DUAL) scn = __ldg(sxnr + s * p.sx_seg_stride);
                }
                if constexpr (PRE == kPreSmooth) {
#pragma unroll
                    for (int i = 0; i < E; ++i) v[i] = v[i] / __ldg(p.smooth + k + i);
                } else if constexpr (PRE != 0) {
#pragma unroll
                    for (int i = 0; i < E; i += 2) pre_activation2<PRE>(v[i], v[i + 1]);
                }
                quant_store<OUT, DUAL, E>(v, sc, scn, qr + k, DUAL ? qnr + k : nullptr);
            }
        }
    }
}

// Dynamic per-token scales: one warp per (row, segment).  Pass 1 reduces |x| (or the positive and
// negative extremes) with warp shuffles, pass 2 re-reads the row segment (at most 24 KB, an L1/L2
// hit) and quantises.  The reference computes `qmax / amax` on a tensor of x's dtype
// (segquant/quantizers/quantizer.py:209-217, :187-203), and torch evaluates scalar / tensor as
// tensor.reciprocal() * scalar: two roundings to that dtype, reproduced here.
template <typename T>
__device__ __forceinline__ void smooth16(float (&v)[16], const float* __restrict__ sm) {
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
        const float4 d = __ldg(reinterpret_cast<const float4*>(sm) + i4);
        v[4 * i4 + 0] = to_float<T>(from_float<T>(__fdiv_rn(v[4 * i4 + 0], d.x)));
        v[4 * i4 + 1] = to_float<T>(from_float<T>(__fdiv_rn(v[4 * i4 + 1], d.y)));
        v[4 * i4 + 2] = to_float<T>(from_float<T>(__fdiv_rn(v[4 * i4 + 2], d.z)));
        v[4 * i4 + 3] = to_float<T>(from_float<T>(__fdiv_rn(v[4 * i4 + 3], d.w)));
    }
}

template <typename T>
__device__ __forceinline__ float scale_like_torch(float qmax, float amax) {
    const float r = to_float<T>(from_float<T>(__frcp_rn(amax)));
    return to_float<T>(from_float<T>(r * qmax));
}

// SMOOTH: every element is first divided by its channel's smoothing factor and rounded to T, as the reference's
// `input_chunk.div_(s.to(dtype))` leaves it (segquant/optimum/optimizer.py:467-470) before the per-token calibration
// sees it; p.smooth holds the factors already rounded to T (as fp32).
template <typename T, int OUT, bool DUAL, bool SMOOTH>
__global__ void __launch_bounds__(256) act_quant_dynamic_kernel(const __grid_constant__ ActQuantParams p) {
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const long long rows = p.batch * p.M;
    const long long items = rows * p.num_segs;
    const T* __restrict__ x = static_cast<const T*>(p.x);
    constexpr float kEps = 1.0f / 16777216.0f;
    constexpr float kQmax = (OUT == SQ_Q_INT8) ? 127.0f : 448.0f;
    constexpr float kQminAbs = (OUT == SQ_Q_INT8) ? 128.0f : 448.0f;

    for (long long item = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5); item < items;
         item += static_cast<long long>(gridDim.x) * warps_per_cta) {
        const long long row = item / p.num_segs;
        const int s = static_cast<int>(item - row * p.num_segs);
        const long long b = row / p.M;
        const long long r = row - b * p.M;
        const int k0 = p.seg_bounds[s], k1 = p.seg_bounds[s + 1];
        const T* xr = x + b * p.x_batch_stride + r * p.x_row_stride;
        uint8_t* qr = p.xq + b * p.xq_batch_stride + r * p.xq_row_stride;
        uint8_t* qnr = DUAL ? p.xq_neg + b * p.xq_batch_stride + r * p.xq_row_stride : nullptr;

        float amax = 0.0f, nmax = 0.0f;
        if constexpr (sizeof(T) == 2 && !SMOOTH) {
            // 16-bit inputs: the extremes are taken on packed pairs (one abs + one max instruction per two elements;
            // max of values is exact in their own format), converted to fp32 once per row
            using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
            uint32_t zero_bits = 0u;
            T2 pmax = *reinterpret_cast<T2*>(&zero_bits), pneg = pmax;
#pragma unroll 4   // several independent 128-bit loads in flight per lane
            for (int k = k0 + (lane << 4); k < k1; k += 512) {
                const uint4 a = __ldg(reinterpret_cast<const uint4*>(xr + k));
                const uint4 c = __ldg(reinterpret_cast<const uint4*>(xr + k + 8));
                const uint32_t w[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const T2 v = *reinterpret_cast<const T2*>(&w[i]);
                    if constexpr (DUAL) {
                        pmax = __hmax2(pmax, v);             // max over x > 0 of x (0 if none)
                        pneg = __hmax2(pneg, __hneg2(v));    // max over x < 0 of |x|
                    } else {
                        pmax = __hmax2(pmax, __habs2(v));
                    }
                }
            }
            amax = fmaxf(to_float<T>(pmax.x), to_float<T>(pmax.y));
            if constexpr (DUAL) nmax = fmaxf(to_float<T>(pneg.x), to_float<T>(pneg.y));
        } else {
#pragma unroll 4
            for (int k = k0 + (lane << 4); k < k1; k += 512) {
                float v[16];
                load16<T>(xr + k, v);
                if constexpr (SMOOTH) smooth16<T>(v, p.smooth + k);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if constexpr (DUAL) {
                        amax = fmaxf(amax, v[i]);    // max over x > 0 of x (0 if none)
                        nmax = fmaxf(nmax, -v[i]);   // max over x < 0 of |x|
                    } else {
                        amax = fmaxf(amax, fabsf(v[i]));
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if constexpr (DUAL) nmax = fmaxf(nmax, __shfl_xor_sync(0xffffffffu, nmax, o));
        }
        const float sc = scale_like_torch<T>(kQmax, fmaxf(amax, kEps));
        float scn = 0.0f;
        if constexpr (DUAL) scn = scale_like_torch<T>(kQminAbs, fmaxf(nmax, kEps));
        if (lane == 0) {
            p.sx_out[(b * p.num_segs + s) * p.M + r] = sc;
            if constexpr (DUAL) p.sx_neg_out[(b * p.num_segs + s) * p.M + r] = scn;
        }
#pragma unroll 4
        for (int k = k0 + (lane << 4); k < k1; k += 512) {
            float v[16];
            load16<T>(xr + k, v);
            if constexpr (SMOOTH) smooth16<T>(v, p.smooth + k);
            if constexpr (!DUAL) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] *= sc;
                *reinterpret_cast<uint4*>(qr + k) = pack16<OUT>(v);
            } else {
                uint4 op, on;
                pack16_dual<OUT>(v, sc, scn, op, on);
                *reinterpret_cast<uint4*>(qr + k) = op;
                *reinterpret_cast<uint4*>(qnr + k) = on;
            }
        }
    }
}

static int validate(const sq_act_quant_args* a, bool dynamic) {
    SQ_REQUIRE(a != nullptr, SQ_ERR_INVALID_ARG, "sq_quantize_act: args is NULL");
    SQ_REQUIRE(a->batch >= 0 && a->M >= 0 && a->K >= 0, SQ_ERR_INVALID_ARG, "sq_quantize_act: negative size");
    if (a->batch * a->M * a->K == 0) return SQ_OK;  // nothing to do: pointers may be NULL
    SQ_REQUIRE(a->x_dev && a->xq_dev, SQ_ERR_INVALID_ARG, "sq_quantize_act: x_dev / xq_dev is NULL");
    SQ_REQUIRE(dynamic || a->sx_dev, SQ_ERR_INVALID_ARG, "sq_quantize_act: sx_dev is NULL");
    SQ_REQUIRE(a->batch >= 0 && a->M >= 0 && a->K >= 0, SQ_ERR_INVALID_ARG, "sq_quantize_act: negative size");
    SQ_REQUIRE(a->x_dtype == SQ_F32 || a->x_dtype == SQ_F16 || a->x_dtype == SQ_BF16, SQ_ERR_INVALID_ARG,
               "sq_quantize_act: unknown x_dtype %d", a->x_dtype);
    SQ_REQUIRE(a->out_kind == SQ_Q_INT8 || a->out_kind == SQ_Q_E4M3, SQ_ERR_UNSUPPORTED,
               "sq_quantize_act: activations quantise to int8 or e4m3 only (got kind %d)", a->out_kind);
    SQ_REQUIRE(a->num_segs >= 1 && a->num_segs <= SQ_MAX_SEGS, SQ_ERR_INVALID_ARG,
               "sq_quantize_act: num_segs %d outside [1, %d]", a->num_segs, SQ_MAX_SEGS);
    SQ_REQUIRE(a->pre_act == SQ_ACT_NONE || a->pre_act == SQ_ACT_GELU_TANH || a->pre_act == SQ_ACT_SILU, SQ_ERR_INVALID_ARG,
               "sq_quantize_act: unknown pre_act %d", a->pre_act);
    SQ_REQUIRE(a->pre_act == SQ_ACT_NONE || (!dynamic && a->smooth_dev == nullptr), SQ_ERR_UNSUPPORTED,
               "sq_quantize_act: pre_act needs static scales and no smoothing vector");
    SQ_REQUIRE(a->K % 16 == 0, SQ_ERR_ALIGNMENT, "sq_quantize_act: K (%lld) must be divisible by 16",
               static_cast<long long>(a->K));
    SQ_REQUIRE(a->K < (1ll << 30), SQ_ERR_TOO_LARGE, "sq_quantize_act: K too large");
    SQ_REQUIRE(a->seg_bounds[0] == 0 && a->seg_bounds[a->num_segs] == a->K, SQ_ERR_INVALID_ARG,
               "sq_quantize_act: seg_bounds must run from 0 to K");
    for (int s = 0; s < a->num_segs; ++s) {
        SQ_REQUIRE(a->seg_bounds[s + 1] > a->seg_bounds[s] || a->K == 0, SQ_ERR_INVALID_ARG,
                   "sq_quantize_act: seg_bounds not increasing at %d", s);
        SQ_REQUIRE(a->seg_bounds[s + 1] % 16 == 0, SQ_ERR_ALIGNMENT,
                   "sq_quantize_act: segment bound %d must be divisible by 16", a->seg_bounds[s + 1]);
    }
    const int esz = a->x_dtype == SQ_F32 ? 4 : 2;
    SQ_REQUIRE((reinterpret_cast<uintptr_t>(a->x_dev) % 16) == 0 && (a->x_row_stride * esz) % 16 == 0 &&
                   (a->x_batch_stride * esz) % 16 == 0,
               SQ_ERR_ALIGNMENT, "sq_quantize_act: x pointer and strides must be 16-byte aligned");
    SQ_REQUIRE((reinterpret_cast<uintptr_t>(a->xq_dev) % 16) == 0 && a->xq_row_stride % 16 == 0 &&
                   a->xq_batch_stride % 16 == 0,
               SQ_ERR_ALIGNMENT, "sq_quantize_act: xq pointer and strides must be 16-byte aligned");
    if (a->xq_neg_dev) {
        SQ_REQUIRE((reinterpret_cast<uintptr_t>(a->xq_neg_dev) % 16) == 0, SQ_ERR_ALIGNMENT,
                   "sq_quantize_act: xq_neg pointer must be 16-byte aligned");
        SQ_REQUIRE(dynamic || a->sx_neg_dev, SQ_ERR_INVALID_ARG, "sq_quantize_act: DualScale needs sx_neg_dev");
    }
    if (a->smooth_dev)
        SQ_REQUIRE((reinterpret_cast<uintptr_t>(a->smooth_dev) % 16) == 0, SQ_ERR_ALIGNMENT,
                   "sq_quantize_act: smooth pointer must be 16-byte aligned");
    return SQ_OK;
}

static void fill_params(const sq_act_quant_args* a, ActQuantParams& p) {
    p.x = a->x_dev; p.sx = a->sx_dev; p.sx_neg = a->sx_neg_dev; p.smooth = a->smooth_dev;
    p.xq = static_cast<uint8_t*>(a->xq_dev); p.xq_neg = static_cast<uint8_t*>(a->xq_neg_dev);
    p.sx_out = nullptr; p.sx_neg_out = nullptr;
    p.batch = a->batch; p.M = a->M; p.K = a->K;
    p.x_batch_stride = a->x_batch_stride; p.x_row_stride = a->x_row_stride;
    p.sx_batch_stride = a->sx_batch_stride; p.sx_seg_stride = a->sx_seg_stride; p.sx_row_stride = a->sx_row_stride;
    p.xq_batch_stride = a->xq_batch_stride; p.xq_row_stride = a->xq_row_stride;
    p.num_segs = a->num_segs;
    p.pre_act = a->pre_act;
    for (int s = 0; s <= SQ_MAX_SEGS; ++s) p.seg_bounds[s] = s <= a->num_segs ? a->seg_bounds[s] : 0;
    int len = a->seg_bounds[1] - a->seg_bounds[0];
    bool uniform = len > 0;
    for (int s = 1; s < a->num_segs && uniform; ++s) uniform = (a->seg_bounds[s + 1] - a->seg_bounds[s]) == len;
    p.uniform_seg = uniform ? len : 0;
}

static int grid_for(long long warp_items) {
    long long ctas = (warp_items + 7) / 8;
    const long long cap = static_cast<long long>(kNumSMs) * 8;  // 8 CTAs of 256 threads per SM
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    return static_cast<int>(ctas);
}

template <typename T, int OUT>
static void launch_static(const ActQuantParams& p, bool dual, bool smooth, cudaStream_t st) {
    // One warp per row.  When all rows fit on the GPU at once (<= 32 warps per SM) small CTAs spread them evenly:
    // 4096 rows as 512 CTAs of 8 warps leave SMs with 4 or 3 CTAs (15 % tail), as 2048 CTAs of 2 warps with 14 or 13.
    const long long rows = p.batch * p.M;
    int block = 256;
    int grid = grid_for(rows);
    if (rows <= static_cast<long long>(kNumSMs) * 32) {
        block = 64;
        grid = static_cast<int>((rows + 1) / 2 < 1 ? 1 : (rows + 1) / 2);
    }
#define SQ_STATIC(PRE)                                                                     \
    do {                                                                                   \
        if (dual) act_quant_kernel<T, OUT, true, PRE><<<grid, block, 0, st>>>(p);           \
        else act_quant_kernel<T, OUT, false, PRE><<<grid, block, 0, st>>>(p);               \
    } while (0)
    if (smooth) SQ_STATIC(kPreSmooth);
    else if (p.pre_act == SQ_ACT_GELU_TANH) SQ_STATIC(SQ_ACT_GELU_TANH);
    else if (p.pre_act == SQ_ACT_SILU) SQ_STATIC(SQ_ACT_SILU);
    else SQ_STATIC(0);
#undef SQ_STATIC
}

template <typename T, int OUT>
static void launch_dynamic(const ActQuantParams& p, bool dual, cudaStream_t st) {
    // Measured alternatives that were NOT faster than this two-pass kernel (161 us on 16384 x 12288 bf16, 0.57 of the
    // copy roofline; DRAM reads are already 1.02x the input, the second pass hits L2): holding residency to 16 warps per
    // SM (164 us), keeping the segment in the registers of a 32-256 thread group (172-203 us), parking it in shared
    // memory between the passes (175 us, 8 warps per SM).
    const int grid = grid_for(p.batch * p.M * p.num_segs);
    if (p.smooth != nullptr) {
        if (dual) act_quant_dynamic_kernel<T, OUT, true, true><<<grid, 256, 0, st>>>(p);
        else act_quant_dynamic_kernel<T, OUT, false, true><<<grid, 256, 0, st>>>(p);
        return;
    }
    if (dual) act_quant_dynamic_kernel<T, OUT, true, false><<<grid, 256, 0, st>>>(p);
    else act_quant_dynamic_kernel<T, OUT, false, false><<<grid, 256, 0, st>>>(p);
}

int quantize_act(const sq_act_quant_args* a, cudaStream_t st) {
    int rc = validate(a, false);
    if (rc != SQ_OK) return rc;
    if (a->batch * a->M * a->K == 0) return SQ_OK;
    ActQuantParams p;
    fill_params(a, p);
    const bool dual = a->xq_neg_dev != nullptr, smooth = a->smooth_dev != nullptr;
#define SQ_DISPATCH(T)                                                          \
    do {                                                                        \
        if (a->out_kind == SQ_Q_INT8) launch_static<T, SQ_Q_INT8>(p, dual, smooth, st); \
        else launch_static<T, SQ_Q_E4M3>(p, dual, smooth, st);                  \
    } while (0)
    if (a->x_dtype == SQ_F32) SQ_DISPATCH(float);
    else if (a->x_dtype == SQ_F16) SQ_DISPATCH(__half);
    else SQ_DISPATCH(__nv_bfloat16);
#undef SQ_DISPATCH
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

int quantize_act_dynamic(const sq_act_quant_args* a, float* sx_out, float* sx_neg_out, cudaStream_t st) {
    int rc = validate(a, true);
    if (rc != SQ_OK) return rc;
    SQ_REQUIRE(sx_out != nullptr, SQ_ERR_INVALID_ARG, "sq_quantize_act_dynamic: sx_out_dev is NULL");
    const bool dual = a->xq_neg_dev != nullptr;
    SQ_REQUIRE(!dual || sx_neg_out != nullptr, SQ_ERR_INVALID_ARG,
               "sq_quantize_act_dynamic: DualScale needs sx_neg_out_dev");
    if (a->batch * a->M * a->K == 0) return SQ_OK;
    ActQuantParams p;
    fill_params(a, p);
    p.sx_out = sx_out; p.sx_neg_out = sx_neg_out;
#define SQ_DISPATCH(T)                                                       \
    do {                                                                     \
        if (a->out_kind == SQ_Q_INT8) launch_dynamic<T, SQ_Q_INT8>(p, dual, st); \
        else launch_dynamic<T, SQ_Q_E4M3>(p, dual, st);                      \
    } while (0)
    if (a->x_dtype == SQ_F32) SQ_DISPATCH(float);
    else if (a->x_dtype == SQ_F16) SQ_DISPATCH(__half);
    else SQ_DISPATCH(__nv_bfloat16);
#undef SQ_DISPATCH
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

// ---- LayerNorm + adaLN modulation + static quantise, one pass -----------------------------------
// y = LN(x) * (1 + scale[b]) + shift[b] (LayerNorm without affine parameters), then the per-segment static
// quantisation of act_quant_kernel.  In a DiT block this is what sits between the residual stream and the q / k / v
// and MLP projections: three torch kernels (layer_norm, the modulation, the quantise) that each read and write the
// whole [tokens, hidden] tensor.  One warp owns a row and keeps it in registers as raw 128-bit words (at most
// kNormWords per lane); x is read once and only bytes are written.  No counterpart in the reference.
//
// Rows this short make the kernel instruction-bound before it is HBM-bound (at 6.5 TB/s and 3 bytes per element the
// SMs have about a dozen issue slots per element), so the arithmetic is trimmed to fit:
//  * statistics in ONE pass over the registers, as sums of d = x - pivot and d * d, pivot = mean of 32 samples of the
//    row (one per lane): var = E[d^2] - E[d]^2 loses nothing to cancellation because |pivot - mean| is a fraction
//    of the standard deviation;
//  * the per-column factors do not depend on the row: each CTA keeps a = (1 + scale) and c = shift of its batch in
//    shared memory as fp32 (for the single-scale case already multiplied by the segment's quantisation scale), and a
//    CTA's rows never straddle two batches, so a row costs two shared loads per four elements instead of two global
//    loads, two unpacks and an add;
//  * all fp32 arithmetic on pairs (fma.rn.f32x2).
constexpr int kNormWords = 8;

// NW = 128-bit words per lane the row needs (4, 6 or 8), a compile-time bound so that short rows do not pay for the
// registers of long ones: with at most 64 registers a thread, four 256-thread CTAs stay resident per SM, and it is the
// number of rows in flight per SM that decides how much of the HBM bandwidth a load -> reduce -> store chain reaches.
// Optional gated residual in front of the normalisation: x' = x + gate[b] * y (the update of the residual stream by the
// previous linear's output, arithmetic and rounding of torch.addcmul), written to x_out and normalised from registers.
struct NormResidual {
    const void* y;       // nullptr: no residual
    const void* gate;
    void* x_out;         // must not alias x
    long long y_bs, y_rs, g_bs, o_bs, o_rs;   // elements
};

template <typename T, int OUT, bool DUAL, int NW, bool RES>
__global__ void __launch_bounds__(256, (NW <= 6 && !RES) ? 4 : 3) norm_quant_kernel(const __grid_constant__ ActQuantParams p, const T* __restrict__ shift,
                                                                                    const T* __restrict__ scale, long long mod_bs, float eps,
                                                                                    const __grid_constant__ NormResidual res) {
    constexpr int E = Unit<T>::E;
    constexpr int H = E / 4;                       // float4 pieces per 128-bit word of x
    constexpr int kMaxWords = 32 * kNormWords;
    __shared__ float4 tab_a[H][kMaxWords];         // (1 + scale[k]) [* sx[seg(k)] unless DUAL]; lane stride 16 bytes
    __shared__ float4 tab_c[H][kMaxWords];         // shift[k] [* sx[seg(k)] unless DUAL]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpc = blockDim.x >> 5;
    const int words = static_cast<int>(p.K / E);
    const T* __restrict__ x = static_cast<const T*>(p.x);
    const float inv_k = 1.0f / static_cast<float>(p.K);
    const float inv_samples = 1.0f / static_cast<float>(words < 32 ? words : 32);

    // work item = wpc consecutive rows of ONE batch, so the table in shared memory serves every warp of the CTA
    const long long blocks_per_batch = (p.M + wpc - 1) / wpc;
    const long long nblk = p.batch * blocks_per_batch;
    long long tab_batch = -1;
    for (long long item = blockIdx.x; item < nblk; item += gridDim.x) {
        const long long b = item / blocks_per_batch;
        const long long r = (item - b * blocks_per_batch) * wpc + warp;
        if (b != tab_batch) {                      // uniform over the CTA
            __syncthreads();
            for (int k = threadIdx.x * 4; k < p.K; k += blockDim.x * 4) {      // segment bounds are multiples of 16
                const float f = DUAL ? 1.0f : __ldg(p.sx + b * p.sx_batch_stride + find_segment(p, k) * p.sx_seg_stride);
                float a[4], c[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    a[i] = shift != nullptr ? (1.0f + to_float<T>(scale[b * mod_bs + k + i])) * f : f;
                    c[i] = shift != nullptr ? to_float<T>(shift[b * mod_bs + k + i]) * f : 0.0f;
                }
                tab_a[(k % E) / 4][k / E] = make_float4(a[0], a[1], a[2], a[3]);
                tab_c[(k % E) / 4][k / E] = make_float4(c[0], c[1], c[2], c[3]);
            }
            tab_batch = b;
            __syncthreads();
        }
        if (r >= p.M) continue;                    // warp-uniform; every warp still runs every iteration of the loop

        const T* xr = x + b * p.x_batch_stride + r * p.x_row_stride;
        uint8_t* qr = p.xq + b * p.xq_batch_stride + r * p.xq_row_stride;
        uint8_t* qnr = DUAL ? p.xq_neg + b * p.xq_batch_stride + r * p.xq_row_stride : nullptr;

        uint4 raw[NW];
#pragma unroll
        for (int j = 0; j < NW; ++j)
            if (lane + 32 * j < words) raw[j] = __ldg(reinterpret_cast<const uint4*>(xr) + lane + 32 * j);
        if constexpr (RES) {
            const uint4* yr = reinterpret_cast<const uint4*>(static_cast<const T*>(res.y) + b * res.y_bs + r * res.y_rs);
            const uint4* gr = reinterpret_cast<const uint4*>(static_cast<const T*>(res.gate) + b * res.g_bs);
            uint4* orow = reinterpret_cast<uint4*>(static_cast<T*>(res.x_out) + b * res.o_bs + r * res.o_rs);
#pragma unroll
            for (int j = 0; j < NW; ++j) {
                const int u = lane + 32 * j;
                if (u < words) {
                    float xv[E], yv[E], gv[E];
                    Unit<T>::unpack(raw[j], xv);
                    Unit<T>::unpack(__ldg(yr + u), yv);
                    Unit<T>::unpack(__ldg(gr + u), gv);
#pragma unroll
                    for (int i = 0; i < E; ++i) xv[i] = __fadd_rn(xv[i], __fmul_rn(gv[i], yv[i]));   // two roundings, like torch
                    raw[j] = Unit<T>::pack(xv);    // the stream stays in T: normalise what was stored
                    orow[u] = raw[j];
                }
            }
        }

        float pivot = 0.0f;
        if (lane < words) {
            float v[E];
            Unit<T>::unpack(raw[0], v);
            pivot = v[0];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pivot += __shfl_xor_sync(0xffffffffu, pivot, o);
        pivot *= inv_samples;

        const float2 neg_pivot = make_float2(-pivot, -pivot);
        float2 s1 = make_float2(0.0f, 0.0f), s2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < NW; ++j) {
            if (lane + 32 * j < words) {
                float v[E];
                Unit<T>::unpack(raw[j], v);
#pragma unroll
                for (int i = 0; i < E; i += 2) {
                    const float2 d = __fadd2_rn(make_float2(v[i], v[i + 1]), neg_pivot);
                    s1 = __fadd2_rn(s1, d);
                    s2 = __ffma2_rn(d, d, s2);
                }
            }
        }
        float sum = s1.x + s1.y, sq = s2.x + s2.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
        }
        const float md = sum * inv_k;              // mean - pivot
        const float rstd = 1.0f / sqrtf(fmaxf(sq * inv_k - md * md, 0.0f) + eps);
        const float nmr = -(pivot + md) * rstd;
        const float2 rstd2 = make_float2(rstd, rstd), nmr2 = make_float2(nmr, nmr);

        // DualScale: the quantisation scale depends on the sign, so it is applied per element; this lane's k only grows
        int s = 0;
        int next_bound = p.seg_bounds[1];
        float sc = 1.0f, scn = 0.0f;
        if constexpr (DUAL) {
            sc = __ldg(p.sx + b * p.sx_batch_stride);
            scn = __ldg(p.sx_neg + b * p.sx_batch_stride);
        }
#pragma unroll
        for (int j = 0; j < NW; ++j) {
            const int u = lane + 32 * j;
            if (u < words) {
                const int k = u * E;
                float v[E];
                Unit<T>::unpack(raw[j], v);
#pragma unroll
                for (int h = 0; h < H; ++h) {
                    const float4 a = tab_a[h][u], c = tab_c[h][u];
                    const float2 n0 = __ffma2_rn(make_float2(v[4 * h], v[4 * h + 1]), rstd2, nmr2);
                    const float2 n1 = __ffma2_rn(make_float2(v[4 * h + 2], v[4 * h + 3]), rstd2, nmr2);
                    const float2 o0 = __ffma2_rn(n0, make_float2(a.x, a.y), make_float2(c.x, c.y));
                    const float2 o1 = __ffma2_rn(n1, make_float2(a.z, a.w), make_float2(c.z, c.w));
                    v[4 * h] = o0.x; v[4 * h + 1] = o0.y; v[4 * h + 2] = o1.x; v[4 * h + 3] = o1.y;
                }
                if constexpr (DUAL) {
                    while (k >= next_bound) {
                        ++s;
                        next_bound = p.seg_bounds[s + 1];
                        sc = __ldg(p.sx + b * p.sx_batch_stride + s * p.sx_seg_stride);
                        scn = __ldg(p.sx_neg + b * p.sx_batch_stride + s * p.sx_seg_stride);
                    }
                }
                quant_store<OUT, DUAL, E>(v, sc, scn, qr + k, DUAL ? qnr + k : nullptr);   // single scale: sc == 1, folded into the table
            }
        }
    }
}

template <typename T, int OUT>
static void launch_norm(const ActQuantParams& p, bool dual, const void* shift, const void* scale, long long mod_bs, float eps,
                        const NormResidual& res, cudaStream_t st) {
    const long long rows = p.batch * p.M;
    int block = 256;
    int grid = grid_for(rows);
    const long long per_lane_words = (p.K / Unit<T>::E + 31) / 32;
    // as many CTAs as are resident at once (3 or 4 per SM, see the kernel's launch bounds): each walks several 8-row items
    // and fills its shared-memory table once per batch sample instead of once per item
    const int resident = kNumSMs * ((per_lane_words <= 6 && res.y == nullptr) ? 4 : 3);
    if (grid > resident) grid = resident;
    if (rows <= static_cast<long long>(kNumSMs) * 32) {
        block = 64;
        grid = static_cast<int>((rows + 1) / 2 < 1 ? 1 : (rows + 1) / 2);
    }
    const T* sh = static_cast<const T*>(shift);
    const T* sc = static_cast<const T*>(scale);
    const long long per_lane = (p.K / Unit<T>::E + 31) / 32;
#define SQ_NORM2(NW, RES)                                                                                  \
    do {                                                                                                   \
        if (dual) norm_quant_kernel<T, OUT, true, NW, RES><<<grid, block, 0, st>>>(p, sh, sc, mod_bs, eps, res);  \
        else norm_quant_kernel<T, OUT, false, NW, RES><<<grid, block, 0, st>>>(p, sh, sc, mod_bs, eps, res);      \
    } while (0)
#define SQ_NORM(NW)                                \
    do {                                           \
        if (res.y != nullptr) SQ_NORM2(NW, true);  \
        else SQ_NORM2(NW, false);                  \
    } while (0)
    if (per_lane <= 4) SQ_NORM(4);
    else if (per_lane <= 6) SQ_NORM(6);
    else SQ_NORM(kNormWords);
#undef SQ_NORM
#undef SQ_NORM2
}

int norm_quantize_act(const sq_act_quant_args* a, const void* shift, const void* scale, long long mod_bs, float eps,
                      const sq_norm_residual* r, cudaStream_t st) {
    int rc = validate(a, false);
    if (rc != SQ_OK) return rc;
    if (a->batch * a->M * a->K == 0) return SQ_OK;
    NormResidual res = {};
    if (r != nullptr) {
        SQ_REQUIRE(r->y_dev && r->gate_dev && r->x_out_dev, SQ_ERR_INVALID_ARG, "sq_norm_quantize_act: residual pointers must not be NULL");
        SQ_REQUIRE(r->x_out_dev != a->x_dev, SQ_ERR_INVALID_ARG, "sq_norm_quantize_act: x_out must not alias x");
        const long long e16 = a->x_dtype == SQ_F32 ? 4 : 8;      // elements per 16 bytes
        SQ_REQUIRE(reinterpret_cast<uintptr_t>(r->y_dev) % 16 == 0 && reinterpret_cast<uintptr_t>(r->gate_dev) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(r->x_out_dev) % 16 == 0 && r->y_batch_stride % e16 == 0 && r->y_row_stride % e16 == 0 &&
                       r->gate_batch_stride % e16 == 0 && r->x_out_batch_stride % e16 == 0 && r->x_out_row_stride % e16 == 0,
                   SQ_ERR_ALIGNMENT, "sq_norm_quantize_act: residual pointers and strides must be 16-byte aligned");
        res.y = r->y_dev; res.gate = r->gate_dev; res.x_out = r->x_out_dev;
        res.y_bs = r->y_batch_stride; res.y_rs = r->y_row_stride; res.g_bs = r->gate_batch_stride;
        res.o_bs = r->x_out_batch_stride; res.o_rs = r->x_out_row_stride;
    }
    SQ_REQUIRE((shift == nullptr) == (scale == nullptr), SQ_ERR_INVALID_ARG, "sq_norm_quantize_act: shift and scale go together");
    SQ_REQUIRE(a->sx_row_stride == 0 && a->smooth_dev == nullptr && a->pre_act == SQ_ACT_NONE, SQ_ERR_UNSUPPORTED,
               "sq_norm_quantize_act: static per-segment scales only, no smoothing vector, no pre_act");
    const long long esz = a->x_dtype == SQ_F32 ? 4 : 2;
    const long long words = a->K * esz / 16;
    SQ_REQUIRE((a->K * esz) % 16 == 0 && words <= 32 * kNormWords, SQ_ERR_UNSUPPORTED,
               "sq_norm_quantize_act: a row must be at most %d bytes (K = %lld)", 32 * kNormWords * 16, static_cast<long long>(a->K));
    SQ_REQUIRE(reinterpret_cast<uintptr_t>(a->x_dev) % 16 == 0 && (a->x_row_stride * esz) % 16 == 0 && (a->x_batch_stride * esz) % 16 == 0,
               SQ_ERR_ALIGNMENT, "sq_norm_quantize_act: x rows must be 16-byte aligned");
    if (shift != nullptr)
        SQ_REQUIRE(reinterpret_cast<uintptr_t>(shift) % 16 == 0 && reinterpret_cast<uintptr_t>(scale) % 16 == 0 && (mod_bs * esz) % 16 == 0,
                   SQ_ERR_ALIGNMENT, "sq_norm_quantize_act: shift / scale rows must be 16-byte aligned");
    ActQuantParams p;
    fill_params(a, p);
    const bool dual = a->xq_neg_dev != nullptr;
#define SQ_DISPATCH(T)                                                                          \
    do {                                                                                        \
        if (a->out_kind == SQ_Q_INT8) launch_norm<T, SQ_Q_INT8>(p, dual, shift, scale, mod_bs, eps, res, st); \
        else launch_norm<T, SQ_Q_E4M3>(p, dual, shift, scale, mod_bs, eps, res, st);                 \
    } while (0)
    if (a->x_dtype == SQ_F32) SQ_DISPATCH(float);
    else if (a->x_dtype == SQ_F16) SQ_DISPATCH(__half);
    else SQ_DISPATCH(__nv_bfloat16);
#undef SQ_DISPATCH
    SQ_CUDA_OK(cudaGetLastError());
    return SQ_OK;
}

}  // namespace sq
