/*
 * CPU oracle for the real-quantized segmented linear path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of the reference's native kernels.  Only tests/,
 * __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may call it; the
 * product never does.  Each function cites the reference lines it follows (paths relative to the
 * reference project root).
 *
 * Parity pin: the reference's own tests hold no golden vectors for this path (test/test_linear.py
 * only prints norms).  The pin is (1) tests/golden/, produced by importing the reference's Python
 * quantizers / SegmentLinear fake-quant path (tests/golden/make_golden.py), against which this file
 * is checked on CPU, and (2) oracle/_ref, the reference's own fake_e4m3fy C++ built from its
 * sources, against which sqo_e4m3_* are checked.
 *
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off -pthread -shared)
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ---- row-parallel helper (plain pthreads; SQO_THREADS overrides the thread count) ------------ */
typedef void (*sqo_row_fn)(int64_t m_begin, int64_t m_end, void* ctx);
typedef struct { sqo_row_fn fn; void* ctx; int64_t b, e; } sqo_job;
static void* sqo_job_run(void* p) { sqo_job* j = (sqo_job*)p; j->fn(j->b, j->e, j->ctx); return NULL; }

int sqo_num_threads(void) {
    const char* env = getenv("SQO_THREADS");
    long n = env ? atol(env) : sysconf(_SC_NPROCESSORS_ONLN);
    if (n < 1) n = 1;
    if (n > 256) n = 256;
    return (int)n;
}

static void sqo_parallel_rows(int64_t M, sqo_row_fn fn, void* ctx) {
    int nt = sqo_num_threads();
    if (nt > M) nt = (int)(M > 0 ? M : 1);
    if (nt <= 1) { fn(0, M, ctx); return; }
    pthread_t th[256];
    sqo_job jobs[256];
    const int64_t per = (M + nt - 1) / nt;
    int started = 0;
    for (int t = 0; t < nt; ++t) {
        jobs[t].fn = fn; jobs[t].ctx = ctx;
        jobs[t].b = t * per; jobs[t].e = (t + 1) * per < M ? (t + 1) * per : M;
        if (jobs[t].b >= jobs[t].e) break;
        if (pthread_create(&th[t], NULL, sqo_job_run, &jobs[t]) != 0) { fn(jobs[t].b, jobs[t].e, ctx); th[t] = 0; }
        ++started;
    }
    for (int t = 0; t < started; ++t) if (th[t]) pthread_join(th[t], NULL);
}

#define SQO_Q_INT8 0
#define SQO_Q_E4M3 1
#define SQO_Q_INT4 2

#define SQO_GEMM_I8 0
#define SQO_GEMM_F8 1
#define SQO_GEMM_W4A8 2

/* ---- fp8 e4m3 (finite-only "fn" variant: no inf, 0x7F/0xFF = NaN, max 448) ------------------
 * static_cast<__nv_fp8_e4m3>(float) is a saturating round-to-nearest-even conversion
 * (segquant/src/real_quant/quantizer.cuh:21-29; segquant/src/fake_quant/quantizer_fp8.cpp:33-35). */
uint8_t sqo_e4m3_from_float(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
    if (isnan(f)) return 0x7F; /* the hardware conversion yields the positive NaN code for every NaN */
    double a = fabs((double)f);
    if (a >= 448.0) return (uint8_t)(sign | 0x7E); /* saturate (also +-inf) */
    if (a == 0.0) return sign;
    /* subnormals: multiples of 2^-9 below 2^-6; normals: 3 mantissa bits */
    int e;
    (void)frexp(a, &e);         /* a = m * 2^e, m in [0.5, 1) -> floor(log2 a) = e - 1 */
    int ex = e - 1;
    if (ex < -6) ex = -6;
    const double ulp = ldexp(1.0, ex - 3);
    double qd = nearbyint(a / ulp); /* default rounding mode = to nearest even; a/ulp is exact */
    double v = qd * ulp;
    if (v >= 448.0) return (uint8_t)(sign | 0x7E); /* unreachable below 448, kept for safety */
    if (v == 0.0) return sign;
    int e2;
    (void)frexp(v, &e2);
    int ex2 = e2 - 1;
    uint8_t out;
    if (ex2 < -6) {
        out = (uint8_t)(v / ldexp(1.0, -9)); /* subnormal: mantissa only */
    } else {
        const int mant = (int)(v / ldexp(1.0, ex2 - 3)) - 8;
        out = (uint8_t)(((ex2 + 7) << 3) | mant);
    }
    return (uint8_t)(sign | out);
}

float sqo_e4m3_to_float(uint8_t b) {
    const int sign = b & 0x80;
    const int ex = (b >> 3) & 0xF;
    const int mant = b & 7;
    double v;
    if (ex == 0xF && mant == 7) return sign ? -NAN : NAN;
    if (ex == 0) v = ldexp((double)mant, -9);
    else v = ldexp(1.0 + mant / 8.0, ex - 7);
    return (float)(sign ? -v : v);
}

void sqo_e4m3_encode(const float* x, uint8_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = sqo_e4m3_from_float(x[i]);
}

void sqo_e4m3_roundtrip(const float* x, float* out, int64_t n) {
    /* fake_e4m3fy CPU branch, segquant/src/fake_quant/quantizer_fp8.cpp:29-37 */
    for (int64_t i = 0; i < n; ++i) out[i] = sqo_e4m3_to_float(sqo_e4m3_from_float(x[i]));
}

/* ---- store rules ------------------------------------------------------------------------------ */
static inline int8_t q_int8(float scaled) {
    /* store_data<int8_t>: clamp then rintf, quantizer.cuh:32-35 */
    float c = fminf(fmaxf(scaled, -128.0f), 127.0f);
    return (int8_t)rintf(c);
}
static inline int q_int4(float scaled) {
    /* store_data<int4b_t>: clamp [-8,7], rintf, & 0xF, quantizer.cuh:37-40 */
    float c = fminf(fmaxf(scaled, -8.0f), 7.0f);
    return ((int)rintf(c)) & 0xF;
}
static inline uint8_t q_byte(float scaled, int kind) {
    return kind == SQO_Q_INT8 ? (uint8_t)q_int8(scaled) : sqo_e4m3_from_float(scaled);
}

/* ---- activation quantise -------------------------------------------------------------------------
 * real_quantize_scaled_kernel / real_quantize_dual_scaled_kernel with (segment, token) scales,
 * quantizer.cuh:148-206.  x is [M, K] row-major with K split by bounds[0..nsegs]; scale of
 * (segment s, row m) is sx[s*sx_seg_stride + m*sx_row_stride].  smooth (nullable): divide x[k] by
 * smooth[k] first (segquant/optimum/optimizer.py:467-470). */
typedef struct {
    const float* x; int64_t M, K; int nsegs; const int32_t* bounds; const float* sx; const float* sx_neg;
    int64_t sx_seg_stride, sx_row_stride; const float* smooth; int out_kind; uint8_t* xq; uint8_t* xq_neg;
} sqo_aq_ctx;

static void sqo_quantize_act_rows(int64_t m0, int64_t m1, void* vp) {
    const sqo_aq_ctx* c = (const sqo_aq_ctx*)vp;
    const int64_t K = c->K;
    for (int64_t m = m0; m < m1; ++m) {
        for (int s = 0; s < c->nsegs; ++s) {
            const float sp = c->sx[s * c->sx_seg_stride + m * c->sx_row_stride];
            const float sn = c->sx_neg ? c->sx_neg[s * c->sx_seg_stride + m * c->sx_row_stride] : 0.0f;
            for (int64_t k = c->bounds[s]; k < c->bounds[s + 1]; ++k) {
                float v = c->x[m * K + k];
                if (c->smooth) v = v / c->smooth[k];
                if (!c->xq_neg) {
                    c->xq[m * K + k] = q_byte(v * sp, c->out_kind);
                } else if (v >= 0) { /* quantizer.cuh:193-197 */
                    c->xq[m * K + k] = q_byte(v * sp, c->out_kind);
                    c->xq_neg[m * K + k] = q_byte(0.0f, c->out_kind);
                } else {             /* quantizer.cuh:198-203 */
                    c->xq_neg[m * K + k] = q_byte(v * sn, c->out_kind);
                    c->xq[m * K + k] = q_byte(0.0f, c->out_kind);
                }
            }
        }
    }
}

void sqo_quantize_act(const float* x, int64_t M, int64_t K, int nsegs, const int32_t* bounds, const float* sx,
                      const float* sx_neg, int64_t sx_seg_stride, int64_t sx_row_stride, const float* smooth, int out_kind,
                      uint8_t* xq, uint8_t* xq_neg) {
    sqo_aq_ctx c = {x, M, K, nsegs, bounds, sx, sx_neg, sx_seg_stride, sx_row_stride, smooth, out_kind, xq, xq_neg};
    sqo_parallel_rows(M, sqo_quantize_act_rows, &c);
}

/* ---- weight quantise ------------------------------------------------------------------------------
 * real_quantized_quantize_weights<T>, real_gemm.cu:538-638 with the kernels quantizer.cuh:55-68
 * (scalar) and :103-118 (per row).  scale_mode 2 (per row and K-group) extends the per-row rule.
 * int4: element idx goes to byte idx/2, low nibble when idx is even (quantizer.cuh:41-49). */
void sqo_quantize_weight(const float* w, int64_t N, int64_t K, int scale_mode, float scale_scalar, const float* scale,
                         int group, int out_kind, uint8_t* out) {
    const int64_t gpr = scale_mode == 2 ? K / group : 0;
    if (out_kind == SQO_Q_INT4) memset(out, 0, (size_t)((N * K + 1) / 2));
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t k = 0; k < K; ++k) {
            float sc = scale_scalar;
            if (scale_mode == 1) sc = scale[n];
            else if (scale_mode == 2) sc = scale[n * gpr + k / group];
            const float v = w[n * K + k] * sc;
            const int64_t idx = n * K + k;
            if (out_kind == SQO_Q_INT4) {
                const int q = q_int4(v);
                if ((idx & 1) == 0) out[idx >> 1] = (uint8_t)((out[idx >> 1] & 0xF0) | q);
                else out[idx >> 1] = (uint8_t)((out[idx >> 1] & 0x0F) | (q << 4));
            } else {
                out[idx] = q_byte(v, out_kind);
            }
        }
    }
}

void sqo_unpack_int4(const uint8_t* packed, int8_t* out, int64_t numel) {
    for (int64_t i = 0; i < numel; ++i) {
        const uint8_t b = packed[i >> 1];
        const int nib = (i & 1) ? (b >> 4) : (b & 0xF);
        out[i] = (int8_t)(nib >= 8 ? nib - 16 : nib);
    }
}

/* ---- segmented GEMM + de-quantise -------------------------------------------------------------------
 * Integer / fp8 products accumulated exactly per accumulation unit (int64 resp. double; the
 * reference accumulates int32 with saturation, real_gemm.cu:172-180, which never saturates at these
 * sizes, and fp32 for e4m3, :192-197), then
 *   y = (float)acc / (sx * sw)                       dequantizer.cuh:8-52  (fp32 multiply, fp32 divide)
 *   y = accp/(sp*sw) + accn/(sn*sw)                  dequantizer.cuh:53-73 (DualScale)
 * summed over units in fp32 in ascending order (segquant/layers/SegmentLinear.py:238-240), + bias
 * (:241).  Units: segments bounds[] refined by weight groups of `group` columns (0 = none).
 * wq is [N, K] int8 / e4m3 bytes, or packed int4 [N, K/2] for SQO_GEMM_W4A8.
 * sw index = s*sw_seg_stride + g*sw_group_stride + n*sw_col_stride.
 * acc_out (nullable): [units][sides][M][N] int32 (fp32 bit patterns of the double sum for e4m3).
 * Returns the number of units. */
typedef struct {
    int kind, sides; int64_t M, N, K, k, ke, g; int s, unit;
    const uint8_t* xq; const uint8_t* xq_neg; const int8_t* w8; const float* wf; float* const* xf;
    const float* sx; const float* sx_neg; int64_t sx_seg_stride, sx_row_stride;
    const float* sw; int64_t sw_seg_stride, sw_group_stride, sw_col_stride;
    float* y; int32_t* acc_out;
} sqo_gemm_ctx;

static void sqo_gemm_unit_rows(int64_t m0, int64_t m1, void* vp) {
    const sqo_gemm_ctx* c = (const sqo_gemm_ctx*)vp;
    const int64_t N = c->N, K = c->K, M = c->M;
    for (int64_t m = m0; m < m1; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            float total = 0.0f;
            for (int sd = 0; sd < c->sides; ++sd) {
                float accf;
                int32_t acc_bits;
                if (c->kind == SQO_GEMM_F8) {
                    double a = 0.0;
                    const float* xr = c->xf[sd] + m * K;
                    const float* wr = c->wf + n * K;
                    for (int64_t kk = c->k; kk < c->ke; ++kk) a += (double)xr[kk] * (double)wr[kk];
                    accf = (float)a;
                    memcpy(&acc_bits, &accf, 4);
                } else {
                    int32_t a = 0; /* |sum| <= K*128*128 < 2^31 for K < 131072 */
                    const int8_t* xr = (const int8_t*)(sd ? c->xq_neg : c->xq) + m * K;
                    const int8_t* wr = c->w8 + n * K;
                    for (int64_t kk = c->k; kk < c->ke; ++kk) a += (int32_t)xr[kk] * (int32_t)wr[kk];
                    acc_bits = a;
                    accf = (float)acc_bits; /* LinearCombination converts int32 -> float, real_gemm.cu:262-267 */
                }
                if (c->acc_out) c->acc_out[(((int64_t)c->unit * c->sides + sd) * M + m) * N + n] = acc_bits;
                const float sxv = (sd ? c->sx_neg : c->sx)[c->s * c->sx_seg_stride + m * c->sx_row_stride];
                const float swv = c->sw[c->s * c->sw_seg_stride + c->g * c->sw_group_stride + n * c->sw_col_stride];
                const float scale = sxv * swv;  /* dequantizer.cuh:32 */
                total = sd == 0 ? accf / scale : total + accf / scale; /* :46, :67-70 */
            }
            c->y[m * N + n] += total;
        }
    }
}

int sqo_seg_gemm(int kind, int64_t M, int64_t N, int64_t K, const uint8_t* xq, const uint8_t* xq_neg, const uint8_t* wq,
                 int nsegs, const int32_t* bounds, int group, const float* sx, const float* sx_neg, int64_t sx_seg_stride,
                 int64_t sx_row_stride, const float* sw, int64_t sw_seg_stride, int64_t sw_group_stride,
                 int64_t sw_col_stride, const float* bias, float* y, int32_t* acc_out) {
    const int sides = xq_neg ? 2 : 1;
    if (K >= 131072) return -1;
    /* expand operands once */
    float* wf = NULL;
    int8_t* wi = NULL;
    float* xf[2] = {NULL, NULL};
    if (kind == SQO_GEMM_F8) {
        wf = (float*)malloc(sizeof(float) * (size_t)(N * K));
        for (int64_t i = 0; i < N * K; ++i) wf[i] = sqo_e4m3_to_float(wq[i]);
        for (int sd = 0; sd < sides; ++sd) {
            const uint8_t* src = sd ? xq_neg : xq;
            xf[sd] = (float*)malloc(sizeof(float) * (size_t)(M * K));
            for (int64_t i = 0; i < M * K; ++i) xf[sd][i] = sqo_e4m3_to_float(src[i]);
        }
    } else if (kind == SQO_GEMM_W4A8) {
        wi = (int8_t*)malloc((size_t)(N * K));
        sqo_unpack_int4(wq, wi, N * K);
    }
    const int8_t* w8 = kind == SQO_GEMM_W4A8 ? wi : (const int8_t*)wq;

    for (int64_t i = 0; i < M * N; ++i) y[i] = 0.0f;
    int unit = 0;
    for (int s = 0; s < nsegs; ++s) {
        int64_t k = bounds[s];
        while (k < bounds[s + 1]) {
            int64_t ke = bounds[s + 1];
            int64_t g = 0;
            if (group > 0) {
                const int64_t ge = (k / group + 1) * group;
                if (ge < ke) ke = ge;
                g = k / group;
            }
            sqo_gemm_ctx c = {kind, sides, M, N, K, k, ke, g, s, unit, xq, xq_neg, w8, wf, xf,
                              sx, sx_neg, sx_seg_stride, sx_row_stride, sw, sw_seg_stride, sw_group_stride, sw_col_stride,
                              y, acc_out};
            sqo_parallel_rows(M, sqo_gemm_unit_rows, &c);
            ++unit;
            k = ke;
        }
    }
    if (bias)
        for (int64_t m = 0; m < M; ++m)
            for (int64_t n = 0; n < N; ++n) y[m * N + n] += bias[n];
    free(wf);
    free(wi);
    free(xf[0]);
    free(xf[1]);
    return unit;
}
