/*
 * segquant_b200 -- C ABI of the B200 (sm_100a) real-quantized segmented linear path.
 *
 * Every entry point takes plain pointers and sizes, enqueues work on the given CUDA stream and
 * returns immediately with a status code (0 = ok, negative = error, see SQ_ERR_*).  Nothing here
 * throws, blocks on the device, or allocates device memory unless its comment says so.
 * All pointers named *_dev are device pointers valid on the device that is current when the call
 * is made; the caller owns them and keeps them alive until the stream has run the work.
 *
 * Scale convention (the reference's): a scale is a MULTIPLIER, q = round(x * scale), and the
 * de-quantised value is q / scale  (segquant/quantizers/quantizer.py:209, :277-279, :442).
 *
 * The entry points replace, one to one, the host pipelines of the reference's native layer:
 *   segquant/src/real_quant/real_gemm.cu      (real_quantized_gemm_scaled, _dual_scaled,
 *                                              real_quantized_quantize_weights)
 *   segquant/src/real_quant/quantizer.cuh     (activation / weight quantise kernels)
 *   segquant/src/real_quant/dequantizer.cuh   (de-quantise kernels, here the GEMM epilogue)
 * which the reference exposes through pybind11 in segquant/src/real_quant/seg_utils.h:82-161.
 */
#ifndef SEGQUANT_B200_H
#define SEGQUANT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SQ_VERSION 100

/* ---- status codes ---------------------------------------------------------------------- */
#define SQ_OK 0
#define SQ_ERR_INVALID_ARG (-1)   /* null pointer, negative size, unknown enum                    */
#define SQ_ERR_ALIGNMENT (-2)     /* K / stride / pointer alignment; the reference raises
                                     std::runtime_error here (real_gemm.cu:237-247)              */
#define SQ_ERR_UNSUPPORTED (-3)   /* a combination this build has no kernel for                   */
#define SQ_ERR_CUDA (-4)          /* a CUDA runtime / driver call failed (real_gemm.cu:300-304)   */
#define SQ_ERR_DEVICE_TIMEOUT (-5)/* a bounded wait inside a kernel ran out (see sq_device_status)*/
#define SQ_ERR_TOO_LARGE (-6)     /* size beyond a stated maximum                                 */

/* ---- enums ----------------------------------------------------------------------------- */
/* floating dtypes of activations / weights / outputs (at::ScalarType Float, Half, BFloat16:
   real_gemm.cu:22-28) */
#define SQ_F32 0
#define SQ_F16 1
#define SQ_BF16 2

/* storage formats of quantised data (StoreType, seg_utils.h:25-46) */
#define SQ_Q_INT8 0  /* int8, clamp [-128,127] then round-to-nearest-even (quantizer.cuh:32-35)   */
#define SQ_Q_E4M3 1  /* fp8 e4m3, saturating RN-even cast (quantizer.cuh:21-29)                   */
#define SQ_Q_INT4 2  /* signed int4, clamp [-8,7], two per byte, element 2j in the LOW nibble
                        (quantizer.cuh:37-50)                                                      */

/* GEMM operand combinations (the reference's module prefixes, quantized_mix.cpp:24-29) */
#define SQ_GEMM_W8A8_I8 0   /* Wint8Aint8      : int8 x int8  -> int32                            */
#define SQ_GEMM_W8A8_F8 1   /* Wfpe4m3Afpe4m3  : e4m3 x e4m3  -> fp32                             */
#define SQ_GEMM_W4A8 2      /* Wint4Aint8      : int8 x int4  -> int32                            */

#define SQ_MAX_SEGS 64      /* most activation-scale segments along K in one call                 */
#define SQ_MAX_PEERS 8      /* most peer GPUs' output buffers one sq_gemm call also writes (fused all-gather) */

typedef void* sq_stream_t;  /* a cudaStream_t */

/* ---- library ----------------------------------------------------------------------------- */
int sq_version(void);
/* Message of the last error on the calling thread ("" if none). */
const char* sq_last_error(void);
/* Short name of a status code. */
const char* sq_status_string(int status);
/* Reads (and clears) the word that kernels of this library write when one of their bounded
   waits ran out on the CURRENT device.  Synchronises the device.  0 = no kernel reported
   anything; otherwise a code identifying the wait that gave up.  Returns SQ_ERR_CUDA (<0) if
   the device cannot be queried. */
int64_t sq_device_status(void);
/* Same read (and clear), as a status: SQ_OK, or SQ_ERR_DEVICE_TIMEOUT with sq_last_error() naming the block and the
   wait that gave up (the kernel that reported it returned early: its output is incomplete), or SQ_ERR_CUDA.
   The reference has no counterpart: its CUTLASS kernels have no waits of their own, and a hung launch there ends
   in the CUDA watchdog or never (real_gemm.cu:300-304 only checks the launch status). */
int sq_check_device(void);
/* Limit, in SM cycles, of every bounded wait inside the GEMM kernels launched after this call (process-wide).
   0 restores the default of 4e9 (about 2 s); accepted range [1e6, 1e12]. */
int sq_set_wait_limit_cycles(int64_t cycles);
/* Launches a one-CTA probe kernel that exercises the bounded-wait / abort path on purpose and safely: one warp waits,
   with the library's wait helper, on a barrier nobody arrives at and gives up after limit_cycles (<= 1e8); a second
   warp with a 64x longer limit must leave early through the CTA's abort flag.  The kernel returns normally; afterwards
   sq_device_status() reports (0 << 8 | 9) once.  out_dev[4] (int32, caller-provided): abort flag, return values of the
   two waits (both 0), and 1 if the second warp left before its own limit.  Test aid; no counterpart in the reference. */
int sq_wait_probe(int64_t limit_cycles, int32_t* out_dev, sq_stream_t stream);
/* Process-wide override of the GEMM schedule the host would pick (tuning and test aid; the environment variables
   SEGQUANT_B200_BN / _CTA2 / _KSUB / _NO_GEMV give the initial values and are read once).  bn: 0 = automatic, or
   128 / 192 / 256 tile columns; two_cta: -1 = automatic, 0 = one-CTA kernel, 1 = CTA-pair kernel; ksub: 0 = automatic,
   1 / 2 = 128-byte K sub-tiles per stage of the pair kernel; no_gemv: 1 = never use the skinny-M kernel.
   Results never depend on the schedule (integer sums are exact, the fp32 steps are the same). */
int sq_set_gemm_schedule(int32_t bn, int32_t two_cta, int32_t ksub, int32_t no_gemv);

/* ---- activation quantise ------------------------------------------------------------------
 * Replaces real_quantize_scaled_kernel / real_quantize_dual_scaled_kernel
 * (segquant/src/real_quant/quantizer.cuh:159-206, launched at real_gemm.cu:701-705, :818-826)
 * together with the torch-side `.contiguous()` copy that feeds them
 * (segquant/optimum/optimizer.py:105, :114).
 *
 * x is `batch` matrices of M rows by K columns, K contiguous, row r of matrix b starting at
 * element  b*x_batch_stride + r*x_row_stride.  Columns are split into num_segs segments by
 * seg_bounds[0..num_segs] (seg_bounds[0]=0, last = K, every bound a multiple of 16).  Segment s
 * of matrix b, row r uses   sx_dev[b*sx_batch_stride + s*sx_seg_stride + r*sx_row_stride].
 * Output has the same [batch, M, K] shape, one byte per element, strides in BYTES.
 * If xq_neg_dev != NULL the DualScale rule applies: x >= 0 goes to xq (scaled by sx), x < 0 goes
 * to xq_neg (scaled by sx_neg), the other side gets 0.
 */
#define SQ_ACT_NONE 0
#define SQ_ACT_GELU_TANH 1      /* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) */
#define SQ_ACT_SILU 2           /* x / (1 + exp(-x)) */

typedef struct sq_act_quant_args {
    const void* x_dev;
    int32_t x_dtype;           /* SQ_F32 / SQ_F16 / SQ_BF16 */
    int32_t out_kind;          /* SQ_Q_INT8 / SQ_Q_E4M3 */
    int64_t batch, M, K;
    int64_t x_batch_stride, x_row_stride;        /* elements */
    int32_t num_segs;
    int32_t seg_bounds[SQ_MAX_SEGS + 1];
    const float* sx_dev;
    const float* sx_neg_dev;   /* NULL unless DualScale */
    int64_t sx_batch_stride, sx_seg_stride, sx_row_stride;
    const float* smooth_dev;   /* NULL, or K per-channel divisors applied before scaling (x / s[k]);
                                  the SmoothQuant pre-op of optimizer.py:467-470, :514-521        */
    void* xq_dev;
    void* xq_neg_dev;          /* NULL unless DualScale */
    int64_t xq_batch_stride, xq_row_stride;      /* bytes */
    int32_t pre_act;           /* SQ_ACT_*: activation applied to x (in fp32) before it is scaled; static scales
                                  only, not together with smooth_dev.  No counterpart in the reference, where the
                                  activation is a separate torch op in front of the layer.                        */
    int32_t reserved0;         /* must be 0 */
} sq_act_quant_args;

int sq_quantize_act(const sq_act_quant_args* args, sq_stream_t stream);

/* Dynamic per-token variant: computes, for every (matrix, segment, row), the scale
 * qmax / max(amax, 2^-24) over that row segment (IntQuantizer.calibrate with axis=-1,
 * segquant/quantizers/quantizer.py:209-217; FloatQuantizer.calibrate :442-452), writes it to
 * sx_out_dev[(b*num_segs + s)*M + r] and quantises with it in the same launch.
 * With DualScale the positive side uses qmax/pos_amax and the negative side |qmin|/neg_amax
 * (quantizer.py:187-203; 448 on both sides for e4m3, :425-440); they go to sx_out_dev and
 * sx_neg_out_dev.  Uses args->x*, batch/M/K, seg_bounds, out_kind, xq*, smooth_dev; ignores args->sx*.
 * With smooth_dev the row is first divided by the K smoothing factors and rounded to the dtype of x, which
 * is the tensor the reference's Smooth / SVD optimizers calibrate on (optimizer.py:467-470, :724-728): pass the
 * factors already rounded to that dtype.
 */
int sq_quantize_act_dynamic(const sq_act_quant_args* args, float* sx_out_dev,
                            float* sx_neg_out_dev, sq_stream_t stream);

/* ---- LayerNorm + adaLN modulation + activation quantise (no counterpart in the reference) ----
 * y = LayerNorm(x) * (1 + scale[b]) + shift[b], LayerNorm over K without affine parameters (eps inside the square
 * root), immediately quantised like sq_quantize_act with the static per-segment scales of `args` (sx_row_stride must
 * be 0, smooth_dev NULL).  Fuses the three torch kernels that sit between the residual stream and the q / k / v and
 * MLP projections of a DiT block (layer_norm, modulation, quantise: each a full pass over [tokens, hidden]) into one
 * read of x.  shift_dev / scale_dev: [batch, K] in the dtype of x, rows mod_batch_stride elements apart, or both NULL
 * for a plain LayerNorm.  A row may be at most 4096 bytes (K <= 2048 for 16-bit inputs); longer rows return
 * SQ_ERR_UNSUPPORTED and the caller keeps the separate kernels.
 */
int sq_norm_quantize_act(const sq_act_quant_args* args, const void* shift_dev, const void* scale_dev,
                         int64_t mod_batch_stride, float eps, sq_stream_t stream);

/* The same with the gated residual update of the stream in front: x' = x + gate[b] * y (arithmetic and rounding of
 * sq_gated_residual / torch.addcmul) is written to x_out_dev and normalised from registers, so the update costs no
 * pass over [tokens, hidden] of its own.  y / x_out: [batch, M, K] in the dtype of x, gate: [batch, K]; strides in
 * elements, 16-byte aligned; x_out must not alias x.  residual == NULL is sq_norm_quantize_act.
 */
typedef struct sq_norm_residual {
    const void* y_dev;
    const void* gate_dev;
    void* x_out_dev;
    int64_t y_batch_stride, y_row_stride;
    int64_t gate_batch_stride;
    int64_t x_out_batch_stride, x_out_row_stride;
} sq_norm_residual;

int sq_residual_norm_quantize_act(const sq_act_quant_args* args, const void* shift_dev, const void* scale_dev,
                                  int64_t mod_batch_stride, float eps, const sq_norm_residual* residual,
                                  sq_stream_t stream);

/* ---- gated residual add (no counterpart in the reference) ---------------------------------------
 * out[b, r, :] = x[b, r, :] + gate[b, :] * y[b, r, :] on 16-bit tensors: the residual-stream update of a DiT block
 * (y = output of a quantised linear, gate = a chunk of the adaLN modulation).  Bit-identical to torch.addcmul; exists
 * because torch runs a gate broadcast over the tokens through its strided-iterator kernel at a fraction of the copy
 * bandwidth.  out may alias x.  K and all strides (elements) are multiples of 8, pointers 16-byte aligned.
 */
typedef struct sq_gated_residual_args {
    const void* x_dev;
    const void* gate_dev;
    const void* y_dev;
    void* out_dev;
    int32_t dtype;             /* SQ_F16 / SQ_BF16 */
    int32_t reserved0;
    int64_t batch, M, K;
    int64_t x_batch_stride, x_row_stride;
    int64_t y_batch_stride, y_row_stride;
    int64_t out_batch_stride, out_row_stride;
    int64_t gate_batch_stride;
} sq_gated_residual_args;

int sq_gated_residual(const sq_gated_residual_args* args, sq_stream_t stream);

/* ---- weight quantise / pack ---------------------------------------------------------------
 * Replaces real_quantized_quantize_weights<T> (real_gemm.cu:538-638; pybind names in
 * seg_utils.h:82-120).  w is [N, K] contiguous.  scale_mode 0: one scalar `scale_scalar`
 * (float overload); 1: scale_dev[N] per output row (Tensor overload); 2: scale_dev[N, K/group]
 * per row and K-group (no counterpart in the reference, whose kernels are per-row at most:
 * segquant/src/README.md:19).  INT4 output is N*K/2 bytes, element 2j of the flattened [N,K]
 * array in the low nibble of byte j.
 */
int sq_quantize_weight(const void* w_dev, int32_t w_dtype, int64_t N, int64_t K,
                       int32_t scale_mode, float scale_scalar, const float* scale_dev,
                       int32_t group_size, int32_t out_kind, void* out_dev, sq_stream_t stream);

/* int4 (two per byte, low nibble first) -> int8, numel = number of int4 elements (even). */
int sq_unpack_int4(const void* packed_dev, void* out_dev, int64_t numel, sq_stream_t stream);

/* ---- segmented GEMM + de-quantise epilogue ------------------------------------------------
 * Replaces launch_universal_gemm_scaled (real_gemm.cu:208-305) and its three wrappers
 * (:424-532), real_dequantize_scaled_kernel / real_dequantize_dual_scaled_kernel
 * (dequantizer.cuh:35-73), and -- when num_segs > 1 or bias_dev != NULL -- the torch-side
 * segment sum and bias add of segquant/layers/SegmentLinear.py:238-241.
 *
 * `batch` independent problems.  Problem b multiplies quantised activations Xq_b [M, K] by the
 * quantised weights Wq_b [N, K] (both K-contiguous, "TN" like the reference: real_gemm.cu:225-227).
 * K is cut into accumulation units: first by the activation segments seg_bounds[], then, if
 * group_size > 0, every group_size columns (weight-scale groups, counted from column 0).
 * Each unit u has an exact int32 (fp32 for e4m3) accumulator acc_u, and
 *
 *   y[b,m,n] = sum_u  float(acc_u[m,n]) / (sx * sw)          (dequantizer.cuh:8-52)
 *            ( + float(accn_u[m,n]) / (sx_neg * sw)  with DualScale, dequantizer.cuh:53-73 )
 *            ( + bias[n] )
 *   sx  = sx_dev [b*sx_batch_stride + s*sx_seg_stride + m*sx_row_stride]
 *   sw  = sw_dev [b*sw_batch_stride + s*sw_seg_stride + g*sw_group_stride + n*sw_col_stride]
 * with s the segment and g = k / group_size the weight group of the unit.  Strides may be 0
 * (broadcast).  sw_dev is fp32, or bf16 when sw_is_bf16 != 0.  Any layout the strides can describe is accepted; with
 * weight groups the group-major one, (K / group_size, N) with sw_col_stride = 1 and sw_group_stride = N, is the fast one:
 * the kernel builds one table of N-tile scales per unit, and in the (N, K / group_size) layout those are strided by the
 * group count (measured: int4 weights, groups of 128, 16384 x 3072 x 12288: 1.28 ms group-major, 1.70 ms column-major).
 *
 * Alignment: K and every segment bound a multiple of 32 (the reference needs K % 16 for
 * 8-bit and K % 32 for int4: real_gemm.cu:199-203); group_size a multiple of 32; operand row and
 * batch strides multiples of 16 bytes; operand base pointers 16-byte aligned.
 *
 * W4A8 weights are packed int4 ([N, K/2] bytes per problem, low nibble = even k).
 * If w_seg_as_batch != 0 the weights of segment s are a separate [N, seg_len] matrix found at
 * batch index s of wq (the reference's packed layout (segments, N*seg/2),
 * segquant/layers/segment_tensor_manager.py:56-66) and `batch` must be 1.
 *
 * acc_dump_dev (NULL in production): if set, unit u's raw accumulator words are also written to
 * acc_dump_dev[((b*units + u)*sides + side)*M*N + m*N + n] (int32, or fp32 bits for e4m3);
 * this is how tests prove bit-exact integer accumulation.
 */
typedef struct sq_gemm_args {
    int32_t kind;              /* SQ_GEMM_* */
    int32_t out_dtype;         /* SQ_F32 / SQ_F16 / SQ_BF16 */
    int64_t batch, M, N, K;
    const void* xq_dev;
    const void* xq_neg_dev;    /* NULL unless DualScale */
    int64_t xq_batch_stride, xq_row_stride;      /* bytes; batch stride 0 = shared by all b */
    const void* wq_dev;
    int64_t wq_batch_stride, wq_row_stride;      /* bytes; batch stride 0 = one weight matrix shared by all b */
    int32_t w_seg_as_batch;
    int32_t num_segs;
    int32_t seg_bounds[SQ_MAX_SEGS + 1];
    int32_t group_size;        /* 0 = no weight groups along K */
    int32_t sw_is_bf16;
    const float* sx_dev;
    const float* sx_neg_dev;
    int64_t sx_batch_stride, sx_seg_stride, sx_row_stride;
    const void* sw_dev;
    int64_t sw_batch_stride, sw_seg_stride, sw_group_stride, sw_col_stride;
    const void* bias_dev;      /* NULL or [N] (per problem: + b*bias_batch_stride), out_dtype or fp32 */
    int32_t bias_dtype;
    int32_t reserved0;
    int64_t bias_batch_stride; /* elements */
    void* y_dev;
    int64_t y_batch_stride, y_row_stride;        /* elements */
    void* acc_dump_dev;
    /* Optional fused all-gather (column-sharded layers, one process per GPU): besides y_dev, every finished
     * tile is also written into num_peer_outputs further [M, *] matrices -- peer GPUs' output buffers mapped
     * into this process (CUDA IPC / symmetric memory) -- at columns [peer_col_offset, peer_col_offset + N)
     * with row stride peer_row_stride (elements of out_dtype; both must keep rows 16-byte aligned).
     * Plain peer stores from the epilogue; no multicast.  batch must be 1.  The caller synchronises the
     * ranks (e.g. an NCCL barrier) before anyone reads its buffer.  No counterpart in the reference. */
    int32_t num_peer_outputs;  /* 0 .. SQ_MAX_PEERS */
    int32_t reserved1;
    void* peer_y_dev[SQ_MAX_PEERS];
    int64_t peer_row_stride, peer_col_offset;
} sq_gemm_args;

int sq_gemm(const sq_gemm_args* args, sq_stream_t stream);

/* ---- exchange step of a column-sharded layer (no counterpart in the reference, which is single-GPU) ----------
 * Copies the [rows, width_bytes] block that starts at src_dev (rows src_row_stride_bytes apart) -- this rank's column
 * block, already in place inside its own [rows, N] result -- to num_peers peer GPUs' matrices: peer_dst_dev[j] points
 * at the block's position in peer j's matrix (HOST array of device pointers into peer memory mapped into this process),
 * rows dst_row_stride_bytes apart.  Plain 16-byte stores over NVLink, whole 512-byte row segments per warp; nothing is
 * read from a peer and nothing waits: order the ranks with a stream-ordered barrier before anyone reads its matrix.
 * width, strides and all pointers must be multiples of 16 bytes. */
int sq_push_columns(const void* src_dev, int64_t rows, int64_t width_bytes, int64_t src_row_stride_bytes,
                    int32_t num_peers, void* const* peer_dst_dev, int64_t dst_row_stride_bytes, sq_stream_t stream);

/* Stream-ordered barrier between the `world` ranks of a sharded layer (one rank per GPU; at most SQ_MAX_PEERS + 1),
 * the step after sq_push_columns or a sq_gemm with peer outputs.  flags_dev is a HOST array of `world` device pointers:
 * entry j is rank j's array of `world` 32-bit words (peer memory mapped into this process; entry `rank` is this rank's own
 * array), all zero before the first call.  `epoch` is the call's number, 1, 2, ... , the same on every rank.  The kernel
 * publishes everything this GPU wrote before it (system-scope fence), stores epoch into word [rank] of every peer's array
 * and waits until its own words have reached epoch.  The wait is bounded like every wait of this library: when it runs
 * out the kernel returns and sq_check_device() reports SQ_ERR_DEVICE_TIMEOUT with wait id 10 and the peer's rank in the
 * place of the block.  No counterpart in the reference. */
int sq_peer_barrier(int32_t rank, int32_t world, void* const* flags_dev, uint32_t epoch, sq_stream_t stream);

/* Number of accumulation units sq_gemm will use for these segment bounds / group size
   (the `units` of the acc_dump layout).  Negative = error. */
int sq_gemm_num_units(int32_t num_segs, const int32_t* seg_bounds, int32_t group_size);

/* ---- fused layer forward --------------------------------------------------------------------
 * One call = SegmentLinear.forward on the real-quant path (segquant/layers/SegmentLinear.py:228-241
 * -> segquant/optimum/optimizer.py:94-118 -> real_gemm.cu:643-894): quantise x with `q`, then
 * run `g` on the result.  q->xq_dev / q->xq_neg_dev are scratch buffers the CALLER provides
 * (batch*M*K bytes each); g->xq_dev / g->xq_neg_dev are ignored and taken from q.
 */
int sq_seg_linear(const sq_act_quant_args* q, const sq_gemm_args* g, sq_stream_t stream);

/* ---- fused layer forward without any device allocation -------------------------------------------
 * No counterpart in the reference (its host pipeline allocates scratch tensors on every call).
 *
 * Same computation as sq_seg_linear, for callers that cannot supply the scratch buffer because they
 * are not allowed to allocate device memory at all -- e.g. a plugin inside a serving process that
 * froze its device-memory budget at start-up, or a latency-critical loop barred from the allocator.
 * The quantised activations go to a fixed array of SQ_STATIC_SCRATCH_BYTES that is part of the
 * library image (each GPU that loads the library holds it until the process exits); q->xq_dev /
 * q->xq_neg_dev are ignored.  DualScale is selected by q->sx_neg_dev != NULL and needs twice the
 * space: batch*M*K (x2) rounded up to 256 must fit, otherwise SQ_ERR_TOO_LARGE is returned and
 * nothing is launched.  The call itself allocates nothing (no cudaMalloc / cudaFree, no allocating
 * library routine).
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current); make that first call before starting any stream capture.  With the runtime's
 * lazy module loading that first call is also where the device reserves the array itself: if the
 * device cannot hold it the call returns SQ_ERR_CUDA and nothing is launched, so a process with a
 * frozen memory budget should make this first call while it still sets that budget up.
 * All calls share the one array, and it keeps whatever the last call left there: two calls whose GPU
 * work can overlap (different streams, or different host threads) race on it and must be ordered by
 * the caller.  Nothing in it needs to be cleared between calls.
 */
#define SQ_STATIC_SCRATCH_BYTES (64u * 1024u * 1024u)
int sq_seg_linear_static(const sq_act_quant_args* q, const sq_gemm_args* g, sq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SEGQUANT_B200_H */
