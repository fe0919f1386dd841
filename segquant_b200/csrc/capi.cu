// extern "C" surface of libsegquant_b200.so (declared in include/segquant_b200.h).
// No torch types: plain pointers, sizes, a cudaStream_t.  Each function maps onto one host
// pipeline of the reference's native layer (see the header for file:line).
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace sq {

static thread_local char g_err[512] = {0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
void clear_error() { g_err[0] = 0; }

// implemented in act_quant.cu / weight_quant.cu / seg_gemm.cu
int quantize_act(const sq_act_quant_args* a, cudaStream_t st);
int quantize_act_dynamic(const sq_act_quant_args* a, float* sx_out, float* sx_neg_out, cudaStream_t st);
int norm_quantize_act(const sq_act_quant_args* a, const void* shift, const void* scale, long long mod_bs, float eps,
                      const sq_norm_residual* r, cudaStream_t st);
int gated_residual(const sq_gated_residual_args* a, cudaStream_t st);
int quantize_weight(const void* w, int w_dtype, long long N, long long K, int scale_mode, float scale_scalar,
                    const float* scale, int group_size, int out_kind, void* out, cudaStream_t st);
int unpack_int4(const void* packed, void* out, long long numel, cudaStream_t st);
int gemm(const sq_gemm_args* a, cudaStream_t st);
int gemm_num_units(int num_segs, const int* seg_bounds, int group_size);
long long read_device_status();
int set_gemm_schedule(int bn, int two_cta, int ksub, int no_gemv);
int set_wait_limit(long long cycles);
int wait_probe(long long limit_cycles, int* out_dev, cudaStream_t st);
int push_columns(const void* src, long long rows, long long width_bytes, long long src_row_stride, int n_peers,
                 void* const* peer_dst, long long dst_row_stride, cudaStream_t st);
int peer_barrier(int rank, int world, void* const* flags, unsigned epoch, cudaStream_t st);

}  // namespace sq

extern "C" {

int sq_version(void) { return SQ_VERSION; }

const char* sq_last_error(void) { return sq::g_err; }

const char* sq_status_string(int status) {
    switch (status) {
        case SQ_OK: return "SQ_OK";
        case SQ_ERR_INVALID_ARG: return "SQ_ERR_INVALID_ARG";
        case SQ_ERR_ALIGNMENT: return "SQ_ERR_ALIGNMENT";
        case SQ_ERR_UNSUPPORTED: return "SQ_ERR_UNSUPPORTED";
        case SQ_ERR_CUDA: return "SQ_ERR_CUDA";
        case SQ_ERR_DEVICE_TIMEOUT: return "SQ_ERR_DEVICE_TIMEOUT";
        case SQ_ERR_TOO_LARGE: return "SQ_ERR_TOO_LARGE";
        default: return "SQ_ERR_UNKNOWN";
    }
}

int64_t sq_device_status(void) {
    sq::clear_error();
    const long long v = sq::read_device_status();
    if (v < 0) sq::set_error("sq_device_status: the device could not be queried");
    return v;
}

int sq_check_device(void) {
    sq::clear_error();
    const long long v = sq::read_device_status();
    if (v < 0) {
        sq::set_error("sq_check_device: the device could not be queried");
        return SQ_ERR_CUDA;
    }
    if (v != 0) {
        sq::set_error("a bounded wait inside a kernel ran out: block %lld, wait id %lld (status word 0x%llx); the launch that "
                      "reported it returned without completing its output", v >> 8, v & 0xff, static_cast<unsigned long long>(v));
        return SQ_ERR_DEVICE_TIMEOUT;
    }
    return SQ_OK;
}

int sq_set_gemm_schedule(int32_t bn, int32_t two_cta, int32_t ksub, int32_t no_gemv) {
    sq::clear_error();
    return sq::set_gemm_schedule(bn, two_cta, ksub, no_gemv);
}

int sq_set_wait_limit_cycles(int64_t cycles) {
    sq::clear_error();
    return sq::set_wait_limit(cycles);
}

int sq_wait_probe(int64_t limit_cycles, int32_t* out_dev, sq_stream_t stream) {
    sq::clear_error();
    return sq::wait_probe(limit_cycles, out_dev, static_cast<cudaStream_t>(stream));
}

int sq_quantize_act(const sq_act_quant_args* args, sq_stream_t stream) {
    sq::clear_error();
    return sq::quantize_act(args, static_cast<cudaStream_t>(stream));
}

int sq_quantize_act_dynamic(const sq_act_quant_args* args, float* sx_out_dev, float* sx_neg_out_dev, sq_stream_t stream) {
    sq::clear_error();
    return sq::quantize_act_dynamic(args, sx_out_dev, sx_neg_out_dev, static_cast<cudaStream_t>(stream));
}

int sq_norm_quantize_act(const sq_act_quant_args* args, const void* shift_dev, const void* scale_dev, int64_t mod_batch_stride,
                         float eps, sq_stream_t stream) {
    sq::clear_error();
    return sq::norm_quantize_act(args, shift_dev, scale_dev, mod_batch_stride, eps, nullptr, static_cast<cudaStream_t>(stream));
}

int sq_residual_norm_quantize_act(const sq_act_quant_args* args, const void* shift_dev, const void* scale_dev, int64_t mod_batch_stride,
                                  float eps, const sq_norm_residual* residual, sq_stream_t stream) {
    sq::clear_error();
    return sq::norm_quantize_act(args, shift_dev, scale_dev, mod_batch_stride, eps, residual, static_cast<cudaStream_t>(stream));
}

int sq_gated_residual(const sq_gated_residual_args* args, sq_stream_t stream) {
    sq::clear_error();
    return sq::gated_residual(args, static_cast<cudaStream_t>(stream));
}

int sq_quantize_weight(const void* w_dev, int32_t w_dtype, int64_t N, int64_t K, int32_t scale_mode, float scale_scalar,
                       const float* scale_dev, int32_t group_size, int32_t out_kind, void* out_dev, sq_stream_t stream) {
    sq::clear_error();
    return sq::quantize_weight(w_dev, w_dtype, N, K, scale_mode, scale_scalar, scale_dev, group_size, out_kind, out_dev,
                               static_cast<cudaStream_t>(stream));
}

int sq_unpack_int4(const void* packed_dev, void* out_dev, int64_t numel, sq_stream_t stream) {
    sq::clear_error();
    return sq::unpack_int4(packed_dev, out_dev, numel, static_cast<cudaStream_t>(stream));
}

int sq_gemm(const sq_gemm_args* args, sq_stream_t stream) {
    sq::clear_error();
    return sq::gemm(args, static_cast<cudaStream_t>(stream));
}

int sq_push_columns(const void* src_dev, int64_t rows, int64_t width_bytes, int64_t src_row_stride_bytes, int32_t num_peers,
                    void* const* peer_dst_dev, int64_t dst_row_stride_bytes, sq_stream_t stream) {
    sq::clear_error();
    return sq::push_columns(src_dev, rows, width_bytes, src_row_stride_bytes, num_peers, peer_dst_dev, dst_row_stride_bytes,
                            static_cast<cudaStream_t>(stream));
}

int sq_peer_barrier(int32_t rank, int32_t world, void* const* flags_dev, uint32_t epoch, sq_stream_t stream) {
    sq::clear_error();
    return sq::peer_barrier(rank, world, flags_dev, epoch, static_cast<cudaStream_t>(stream));
}

int sq_gemm_num_units(int32_t num_segs, const int32_t* seg_bounds, int32_t group_size) {
    return sq::gemm_num_units(num_segs, seg_bounds, group_size);
}

int sq_seg_linear(const sq_act_quant_args* q, const sq_gemm_args* g, sq_stream_t stream) {
    sq::clear_error();
    if (q == nullptr || g == nullptr) {
        sq::set_error("sq_seg_linear: NULL argument block");
        return SQ_ERR_INVALID_ARG;
    }
    if (q->batch != g->batch || q->M != g->M || q->K != g->K) {
        sq::set_error("sq_seg_linear: quantise and GEMM blocks disagree on batch/M/K");
        return SQ_ERR_INVALID_ARG;
    }
    int rc = sq::quantize_act(q, static_cast<cudaStream_t>(stream));
    if (rc != SQ_OK) return rc;
    sq_gemm_args gg = *g;
    gg.xq_dev = q->xq_dev;
    gg.xq_neg_dev = q->xq_neg_dev;
    gg.xq_batch_stride = q->xq_batch_stride;
    gg.xq_row_stride = q->xq_row_stride;
    return sq::gemm(&gg, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
