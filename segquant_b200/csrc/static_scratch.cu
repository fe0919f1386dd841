// sq_seg_linear_static: the fused layer forward for callers that must not allocate device memory.
//
// sq_seg_linear needs a scratch buffer for the quantised activation bytes (batch*M*K bytes, twice
// that with DualScale) and expects the caller to bring it.  Some callers cannot: a plugin loaded
// into a serving process that fixed its device-memory budget at start-up and forbids any later
// cudaMalloc (an allocation there synchronises the device and stalls every other tenant), or a
// latency-critical decode loop that is simply not allowed to touch an allocator.  For them the
// scratch lives in the array below, which is part of the library image: every GPU that loads the
// library holds SQ_STATIC_SCRATCH_BYTES of it until the process exits.
//
// This entry point has no counterpart in the reference, whose host pipeline allocates its
// scratch tensors on every call (segquant/src/real_quant/real_gemm.cu:694-696, :714-715).
#include <mutex>

#include "common.cuh"

namespace sq {
int quantize_act(const sq_act_quant_args* a, cudaStream_t st);
int gemm(const sq_gemm_args* a, cudaStream_t st);
}  // namespace sq

// The scratch itself.  In host code this name is only a handle for the runtime, not a device
// address: the address a kernel can use is obtained once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[SQ_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_dev[kMaxDevices] = {};  // device address of g_static_scratch, per device

// Set-up, once per device, with that device current.  Returns nullptr (and sets the error) on failure.
unsigned char* scratch_for_current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        sq::set_error("sq_seg_linear_static: cannot identify the current device (%s)", cudaGetErrorString(e));
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_dev[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            sq::set_error("sq_seg_linear_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return nullptr;
        }
        g_scratch_dev[dev] = static_cast<unsigned char*>(ptr);
    }
    return g_scratch_dev[dev];
}

}  // namespace

extern "C" int sq_seg_linear_static(const sq_act_quant_args* q, const sq_gemm_args* g, sq_stream_t stream) {
    sq::clear_error();
    if (q == nullptr || g == nullptr) {
        sq::set_error("sq_seg_linear_static: NULL argument block");
        return SQ_ERR_INVALID_ARG;
    }
    if (q->batch != g->batch || q->M != g->M || q->K != g->K || q->batch < 0 || q->M < 0 || q->K < 0) {
        sq::set_error("sq_seg_linear_static: quantise and GEMM blocks disagree on batch/M/K");
        return SQ_ERR_INVALID_ARG;
    }
    const bool dual = q->sx_neg_dev != nullptr;
    if (dual != (g->sx_neg_dev != nullptr)) {
        sq::set_error("sq_seg_linear_static: DualScale must be set in both argument blocks (sx_neg_dev)");
        return SQ_ERR_INVALID_ARG;
    }
    // one quantised tensor (two with DualScale), each rounded up to the array's 256-byte alignment
    const unsigned long long one = (static_cast<unsigned long long>(q->batch) * q->M * q->K + 255ull) & ~255ull;
    const unsigned long long need = one * (dual ? 2ull : 1ull);
    if (need > SQ_STATIC_SCRATCH_BYTES) {
        sq::set_error("sq_seg_linear_static: batch*M*K%s = %llu bytes of scratch exceed the built-in %llu bytes; "
                      "use sq_seg_linear with a caller-provided buffer",
                      dual ? " (x2 for DualScale)" : "", need, static_cast<unsigned long long>(SQ_STATIC_SCRATCH_BYTES));
        return SQ_ERR_TOO_LARGE;
    }
    unsigned char* scratch = scratch_for_current_device();
    if (scratch == nullptr) return SQ_ERR_CUDA;

    // Nothing in the scratch has to start at zero: the quantise kernel overwrites every byte the GEMM
    // reads, and rows beyond M are zero-filled by the TMA unit from the tensor map's bounds.
    sq_act_quant_args qq = *q;
    qq.xq_dev = scratch;
    qq.xq_neg_dev = dual ? scratch + one : nullptr;
    qq.xq_batch_stride = q->M * q->K;
    qq.xq_row_stride = q->K;
    int rc = sq::quantize_act(&qq, static_cast<cudaStream_t>(stream));
    if (rc != SQ_OK) return rc;
    sq_gemm_args gg = *g;
    gg.xq_dev = qq.xq_dev;
    gg.xq_neg_dev = qq.xq_neg_dev;
    gg.xq_batch_stride = q->batch > 1 ? qq.xq_batch_stride : 0;
    gg.xq_row_stride = qq.xq_row_stride;
    return sq::gemm(&gg, static_cast<cudaStream_t>(stream));
}
