// Host side of the segmented quantised GEMM: argument validation, schedule choice, TMA descriptors
// and dispatch to the kernel translation units (seg_gemm_tu_*.cu; device code in seg_gemm_kernels.cuh).
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "seg_gemm_params.cuh"

namespace sq {

// skinny-M path (seg_gemv.cu)
bool gemv_applies(const sq_gemm_args* a, bool dual);
int launch_gemv(const GemmParams& p, const sq_gemm_args* a, bool dual, cudaStream_t st);

static int g_last_tu = 0;   // (kind * 2 + dual) of the last launch; the trace reader of -DSQ_TRACE builds uses it

#define SQ_FOR_EACH_TU(X) X(SQ_GEMM_W8A8_I8, false) X(SQ_GEMM_W8A8_I8, true) X(SQ_GEMM_W8A8_F8, false) X(SQ_GEMM_W8A8_F8, true) \
                          X(SQ_GEMM_W4A8, false) X(SQ_GEMM_W4A8, true)

long long push_read_status();   // peer_push.cu

long long read_device_status() {
    if (cudaDeviceSynchronize() != cudaSuccess) return SQ_ERR_CUDA;
    long long first = 0;
#define SQ_X(K, D)                                        \
    {                                                     \
        const long long v = tu_read_status<K, D>();       \
        if (v < 0) return v;                              \
        if (first == 0) first = v;                        \
    }
    SQ_FOR_EACH_TU(SQ_X)
#undef SQ_X
    {
        const long long v = push_read_status();   // the peer barrier's word (peer_push.cu)
        if (v < 0) return v;
        if (first == 0) first = v;
    }
    return first;
}

int wait_probe(long long limit_cycles, int* out_dev, cudaStream_t st) {
    SQ_REQUIRE(out_dev != nullptr, SQ_ERR_INVALID_ARG, "sq_wait_probe: out_dev is NULL");
    SQ_REQUIRE(limit_cycles > 0 && limit_cycles <= 100000000ll, SQ_ERR_INVALID_ARG,
               "sq_wait_probe: limit_cycles must lie in (0, 1e8] (the probe is meant to give up within milliseconds)");
    return tu_wait_probe<SQ_GEMM_W8A8_I8, false>(limit_cycles, out_dev, st);
}

int set_wait_limit(long long cycles);

#ifdef SQ_TRACE
extern "C" int sq_trace_read(long long* out, int n) {
    if (cudaDeviceSynchronize() != cudaSuccess) return SQ_ERR_CUDA;
#define SQ_X(K, D) \
    if (g_last_tu == static_cast<int>(K) * 2 + (D ? 1 : 0)) return tu_trace_read<K, D>(out, n);
    SQ_FOR_EACH_TU(SQ_X)
#undef SQ_X
    return SQ_ERR_INVALID_ARG;
}
#endif

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

// Encoded descriptors are cached by everything that goes into them: a layer that is called again with the same
// buffers (a serving loop, a CUDA-graph capture of many layers that share weights) pays a hash lookup instead of a
// driver call per operand.  A descriptor holds no reference to the memory, so a stale entry is harmless: the key
// includes the address and every extent.  Bounded: the table is emptied when it reaches kMapCacheMax entries.
struct MapKey {
    uint64_t v[9];
    bool operator==(const MapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = 1469598103934665603ull;
        for (uint64_t x : k.v) { h ^= x; h *= 1099511628211ull; }
        return static_cast<size_t>(h);
    }
};
constexpr size_t kMapCacheMax = 8192;
static std::mutex g_map_mutex;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash>& map_cache() {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> m;
    return m;
}

// 3-D uint8 tensor {inner bytes, rows, batch}.
static int make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t batch, uint64_t row_stride,
                    uint64_t batch_stride, uint32_t box_inner, uint32_t box_rows, bool swizzle128, const char* what) {
    const MapKey key{{reinterpret_cast<uint64_t>(base), inner, rows, batch, row_stride, batch_stride, box_inner, box_rows,
                      swizzle128 ? 1ull : 0ull}};
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        auto it = map_cache().find(key);
        if (it != map_cache().end()) { *map = it->second; return SQ_OK; }
    }
    auto fn = get_encode_fn();
    SQ_REQUIRE(fn != nullptr, SQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {inner, rows, batch};
    cuuint64_t strides[2] = {row_stride, batch_stride};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SQ_REQUIRE(r == CUDA_SUCCESS, SQ_ERR_CUDA,
               "cuTensorMapEncodeTiled(%s) failed with CUresult %d (dims %llu x %llu x %llu, strides %llu, %llu)", what,
               static_cast<int>(r), (unsigned long long)inner, (unsigned long long)rows, (unsigned long long)batch,
               (unsigned long long)row_stride, (unsigned long long)batch_stride);
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        if (map_cache().size() >= kMapCacheMax) map_cache().clear();
        map_cache().emplace(key, *map);
    }
    return SQ_OK;
}

// Process-wide schedule overrides (tuning and test aids).  The environment variables SEGQUANT_B200_BN=128|192|256,
// SEGQUANT_B200_CTA2=0|1, SEGQUANT_B200_KSUB=1|2 and SEGQUANT_B200_NO_GEMV=1 are read ONCE, on first use;
// sq_set_gemm_schedule() changes the choice afterwards.  0 / negative = automatic.
struct Overrides {
    int bn = 0;        // 128 / 192 / 256, 0 = automatic
    int cta2 = -1;     // 0 / 1, -1 = automatic
    int ksub = 0;      // 1 / 2, 0 = automatic
    int no_gemv = 0;   // 1: never take the skinny-M kernel
    long long wait_cycles = 4000000000ll;   // limit of every bounded wait inside the GEMM kernels (SM cycles)
};
static Overrides& overrides() {
    static Overrides ov = [] {
        Overrides o;
        if (const char* env = getenv("SEGQUANT_B200_BN")) {
            const int v = atoi(env);
            if (v == 128 || v == 192 || v == 256) o.bn = v;
        }
        if (const char* env = getenv("SEGQUANT_B200_CTA2")) o.cta2 = atoi(env) ? 1 : 0;
        if (const char* env = getenv("SEGQUANT_B200_KSUB")) o.ksub = atoi(env) == 1 ? 1 : (atoi(env) == 2 ? 2 : 0);
        if (const char* env = getenv("SEGQUANT_B200_NO_GEMV")) o.no_gemv = env[0] == '1' ? 1 : 0;
        return o;
    }();
    return ov;
}
int set_gemm_schedule(int bn, int two_cta, int ksub, int no_gemv) {
    SQ_REQUIRE(bn == 0 || bn == 128 || bn == 192 || bn == 256, SQ_ERR_INVALID_ARG, "sq_set_gemm_schedule: bn must be 0, 128, 192 or 256");
    SQ_REQUIRE(ksub >= 0 && ksub <= 2, SQ_ERR_INVALID_ARG, "sq_set_gemm_schedule: ksub must be 0, 1 or 2");
    Overrides& o = overrides();
    o.bn = bn;
    o.cta2 = two_cta < 0 ? -1 : (two_cta ? 1 : 0);
    o.ksub = ksub;
    o.no_gemv = no_gemv > 0 ? 1 : 0;
    return SQ_OK;
}
int set_wait_limit(long long cycles) {
    SQ_REQUIRE(cycles == 0 || (cycles >= 1000000ll && cycles <= 1000000000000ll), SQ_ERR_INVALID_ARG,
               "sq_set_wait_limit_cycles: 0 (default) or a value in [1e6, 1e12]");
    overrides().wait_cycles = cycles == 0 ? 4000000000ll : cycles;
    return SQ_OK;
}
int forced_ksub() { return overrides().ksub; }
long long wait_limit_cycles() { return overrides().wait_cycles; }
bool gemv_disabled() { return overrides().no_gemv != 0; }

// Schedule choice against wave quantisation.  The persistent grid runs ceil(tiles / slots) rounds
// (148 CTAs, or 74 CTA pairs each covering twice the rows); a round costs about (bn + fixed) per
// tile divided by the efficiency of the mode (a single CTA is limited by shared-memory bandwidth,
// see seg_gemm_2cta.cuh).  Narrow tiles re-read more operands, which the fixed term also stands for.
struct Schedule {
    int bn;
    bool two_cta;
};
static Schedule pick_schedule(long long M, long long N, long long K, long long batch, bool dual, int kind, bool no192 = false, int longest_unit = 1 << 30) {
    const int force_bn = overrides().bn, force_cta2 = overrides().cta2;
    const int widths[3] = {256, 192, 128};
    Schedule best{256, false};
    double best_cost = 1e300;
    const double nst = static_cast<double>((K + BK - 1) / BK);   // 128-byte K stages per tile
    for (int mode = 0; mode < 2; ++mode) {
        if (force_cta2 >= 0 && mode != force_cta2) continue;
        // measured on B200: the CTA pair wins once K is long enough to amortise its longer prologue.  Below K = 2048 the
        // two are within noise of each other in situ for 8-bit weights (8192 x 6144 x 1536 alone, operands L2-resident:
        // 64.6 us on pairs, 71.7 us on single CTAs; the same layers inside the MMDiT step: 0.1 ms per step slower on
        // pairs), so single CTAs stay; int4 weights gain from K = 1024 wherever there are two full rounds of pair tiles,
        // because each CTA expands only its half of the weight tile (4608 x 9216 x 1536: 64 us against 84 us; with
        // K = 3072: 103 us against 146 us).
        if (force_cta2 < 0 && mode == 1 && K < 2048) {
            const long long pair_tiles = batch * ((M + BM2 - 1) / BM2) * ((N + 255) / 256);
            if (kind != SQ_GEMM_W4A8 || K < 1024 || pair_tiles < 2 * (kNumSMs / 2)) continue;
        }
        // units of one or two K stages (weight-scale groups of 128 / 256): every unit is a hand-over between the issuing
        // thread and both CTAs' epilogues, and the layer is bound by its epilogue either way (measured: INT8 with groups of
        // 128 at 4608 x 9216 x 3072 takes 281-294 us on pairs, 284 us on single CTAs)
        // int4 weights are the exception: with 128-byte K stages (launch_2cta) a pair's CTAs expand half a tile each, and
        // the layer is 3-5 % faster than on single CTAs (groups of 128: 297 against 311 us at 4608 x 9216 x 3072, DualScale
        // 4608 x 3072 x 12288 759 against 783 us)
        const bool w4_short = kind == SQ_GEMM_W4A8 && longest_unit <= 256;
        if (force_cta2 < 0 && mode == 1 && longest_unit <= 256 && !w4_short) continue;
        if (force_cta2 < 0 && mode == 0 && w4_short) continue;
        const long long rows = mode ? BM2 : BM;
        const long long slots = mode ? kNumSMs / 2 : kNumSMs;
        for (int w : widths) {
            if (force_bn && w != force_bn) continue;
            if (no192 && w == 192) continue;
            // DualScale with units of one or two K stages: only 128-column tiles leave room for two accumulator pairs in
            // tensor memory, so that a unit's drain overlaps the next unit's MMAs (int4, groups of 128, 4608 x 3072 x 12288:
            // 783 us against 858 us with 256-column tiles)
            if (!force_bn && dual && longest_unit <= 256 && w > 128) continue;
            const long long tiles = batch * ((M + rows - 1) / rows) * ((N + w - 1) / w);
            const long long rounds = (tiles + slots - 1) / slots;
            // SM cycles, fitted to in-kernel timelines: a K stage costs the issuing thread a fixed ~500 cycles
            // (barrier wait, commit, issue) plus ~1.2 per tile column (twice with DualScale); a pair is ~17 % cheaper
            // per stage; every tile pays ~3400 cycles of prologue / hand-over, and a wide DualScale tile, whose two
            // accumulators fill tensor memory, also pays its un-overlapped drain and store
            double stage = 500.0 + 1.2 * w * (dual ? 2.0 : 1.0);
            if (mode) stage *= 0.83;
            const double fixed = 3400.0 + ((dual && w > 128) ? 4600.0 : 0.0);
            const double cost = static_cast<double>(rounds) * (nst * stage + fixed);
            if (cost < best_cost * 0.97) { best_cost = cost; best = Schedule{w, mode == 1}; }
        }
    }
    return best;
}

// longest accumulation unit (K elements) of a segment / group layout
static int max_unit_k(int num_segs, const int* seg_bounds, int group_size) {
    int longest = 0;
    for (int s = 0; s < num_segs; ++s) {
        int k = seg_bounds[s];
        const int e = seg_bounds[s + 1];
        while (k < e) {
            int ue = e;
            if (group_size > 0) {
                const int ge = (k / group_size + 1) * group_size;
                ue = ge < e ? ge : e;
            }
            longest = ue - k > longest ? ue - k : longest;
            k = ue;
        }
    }
    return longest;
}

int gemm_num_units(int num_segs, const int* seg_bounds, int group_size) {
    if (num_segs < 1 || num_segs > SQ_MAX_SEGS || seg_bounds == nullptr || group_size < 0) return SQ_ERR_INVALID_ARG;
    int units = 0;
    for (int s = 0; s < num_segs; ++s) {
        int k = seg_bounds[s];
        const int e = seg_bounds[s + 1];
        if (e <= k) return SQ_ERR_INVALID_ARG;
        while (k < e) {
            int ue = e;
            if (group_size > 0) {
                const int ge = (k / group_size + 1) * group_size;
                ue = ge < e ? ge : e;
            }
            ++units;
            k = ue;
        }
    }
    return units;
}

int gemm(const sq_gemm_args* a, cudaStream_t st) {
    SQ_REQUIRE(a != nullptr, SQ_ERR_INVALID_ARG, "sq_gemm: args is NULL");
    SQ_REQUIRE(a->kind == SQ_GEMM_W8A8_I8 || a->kind == SQ_GEMM_W8A8_F8 || a->kind == SQ_GEMM_W4A8, SQ_ERR_INVALID_ARG,
               "sq_gemm: unknown kind %d", a->kind);
    SQ_REQUIRE(a->out_dtype == SQ_F32 || a->out_dtype == SQ_F16 || a->out_dtype == SQ_BF16, SQ_ERR_INVALID_ARG,
               "sq_gemm: unknown out_dtype %d", a->out_dtype);
    SQ_REQUIRE(a->batch >= 0 && a->M >= 0 && a->N >= 0 && a->K >= 0, SQ_ERR_INVALID_ARG, "sq_gemm: negative size");
    if (a->batch == 0 || a->M == 0 || a->N == 0) return SQ_OK;
    SQ_REQUIRE(a->xq_dev && a->wq_dev && a->sx_dev && a->sw_dev && a->y_dev, SQ_ERR_INVALID_ARG, "sq_gemm: NULL operand pointer");
    const bool dual = a->xq_neg_dev != nullptr;
    SQ_REQUIRE(!dual || a->sx_neg_dev, SQ_ERR_INVALID_ARG, "sq_gemm: DualScale needs sx_neg_dev");
    SQ_REQUIRE(a->K > 0, SQ_ERR_INVALID_ARG, "sq_gemm: K must be positive");
    SQ_REQUIRE(a->K % 32 == 0, SQ_ERR_ALIGNMENT, "sq_gemm: K (%lld) must be divisible by 32", static_cast<long long>(a->K));
    SQ_REQUIRE(a->M < (1ll << 31) - BM && a->N < (1ll << 31) - BN && a->K < (1ll << 30) && a->batch < (1 << 20),
               SQ_ERR_TOO_LARGE, "sq_gemm: problem dimension too large");
    SQ_REQUIRE(a->num_segs >= 1 && a->num_segs <= SQ_MAX_SEGS, SQ_ERR_INVALID_ARG, "sq_gemm: num_segs %d outside [1, %d]",
               a->num_segs, SQ_MAX_SEGS);
    SQ_REQUIRE(a->seg_bounds[0] == 0 && a->seg_bounds[a->num_segs] == a->K, SQ_ERR_INVALID_ARG,
               "sq_gemm: seg_bounds must run from 0 to K");
    for (int s = 0; s < a->num_segs; ++s) {
        SQ_REQUIRE(a->seg_bounds[s + 1] > a->seg_bounds[s], SQ_ERR_INVALID_ARG, "sq_gemm: seg_bounds not increasing at %d", s);
        SQ_REQUIRE(a->seg_bounds[s + 1] % 32 == 0, SQ_ERR_ALIGNMENT, "sq_gemm: segment bound %d must be divisible by 32",
                   a->seg_bounds[s + 1]);
    }
    SQ_REQUIRE(a->group_size >= 0 && a->group_size % 32 == 0, SQ_ERR_ALIGNMENT, "sq_gemm: group_size %d must be a multiple of 32",
               a->group_size);
    const bool w4 = a->kind == SQ_GEMM_W4A8;
    auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    SQ_REQUIRE(aligned16(a->xq_dev) && (!dual || aligned16(a->xq_neg_dev)) && aligned16(a->wq_dev), SQ_ERR_ALIGNMENT,
               "sq_gemm: operand pointers must be 16-byte aligned");
    SQ_REQUIRE(a->xq_row_stride % 16 == 0 && a->xq_batch_stride % 16 == 0 && a->wq_row_stride % 16 == 0 &&
                   a->wq_batch_stride % 16 == 0,
               SQ_ERR_ALIGNMENT, "sq_gemm: operand strides must be multiples of 16 bytes");
    SQ_REQUIRE(a->xq_row_stride >= a->K && a->xq_batch_stride >= 0, SQ_ERR_INVALID_ARG, "sq_gemm: xq_row_stride smaller than K");

    long long w_k = a->K;  // K extent of one weight matrix
    long long w_batches = a->batch;
    if (a->w_seg_as_batch) {
        SQ_REQUIRE(a->batch == 1, SQ_ERR_INVALID_ARG, "sq_gemm: w_seg_as_batch needs batch == 1");
        const int len = a->seg_bounds[1];
        for (int s = 0; s < a->num_segs; ++s)
            SQ_REQUIRE(a->seg_bounds[s + 1] - a->seg_bounds[s] == len, SQ_ERR_UNSUPPORTED,
                       "sq_gemm: w_seg_as_batch needs equal segments (SegmentLinear.py:80-82)");
        w_k = len;
        w_batches = a->num_segs;
    }
    const long long w_row_bytes = w4 ? w_k / 2 : w_k;
    SQ_REQUIRE(a->wq_row_stride >= w_row_bytes, SQ_ERR_INVALID_ARG, "sq_gemm: wq_row_stride smaller than a weight row");

    const int units = gemm_num_units(a->num_segs, a->seg_bounds, a->group_size);
    SQ_REQUIRE(units > 0, SQ_ERR_INVALID_ARG, "sq_gemm: bad segment description");

    GemmParams p;
    p.M = a->M; p.N = a->N; p.K = a->K; p.batch = static_cast<int>(a->batch);
    p.num_segs = a->num_segs;
    for (int s = 0; s <= SQ_MAX_SEGS; ++s) p.seg_bounds[s] = s <= a->num_segs ? a->seg_bounds[s] : 0;
    p.group_size = a->group_size;
    p.w_seg_as_batch = a->w_seg_as_batch ? 1 : 0;
    p.a_batched = a->xq_batch_stride != 0 ? 1 : 0;
    p.sx = a->sx_dev; p.sx_neg = a->sx_neg_dev;
    p.sx_bs = a->sx_batch_stride; p.sx_ss = a->sx_seg_stride; p.sx_rs = a->sx_row_stride;
    p.sw = a->sw_dev; p.sw_is_bf16 = a->sw_is_bf16 ? 1 : 0;
    p.sw_bs = a->sw_batch_stride; p.sw_ss = a->sw_seg_stride; p.sw_gs = a->sw_group_stride; p.sw_cs = a->sw_col_stride;
    p.bias = a->bias_dev; p.bias_dtype = a->bias_dtype; p.bias_bs = a->bias_batch_stride;
    p.y = a->y_dev; p.out_dtype = a->out_dtype; p.y_bs = a->y_batch_stride; p.y_rs = a->y_row_stride;
    p.acc_dump = a->acc_dump_dev; p.units = units;
    p.n_peers = a->num_peer_outputs;
    p.peer_rs = a->peer_row_stride;
    p.peer_co = a->peer_col_offset;
    for (int j = 0; j < SQ_MAX_PEERS; ++j) p.peer_y[j] = j < a->num_peer_outputs ? a->peer_y_dev[j] : nullptr;
    if (a->num_peer_outputs != 0) {
        const long long pesz = a->out_dtype == SQ_F32 ? 4 : 2;
        SQ_REQUIRE(a->num_peer_outputs > 0 && a->num_peer_outputs <= SQ_MAX_PEERS, SQ_ERR_INVALID_ARG,
                   "sq_gemm: num_peer_outputs %d out of range", a->num_peer_outputs);
        SQ_REQUIRE(a->batch == 1, SQ_ERR_UNSUPPORTED, "sq_gemm: peer outputs need batch == 1");
        SQ_REQUIRE(a->acc_dump_dev == nullptr, SQ_ERR_UNSUPPORTED, "sq_gemm: peer outputs cannot be combined with acc_dump_dev");
        SQ_REQUIRE(a->peer_row_stride >= a->peer_col_offset + a->N && a->peer_col_offset >= 0, SQ_ERR_INVALID_ARG,
                   "sq_gemm: peer_row_stride / peer_col_offset do not hold N columns");
        SQ_REQUIRE((a->peer_row_stride * pesz) % 16 == 0 && (a->peer_col_offset * pesz) % 16 == 0 && (a->N * pesz) % 16 == 0,
                   SQ_ERR_ALIGNMENT, "sq_gemm: peer outputs need 16-byte aligned rows and column offset");
        for (int j = 0; j < a->num_peer_outputs; ++j)
            SQ_REQUIRE(a->peer_y_dev[j] != nullptr && reinterpret_cast<uintptr_t>(a->peer_y_dev[j]) % 16 == 0, SQ_ERR_INVALID_ARG,
                       "sq_gemm: peer_y_dev[%d] is NULL or not 16-byte aligned", j);
    }
    if (a->bias_dev)
        SQ_REQUIRE(a->bias_dtype == SQ_F32 || a->bias_dtype == SQ_F16 || a->bias_dtype == SQ_BF16, SQ_ERR_INVALID_ARG,
                   "sq_gemm: unknown bias_dtype %d", a->bias_dtype);
    p.wait_cycles = overrides().wait_cycles;
    // a handful of rows: stream the weights once on the CUDA cores instead of padding 128-row tensor-core tiles
    if (gemv_applies(a, dual)) return launch_gemv(p, a, dual, st);
    // Fused all-gather: stores to peers should be whole 128-byte lines ([16 rows x 128 bytes] boxes, see store_output).
    // That needs TMA-storable outputs and a tile whose per-warp column count is a multiple of the box (not 192 wide);
    // otherwise peers get the 16-column boxes of the plain store path.
    const long long oesz = a->out_dtype == SQ_F32 ? 4 : 2;
    const bool y_tma_ok = (reinterpret_cast<uintptr_t>(a->y_dev) & 15u) == 0 && (a->y_row_stride * oesz) % 16 == 0 &&
                          a->y_row_stride >= a->N;
    const bool want_wide = a->num_peer_outputs > 0 && y_tma_ok && overrides().bn != 192;
    const int longest_unit = max_unit_k(a->num_segs, a->seg_bounds, a->group_size);
    const Schedule sched = pick_schedule(a->M, a->N, a->K, a->batch, dual, a->kind, want_wide, longest_unit);
    p.peer_wide = want_wide ? 1 : 0;
    p.short_units = longest_unit <= 256 ? 1 : 0;
    const int tile_rows = sched.two_cta ? BM2 : BM;
    p.tiles_m = static_cast<int>((a->M + tile_rows - 1) / tile_rows);
    p.bn = sched.bn;
    p.dual_db = (dual && p.bn <= 128) ? 1 : 0;
    // short units of an integer kind: accumulators start from a magic bit pattern and are read as floats (seg_gemm_kernels.cuh);
    // the dump (tests) and peer-store variants of the epilogue use plain conversions on accumulators that start from zero
    p.all_magic = (a->kind != SQ_GEMM_W8A8_F8 && a->acc_dump_dev == nullptr && a->num_peer_outputs == 0 &&
                   longest_unit <= 224) ? 1 : 0;
    p.tiles_n = static_cast<int>((a->N + p.bn - 1) / p.bn);
    p.total_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * a->batch;

    CUtensorMap ma, man, mw;
    const uint64_t a_batches = p.a_batched ? a->batch : 1;
    const uint64_t a_bstride = p.a_batched ? a->xq_batch_stride : static_cast<uint64_t>(a->xq_row_stride) * a->M;
    int rc = make_map(&ma, a->xq_dev, a->K, a->M, a_batches, a->xq_row_stride, a_bstride, BK, BM, true, "xq");
    if (rc != SQ_OK) return rc;
    man = ma;
    if (dual) {
        rc = make_map(&man, a->xq_neg_dev, a->K, a->M, a_batches, a->xq_row_stride, a_bstride, BK, BM, true, "xq_neg");
        if (rc != SQ_OK) return rc;
    }
    const uint64_t w_bstride = (w_batches > 1 && a->wq_batch_stride != 0) ? a->wq_batch_stride
                                                                         : static_cast<uint64_t>(a->wq_row_stride) * a->N;
    const uint64_t w_nb = (w_batches > 1 && a->wq_batch_stride != 0) ? w_batches : 1;
    SQ_REQUIRE(w_nb == static_cast<uint64_t>(w_batches) || !a->w_seg_as_batch, SQ_ERR_INVALID_ARG,
               "sq_gemm: w_seg_as_batch needs a non-zero wq_batch_stride");
    p.w_batched = (w_nb > 1 && !a->w_seg_as_batch) ? 1 : 0;   // wq_batch_stride == 0: one weight matrix for all problems
    // output: TMA stores need a 16-byte aligned base and strides; anything else is written by the threads
    OutMaps my;
    my.y = ma;
    for (int j = 0; j < SQ_MAX_PEERS; ++j) my.peer[j] = ma;
    p.peer_tma = 0;
    {
        const long long esz = a->out_dtype == SQ_F32 ? 4 : 2;
        const bool aligned = (reinterpret_cast<uintptr_t>(a->y_dev) & 15u) == 0 && (a->y_row_stride * esz) % 16 == 0 &&
                             a->y_row_stride >= a->N && (a->batch == 1 || ((a->y_batch_stride * esz) % 16 == 0 && a->y_batch_stride > 0));
        p.y_tma = 0;
        if (aligned) {
            const uint64_t y_bstride = a->batch > 1 ? a->y_batch_stride * esz : static_cast<uint64_t>(a->y_row_stride) * esz * a->M;
            // box: [32 rows x 16 columns], or with wide peer stores [16 rows x 128 bytes] read from a swizzled staging area
            const uint32_t box_bytes = p.peer_wide ? 128u : static_cast<uint32_t>(16 * esz);
            const uint32_t box_rows = p.peer_wide ? 16u : 32u;
            const bool box_swz = p.peer_wide != 0;
            rc = make_map(&my.y, a->y_dev, a->N * esz, a->M, a->batch, a->y_row_stride * esz, y_bstride, box_bytes, box_rows, box_swz, "y");
            if (rc != SQ_OK) return rc;
            p.y_tma = 1;
            // peers: the map starts at their column offset, so the kernel uses the coordinates of y
            for (int j = 0; j < a->num_peer_outputs; ++j) {
                const uint8_t* base = static_cast<const uint8_t*>(a->peer_y_dev[j]) + a->peer_col_offset * esz;
                rc = make_map(&my.peer[j], base, a->N * esz, a->M, 1, a->peer_row_stride * esz,
                              static_cast<uint64_t>(a->peer_row_stride) * esz * a->M, box_bytes, box_rows, box_swz, "peer_y");
                if (rc != SQ_OK) return rc;
            }
            p.peer_tma = a->num_peer_outputs > 0 ? 1 : 0;
        }
    }
    if (!p.y_tma) p.peer_wide = 0;
    // B tile rows staged per CTA: the whole tile, or half of it in a CTA pair
    const uint32_t w_box_rows = sched.two_cta ? p.bn / 2 : p.bn;
    if (w4) rc = make_map(&mw, a->wq_dev, w_row_bytes, a->N, w_nb, a->wq_row_stride, w_bstride, BK / 2, w_box_rows, false, "wq(int4)");
    else rc = make_map(&mw, a->wq_dev, w_row_bytes, a->N, w_nb, a->wq_row_stride, w_bstride, BK, w_box_rows, true, "wq");
    if (rc != SQ_OK) return rc;

    g_last_tu = a->kind * 2 + (dual ? 1 : 0);
    switch (a->kind) {
        case SQ_GEMM_W8A8_I8:
            return dual ? launch_gemm<SQ_GEMM_W8A8_I8, true>(sched.two_cta, ma, man, mw, my, p, st)
                        : launch_gemm<SQ_GEMM_W8A8_I8, false>(sched.two_cta, ma, man, mw, my, p, st);
        case SQ_GEMM_W8A8_F8:
            return dual ? launch_gemm<SQ_GEMM_W8A8_F8, true>(sched.two_cta, ma, man, mw, my, p, st)
                        : launch_gemm<SQ_GEMM_W8A8_F8, false>(sched.two_cta, ma, man, mw, my, p, st);
        default:
            return dual ? launch_gemm<SQ_GEMM_W4A8, true>(sched.two_cta, ma, man, mw, my, p, st)
                        : launch_gemm<SQ_GEMM_W4A8, false>(sched.two_cta, ma, man, mw, my, p, st);
    }
}

}  // namespace sq
