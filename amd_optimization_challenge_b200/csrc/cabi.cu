// extern "C" boundary of libb200mla.so: argument validation, workspace layout, kernel selection
// and launches.  Declarations and the reference interfaces they replace: include/b200_mla.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/b200_mla.h"
#include "mla_common.cuh"

namespace b200mla {
cudaError_t launch_generic(const MlaParams& p, cudaStream_t stream);
size_t generic_smem_bytes(int batch);
cudaError_t launch_sm100(const MlaParams& p, int* status, cudaStream_t stream);
bool sm100_supported(const MlaParams& p);
int sm100_rows_per_cta(const MlaParams& p);
int sm100_tile_tokens(const MlaParams& p);
cudaError_t launch_sm100x(const MlaParams& p, int* status, cudaStream_t stream);
bool sm100x_supported(const MlaParams& p);
int sm100x_rows_per_cta(const MlaParams& p);
long long sm100x_q_split_bytes(int batch, int rows);
long long sm100x_q_scale_bytes(int batch, int rows);
cudaError_t launch_combine_spans(const MlaParams& p, cudaStream_t stream);
cudaError_t launch_combine_parts(const float* o_parts, const float* lse_parts, int parts, long long rows,
                                 long long o_stride, long long lse_stride, __nv_bfloat16* out, float* out_lse,
                                 cudaStream_t stream);
cudaError_t launch_quantize_fp8(const __nv_bfloat16* x, long long n, uint8_t* out, float* scale_out,
                                unsigned int* scratch, cudaStream_t stream);
cudaError_t launch_kv_append(const void* src, long long n, long long src_stride, const int* slots, long long base_slot,
                             long long num_slots, int kv_format, void* codes, long long codes_stride, void* bs,
                             long long bs_stride, void* rope, long long rope_stride, const float* scale, int* bad,
                             cudaStream_t stream);
long long peer_part_bytes(long long rows);
long long peer_exchange_bytes(long long rows);
long long peer_partial_offset(long long rows, unsigned int epoch);
cudaError_t launch_peer_merge(const void* const* bases, int world, int rank, unsigned int epoch, unsigned long long limit_ns,
                              long long rows, void* out, int* status, cudaStream_t stream);
cudaError_t launch_q_amax_parts(const __nv_bfloat16* x, long long n, unsigned int* parts, cudaStream_t stream);
}  // namespace b200mla

using namespace b200mla;

namespace {

thread_local char g_err[512] = "";
thread_local cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

constexpr int kMaxCtasPerSm = 2;
inline long long align256(long long x) { return (x + 255) & ~255LL; }

// workspace: [status word | tile prefix | split-Q scales | split-Q planes | partial LSE | partial O]
struct WsLayout { long long status_off, prefix_off, qscale_off, qsplit_off, lse_off, o_off, total; };

WsLayout ws_layout(int batch, int rows, int g_max) {
    WsLayout L;
    const long long slots = (long long)g_max + batch;
    L.status_off = 0;
    L.prefix_off = 256;
    L.qscale_off = L.prefix_off + align256((long long)(batch + 1) * 4);
    L.qsplit_off = L.qscale_off + align256(sm100x_q_scale_bytes(batch, rows));
    L.lse_off = L.qsplit_off + align256(sm100x_q_split_bytes(batch, rows));
    L.o_off = L.lse_off + align256(slots * rows * 4);
    L.total = L.o_off + align256(slots * rows * (long long)V_DIM * 4);
    return L;
}

}  // namespace

extern "C" {

int32_t b200_mla_version(void) { return 1000; }

const char* b200_mla_last_error(void) { return g_err; }

int64_t b200_mla_workspace_bytes(int32_t batch, int32_t heads, int32_t q_len) {
    if (batch <= 0 || heads <= 0 || q_len <= 0) return 0;
    return ws_layout(batch, heads * q_len, kMaxCtasPerSm * sm_count()).total;
}

int32_t b200_mla_decode(const b200_mla_decode_args* a, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!a) return fail(B200_MLA_ERR_INVALID_ARG, "args is NULL");
    if (a->batch <= 0 || a->heads <= 0 || a->q_len <= 0)
        return fail(B200_MLA_ERR_INVALID_ARG, "batch/heads/q_len must be positive (got %d/%d/%d)", a->batch, a->heads, a->q_len);
    if (a->batch > MAX_BATCH) return fail(B200_MLA_ERR_TOO_LARGE, "batch %d exceeds %d", a->batch, MAX_BATCH);
    if (a->heads % 16 != 0) return fail(B200_MLA_ERR_UNSUPPORTED, "heads must be a multiple of 16 (got %d)", a->heads);
    if (a->q_len > 8) return fail(B200_MLA_ERR_UNSUPPORTED, "q_len > 8 is not a decode shape (got %d)", a->q_len);
    if (a->q_format < B200_MLA_Q_BF16 || a->q_format > B200_MLA_Q_BF16_CAST_E4M3)
        return fail(B200_MLA_ERR_INVALID_ARG, "bad q_format %d", a->q_format);
    if (a->kv_format < B200_MLA_KV_E4M3 || a->kv_format > B200_MLA_KV_HYBRID)
        return fail(B200_MLA_ERR_INVALID_ARG, "bad kv_format %d", a->kv_format);
    if (!a->q || !a->kv_codes || !a->kv_indptr) return fail(B200_MLA_ERR_INVALID_ARG, "q, kv_codes and kv_indptr are required");
    if (a->q_format != B200_MLA_Q_BF16 && !a->q_scale)
        return fail(B200_MLA_ERR_INVALID_ARG, "q_scale is required for e4m3 Q (the scale, or the amax partials when Q is cast on load)");
    if ((a->kv_format == B200_MLA_KV_E4M3 || a->kv_format == B200_MLA_KV_HYBRID) && !a->kv_scale)
        return fail(B200_MLA_ERR_INVALID_ARG, "kv_scale is required for e4m3 / hybrid caches");
    if (a->kv_format != B200_MLA_KV_E4M3 && !a->kv_block_scales)
        return fail(B200_MLA_ERR_INVALID_ARG, "kv_block_scales is required for mxfp4 / hybrid caches");
    if (a->kv_format == B200_MLA_KV_HYBRID && !a->kv_rope) return fail(B200_MLA_ERR_INVALID_ARG, "kv_rope is required for hybrid caches");
    if (a->q_row_stride % 16 || a->q_head_stride % 16) return fail(B200_MLA_ERR_INVALID_ARG, "Q strides must be multiples of 16 elements");
    if (a->kv_codes_stride % 16 || ((uintptr_t)a->kv_codes & 15)) return fail(B200_MLA_ERR_INVALID_ARG, "kv_codes must be 16-byte aligned with a stride multiple of 16");
    if (a->kv_format == B200_MLA_KV_HYBRID && (a->kv_rope_stride % 16 || ((uintptr_t)a->kv_rope & 15)))
        return fail(B200_MLA_ERR_INVALID_ARG, "kv_rope must be 16-byte aligned with a stride multiple of 16");
    if ((uintptr_t)a->q & 15) return fail(B200_MLA_ERR_INVALID_ARG, "q must be 16-byte aligned");
    if (a->page_size < 1) return fail(B200_MLA_ERR_INVALID_ARG, "page_size must be >= 1");
    if (a->page_size > 1 && a->kv_indices && !a->kv_page_indptr)
        return fail(B200_MLA_ERR_INVALID_ARG, "kv_page_indptr is required when page_size > 1");
    if (!a->out && !a->out_o_f32) return fail(B200_MLA_ERR_INVALID_ARG, "one of out / out_o_f32 is required");
    if (!a->workspace || ((uintptr_t)a->workspace & 255)) return fail(B200_MLA_ERR_INVALID_ARG, "workspace must be non-NULL and 256-byte aligned");
    if (a->num_slots <= 0) return fail(B200_MLA_ERR_INVALID_ARG, "num_slots (rows of the cache planes) must be positive: page ids are checked against it");

    MlaParams p;
    memset(&p, 0, sizeof(p));
    p.batch = a->batch; p.heads = a->heads; p.q_len = a->q_len; p.rows = a->heads * a->q_len;
    // bf16 Q cast on load: for every kernel that is an e4m3 Q whose bytes are made while they are loaded
    p.q_cast = a->q_format == B200_MLA_Q_BF16_CAST_E4M3 ? 1 : 0;
    p.q_amax_parts = p.q_cast ? reinterpret_cast<const unsigned int*>(a->q_scale) : nullptr;
    p.q_format = p.q_cast ? (int)Q_E4M3 : a->q_format; p.kv_format = a->kv_format; p.causal = a->causal ? 1 : 0; p.page_size = a->page_size;
    p.sm_scale = a->sm_scale;
    p.q = a->q; p.q_row_stride = a->q_row_stride; p.q_head_stride = a->q_head_stride; p.q_scale = p.q_cast ? nullptr : a->q_scale;
    p.kv_codes = (const uint8_t*)a->kv_codes; p.kv_codes_stride = a->kv_codes_stride;
    p.kv_bs = (const uint8_t*)a->kv_block_scales; p.kv_bs_stride = a->kv_block_scales_stride;
    p.kv_rope = (const uint8_t*)a->kv_rope; p.kv_rope_stride = a->kv_rope_stride;
    p.kv_scale = a->kv_scale; p.num_slots = a->num_slots; p.total_kv_hint = a->total_kv_hint > 0 ? a->total_kv_hint : 0;
    p.last_slot = (unsigned int)((a->num_slots < 0x80000000LL ? a->num_slots : 0x80000000LL) - 1);
    p.kv_indptr = a->kv_indptr; p.kv_indices = a->kv_indices; p.kv_page_indptr = a->kv_page_indptr;
    p.kv_pos_offset = a->kv_pos_offset; p.kv_total_len = a->kv_total_len;
    p.out = (__nv_bfloat16*)a->out; p.out_o_f32 = a->out_o_f32; p.out_lse = a->out_lse;

    const int sms = sm_count();
    // two tcgen05 kernels: the plain one for e4m3 Q x e4m3 cache, the transforming one for every other pair
    const bool plain = sm100_supported(p), xform = !plain && sm100x_supported(p);
    bool use_sm100 = false;
    if (a->impl == B200_MLA_IMPL_TCGEN05) {
        if (!plain && !xform) return fail(B200_MLA_ERR_UNSUPPORTED, "the tcgen05 kernels do not cover this shape");
        use_sm100 = true;
    } else if (a->impl == B200_MLA_IMPL_AUTO) {
        use_sm100 = plain || xform;
    } else if (a->impl != B200_MLA_IMPL_GENERIC) {
        return fail(B200_MLA_ERR_INVALID_ARG, "bad impl %d", a->impl);
    }

    int ctas_per_sm;
    if (use_sm100) {
        p.tile_tokens = plain ? sm100_tile_tokens(p) : 128;
        p.rows_per_cta = plain ? sm100_rows_per_cta(p) : sm100x_rows_per_cta(p);
        ctas_per_sm = 1;
    }
    else { p.tile_tokens = 64; p.rows_per_cta = 16; ctas_per_sm = 2; }
    const int groups = p.rows / p.rows_per_cta;
    const long long hint = a->total_kv_hint > 0 ? a->total_kv_hint : a->num_slots;
    const long long tiles_bound = (hint + p.tile_tokens - 1) / p.tile_tokens + a->batch;
    long long G = (long long)ctas_per_sm * sms / groups;
    if (G < 1) G = 1;
    if (G > tiles_bound) G = tiles_bound;
    if (a->max_ctas > 0 && G > a->max_ctas) G = a->max_ctas;
    p.num_ctas = (int)G;

    const WsLayout L = ws_layout(a->batch, p.rows, kMaxCtasPerSm * sms);
    if (a->workspace_bytes < L.total)
        return fail(B200_MLA_ERR_WORKSPACE, "workspace of %lld bytes is smaller than the %lld required", (long long)a->workspace_bytes, L.total);
    char* ws = (char*)a->workspace;
    p.status = (int*)(ws + L.status_off);
    p.tile_prefix = (int*)(ws + L.prefix_off);
    p.part_lse = (float*)(ws + L.lse_off);
    p.part_o = (float*)(ws + L.o_off);
    p.q_split_scale = (float*)(ws + L.qscale_off);
    p.q_split = (uint8_t*)(ws + L.qsplit_off);

    const bool prof = g_ev_start && g_ev_stop;
    if (prof) cudaEventRecord(g_ev_start, stream);
    cudaError_t e = !use_sm100 ? launch_generic(p, stream)
                    : plain    ? launch_sm100(p, (int*)(ws + L.status_off), stream)
                               : launch_sm100x(p, (int*)(ws + L.status_off), stream);
    if (prof) cudaEventRecord(g_ev_stop, stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "stage-1 launch failed: %s", cudaGetErrorString(e));
    e = launch_combine_spans(p, stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "combine launch failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

}  // extern "C"

// Scratch of the allocation-free entry point: lives in the library image, one copy per GPU.
static __device__ __align__(256) unsigned char g_static_workspace[B200_MLA_STATIC_WORKSPACE_BYTES];

// Device address of the built-in scratch on the current device.  In host code the array's name is
// only a handle; its device address is looked up once per device, with that device current.
static int static_workspace_ptr(void** out) {
    constexpr int kMaxDevices = 64;
    static void* dev_ptr[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(B200_MLA_ERR_UNSUPPORTED, "device ordinal %d is beyond %d", dev, kMaxDevices);
    void* ptr = __atomic_load_n(&dev_ptr[dev], __ATOMIC_ACQUIRE);
    if (!ptr) {
        e = cudaGetSymbolAddress(&ptr, g_static_workspace);
        if (e != cudaSuccess || !ptr)
            return fail(B200_MLA_ERR_CUDA, "cudaGetSymbolAddress(static workspace) failed: %s", cudaGetErrorString(e));
        __atomic_store_n(&dev_ptr[dev], ptr, __ATOMIC_RELEASE);
    }
    *out = ptr;
    return B200_MLA_OK;
}

extern "C" {

int32_t b200_mla_decode_static(const b200_mla_decode_args* args, void* stream) {
    if (!args) return fail(B200_MLA_ERR_INVALID_ARG, "args is NULL");
    if (args->batch <= 0 || args->heads <= 0 || args->q_len <= 0)
        return fail(B200_MLA_ERR_INVALID_ARG, "batch/heads/q_len must be positive");
    const long long need = b200_mla_workspace_bytes(args->batch, args->heads, args->q_len);
    if (need > (long long)B200_MLA_STATIC_WORKSPACE_BYTES)
        return fail(B200_MLA_ERR_TOO_LARGE,
                    "this problem needs %lld bytes of scratch, the built-in scratch of b200_mla_decode_static holds %u; "
                    "use b200_mla_decode with a caller-provided workspace", need, (unsigned)B200_MLA_STATIC_WORKSPACE_BYTES);
    void* ptr = nullptr;
    const int rc = static_workspace_ptr(&ptr);
    if (rc != B200_MLA_OK) return rc;
    b200_mla_decode_args a = *args;
    a.workspace = ptr;
    a.workspace_bytes = B200_MLA_STATIC_WORKSPACE_BYTES;
    return b200_mla_decode(&a, stream);
}

int32_t b200_mla_read_status(const void* workspace, int32_t* out, void* stream) {
    if (!out) return fail(B200_MLA_ERR_INVALID_ARG, "out is NULL");
    void* ws = const_cast<void*>(workspace);
    if (!ws) {
        const int rc = static_workspace_ptr(&ws);
        if (rc != B200_MLA_OK) return rc;
    }
    cudaError_t e = cudaMemcpyAsync(out, ws, sizeof(int32_t), cudaMemcpyDefault, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "status copy failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int32_t b200_mla_reset_status(void* workspace, void* stream) {
    if (!workspace) {
        const int rc = static_workspace_ptr(&workspace);
        if (rc != B200_MLA_OK) return rc;
    }
    cudaError_t e = cudaMemsetAsync(workspace, 0, 256, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "status reset failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int32_t b200_mla_set_stage1_events(void* start_event, void* stop_event) {
    g_ev_start = (cudaEvent_t)start_event;
    g_ev_stop = (cudaEvent_t)stop_event;
    return B200_MLA_OK;
}

int32_t b200_mla_combine(const float* o_parts, const float* lse_parts, int32_t parts, int64_t rows,
                         int64_t o_part_stride, int64_t lse_part_stride, void* out, float* out_lse, void* stream) {
    if (!o_parts || !lse_parts || !out) return fail(B200_MLA_ERR_INVALID_ARG, "o_parts, lse_parts and out are required");
    if (parts <= 0 || rows <= 0) return fail(B200_MLA_ERR_INVALID_ARG, "parts and rows must be positive");
    if (rows > 0x7fffffffLL) return fail(B200_MLA_ERR_TOO_LARGE, "rows exceeds 2^31-1");
    if (((uintptr_t)o_parts & 15) || ((uintptr_t)out & 7)) return fail(B200_MLA_ERR_INVALID_ARG, "o_parts must be 16-byte and out 8-byte aligned");
    if (o_part_stride == 0) o_part_stride = rows * V_DIM;
    if (lse_part_stride == 0) lse_part_stride = rows;
    if (o_part_stride < rows * V_DIM || lse_part_stride < rows || (o_part_stride & 3))
        return fail(B200_MLA_ERR_INVALID_ARG, "part strides must cover a part; the O stride must be a multiple of 4 elements");
    cudaError_t e = launch_combine_parts(o_parts, lse_parts, parts, rows, o_part_stride, lse_part_stride,
                                        (__nv_bfloat16*)out, out_lse, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "combine launch failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int64_t b200_mla_peer_exchange_bytes(int64_t rows) { return rows > 0 ? peer_exchange_bytes(rows) : 0; }

int64_t b200_mla_peer_partial_offset(int64_t rows, uint32_t epoch) { return rows > 0 ? peer_partial_offset(rows, epoch) : 0; }

int32_t b200_mla_peer_alloc(int64_t rows, void** base, unsigned char* handle) {
    if (!base || !handle) return fail(B200_MLA_ERR_INVALID_ARG, "base and handle are required");
    if (rows <= 0) return fail(B200_MLA_ERR_INVALID_ARG, "rows must be positive");
    static_assert(sizeof(cudaIpcMemHandle_t) == B200_MLA_PEER_HANDLE_BYTES, "handle size");
    void* ptr = nullptr;
    const size_t bytes = (size_t)peer_exchange_bytes(rows);
    cudaError_t e = cudaMalloc(&ptr, bytes);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "exchange allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    e = cudaMemset(ptr, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) {
        cudaFree(ptr);
        return fail(B200_MLA_ERR_CUDA, "exchange allocation cannot be exported: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof(h));
    *base = ptr;
    return B200_MLA_OK;
}

int32_t b200_mla_peer_open(const unsigned char* handle, void** base) {
    if (!base || !handle) return fail(B200_MLA_ERR_INVALID_ARG, "base and handle are required");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(B200_MLA_ERR_CUDA, "peer allocation cannot be mapped: %s", cudaGetErrorString(e));
    }
    *base = ptr;
    return B200_MLA_OK;
}

int32_t b200_mla_peer_close(void* base) {
    if (!base) return B200_MLA_OK;
    cudaError_t e = cudaIpcCloseMemHandle(base);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "peer mapping cannot be closed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int32_t b200_mla_peer_free(void* base) {
    if (!base) return B200_MLA_OK;
    cudaError_t e = cudaFree(base);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "exchange allocation cannot be freed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int32_t b200_mla_peer_merge(const b200_mla_peer_merge_args* a, void* stream) {
    if (!a) return fail(B200_MLA_ERR_INVALID_ARG, "args is NULL");
    if (a->world != 1 && a->world != 2 && a->world != 4 && a->world != 8)
        return fail(B200_MLA_ERR_UNSUPPORTED, "world must be 1, 2, 4 or 8 (got %d)", a->world);
    if (a->rank < 0 || a->rank >= a->world) return fail(B200_MLA_ERR_INVALID_ARG, "rank %d outside [0, %d)", a->rank, a->world);
    if (a->epoch == 0) return fail(B200_MLA_ERR_INVALID_ARG, "epoch starts at 1");
    if (a->rows <= 0 || a->rows > 0x7fffffffLL) return fail(B200_MLA_ERR_INVALID_ARG, "rows must be in [1, 2^31)");
    if (!a->bases || !a->out || ((uintptr_t)a->out & 7)) return fail(B200_MLA_ERR_INVALID_ARG, "bases and out (8-byte aligned) are required");
    for (int i = 0; i < a->world; ++i)
        if (!a->bases[i] || ((uintptr_t)a->bases[i] & 255)) return fail(B200_MLA_ERR_INVALID_ARG, "bases[%d] must be a 256-byte aligned device pointer", i);
    void* ws = a->workspace;
    if (!ws) {
        const int rc = static_workspace_ptr(&ws);
        if (rc != B200_MLA_OK) return rc;
    }
    const unsigned long long limit_ns = a->wait_limit_ms > 0 ? (unsigned long long)a->wait_limit_ms * 1000000ULL : 2000000000ULL;
    cudaError_t e = launch_peer_merge(a->bases, a->world, a->rank, a->epoch, limit_ns, a->rows, a->out, (int*)ws, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "peer merge launch failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int32_t b200_mla_q_amax(const void* x_bf16, int64_t n, uint32_t* parts_out, void* stream) {
    if (!x_bf16 || !parts_out) return fail(B200_MLA_ERR_INVALID_ARG, "NULL argument");
    if (n <= 0) return fail(B200_MLA_ERR_INVALID_ARG, "n must be positive");
    if (((uintptr_t)x_bf16 & 15) || ((uintptr_t)parts_out & 3))
        return fail(B200_MLA_ERR_INVALID_ARG, "x must be 16-byte and parts_out 4-byte aligned");
    cudaError_t e = launch_q_amax_parts((const __nv_bfloat16*)x_bf16, n, parts_out, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "amax launch failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int32_t b200_mla_kv_append(const b200_mla_kv_append_args* a, void* stream) {
    if (!a) return fail(B200_MLA_ERR_INVALID_ARG, "args is NULL");
    if (a->n < 0) return fail(B200_MLA_ERR_INVALID_ARG, "n must be >= 0");
    if (a->n == 0) return B200_MLA_OK;
    if (a->kv_format < B200_MLA_KV_E4M3 || a->kv_format > B200_MLA_KV_HYBRID) return fail(B200_MLA_ERR_INVALID_ARG, "bad kv_format %d", a->kv_format);
    if (!a->rows_bf16 || !a->kv_codes) return fail(B200_MLA_ERR_INVALID_ARG, "rows_bf16 and kv_codes are required");
    if (((uintptr_t)a->rows_bf16 & 15) || a->row_stride % 8 || a->row_stride < B200_MLA_QK_DIM)
        return fail(B200_MLA_ERR_INVALID_ARG, "rows_bf16 must be 16-byte aligned with a row stride >= 576 that is a multiple of 8 elements");
    if (((uintptr_t)a->kv_codes & 15) || a->kv_codes_stride % 16) return fail(B200_MLA_ERR_INVALID_ARG, "kv_codes must be 16-byte aligned with a stride multiple of 16");
    const int min_codes = a->kv_format == B200_MLA_KV_E4M3 ? 576 : (a->kv_format == B200_MLA_KV_MXFP4 ? 288 : 256);
    if (a->kv_codes_stride < min_codes) return fail(B200_MLA_ERR_INVALID_ARG, "kv_codes_stride is smaller than a row (%d bytes)", min_codes);
    if (a->kv_format != B200_MLA_KV_MXFP4 && !a->kv_scale) return fail(B200_MLA_ERR_INVALID_ARG, "kv_scale is required for e4m3 / hybrid caches");
    if (a->kv_format != B200_MLA_KV_E4M3 && (!a->kv_block_scales || a->kv_block_scales_stride < (a->kv_format == B200_MLA_KV_MXFP4 ? 18 : 16)))
        return fail(B200_MLA_ERR_INVALID_ARG, "kv_block_scales (stride >= 18 for mxfp4, >= 16 for hybrid) is required");
    if (a->kv_format == B200_MLA_KV_HYBRID && (!a->kv_rope || ((uintptr_t)a->kv_rope & 15) || a->kv_rope_stride % 16 || a->kv_rope_stride < 64))
        return fail(B200_MLA_ERR_INVALID_ARG, "kv_rope must be 16-byte aligned with a stride >= 64 that is a multiple of 16");
    if (a->num_slots <= 0) return fail(B200_MLA_ERR_INVALID_ARG, "num_slots must be positive");
    if (!a->slots && (a->base_slot < 0 || a->base_slot + a->n > a->num_slots))
        return fail(B200_MLA_ERR_INVALID_ARG, "rows [base_slot, base_slot + n) do not fit in num_slots");
    if (a->slots && !a->status) return fail(B200_MLA_ERR_INVALID_ARG, "status (device int32) is required with a slot list: it reports slots outside the cache");
    cudaError_t e = launch_kv_append(a->rows_bf16, a->n, a->row_stride, a->slots, a->base_slot, a->num_slots, a->kv_format,
                                     a->kv_codes, a->kv_codes_stride, a->kv_block_scales, a->kv_block_scales_stride,
                                     a->kv_rope, a->kv_rope_stride, a->kv_scale, a->status, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "kv append launch failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

int32_t b200_mla_quantize_fp8(const void* x_bf16, int64_t n, void* codes_out, float* scale_out, void* scratch,
                              void* stream) {
    if (!x_bf16 || !codes_out || !scale_out || !scratch) return fail(B200_MLA_ERR_INVALID_ARG, "NULL argument");
    if (n <= 0) return fail(B200_MLA_ERR_INVALID_ARG, "n must be positive");
    if (((uintptr_t)x_bf16 & 15) || ((uintptr_t)codes_out & 7) || ((uintptr_t)scratch & 3))
        return fail(B200_MLA_ERR_INVALID_ARG, "x must be 16-byte, codes 8-byte and scratch 4-byte aligned");
    cudaError_t e = launch_quantize_fp8((const __nv_bfloat16*)x_bf16, n, (uint8_t*)codes_out, scale_out,
                                        (unsigned int*)scratch, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(B200_MLA_ERR_CUDA, "quantize launch failed: %s", cudaGetErrorString(e));
    return B200_MLA_OK;
}

}  // extern "C"
