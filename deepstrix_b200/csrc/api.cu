// C ABI of the library: device verbs, expert store, MoE operators and the
// whole-layer call.  Declarations and reference citations: include/dsx_moe.h.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "dsx_common.cuh"
#include "prefill.cuh"

namespace dsx {

static thread_local char g_err[768] = "";
static thread_local uint64_t g_launches = 0;

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
void count_launch() { g_launches++; }

}  // namespace dsx

using namespace dsx;

struct dsx_expert_store {
    int fmt = 0, n_slots = 0, device = 0;
    int64_t H = 0, F = 0;
    uint8_t *gu_nib = nullptr, *gu_sc = nullptr, *dn_nib = nullptr, *dn_sc = nullptr;
    int64_t gu_nib_stride = 0, gu_sc_stride = 0, dn_nib_stride = 0, dn_sc_stride = 0;  // bytes per slot
    // MXFP4 only (null for a decode-only store): the tensor-core planes of prefill_mx.cu.  Codes K-major
    // ([slot][gate|up][ffn][hidden/2] and [slot][hidden][ffn/2], the HF byte layout) and the block scales as
    // 512-byte scale-factor chunks (layout: kmajor_mxfp4_kernel in repack.cu).
    uint8_t *km_gu = nullptr, *km_dn = nullptr, *sf_gu = nullptr, *sf_dn = nullptr;
    int64_t km_gu_stride = 0, km_dn_stride = 0, sf_gu_stride = 0, sf_dn_stride = 0;  // bytes per slot
    uint8_t* stage = nullptr;  // device staging for host sources
    size_t stage_bytes = 0;
    size_t device_bytes = 0;
    // largest E8M0 scale byte seen by a load (device word, folded by every load); the host copy is
    // refreshed lazily.  The tensor-core path holds weights as f16 and needs every scale <= 2^13.
    uint32_t* d_scale_max = nullptr;
    mutable uint32_t h_scale_max = 0;
    mutable bool scale_dirty = false;
};

struct dsx_moe_layer {
    dsx_moe_config cfg{};
    const dsx_expert_store* routed = nullptr;
    const dsx_expert_store* shared = nullptr;
    const float* router_w = nullptr;
    const float* router_bias = nullptr;
    int sm_count = 0;
    // workspace (device)
    float* logits = nullptr;
    int32_t* sel_local = nullptr;   // picks translated through an ownership table (dsx_moe_layer_forward_remap)
    // A shared expert whose format or width differs from the routed experts' (the reference's own layout: MXFP4 routed,
    // Q8_0 shared) cannot ride in the routed kernels' launches.  It then runs as a one-expert, one-pick layer of its
    // own (picks all 0, weights all 1) that writes the shared rows of this layer's partial buffer.
    dsx_moe_layer* sh_layer = nullptr;
    int32_t* sh_sel = nullptr;      // [max_tokens] zeros
    float* sh_w = nullptr;          // [max_tokens] ones
    int32_t *selected = nullptr, *hist = nullptr, *offsets = nullptr, *perm = nullptr, *work_items = nullptr, *n_work_items = nullptr;
    float* weights = nullptr;
    int32_t work_cap = 0;
    ItemRec* item_recs = nullptr;   // one record per work item, written by the one-launch decode router for batches below 8 tokens
    GroupScratch gs{};
    __half* mid = nullptr;
    float* partial = nullptr;
    uint32_t* error_word = nullptr;
    unsigned int* router_counters = nullptr;   // ticket counters of the one-launch decode router
    __nv_bfloat16 *x_stage = nullptr, *out_stage = nullptr;
    PrefillWorkspace pf{};
    // optional per-stage event pairs (dsx_moe_layer_profile)
    bool profile = false;
    cudaEvent_t ev[2 * DSX_STAGE_COUNT] = {};
    bool ev_used[DSX_STAGE_COUNT] = {};
    // what the last forward used (for dsx_moe_layer_routing)
    const float* last_logits = nullptr;
    const int32_t* last_selected = nullptr;
    const float* last_weights = nullptr;
};

extern "C" {

const char* dsx_last_error(void) { return g_err; }
uint64_t dsx_launch_count(int reset) {
    const uint64_t v = g_launches;
    if (reset) g_launches = 0;
    return v;
}

// ------------------------------------------------------------ device verbs
int dsx_device_count(int* count) { DSX_CUDA(cudaGetDeviceCount(count)); return DSX_OK; }
int dsx_device_set(int device) { DSX_CUDA(cudaSetDevice(device)); return DSX_OK; }
int dsx_device_get(int* device) { DSX_CUDA(cudaGetDevice(device)); return DSX_OK; }
int dsx_device_sync(void) { DSX_CUDA(cudaDeviceSynchronize()); return DSX_OK; }
int dsx_device_props(int device, char* name256, int* sm_count, size_t* total_mem, int* cc_major, int* cc_minor) {
    cudaDeviceProp p;
    DSX_CUDA(cudaGetDeviceProperties(&p, device));
    if (name256) { strncpy(name256, p.name, 255); name256[255] = 0; }
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (total_mem) *total_mem = p.totalGlobalMem;
    if (cc_major) *cc_major = p.major;
    if (cc_minor) *cc_minor = p.minor;
    return DSX_OK;
}
int dsx_device_enable_peer(int peer_device) {
    int dev = 0, can = 0;
    DSX_CUDA(cudaGetDevice(&dev));
    DSX_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
    if (!can) return set_error(DSX_ERR_UNSUPPORTED, "device %d cannot access peer %d", dev, peer_device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return DSX_OK; }
    DSX_CUDA(e);
    return DSX_OK;
}

int dsx_malloc(void** dptr, size_t bytes) { DSX_CUDA(cudaMalloc(dptr, bytes)); return DSX_OK; }
int dsx_free(void* dptr) { DSX_CUDA(cudaFree(dptr)); return DSX_OK; }
int dsx_mem_get_info(size_t* free_bytes, size_t* total_bytes) { DSX_CUDA(cudaMemGetInfo(free_bytes, total_bytes)); return DSX_OK; }
int dsx_host_malloc(void** hptr, size_t bytes) { DSX_CUDA(cudaHostAlloc(hptr, bytes, cudaHostAllocDefault)); return DSX_OK; }
int dsx_host_free(void* hptr) { DSX_CUDA(cudaFreeHost(hptr)); return DSX_OK; }

static cudaMemcpyKind to_kind(int kind) {
    return kind == 1 ? cudaMemcpyHostToDevice : kind == 2 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
}
int dsx_memcpy(void* dst, const void* src, size_t bytes, int kind) {
    DSX_REQUIRE(kind >= 1 && kind <= 3, "memcpy: kind %d", kind);
    DSX_CUDA(cudaMemcpy(dst, src, bytes, to_kind(kind)));
    return DSX_OK;
}
int dsx_memcpy_async(void* dst, const void* src, size_t bytes, int kind, dsx_stream_t stream) {
    DSX_REQUIRE(kind >= 1 && kind <= 3, "memcpy_async: kind %d", kind);
    DSX_CUDA(cudaMemcpyAsync(dst, src, bytes, to_kind(kind), (cudaStream_t)stream));
    return DSX_OK;
}
int dsx_memcpy_peer_async(void* dst, int dst_device, const void* src, int src_device, size_t bytes, dsx_stream_t stream) {
    DSX_CUDA(cudaMemcpyPeerAsync(dst, dst_device, src, src_device, bytes, (cudaStream_t)stream));
    return DSX_OK;
}
int dsx_memset(void* dptr, int value, size_t bytes) { DSX_CUDA(cudaMemset(dptr, value, bytes)); return DSX_OK; }
int dsx_memset_async(void* dptr, int value, size_t bytes, dsx_stream_t stream) {
    DSX_CUDA(cudaMemsetAsync(dptr, value, bytes, (cudaStream_t)stream));
    return DSX_OK;
}

int dsx_stream_create(dsx_stream_t* stream, int non_blocking, int priority) {
    cudaStream_t s;
    DSX_CUDA(cudaStreamCreateWithPriority(&s, non_blocking ? cudaStreamNonBlocking : cudaStreamDefault, priority));
    *stream = s;
    return DSX_OK;
}
int dsx_stream_destroy(dsx_stream_t stream) { DSX_CUDA(cudaStreamDestroy((cudaStream_t)stream)); return DSX_OK; }
int dsx_stream_sync(dsx_stream_t stream) { DSX_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); return DSX_OK; }
int dsx_stream_query(dsx_stream_t stream, int* done) {
    cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
    if (e == cudaErrorNotReady) { *done = 0; return DSX_OK; }
    DSX_CUDA(e);
    *done = 1;
    return DSX_OK;
}
int dsx_stream_wait_event(dsx_stream_t stream, dsx_event_t event) {
    DSX_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
    return DSX_OK;
}

int dsx_event_create(dsx_event_t* event, int timing) {
    cudaEvent_t e;
    DSX_CUDA(cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming));
    *event = e;
    return DSX_OK;
}
int dsx_event_destroy(dsx_event_t event) { DSX_CUDA(cudaEventDestroy((cudaEvent_t)event)); return DSX_OK; }
int dsx_event_record(dsx_event_t event, dsx_stream_t stream) { DSX_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); return DSX_OK; }
int dsx_event_sync(dsx_event_t event) { DSX_CUDA(cudaEventSynchronize((cudaEvent_t)event)); return DSX_OK; }
int dsx_event_query(dsx_event_t event, int* done) {
    cudaError_t e = cudaEventQuery((cudaEvent_t)event);
    if (e == cudaErrorNotReady) { *done = 0; return DSX_OK; }
    DSX_CUDA(e);
    *done = 1;
    return DSX_OK;
}
int dsx_event_elapsed_ms(dsx_event_t start, dsx_event_t stop, float* ms) {
    DSX_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return DSX_OK;
}

int dsx_graph_begin_capture(dsx_stream_t stream) {
    DSX_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    return DSX_OK;
}
int dsx_graph_end_capture(dsx_stream_t stream, dsx_graph_t* graph_exec) {
    cudaGraph_t g = nullptr;
    DSX_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t ge = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    DSX_CUDA(e);
    *graph_exec = ge;
    return DSX_OK;
}
int dsx_graph_launch(dsx_graph_t graph_exec, dsx_stream_t stream) {
    DSX_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream));
    return DSX_OK;
}
int dsx_graph_destroy(dsx_graph_t graph_exec) { DSX_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec)); return DSX_OK; }

// ------------------------------------------------------------ expert store
int dsx_bytes_per_expert(int fmt, int64_t k, int64_t rows, size_t* bytes) {
    DSX_REQUIRE(k % 32 == 0 && rows > 0, "bytes_per_expert: k %lld rows %lld", (long long)k, (long long)rows);
    DSX_REQUIRE(fmt == DSX_FMT_MXFP4 || fmt == DSX_FMT_Q8_0, "bytes_per_expert: format %d", fmt);
    *bytes = (size_t)rows * (size_t)(k / 32) * (fmt == DSX_FMT_MXFP4 ? 17 : 34);
    return DSX_OK;
}

int dsx_expert_store_create(dsx_expert_store** store, int fmt, int n_slots, int64_t hidden, int64_t ffn) {
    return dsx_expert_store_create_ex(store, fmt, n_slots, hidden, ffn, 0);
}

int dsx_expert_store_create_ex(dsx_expert_store** store, int fmt, int n_slots, int64_t hidden, int64_t ffn, uint32_t flags) {
    DSX_REQUIRE(fmt == DSX_FMT_MXFP4 || fmt == DSX_FMT_Q8_0, "expert_store: format %d", fmt);
    DSX_REQUIRE((flags & ~(uint32_t)DSX_STORE_DECODE_ONLY) == 0, "expert_store: unknown flags 0x%x", flags);
    DSX_REQUIRE(n_slots >= 1 && hidden > 0 && ffn > 0 && hidden % 256 == 0 && ffn % 256 == 0,
                "expert_store: %d slots, hidden %lld, ffn %lld (both must be multiples of 256)", n_slots, (long long)hidden, (long long)ffn);
    dsx_expert_store* s = new (std::nothrow) dsx_expert_store();
    if (!s) return set_error(DSX_ERR_NOMEM, "expert_store: out of host memory");
    s->fmt = fmt; s->n_slots = n_slots; s->H = hidden; s->F = ffn;
    cudaGetDevice(&s->device);
    const int tk = tile_k(fmt);
    const int64_t sub_gu = (ffn / 16) * (hidden / tk) * 2, sub_dn = (hidden / 16) * (ffn / tk);
    s->gu_nib_stride = sub_gu * kSubNibBytes; s->gu_sc_stride = sub_gu * kSubScBytes;
    s->dn_nib_stride = sub_dn * kSubNibBytes; s->dn_sc_stride = sub_dn * kSubScBytes;
    const size_t n = (size_t)n_slots;
    cudaError_t e = cudaMalloc(&s->gu_nib, n * s->gu_nib_stride);
    if (e == cudaSuccess) e = cudaMalloc(&s->gu_sc, n * s->gu_sc_stride);
    if (e == cudaSuccess) e = cudaMalloc(&s->dn_nib, n * s->dn_nib_stride);
    if (e == cudaSuccess) e = cudaMalloc(&s->dn_sc, n * s->dn_sc_stride);
    // the tensor-core kernel tiles 256 gate/up rows and 512 down rows (other shapes keep the decode layout only)
    const bool tensor_planes = fmt == DSX_FMT_MXFP4 && !(flags & DSX_STORE_DECODE_ONLY) && ffn % 256 == 0 && hidden % 512 == 0;
    if (tensor_planes) {
        s->km_gu_stride = ffn * hidden;          // two matrices of ffn x hidden / 2 bytes
        s->km_dn_stride = hidden * ffn / 2;
        s->sf_gu_stride = ffn * hidden / 16;     // one byte per 32 weights, two matrices
        s->sf_dn_stride = hidden * ffn / 32;
        if (e == cudaSuccess) e = cudaMalloc(&s->km_gu, n * s->km_gu_stride);
        if (e == cudaSuccess) e = cudaMalloc(&s->km_dn, n * s->km_dn_stride);
        if (e == cudaSuccess) e = cudaMalloc(&s->sf_gu, n * s->sf_gu_stride);
        if (e == cudaSuccess) e = cudaMalloc(&s->sf_dn, n * s->sf_dn_stride);
    }
    if (e == cudaSuccess) e = cudaMalloc((void**)&s->d_scale_max, 256);
    if (e == cudaSuccess) e = cudaMemset(s->d_scale_max, 0, 256);
    // scale planes start at zero: the largest-scale scan covers whole planes, slots not loaded yet included
    if (e == cudaSuccess) e = cudaMemset(s->gu_sc, 0, n * s->gu_sc_stride);
    if (e == cudaSuccess) e = cudaMemset(s->dn_sc, 0, n * s->dn_sc_stride);
    if (e != cudaSuccess) {
        dsx_expert_store_destroy(s);
        return set_error((int)e, "expert_store: cudaMalloc failed: %s", cudaGetErrorString(e));
    }
    s->device_bytes = n * (size_t)(s->gu_nib_stride + s->gu_sc_stride + s->dn_nib_stride + s->dn_sc_stride + s->km_gu_stride +
                                   s->km_dn_stride + s->sf_gu_stride + s->sf_dn_stride);
    *store = s;
    return DSX_OK;
}

int dsx_expert_store_destroy(dsx_expert_store* s) {
    if (!s) return DSX_OK;
    cudaFree(s->gu_nib); cudaFree(s->gu_sc); cudaFree(s->dn_nib); cudaFree(s->dn_sc); cudaFree(s->stage); cudaFree(s->d_scale_max);
    cudaFree(s->km_gu); cudaFree(s->km_dn); cudaFree(s->sf_gu); cudaFree(s->sf_dn);
    delete s;
    return DSX_OK;
}

static void src_bytes(int layout, int64_t rows, int64_t K, size_t* qb, size_t* sb) {
    const size_t nb = (size_t)rows * (size_t)(K / 32);
    switch (layout) {
        case DSX_SRC_MXFP4_HF: *qb = nb * 16; *sb = nb; break;
        case DSX_SRC_MXFP4_GGML: case DSX_SRC_MXFP4_SB2: *qb = nb * 17; *sb = 0; break;
        case DSX_SRC_Q8_0_BLOCKS: *qb = nb * 34; *sb = 0; break;
        default: *qb = nb * 32; *sb = nb * 2; break;
    }
}

int dsx_expert_store_load(dsx_expert_store* st, int slot, int which, int src_layout, const void* q, const void* s,
                          int src_on_device, dsx_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(st != nullptr && q != nullptr, "expert_store_load: null store or source");
    DSX_REQUIRE(slot >= -1 && slot < st->n_slots, "expert_store_load: slot %d of %d", slot, st->n_slots);
    DSX_REQUIRE(which >= DSX_MAT_GATE && which <= DSX_MAT_DOWN, "expert_store_load: matrix kind %d", which);
    DSX_REQUIRE(src_layout >= 0 && src_layout <= DSX_SRC_Q8_0_SPLIT, "expert_store_load: layout %d", src_layout);
    const bool down = which == DSX_MAT_DOWN;
    const int64_t rows = down ? st->H : st->F, K = down ? st->F : st->H;
    size_t qb, sb;
    src_bytes(src_layout, rows, K, &qb, &sb);
    DSX_REQUIRE(sb == 0 || s != nullptr, "expert_store_load: this layout needs a scale array");
    uint8_t* nib = down ? st->dn_nib : st->gu_nib;
    uint8_t* sc = down ? st->dn_sc : st->gu_sc;
    const int64_t nstr = down ? st->dn_nib_stride : st->gu_nib_stride, sstr = down ? st->dn_sc_stride : st->gu_sc_stride;
    const int pair_stride = down ? 1 : 2, pair_index = which == DSX_MAT_UP ? 1 : 0;
    const int first = slot < 0 ? 0 : slot, count = slot < 0 ? st->n_slots : 1;
    auto fold_scales = [&]() -> int {  // the largest scale is recomputed over the whole planes before the next use
        st->scale_dirty = true;
        return DSX_OK;
    };
    // the same source once more into the tensor-core planes (MXFP4 stores that keep them)
    auto tensor_planes = [&](const uint8_t* dq, const uint8_t* ds, int slot0, int n_mats) -> int {
        if (!st->km_gu) return DSX_OK;
        uint8_t* km = down ? st->km_dn : st->km_gu;
        uint8_t* sf = down ? st->sf_dn : st->sf_gu;
        const int64_t kstr = down ? st->km_dn_stride : st->km_gu_stride, fstr = down ? st->sf_dn_stride : st->sf_gu_stride;
        return launch_kmajor_mxfp4(src_layout, dq, ds, rows, K, down ? -1 : pair_index, n_mats, (int64_t)qb, (int64_t)sb, km + slot0 * kstr, kstr,
                                   sf + slot0 * fstr, fstr, stream);
    };
    if (src_on_device) {
        if (int rc = launch_repack(st->fmt, src_layout, (const uint8_t*)q, (const uint8_t*)s, rows, K, nib + first * nstr,
                                   sc + first * sstr, pair_stride, pair_index, count, (int64_t)qb, (int64_t)sb, nstr, sstr, stream))
            return rc;
        if (int rc = tensor_planes((const uint8_t*)q, (const uint8_t*)s, first, count)) return rc;
        return fold_scales();
    }
    // host source: stage through device memory in batches
    const size_t qpad = (qb + 255) & ~(size_t)255, spad = (sb + 255) & ~(size_t)255;
    const int batch = (int)std::max<size_t>(1, std::min<size_t>((size_t)count, ((size_t)192 << 20) / (qpad + spad)));
    const size_t need = (size_t)batch * (qpad + spad);
    if (st->stage_bytes < need) {
        DSX_CUDA(cudaStreamSynchronize(stream));
        cudaFree(st->stage);
        st->stage = nullptr; st->stage_bytes = 0;
        DSX_CUDA(cudaMalloc(&st->stage, need));
        st->stage_bytes = need;
    }
    for (int b0 = 0; b0 < count; b0 += batch) {
        const int nb = std::min(batch, count - b0);
        uint8_t* dq = st->stage;
        uint8_t* ds = st->stage + (size_t)batch * qpad;
        // per-expert sources are contiguous (stride qb / sb); device copies keep that stride
        DSX_CUDA(cudaMemcpyAsync(dq, (const uint8_t*)q + (size_t)b0 * qb, (size_t)nb * qb, cudaMemcpyHostToDevice, stream));
        if (sb) DSX_CUDA(cudaMemcpyAsync(ds, (const uint8_t*)s + (size_t)b0 * sb, (size_t)nb * sb, cudaMemcpyHostToDevice, stream));
        if (int rc = launch_repack(st->fmt, src_layout, dq, sb ? ds : nullptr, rows, K, nib + (first + b0) * nstr,
                                   sc + (first + b0) * sstr, pair_stride, pair_index, nb, (int64_t)qb, (int64_t)sb, nstr, sstr, stream))
            return rc;
        if (int rc = tensor_planes(dq, sb ? ds : nullptr, first + b0, nb)) return rc;
        DSX_CUDA(cudaStreamSynchronize(stream));  // the staging buffer is reused
    }
    return fold_scales();
}

int dsx_expert_store_unpack(const dsx_expert_store* st, int slot, int which, void* q_out, void* s_out, dsx_stream_t stream) {
    DSX_REQUIRE(st && slot >= 0 && slot < st->n_slots && which >= 0 && which <= 2 && q_out && s_out, "expert_store_unpack: bad argument");
    const bool down = which == DSX_MAT_DOWN;
    const int64_t rows = down ? st->H : st->F, K = down ? st->F : st->H;
    const uint8_t* nib = (down ? st->dn_nib : st->gu_nib) + slot * (down ? st->dn_nib_stride : st->gu_nib_stride);
    const uint8_t* sc = (down ? st->dn_sc : st->gu_sc) + slot * (down ? st->dn_sc_stride : st->gu_sc_stride);
    return launch_unpack(st->fmt, nib, sc, rows, K, down ? 1 : 2, which == DSX_MAT_UP ? 1 : 0, (uint8_t*)q_out, (uint8_t*)s_out,
                         (cudaStream_t)stream);
}

int dsx_expert_store_clone(const dsx_expert_store* src, dsx_expert_store** dst, dsx_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(src && dst, "expert_store_clone: null argument");
    dsx_expert_store* d = nullptr;
    if (int rc = dsx_expert_store_create_ex(&d, src->fmt, src->n_slots, src->H, src->F,
                                            (src->fmt == DSX_FMT_MXFP4 && !src->km_gu) ? DSX_STORE_DECODE_ONLY : 0))
        return rc;
    const size_t n = (size_t)src->n_slots;
    cudaError_t e = cudaMemcpyAsync(d->gu_nib, src->gu_nib, n * src->gu_nib_stride, cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d->gu_sc, src->gu_sc, n * src->gu_sc_stride, cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d->dn_nib, src->dn_nib, n * src->dn_nib_stride, cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d->dn_sc, src->dn_sc, n * src->dn_sc_stride, cudaMemcpyDeviceToDevice, stream);
    if (src->km_gu) {
        if (e == cudaSuccess) e = cudaMemcpyAsync(d->km_gu, src->km_gu, n * src->km_gu_stride, cudaMemcpyDeviceToDevice, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d->km_dn, src->km_dn, n * src->km_dn_stride, cudaMemcpyDeviceToDevice, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d->sf_gu, src->sf_gu, n * src->sf_gu_stride, cudaMemcpyDeviceToDevice, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d->sf_dn, src->sf_dn, n * src->sf_dn_stride, cudaMemcpyDeviceToDevice, stream);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(d->d_scale_max, src->d_scale_max, 4, cudaMemcpyDeviceToDevice, stream);
    d->scale_dirty = true;
    if (e != cudaSuccess) {
        dsx_expert_store_destroy(d);
        return set_error((int)e, "expert_store_clone: copy failed: %s", cudaGetErrorString(e));
    }
    *dst = d;
    return DSX_OK;
}

int dsx_expert_store_info(const dsx_expert_store* st, int* fmt, int* n_slots, int64_t* hidden, int64_t* ffn, size_t* device_bytes) {
    DSX_REQUIRE(st, "expert_store_info: null store");
    if (fmt) *fmt = st->fmt;
    if (n_slots) *n_slots = st->n_slots;
    if (hidden) *hidden = st->H;
    if (ffn) *ffn = st->F;
    if (device_bytes) *device_bytes = st->device_bytes;
    return DSX_OK;
}

// ------------------------------------------------------------------ router
int dsx_router_logits(const void* x_bf16, int64_t T, const float* W, int n_expert, int64_t hidden, float* logits, dsx_stream_t stream) {
    DSX_REQUIRE(T >= 0, "router_logits: negative token count");
    if (T == 0) return DSX_OK;   // an empty batch has no rows to point at
    DSX_REQUIRE(x_bf16 && W && logits, "router_logits: null argument");
    return launch_router_logits((const __nv_bfloat16*)x_bf16, T, W, n_expert, hidden, logits, (cudaStream_t)stream);
}
int dsx_router_topk(const float* logits, const float* bias, int64_t T, const dsx_router_config* cfg, int32_t* selected,
                    float* weights, dsx_stream_t stream) {
    DSX_REQUIRE(logits && cfg && selected && weights && T >= 0, "router_topk: null argument");
    return launch_router_topk(logits, bias, T, *cfg, selected, weights, 0, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}
int dsx_router_topk_ex(const float* logits, const float* bias, int64_t T, const dsx_router_config* cfg, int32_t* selected,
                       float* weights, int n_alt, int32_t* alts, float* alt_w, float* range_out, dsx_stream_t stream) {
    DSX_REQUIRE(logits && cfg && selected && weights && T >= 0, "router_topk_ex: null argument");
    DSX_REQUIRE(alts != nullptr || alt_w == nullptr, "router_topk_ex: alt_w without alts");
    return launch_router_topk(logits, bias, T, *cfg, selected, weights, n_alt, alts, alt_w, range_out, (cudaStream_t)stream);
}
int dsx_expert_sel_count(uint32_t* counts, const int32_t* selected, uint32_t layer_off, uint32_t n_expert, int64_t total,
                         dsx_stream_t stream) {
    DSX_REQUIRE(total >= 0 && n_expert > 0, "expert_sel_count: %lld picks, %u experts", (long long)total, n_expert);
    if (total == 0) return DSX_OK;
    DSX_REQUIRE(counts && selected, "expert_sel_count: null argument");
    return launch_expert_sel_count(counts, selected, layer_off, n_expert, total, (cudaStream_t)stream);
}
int dsx_router_topk_prior(const float* logits, const float* bias, int64_t T, const dsx_router_config* cfg, int32_t* selected,
                          float* weights, int n_alt, int32_t* alts, float* alt_w, float* range_out, const float* prior, int n_protect,
                          int prior_dry, int32_t* orig_sel, dsx_stream_t stream) {
    DSX_REQUIRE(logits && cfg && selected && weights && prior && T >= 0, "router_topk_prior: null argument");
    DSX_REQUIRE(alts != nullptr || alt_w == nullptr, "router_topk_prior: alt_w without alts");
    return launch_router_topk_prior(logits, bias, T, *cfg, selected, weights, n_alt, alts, alt_w, range_out, prior, n_protect, prior_dry,
                                    orig_sel, (cudaStream_t)stream);
}

uint32_t dsx_wi_upper_bound(uint64_t members, uint32_t groups, uint32_t chunk, uint64_t cap) {
    const uint64_t m = members, g = std::min<uint64_t>(m, groups), c = chunk ? chunk : 1;
    return (uint32_t)std::min(std::min(m, g + (m + c - 1) / c), cap);
}

int dsx_moe_group_build(const int32_t* selected, int64_t T, int n_used, int n_expert, int chunk, int32_t* hist,
                        int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, dsx_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(selected && hist && offsets && perm && T >= 0 && n_used >= 1, "group_build: null argument");
    DSX_REQUIRE((work_items == nullptr) == (n_work_items == nullptr), "group_build: work_items and n_work_items go together");
    GroupScratch gs{};
    const int64_t P = T * n_used;
    if (P > kGroupChunk) {
        gs.capacity_chunks = (P + kGroupChunk - 1) / kGroupChunk;
        DSX_CUDA(cudaMallocAsync((void**)&gs.chunk_hist, sizeof(int32_t) * (size_t)gs.capacity_chunks * (size_t)n_expert, stream));
    }
    const int32_t cap = work_items ? (int32_t)dsx_wi_upper_bound((uint64_t)P, (uint32_t)n_expert, (uint32_t)chunk, 1u << 30) : 0;
    const int rc = launch_group_build(selected, T, n_used, n_expert, 0, chunk, 0, hist, offsets, perm, work_items, n_work_items, cap, gs, stream);
    if (gs.chunk_hist) cudaFreeAsync(gs.chunk_hist, stream);
    return rc;
}

int dsx_moe_group_build_static(const int32_t* selected, int64_t T, int n_used, int n_expert, int chunk, int32_t* hist,
                               int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, dsx_stream_t stream) {
    DSX_REQUIRE(selected && hist && offsets && perm && T >= 0 && n_used >= 1, "group_build_static: null argument");
    DSX_REQUIRE((work_items == nullptr) == (n_work_items == nullptr), "group_build_static: work_items and n_work_items go together");
    const int32_t cap = work_items ? (int32_t)dsx_wi_upper_bound((uint64_t)(T * n_used), (uint32_t)n_expert, (uint32_t)chunk, 1u << 30) : 0;
    return launch_group_build_static(selected, T, n_used, n_expert, chunk, hist, offsets, perm, work_items, n_work_items, cap,
                                     (cudaStream_t)stream);
}

int dsx_reduce_partials_to(const float* partial, int64_t T, int n_used, int64_t hidden, int with_shared, const int32_t* selected,
                           int expert_lo, int n_local, void* const* out_rows, dsx_stream_t stream) {
    DSX_REQUIRE(T >= 0 && n_used >= 1 && n_used <= 32 && hidden >= 8, "reduce_partials_to: %lld tokens, %d slots, %lld columns", (long long)T, n_used,
                (long long)hidden);
    if (T == 0) return DSX_OK;
    DSX_REQUIRE(partial && out_rows, "reduce_partials_to: null argument");
    DSX_REQUIRE(((uintptr_t)partial & 15) == 0, "reduce_partials_to: rows must be 16-byte aligned");
    return launch_combine(partial, T, n_used, hidden, with_shared ? 1 : 0, selected, expert_lo, n_local, nullptr, (cudaStream_t)stream,
                          (__nv_bfloat16* const*)out_rows);
}

int dsx_reduce_partials(const float* partial, int64_t T, int n_used, int64_t hidden, int with_shared, const int32_t* selected,
                        int expert_lo, int n_local, void* out_bf16, dsx_stream_t stream) {
    DSX_REQUIRE(T >= 0 && n_used >= 1 && n_used <= 32 && hidden >= 8, "reduce_partials: %lld tokens, %d slots, %lld columns", (long long)T, n_used,
                (long long)hidden);
    if (T == 0) return DSX_OK;
    DSX_REQUIRE(partial && out_bf16, "reduce_partials: null argument");
    DSX_REQUIRE((((uintptr_t)partial | (uintptr_t)out_bf16) & 15) == 0, "reduce_partials: rows must be 16-byte aligned");
    return launch_combine(partial, T, n_used, hidden, with_shared ? 1 : 0, selected, expert_lo, n_local, (__nv_bfloat16*)out_bf16,
                          (cudaStream_t)stream);
}

// ------------------------------------------------------------------- layer
struct StageTimer {  // brackets one stage with an event pair when profiling is on
    dsx_moe_layer* L; int stage; cudaStream_t stream;
    StageTimer(dsx_moe_layer* l, int s, cudaStream_t st) : L(l), stage(s), stream(st) {
        if (L->profile) { cudaEventRecord(L->ev[2 * stage], stream); L->ev_used[stage] = true; }
    }
    ~StageTimer() { if (L->profile) cudaEventRecord(L->ev[2 * stage + 1], stream); }
};

static void layer_free(dsx_moe_layer* L) {
    if (L->sh_layer) {
        L->sh_layer->partial = nullptr;   // a view into this layer's buffer
        dsx_moe_layer_destroy(L->sh_layer);
        L->sh_layer = nullptr;
    }
    cudaFree(L->sh_sel); cudaFree(L->sh_w);
    for (cudaEvent_t e : L->ev) if (e) cudaEventDestroy(e);
    cudaFree(L->sel_local);
    cudaFree(L->logits); cudaFree(L->selected); cudaFree(L->weights); cudaFree(L->hist); cudaFree(L->offsets);
    cudaFree(L->perm); cudaFree(L->work_items); cudaFree(L->n_work_items); cudaFree(L->gs.chunk_hist); cudaFree(L->mid);
    cudaFree(L->partial); cudaFree(L->error_word); cudaFree(L->router_counters); cudaFree(L->item_recs); cudaFree(L->x_stage); cudaFree(L->out_stage);
    prefill_mx_workspace_free(&L->pf);
    prefill_workspace_free(&L->pf);
}

static int check_weights(const dsx_moe_config& c, const dsx_expert_store* routed, const dsx_expert_store* shared,
                         const float* router_w) {
    DSX_REQUIRE(routed && router_w, "moe_layer: routed store and router weights are required");
    DSX_REQUIRE(routed->H == c.hidden && routed->F == c.ffn, "moe_layer: routed store is %lldx%lld, config says %dx%d",
                (long long)routed->H, (long long)routed->F, c.hidden, c.ffn);
    DSX_REQUIRE(routed->n_slots <= c.router.n_expert, "moe_layer: store has %d slots for %d experts", routed->n_slots, c.router.n_expert);
    if (c.shared_ffn > 0) {
        DSX_REQUIRE(shared && shared->n_slots >= 1 && shared->H == c.hidden && shared->F == c.shared_ffn,
                    "moe_layer: shared store missing or of the wrong shape");
        // a shared expert of another format or width is allowed: it runs as its own pass (see dsx_moe_layer::sh_layer)
    }
    return DSX_OK;
}

// Stores whose prefill-size batches run on block-scaled FP4 MMAs (the others take the f16-operand kernels).
static bool takes_block_scaled(const dsx_expert_store* routed, const dsx_expert_store* shared) {
    return routed->fmt == DSX_FMT_MXFP4 && routed->km_gu != nullptr && (!shared || (shared->fmt == DSX_FMT_MXFP4 && shared->km_gu != nullptr));
}

int dsx_moe_layer_create(dsx_moe_layer** layer, const dsx_moe_config* cfg, const dsx_expert_store* routed,
                         const dsx_expert_store* shared, const float* router_w, const float* router_bias) {
    DSX_REQUIRE(layer && cfg, "moe_layer_create: null argument");
    const dsx_moe_config& c = *cfg;
    DSX_REQUIRE(c.hidden > 0 && c.hidden % 256 == 0 && c.ffn > 0 && c.ffn % 256 == 0, "moe_layer: hidden/ffn must be multiples of 256");
    DSX_REQUIRE(c.max_tokens >= 1 && c.max_tokens < 65536, "moe_layer: max_tokens %d out of range (1..65535)", c.max_tokens);
    DSX_REQUIRE(c.router.n_used >= 1 && c.router.n_used <= 16, "moe_layer: n_used %d", c.router.n_used);
    if (int rc = check_weights(c, routed, shared, router_w)) return rc;
    dsx_moe_layer* L = new (std::nothrow) dsx_moe_layer();
    if (!L) return set_error(DSX_ERR_NOMEM, "moe_layer: out of host memory");
    L->cfg = c; L->routed = routed; L->shared = c.shared_ffn > 0 ? shared : nullptr;
    L->router_w = router_w; L->router_bias = router_bias;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&L->sm_count, cudaDevAttrMultiProcessorCount, dev);
    const size_t Tm = (size_t)c.max_tokens, E = (size_t)c.router.n_expert, k = (size_t)c.router.n_used, P = Tm * k;
    L->work_cap = (int32_t)(dsx_wi_upper_bound(P, (uint32_t)E, 8, 1u << 30) + (Tm + 7) / 8);
    L->gs.capacity_chunks = (int64_t)((P + kGroupChunk - 1) / kGroupChunk);
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, std::max<size_t>(bytes, 256)); };
    alloc((void**)&L->logits, Tm * E * 4);
    alloc((void**)&L->selected, P * 4);
    alloc((void**)&L->sel_local, P * 4);
    alloc((void**)&L->weights, P * 4);
    alloc((void**)&L->hist, E * 4);
    alloc((void**)&L->offsets, (E + 1) * 4);
    alloc((void**)&L->perm, P * 4);
    alloc((void**)&L->work_items, (size_t)L->work_cap * 4);
    alloc((void**)&L->item_recs, (size_t)128 * sizeof(ItemRec));   // at most 7 * n_used + 1 items, n_used <= 16
    alloc((void**)&L->n_work_items, 256);
    alloc((void**)&L->gs.chunk_hist, (size_t)L->gs.capacity_chunks * E * 4);
    alloc((void**)&L->mid, (P + Tm) * (size_t)std::max(c.ffn, c.shared_ffn) * 2);
    alloc((void**)&L->partial, (P + Tm) * (size_t)c.hidden * 4);
    alloc((void**)&L->error_word, 256);
    alloc((void**)&L->router_counters, 256);
    alloc((void**)&L->x_stage, Tm * (size_t)c.hidden * 2);
    alloc((void**)&L->out_stage, Tm * (size_t)c.hidden * 2);
    if (e == cudaSuccess) e = cudaMemset(L->error_word, 0, 256);
    if (e == cudaSuccess) e = cudaMemset(L->router_counters, 0, 256);
    if (e != cudaSuccess) {
        layer_free(L);
        delete L;
        return set_error((int)e, "moe_layer: workspace allocation failed: %s", cudaGetErrorString(e));
    }
    if (int rc = router_configure()) {
        layer_free(L);
        delete L;
        return rc;
    }
    if (int rc = gemv_configure()) {
        layer_free(L);
        delete L;
        return rc;
    }
    const bool split_shared = L->shared != nullptr && (shared->fmt != routed->fmt || c.shared_ffn != c.ffn);
    dsx_moe_config c_ws = c;
    if (split_shared) c_ws.shared_ffn = 0;   // this layer's own launches carry no shared rows
    if (int rc = prefill_workspace_create(&L->pf, c_ws, c.router.n_used, L->mid, !takes_block_scaled(routed, split_shared ? nullptr : L->shared))) {
        layer_free(L);
        delete L;
        return rc;
    }
    if (L->pf.ready && routed->km_gu != nullptr)
        if (int rc = prefill_mx_workspace_create(&L->pf, c_ws, c.router.n_used)) {
            layer_free(L);
            delete L;
            return rc;
        }
    if (split_shared) {
        dsx_moe_config cs = c;
        cs.ffn = c.shared_ffn; cs.shared_ffn = 0;
        cs.router.n_expert = 1; cs.router.n_used = 1; cs.router.n_group = 1; cs.router.topk_group = 1;
        int rc = dsx_moe_layer_create(&L->sh_layer, &cs, shared, nullptr, router_w, nullptr);
        if (rc == DSX_OK) {
            cudaFree(L->sh_layer->partial);   // its rows live in this layer's buffer (set per call)
            L->sh_layer->partial = nullptr;
            cudaError_t e2 = cudaMalloc((void**)&L->sh_sel, Tm * 4);
            if (e2 == cudaSuccess) e2 = cudaMalloc((void**)&L->sh_w, Tm * 4);
            if (e2 == cudaSuccess) e2 = cudaMemset(L->sh_sel, 0, Tm * 4);
            if (e2 == cudaSuccess) {
                std::vector<float> ones(Tm, 1.0f);
                e2 = cudaMemcpy(L->sh_w, ones.data(), Tm * 4, cudaMemcpyHostToDevice);
            }
            if (e2 != cudaSuccess) rc = set_error((int)e2, "moe_layer: shared-expert workspace allocation failed: %s", cudaGetErrorString(e2));
        }
        if (rc != DSX_OK) {
            layer_free(L);
            delete L;
            return rc;
        }
    }
    *layer = L;
    return DSX_OK;
}

int dsx_moe_layer_destroy(dsx_moe_layer* L) {
    if (!L) return DSX_OK;
    layer_free(L);
    delete L;
    return DSX_OK;
}

int dsx_moe_layer_set_weights(dsx_moe_layer* L, const dsx_expert_store* routed, const dsx_expert_store* shared,
                              const float* router_w, const float* router_bias) {
    DSX_REQUIRE(L, "moe_layer_set_weights: null layer");
    if (int rc = check_weights(L->cfg, routed, shared, router_w)) return rc;
    const bool split_shared = L->cfg.shared_ffn > 0 && (shared->fmt != routed->fmt || L->cfg.shared_ffn != L->cfg.ffn);
    if (split_shared != (L->sh_layer != nullptr))
        return set_error(DSX_ERR_UNSUPPORTED, "moe_layer_set_weights: the layer was built for a shared expert that %s the routed experts' format; "
                                              "create a new layer", L->sh_layer ? "differs from" : "matches");
    if (L->sh_layer)
        if (int rc = dsx_moe_layer_set_weights(L->sh_layer, shared, nullptr, router_w, nullptr)) return rc;
    L->routed = routed; L->shared = L->cfg.shared_ffn > 0 ? shared : nullptr;
    L->router_w = router_w; L->router_bias = router_bias;
    if (!takes_block_scaled(routed, L->sh_layer ? nullptr : L->shared))
        if (int rc = prefill_f16_rows_ensure(&L->pf)) return rc;
    // the tensor maps of the prefill path describe the previous stores (a new store may even sit at a freed
    // store's address with another slot count): encode them again on the next use
    for (int i = 0; i < 2; i++) L->pf.mapped_gu_nib[i] = L->pf.mapped_dn_nib[i] = L->pf.mapped_km_gu[i] = L->pf.mapped_km_dn[i] = nullptr;
    return DSX_OK;
}

// The tensor-core path multiplies f16 weights: E2M1 (<= 6) x 2^(e-127) must stay finite in f16, i.e.
// e <= 140.  Reads the store's folded maximum once after its last load (synchronises then).
static bool scales_fit_f16(const dsx_expert_store* st) {
    if (st->fmt != DSX_FMT_MXFP4) return true;
    if (st->scale_dirty) {
        // MXFP4 scale planes hold nothing but E8M0 bytes: one maximum over both planes as they are now
        // (a slot reloaded with smaller scales lowers it again)
        uint32_t v = 255;
        const size_t n = (size_t)st->n_slots;
        if (cudaMemset(st->d_scale_max, 0, 4) != cudaSuccess) return false;
        if (launch_max_byte(st->gu_sc, (int64_t)(n * st->gu_sc_stride), st->d_scale_max, nullptr) != DSX_OK) return false;
        if (launch_max_byte(st->dn_sc, (int64_t)(n * st->dn_sc_stride), st->d_scale_max, nullptr) != DSX_OK) return false;
        if (cudaMemcpy(&v, st->d_scale_max, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
        st->h_scale_max = v;
        st->scale_dirty = false;
    }
    return st->h_scale_max <= 140u;
}

// picks -> out.  expert_lo / n_local select the owned id range (0 / n_expert for a full layer).
static int forward_core(dsx_moe_layer* L, const __nv_bfloat16* x, int64_t T, const int32_t* selected, const float* weights,
                        int expert_lo, bool filter_picks, int with_shared, __nv_bfloat16* out, cudaStream_t stream,
                        bool groups_ready = false, bool skip_combine = false, __nv_bfloat16* const* out_rows = nullptr) {
    const dsx_moe_config& c = L->cfg;
    const int k = c.router.n_used, n_local = L->routed->n_slots;
    // split: the shared expert runs as a pass of its own (sh_layer) between this layer's kernels and the combine
    const bool split = with_shared && L->sh_layer != nullptr;
    const bool shared = with_shared && L->shared != nullptr && !split;
    auto shared_pass_and_combine = [&]() -> int {
        if (split) {
            dsx_moe_layer* S = L->sh_layer;
            S->partial = L->partial + (size_t)T * k * c.hidden;   // the shared rows of this layer's partial buffer
            if (int rc = forward_core(S, x, T, L->sh_sel, L->sh_w, 0, false, 0, nullptr, stream, false, true)) return rc;
        }
        if (skip_combine) return DSX_OK;
        StageTimer tm(L, DSX_STAGE_COMBINE, stream);
        return launch_combine(L->partial, T, k, c.hidden, (shared || split) ? 1 : 0, filter_picks ? selected : nullptr, expert_lo, n_local, out,
                              stream, out_rows);
    };
    // MXFP4 stores with tensor-core planes: block-scaled FP4 MMAs on the stored codes and scales (any E8M0 scale);
    // otherwise f16 operands expanded in shared memory (Q8_0; MXFP4 scales must then fit f16)
    const bool mx = L->pf.mx_ready && takes_block_scaled(L->routed, shared ? L->shared : nullptr);
    if (prefill_wanted(L->pf, c, L->routed->fmt, T) &&
        (mx || (L->pf.xperm != nullptr && scales_fit_f16(L->routed) && (!shared || scales_fit_f16(L->shared))))) {
        PrefillCall pc{};
        pc.x = x; pc.T = T; pc.selected = selected; pc.route_w = weights; pc.expert_lo = expert_lo; pc.n_local = n_local;
        pc.filter_picks = filter_picks; pc.with_shared = shared; pc.out = out; pc.out_rows = out_rows;
        pc.skip_combine = skip_combine || split;
        pc.hist = L->hist; pc.offsets = L->offsets; pc.perm = L->perm; pc.gs = L->gs;
        pc.mid = L->mid; pc.partial = L->partial; pc.error_word = L->error_word; pc.sm_count = L->sm_count;
        pc.n_used = k; pc.clamp = c.clamp;
        pc.gu_nib = L->routed->gu_nib; pc.gu_sc = L->routed->gu_sc; pc.dn_nib = L->routed->dn_nib; pc.dn_sc = L->routed->dn_sc;
        pc.gu_nib_stride = L->routed->gu_nib_stride; pc.gu_sc_stride = L->routed->gu_sc_stride;
        pc.dn_nib_stride = L->routed->dn_nib_stride; pc.dn_sc_stride = L->routed->dn_sc_stride;
        if (shared) { pc.sh_gu_nib = L->shared->gu_nib; pc.sh_gu_sc = L->shared->gu_sc; pc.sh_dn_nib = L->shared->dn_nib; pc.sh_dn_sc = L->shared->dn_sc; }
        pc.fmt = L->routed->fmt;
        StageTimer tm(L, DSX_STAGE_GATE_UP, stream);
        if (mx) {
            pc.km_gu = L->routed->km_gu; pc.km_dn = L->routed->km_dn; pc.sf_gu = L->routed->sf_gu; pc.sf_dn = L->routed->sf_dn;
            pc.km_gu_stride = L->routed->km_gu_stride; pc.km_dn_stride = L->routed->km_dn_stride;
            pc.sf_gu_stride = L->routed->sf_gu_stride; pc.sf_dn_stride = L->routed->sf_dn_stride;
            if (shared) { pc.sh_km_gu = L->shared->km_gu; pc.sh_km_dn = L->shared->km_dn; pc.sh_sf_gu = L->shared->sf_gu; pc.sh_sf_dn = L->shared->sf_dn; }
            if (int rc = prefill_mx_forward(&L->pf, c, pc, stream)) return rc;
        } else if (int rc = prefill_forward(&L->pf, c, pc, stream)) {
            return rc;
        }
        return split ? shared_pass_and_combine() : DSX_OK;
    }
    if (!groups_ready) {   // the one-launch decode router has already built them
        StageTimer tm(L, DSX_STAGE_GROUP_BUILD, stream);
        if (int rc = launch_group_build(selected, T, k, n_local, expert_lo, 8, shared ? (int)T : 0, L->hist, L->offsets, L->perm,
                                        L->work_items, L->n_work_items, L->work_cap, L->gs, stream))
            return rc;
    }
    GemvArgs a{};
    a.fmt = L->routed->fmt; a.shared_fmt = shared ? L->shared->fmt : a.fmt; a.n_expert = n_local;
    a.work_items = L->work_items; a.n_work_items = L->n_work_items; a.offsets = L->offsets; a.perm = L->perm;
    // the decode router writes them for batches below 8 tokens; both kernels must have a small-batch form
    a.item_recs = (groups_ready && T < 8 && gemv_small_batch_ok(L->routed->fmt, c.hidden, c.ffn, T)) ? L->item_recs : nullptr;
    a.route_w = weights; a.n_used = k; a.T = T; a.clamp = c.clamp; a.x = x; a.mid = L->mid; a.mid_stride = c.ffn;
    a.partial = L->partial; a.error_word = L->error_word;
    // gate/up: rows = ffn, K = hidden
    a.K = c.hidden; a.rows = c.ffn; a.sh_rows = c.ffn;
    a.nib = L->routed->gu_nib; a.sc = L->routed->gu_sc; a.nib_slot_stride = L->routed->gu_nib_stride; a.sc_slot_stride = L->routed->gu_sc_stride;
    a.sh_nib = shared ? L->shared->gu_nib : nullptr; a.sh_sc = shared ? L->shared->gu_sc : nullptr;
    {
        StageTimer tm(L, DSX_STAGE_GATE_UP, stream);
        if (int rc = launch_gemv_gate_up(a, L->sm_count, stream)) return rc;
    }
    // down: rows = hidden, K = ffn
    a.K = c.ffn; a.rows = c.hidden; a.sh_rows = c.hidden;
    a.nib = L->routed->dn_nib; a.sc = L->routed->dn_sc; a.nib_slot_stride = L->routed->dn_nib_stride; a.sc_slot_stride = L->routed->dn_sc_stride;
    a.sh_nib = shared ? L->shared->dn_nib : nullptr; a.sh_sc = shared ? L->shared->dn_sc : nullptr;
    {
        StageTimer tm(L, DSX_STAGE_DOWN, stream);
        if (int rc = launch_gemv_down(a, L->sm_count, stream)) return rc;
    }
    return shared_pass_and_combine();
}

int dsx_moe_layer_forward(dsx_moe_layer* L, const void* x_bf16, int64_t T, void* out_bf16, const float* logits_in, dsx_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(L, "moe_layer_forward: null layer");
    DSX_REQUIRE(T >= 0 && T <= L->cfg.max_tokens, "moe_layer_forward: %lld tokens, workspace holds %d", (long long)T, L->cfg.max_tokens);
    if (T == 0) return DSX_OK;   // an empty batch has no rows to point at
    DSX_REQUIRE(x_bf16 && out_bf16, "moe_layer_forward: null argument");
    DSX_REQUIRE(L->routed->n_slots == L->cfg.router.n_expert, "moe_layer_forward: store holds %d of %d experts; use forward_picks",
                L->routed->n_slots, L->cfg.router.n_expert);
    const __nv_bfloat16* x = (const __nv_bfloat16*)x_bf16;
    const float* logits = logits_in;
    if (L->profile) for (bool& u : L->ev_used) u = false;
    if (!logits && router_fused_ok(T, L->cfg.router, L->cfg.hidden)) {
        // decode: logits, top-k and the group build in one launch
        {
            StageTimer tm(L, DSX_STAGE_ROUTER_LOGITS, stream);
            if (int rc = launch_router_fused(x, T, L->router_w, L->router_bias, L->cfg.hidden, L->cfg.router, L->logits, L->selected,
                                             L->weights, 8, (L->shared && !L->sh_layer) ? (int)T : 0, L->hist, L->offsets, L->perm, L->work_items,
                                             L->n_work_items, L->work_cap, T < 8 ? L->item_recs : nullptr, L->router_counters, L->error_word, stream))
                return rc;
        }
        L->last_logits = L->logits; L->last_selected = L->selected; L->last_weights = L->weights;
        return forward_core(L, x, T, L->selected, L->weights, 0, false, 1, (__nv_bfloat16*)out_bf16, stream, true);
    }
    if (!logits) {
        StageTimer tm(L, DSX_STAGE_ROUTER_LOGITS, stream);
        if (int rc = launch_router_logits(x, T, L->router_w, L->cfg.router.n_expert, L->cfg.hidden, L->logits, stream)) return rc;
        logits = L->logits;
    }
    {
        StageTimer tm(L, DSX_STAGE_ROUTER_TOPK, stream);
        if (int rc = launch_router_topk(logits, L->router_bias, T, L->cfg.router, L->selected, L->weights, 0, nullptr, nullptr, nullptr, stream)) return rc;
    }
    L->last_logits = logits; L->last_selected = L->selected; L->last_weights = L->weights;
    return forward_core(L, x, T, L->selected, L->weights, 0, false, 1, (__nv_bfloat16*)out_bf16, stream);
}

int dsx_moe_layer_forward_host(dsx_moe_layer* L, const void* x_host, int64_t T, void* out_host, dsx_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(L && x_host && out_host, "moe_layer_forward_host: null argument");
    DSX_REQUIRE(T >= 0 && T <= L->cfg.max_tokens, "moe_layer_forward_host: %lld tokens, workspace holds %d", (long long)T, L->cfg.max_tokens);
    const size_t bytes = (size_t)T * (size_t)L->cfg.hidden * 2;
    DSX_CUDA(cudaMemcpyAsync(L->x_stage, x_host, bytes, cudaMemcpyHostToDevice, stream));
    if (int rc = dsx_moe_layer_forward(L, L->x_stage, T, L->out_stage, nullptr, stream_)) return rc;
    DSX_CUDA(cudaMemcpyAsync(out_host, L->out_stage, bytes, cudaMemcpyDeviceToHost, stream));
    DSX_CUDA(cudaStreamSynchronize(stream));
    return DSX_OK;
}

int dsx_moe_layer_forward_picks(dsx_moe_layer* L, const void* x_bf16, int64_t T, const int32_t* selected, const float* weights,
                                int expert_lo, int with_shared, void* out_bf16, dsx_stream_t stream) {
    DSX_REQUIRE(L, "moe_layer_forward_picks: null layer");
    DSX_REQUIRE(T >= 0 && T <= L->cfg.max_tokens, "moe_layer_forward_picks: %lld tokens, workspace holds %d", (long long)T, L->cfg.max_tokens);
    if (T == 0) return DSX_OK;
    DSX_REQUIRE(x_bf16 && selected && weights && out_bf16, "moe_layer_forward_picks: null argument");
    L->last_logits = nullptr; L->last_selected = selected; L->last_weights = weights;
    return forward_core(L, (const __nv_bfloat16*)x_bf16, T, selected, weights, expert_lo, true, with_shared, (__nv_bfloat16*)out_bf16,
                        (cudaStream_t)stream);
}

int dsx_moe_layer_forward_picks_to(dsx_moe_layer* L, const void* x_bf16, int64_t T, const int32_t* selected, const float* weights,
                                   int expert_lo, int with_shared, void* const* out_rows, dsx_stream_t stream) {
    DSX_REQUIRE(L, "moe_layer_forward_picks_to: null layer");
    DSX_REQUIRE(T >= 0 && T <= L->cfg.max_tokens, "moe_layer_forward_picks_to: %lld tokens, workspace holds %d", (long long)T, L->cfg.max_tokens);
    if (T == 0) return DSX_OK;
    DSX_REQUIRE(x_bf16 && selected && weights && out_rows, "moe_layer_forward_picks_to: null argument");
    DSX_REQUIRE(L->cfg.hidden % 8 == 0, "moe_layer_forward_picks_to: hidden must be a multiple of 8");
    L->last_logits = nullptr; L->last_selected = selected; L->last_weights = weights;
    return forward_core(L, (const __nv_bfloat16*)x_bf16, T, selected, weights, expert_lo, true, with_shared, nullptr, (cudaStream_t)stream, false, false,
                        (__nv_bfloat16* const*)out_rows);
}

// picks (global expert ids) -> local slots of this owner: remap[e] < 0 means slot -(remap[e] + 1) is held here,
// remap[e] >= 0 means another device holds e (its slot there), ids outside [0, n_expert) -- NO_PICK, or the
// sentinel n_expert that pads fixed-shape launches -- are nobody's.  Everything not held here becomes -1.
__global__ void remap_picks_kernel(const int32_t* __restrict__ selected, const int32_t* __restrict__ remap, int n_expert, int n_slots,
                                   int64_t n, int32_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = selected[i];
    int slot = -1;
    if (e >= 0 && e < n_expert) {
        const int r = remap[e];
        if (r < 0 && -(r + 1) < n_slots) slot = -(r + 1);
    }
    out[i] = slot;
}

int dsx_moe_layer_forward_remap(dsx_moe_layer* L, const void* x_bf16, int64_t T, const int32_t* selected, const float* weights,
                                const int32_t* remap, int n_expert, int with_shared, void* out_bf16, dsx_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(L, "moe_layer_forward_remap: null layer");
    DSX_REQUIRE(T >= 0 && T <= L->cfg.max_tokens, "moe_layer_forward_remap: %lld tokens, workspace holds %d", (long long)T, L->cfg.max_tokens);
    if (T == 0) return DSX_OK;
    DSX_REQUIRE(x_bf16 && selected && weights && remap && out_bf16 && n_expert >= 1, "moe_layer_forward_remap: null argument");
    const int64_t n = T * L->cfg.router.n_used;
    remap_picks_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(selected, remap, n_expert, L->routed->n_slots, n, L->sel_local);
    DSX_LAUNCHED();
    L->last_logits = nullptr; L->last_selected = L->sel_local; L->last_weights = weights;
    return forward_core(L, (const __nv_bfloat16*)x_bf16, T, L->sel_local, weights, 0, true, with_shared, (__nv_bfloat16*)out_bf16, stream);
}

int dsx_moe_layer_routing(const dsx_moe_layer* L, const float** logits, const int32_t** selected, const float** weights,
                          const int32_t** hist, const int32_t** offsets, const int32_t** perm) {
    DSX_REQUIRE(L, "moe_layer_routing: null layer");
    if (logits) *logits = L->last_logits;
    if (selected) *selected = L->last_selected;
    if (weights) *weights = L->last_weights;
    if (hist) *hist = L->hist;
    if (offsets) *offsets = L->offsets;
    if (perm) *perm = L->perm;
    return DSX_OK;
}

int dsx_moe_layer_profile(dsx_moe_layer* L, int enable) {
    DSX_REQUIRE(L, "moe_layer_profile: null layer");
    if (enable)
        for (cudaEvent_t& e : L->ev)
            if (!e) DSX_CUDA(cudaEventCreate(&e));
    L->profile = enable != 0;
    return DSX_OK;
}

int dsx_moe_layer_stage_ms(dsx_moe_layer* L, float* ms) {
    DSX_REQUIRE(L && ms && L->profile, "moe_layer_stage_ms: profiling is off");
    for (int s = 0; s < DSX_STAGE_COUNT; s++) {
        ms[s] = -1.0f;
        if (!L->ev_used[s]) continue;
        DSX_CUDA(cudaEventSynchronize(L->ev[2 * s + 1]));
        DSX_CUDA(cudaEventElapsedTime(&ms[s], L->ev[2 * s], L->ev[2 * s + 1]));
    }
    return DSX_OK;
}

int dsx_moe_layer_check(dsx_moe_layer* L, dsx_stream_t stream_, uint32_t* error_word) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(L, "moe_layer_check: null layer");
    uint32_t w = 0;
    DSX_CUDA(cudaMemcpyAsync(&w, L->error_word, 4, cudaMemcpyDeviceToHost, stream));
    DSX_CUDA(cudaStreamSynchronize(stream));
    if (w) DSX_CUDA(cudaMemsetAsync(L->error_word, 0, 4, stream));
    if (L->sh_layer) {   // the shared expert's own pass reports into its own word
        uint32_t ws = 0;
        dsx_moe_layer_check(L->sh_layer, stream_, &ws);
        w |= ws;
    }
    if (error_word) *error_word = w;
    if (w)
        return set_error(DSX_ERR_DEVICE, "a kernel reported error word 0x%x (%s%s)", w, (w & 15u) ? "a bounded wait ran out" : "",
                         (w & 16u) ? ((w & 15u) ? "; a value left the f16 range" : "a value left the f16 range") : "");
    return DSX_OK;
}

}  // extern "C"
