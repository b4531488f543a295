/*
 * dsx_moe.h -- C ABI of the B200 (sm_100a) routed-MoE path for deepstrix.
 *
 * Two groups of entry points, matching the two interfaces the MoE path sits
 * behind in the reference (paths are relative to the deepstrix repository):
 *
 *   1. Device verbs ("v4flash-cuda"): the runtime calls that
 *      crates/v4flash-hip/src/sys.rs:206-382 declares against libamdhip64 and
 *      that buffer.rs / stream.rs / event.rs / graph.rs wrap.
 *   2. MoE operators: what crates/v4flash-kernels/src/{router_topk.rs,
 *      moe_group_builder.rs, mxfp4_pair.rs, mxfp4.rs, q2_k.rs, mxfp4_repack.rs,
 *      model_weights.rs} and het/dispatch.rs expose to the engine.
 *
 * Conventions: plain pointers and sizes only; every function returns 0 on
 * success or a negative dsx_status / positive cudaError_t; dsx_last_error()
 * returns a thread-local message.  No function synchronises the device unless
 * its comment says so.  All "device" pointers are CUDA device pointers of the
 * current device; streams are cudaStream_t passed as void*.
 *
 * There is no CPU fallback anywhere behind this header.
 */
#ifndef DSX_MOE_H
#define DSX_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSX_API __attribute__((visibility("default")))

typedef void* dsx_stream_t; /* cudaStream_t; NULL = default stream */
typedef void* dsx_event_t;  /* cudaEvent_t */
typedef void* dsx_graph_t;  /* cudaGraphExec_t */

enum dsx_status {
    DSX_OK = 0,
    DSX_ERR_INVALID = -1,     /* bad argument / size mismatch (launcher-side validation) */
    DSX_ERR_UNSUPPORTED = -2, /* shape or format outside what the kernels cover */
    DSX_ERR_DEVICE = -3,      /* a kernel reported a device-side error word (e.g. a bounded wait ran out) */
    DSX_ERR_NOMEM = -4
};

/* Thread-local text of the last failure (never NULL).
 * Replaces HipError{code,name,message,context}, crates/v4flash-hip/src/error.rs:10-78. */
DSX_API const char* dsx_last_error(void);

/* ------------------------------------------------------------------------
 * 1. Device verbs
 * ---------------------------------------------------------------------- */

/* hipGetDeviceCount / hipSetDevice / hipDeviceSynchronize -- sys.rs:206-222, device.rs:41-104 */
DSX_API int dsx_device_count(int* count);
DSX_API int dsx_device_set(int device);
DSX_API int dsx_device_get(int* device);
DSX_API int dsx_device_sync(void);
/* hipGetDeviceProperties subset: name (<=255 chars), SM count, total memory, cc major/minor -- device.rs */
DSX_API int dsx_device_props(int device, char* name256, int* sm_count, size_t* total_mem, int* cc_major, int* cc_minor);
/* hipDeviceCanAccessPeer / hipDeviceEnablePeerAccess -- sys.rs (peer access) */
DSX_API int dsx_device_enable_peer(int peer_device);

/* hipMalloc / hipFree / hipMemGetInfo / hipHostMalloc / hipHostFree -- sys.rs, buffer.rs:19-120,450-518 */
DSX_API int dsx_malloc(void** dptr, size_t bytes);
DSX_API int dsx_free(void* dptr);
DSX_API int dsx_mem_get_info(size_t* free_bytes, size_t* total_bytes);
DSX_API int dsx_host_malloc(void** hptr, size_t bytes); /* pinned */
DSX_API int dsx_host_free(void* hptr);

/* hipMemcpy / hipMemcpyAsync / hipMemcpyPeerAsync / hipMemset(Async) -- buffer.rs:121-434, het/sync.rs:1-7.
 * kind: 1 = host->device, 2 = device->host, 3 = device->device.  The blocking forms synchronise. */
DSX_API int dsx_memcpy(void* dst, const void* src, size_t bytes, int kind);
DSX_API int dsx_memcpy_async(void* dst, const void* src, size_t bytes, int kind, dsx_stream_t stream);
DSX_API int dsx_memcpy_peer_async(void* dst, int dst_device, const void* src, int src_device, size_t bytes, dsx_stream_t stream);
DSX_API int dsx_memset(void* dptr, int value, size_t bytes);
DSX_API int dsx_memset_async(void* dptr, int value, size_t bytes, dsx_stream_t stream);

/* Stream -- stream.rs:15-173 (create with priority, destroy, synchronize, query, wait_event) */
DSX_API int dsx_stream_create(dsx_stream_t* stream, int non_blocking, int priority);
DSX_API int dsx_stream_destroy(dsx_stream_t stream);
DSX_API int dsx_stream_sync(dsx_stream_t stream);
DSX_API int dsx_stream_query(dsx_stream_t stream, int* done);
DSX_API int dsx_stream_wait_event(dsx_stream_t stream, dsx_event_t event);

/* Event -- event.rs (create, record, synchronize, query, elapsed ms) */
DSX_API int dsx_event_create(dsx_event_t* event, int timing);
DSX_API int dsx_event_destroy(dsx_event_t event);
DSX_API int dsx_event_record(dsx_event_t event, dsx_stream_t stream);
DSX_API int dsx_event_sync(dsx_event_t event);
DSX_API int dsx_event_query(dsx_event_t event, int* done);
DSX_API int dsx_event_elapsed_ms(dsx_event_t start, dsx_event_t stop, float* ms);

/* Stream capture -> executable graph -- graph.rs:36-127 (begin/end capture, instantiate, launch) */
DSX_API int dsx_graph_begin_capture(dsx_stream_t stream);
DSX_API int dsx_graph_end_capture(dsx_stream_t stream, dsx_graph_t* graph_exec);
DSX_API int dsx_graph_launch(dsx_graph_t graph_exec, dsx_stream_t stream);
DSX_API int dsx_graph_destroy(dsx_graph_t graph_exec);
/* Re-pointing the kernels of an instantiated graph -- sys.rs:360-382 (hipGraphGetNodes, hipGraphKernelNodeGetParams,
 * hipGraphExecKernelNodeSetParams).  end_capture_keep also hands back the captured graph (the template; destroy it
 * with dsx_graph_template_destroy once no more updates are needed).  kernel_nodes lists its kernel nodes in the
 * driver's node order: call with nodes = NULL to get the count, then with room for *count handles.
 * set_params replaces a node's arguments in the executable graph; fn / grid / block may be NULL to keep the
 * node's kernel / grid / block and shared-memory size.  params uses the kernelParams ABI and is read during the call. */
DSX_API int dsx_graph_end_capture_keep(dsx_stream_t stream, dsx_graph_t* graph_exec, void** graph);
DSX_API int dsx_graph_template_destroy(void* graph);
DSX_API int dsx_graph_kernel_nodes(void* graph, void** nodes, size_t* count);
DSX_API int dsx_graph_exec_kernel_node_set_params(dsx_graph_t graph_exec, void* node, void* fn, const uint32_t grid[3],
                                                  const uint32_t block[3], uint32_t shared_bytes, void** params);

/* Code objects -- module.rs:28-57,141-171, launch.rs:25-40, sys.rs:317-330 (hipModuleLoadData / Unload /
 * GetFunction / LaunchKernel).  `image` is a cubin or fatbin in host memory (what `nvcc -cubin
 * -gencode arch=compute_100a,code=sm_100a` writes; a Rust crate embeds it with include_bytes!, as
 * crates/v4flash-kernels/build.rs:114-119 does for its code objects).  The module belongs to the device that
 * is current at load.  get_function keeps a name -> handle table per module (module.rs:37-57), so a lookup
 * per launch costs a map probe.  launch takes the CUDA "kernelParams" ABI: params[i] points at the i-th
 * argument, read during the call.  Kernels that use more than 48 KB of dynamic shared memory need
 * dsx_function_set_max_shared once.  deepstrix_b200/kernels/dsx_combine.cubin (kernel "dsx_combine_kernel")
 * is built beside the library as a loadable example of the library's own kernels. */
typedef struct dsx_module dsx_module;
typedef void* dsx_function_t; /* CUfunction, owned by its module */
DSX_API int dsx_module_load_data(const void* image, dsx_module** module);
DSX_API int dsx_module_unload(dsx_module* module);
DSX_API int dsx_module_get_function(dsx_module* module, const char* name, dsx_function_t* fn);
DSX_API int dsx_function_set_max_shared(dsx_function_t fn, uint32_t bytes);
DSX_API int dsx_function_launch(dsx_function_t fn, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_bytes,
                                dsx_stream_t stream, void** params);
/* hipStreamWaitValue32 / hipStreamWriteValue32 -- sys.rs:290-302; used to gate one stream on a value another
 * stream (or device) writes, het/forward_layer.rs:436-449.  The comparison happens when the stream reaches the
 * operation, not at the call.  flags: 0 = *addr >= value, 1 = ==, 2 = (*addr & value) != 0, 3 = ~(*addr | value) != 0.
 * addr is a 4-byte aligned device address. */
DSX_API int dsx_stream_wait_value32(dsx_stream_t stream, void* addr, uint32_t value, uint32_t flags);
DSX_API int dsx_stream_write_value32(dsx_stream_t stream, void* addr, uint32_t value);

/* ------------------------------------------------------------------------
 * 2. MoE operators
 * ---------------------------------------------------------------------- */

enum dsx_weight_fmt {
    DSX_FMT_MXFP4 = 0, /* E2M1 codes + E8M0 scale per 32 (src/mxfp4_tables.rs) */
    DSX_FMT_Q8_0 = 1   /* int8 + f16 scale per 32 (kernels/q8_0_matvec.hip:5-16) */
};

/* Source layouts accepted by dsx_expert_store_load (the loader's job,
 * v4flash-core/src/weight_src.rs:75-98 and hf_v41.rs:1150-1233). */
enum dsx_src_layout {
    DSX_SRC_MXFP4_HF = 0,   /* q: [rows, K/2] bytes, element 2i = low nibble; s: [rows, K/32] E8M0 (2^(e-127)) */
    DSX_SRC_MXFP4_GGML = 1, /* q: [rows, K/32] blocks of 17 B `e | qs[16]`; s unused */
    DSX_SRC_MXFP4_SB2 = 2,  /* q: [rows, K/256] super-blocks of 136 B (mxfp4_tables.rs:10-35); s unused */
    DSX_SRC_Q8_0_BLOCKS = 3,/* q: [rows, K/32] blocks of 34 B `f16 d | i8[32]`; s unused */
    DSX_SRC_Q8_0_SPLIT = 4  /* q: int8 [rows, K]; s: f16 [rows, K/32] (src/weights.rs:215-240 per-row split) */
};

enum dsx_matrix_kind { DSX_MAT_GATE = 0, DSX_MAT_UP = 1, DSX_MAT_DOWN = 2 };

enum dsx_score_fn {
    DSX_SCORE_SQRT_SOFTPLUS = 0, /* kernels/router_topk.hip:32-36,71 */
    DSX_SCORE_SIGMOID = 1        /* kernels/laguna_ops.hip:59 */
};

/* bytes_per_expert(dtype, k, rows): rows*(k/32)*17 for MXFP4, rows*(k/32)*34 for Q8_0
 * -- crates/v4flash-kernels/src/weight_contract.rs:146,363-366. */
DSX_API int dsx_bytes_per_expert(int fmt, int64_t k, int64_t rows, size_t* bytes);

/* --- Expert store: RoutedExpertWeights (src/model_weights.rs:41-52) ------
 * n_slots experts, each with gate [ffn, hidden], up [ffn, hidden] and
 * down [hidden, ffn], kept in HBM in this library's tile layout (16-row x
 * 64-column tiles for MXFP4, 16 x 32 for Q8_0; gate and up tiles interleaved
 * so one stream feeds the fused gate/up kernel).  Same byte count as the
 * reference (17 or 34 bytes per 32 weights). */
typedef struct dsx_expert_store dsx_expert_store;

DSX_API int dsx_expert_store_create(dsx_expert_store** store, int fmt, int n_slots, int64_t hidden, int64_t ffn);
/* An MXFP4 store holds every matrix twice: in the decode kernels' tile layout, and K-major (the HF
 * byte layout) with its E8M0 scales cut into the scale-factor chunks of the block-scaled tensor-core
 * kernel that runs batches above 64 tokens -- 34 bytes per 32 weights in all.  DSX_STORE_DECODE_ONLY
 * leaves the second copy out (17 bytes per 32 weights, the reference's byte count); large batches on
 * such a store run on the grouped-GEMV kernels.  Q8_0 stores have one copy either way. */
enum dsx_store_flags { DSX_STORE_DECODE_ONLY = 1 };
DSX_API int dsx_expert_store_create_ex(dsx_expert_store** store, int fmt, int n_slots, int64_t hidden, int64_t ffn, uint32_t flags);
DSX_API int dsx_expert_store_destroy(dsx_expert_store* store);
/* Repack one matrix of one slot from a source layout into the tile layout
 * (the role of mxfp4_repack_hf_to_ggml, kernels/mxfp4_repack.hip:35-65 and
 * load_experts_packed, het/weights.rs:1014-1203).  q/s are DEVICE pointers when
 * src_on_device != 0, host pointers otherwise (then the call stages them through
 * an internal device buffer and synchronises the stream). */
DSX_API int dsx_expert_store_load(dsx_expert_store* store, int slot, int which, int src_layout,
                                  const void* q, const void* s, int src_on_device, dsx_stream_t stream);
/* Inverse of the repack, for bit-parity tests: writes HF layout (MXFP4) or the
 * split layout (Q8_0) to DEVICE buffers q_out/s_out. */
DSX_API int dsx_expert_store_unpack(const dsx_expert_store* store, int slot, int which,
                                    void* q_out, void* s_out, dsx_stream_t stream);
/* Device-to-device clone of every plane (used to keep several layers resident). */
DSX_API int dsx_expert_store_clone(const dsx_expert_store* src, dsx_expert_store** dst, dsx_stream_t stream);
DSX_API int dsx_expert_store_info(const dsx_expert_store* store, int* fmt, int* n_slots, int64_t* hidden,
                                  int64_t* ffn, size_t* device_bytes);

/* --- Router --------------------------------------------------------------
 * logits[T,E] = x[T,H] (bf16) . W[E,H]^T (f32), f32 accumulate in an order
 * that does not depend on T (F16Matvec::matvec / matvec_batched_router,
 * kernels/f16_matvec.hip:26-45; het/forward_prefill.rs:8951-8973). */
DSX_API int dsx_router_logits(const void* x_bf16, int64_t T, const float* W, int n_expert, int64_t hidden,
                              float* logits, dsx_stream_t stream);

typedef struct {
    int32_t n_expert;    /* <= 512, multiple of 32 */
    int32_t n_used;      /* <= 16 (ROUTER_MAX_USED is 8 in router_topk_par.hip:14-22) */
    int32_t n_group;     /* <=1: no group limit (the reference); else experts split into contiguous groups */
    int32_t topk_group;  /* groups kept when n_group > 1 */
    int32_t score_fn;    /* dsx_score_fn */
    float route_scale;   /* expert_weight_scale */
    float weight_eps;    /* 6.103515625e-5 in het/forward_layer.rs:36 */
} dsx_router_config;

/* RouterTopk::launch_batched (src/router_topk.rs:245-364; kernels
 * router_topk_par.hip:66-238): p = f(logit); s = p + bias; k argmax passes,
 * equal scores -> lower index; w_j = p[sel_j] / max(sum, eps) * scale.
 * bias may be NULL.  selected: int32 [T, n_used] in rank order; weights f32. */
DSX_API int dsx_router_topk(const float* logits, const float* bias, int64_t T, const dsx_router_config* cfg,
                            int32_t* selected, float* weights, dsx_stream_t stream);
/* RouterTopk::launch_batched_ex (src/router_topk.rs:245-364; router_topk_par.hip:18-21,75-81,140-160,
 * 231-236): the same picks and weights, plus
 *   alts      int32 [T, n_alt]  ranks n_used+1 .. n_used+n_alt (further argmax passes; what box 2
 *                               substitutes for a pick it does not hold); NULL -> no alternatives
 *   alt_w     f32 [T, n_alt]    prob(alt) / (sum of the picks' probs) * scale; may be NULL
 *   range_out f32 [T]           max - min of the selection scores over all experts; may be NULL
 * n_used + n_alt <= 16.  The cache prior of the reference has its own entry point below. */
DSX_API int dsx_router_topk_ex(const float* logits, const float* bias, int64_t T, const dsx_router_config* cfg,
                               int32_t* selected, float* weights, int n_alt, int32_t* alts, float* alt_w,
                               float* range_out, dsx_stream_t stream);

/* The cache prior of RouterTopk::launch_batched_ex (router_topk_par.hip:82-99,173-210): prior[n_expert] is
 * added to the SELECTION score; the first n_protect picks of the plain ranking are always kept, the other
 * slots and the alternatives are the argmax of score + prior; weights come from the unbiased probabilities
 * of the emitted picks.  orig_sel (may be NULL): int32 [T, n_used], the plain top-n_used.  prior_dry != 0
 * swaps the roles: the plain picks are emitted and weighted, orig_sel carries the prior's choice.
 * No group limit (cfg->n_group <= 1); n_used + n_alt <= 32. */
DSX_API int dsx_router_topk_prior(const float* logits, const float* bias, int64_t T, const dsx_router_config* cfg,
                                  int32_t* selected, float* weights, int n_alt, int32_t* alts, float* alt_w,
                                  float* range_out, const float* prior, int n_protect, int prior_dry, int32_t* orig_sel,
                                  dsx_stream_t stream);

/* ExpertSelCount::launch (src/expert_sel_count.rs:34; kernels/expert_sel_count.hip:17-28): the selection
 * statistics bank, counts[layer_off + selected[i]] += 1 for every pick (u32, n_layer x n_expert, kept across
 * steps and harvested by the caller); ids outside [0, n_expert) are dropped. */
DSX_API int dsx_expert_sel_count(uint32_t* counts, const int32_t* selected, uint32_t layer_off, uint32_t n_expert,
                                 int64_t total, dsx_stream_t stream);

/* --- Histogram / permute / work items ------------------------------------
 * MoeGroupBuilder::launch + launch_work_items_split (src/moe_group_builder.rs:72-259;
 * kernels/moe_group_builder.hip:32-51, moe_work_items_builder.hip:61-145) with the
 * deterministic member order of b2_moe_group_wi_builder (kernels/b2_fast_chain.hip:94-105):
 *   hist[e]      picks of expert e (ids < 0 or >= n_expert are dropped)
 *   offsets[e]   exclusive prefix sum, n_expert+1 entries
 *   perm[offsets[e]+pos] = t*n_used+s, ascending inside each expert
 *   work_items[i] = (e << 16) | member_start, ceil(hist[e]/chunk) per expert,
 *                   sorted by expert; n_work_items[0] = their count
 * work_items needs room for dsx_wi_upper_bound(...) entries.  Limits as in
 * moe_group_builder.rs:18-31: T and every member_start must stay below 65536
 * for the packed work items (larger T: pass work_items = NULL). */
DSX_API int dsx_moe_group_build(const int32_t* selected, int64_t T, int n_used, int n_expert, int chunk,
                                int32_t* hist, int32_t* offsets, int32_t* perm,
                                int32_t* work_items, int32_t* n_work_items, dsx_stream_t stream);
/* Same operation and outputs as dsx_moe_group_build, for callers that must not
 * allocate device memory.  This entry point has no counterpart in the
 * reference.  Who needs it: an engine that hands the whole GPU to its own arena
 * at start-up (the way deepstrix sizes its per-layer scratch once), so that a
 * cudaMalloc made behind its back fails or eats into memory it has planned for;
 * and a serving loop that cannot afford the device-wide synchronisation an
 * allocation or a free may imply.  dsx_moe_group_build borrows a temporary
 * buffer from the driver when T * n_used exceeds 2048; this variant keeps that
 * buffer inside the library instead, as a fixed 128 KiB array in device memory
 * that every GPU which loads the library holds until the process exits.
 *   - Limit: T * n_used <= 131072 picks (for example 16384 tokens x top-8) and
 *     n_expert <= 512.  Larger inputs are refused with DSX_ERR_UNSUPPORTED and a
 *     message; nothing is launched.
 *   - It calls no cudaMalloc / cudaFree / cudaMallocAsync and no library routine
 *     that allocates.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and caches it; make that
 *     first call before starting any stream capture on that device.
 *   - All calls on one device share the one array.  Its previous contents never
 *     matter (every entry a call reads is first written by that call), but two
 *     calls that overlap on the GPU -- different streams, or different threads --
 *     race on it: issue them on one stream, or order them with events. */
DSX_API int dsx_moe_group_build_static(const int32_t* selected, int64_t T, int n_used, int n_expert, int chunk,
                                       int32_t* hist, int32_t* offsets, int32_t* perm,
                                       int32_t* work_items, int32_t* n_work_items, dsx_stream_t stream);
/* Q2KAccumulateMatvec::launch_reduce_partials[_hetsplit] (kernels/q2_k_accumulate_matvec_par.hip:705-766;
 * b2_reduce_partials_zero, b2_fast_chain.hip:137-189) followed by VecAddInplace (src/ffn.rs:118-151):
 *   out[t, :] = 0 + partial[t*n_used + 0, :] + ... + partial[t*n_used + n_used-1, :]   (slot order, f32 adds)
 *             + partial[T*n_used + t, :]                                              (when with_shared != 0)
 * written as bf16 [T, hidden].  partial: f32 [T*n_used (+ T), hidden], hidden a multiple of 8, both buffers 16-byte
 * aligned, n_used <= 32.  selected (optional, int32 [T, n_used]): slots whose pick lies outside
 * [expert_lo, expert_lo + n_local) are skipped (rows another owner computes). */
DSX_API int dsx_reduce_partials(const float* partial, int64_t T, int n_used, int64_t hidden, int with_shared,
                                const int32_t* selected, int expert_lo, int n_local, void* out_bf16, dsx_stream_t stream);
/* The same reduction with the result rows stored through a table: out_rows is a device array of T row pointers (bf16
 * [hidden] each, 16-byte aligned, possibly in another GPU's mapped memory); rows with a NULL entry are skipped. */
DSX_API int dsx_reduce_partials_to(const float* partial, int64_t T, int n_used, int64_t hidden, int with_shared,
                                   const int32_t* selected, int expert_lo, int n_local, void* const* out_rows, dsx_stream_t stream);
/* moe_wi_upper_bound, het/dispatch.rs:444-454 */
DSX_API uint32_t dsx_wi_upper_bound(uint64_t members, uint32_t groups, uint32_t chunk, uint64_t cap);

/* --- Whole layer ---------------------------------------------------------
 * One call = router GEMV -> top-k -> histogram/permute -> grouped gate/up +
 * clamp + SwiGLU + routing weight -> grouped down -> slot-order combine (+
 * shared expert).  The template in the reference is MtpState::moe
 * (het/mtp.rs:1606-1730) / MoeExecutor::run (het/remote_experts.rs:7428-7442). */
typedef struct {
    int32_t hidden;       /* multiple of 256 */
    int32_t ffn;          /* routed expert width, multiple of 256 */
    int32_t shared_ffn;   /* 0 = no shared expert */
    int32_t max_tokens;   /* workspace is sized for this many tokens per call */
    float clamp;          /* SwiGLU clamp (10.0 in config.rs:104); <= 1e-6 disables */
    dsx_router_config router;
} dsx_moe_config;

typedef struct dsx_moe_layer dsx_moe_layer;

/* routed: store with n_expert slots.  shared: store with 1 slot (or NULL).
 * router_w: DEVICE f32 [n_expert, hidden]; router_bias: DEVICE f32 [n_expert] or NULL.
 * The layer borrows all four (they must outlive it) and owns its workspace. */
DSX_API int dsx_moe_layer_create(dsx_moe_layer** layer, const dsx_moe_config* cfg,
                                 const dsx_expert_store* routed, const dsx_expert_store* shared,
                                 const float* router_w, const float* router_bias);
DSX_API int dsx_moe_layer_destroy(dsx_moe_layer* layer);
/* Re-point an existing layer (and its workspace) at another set of weights. */
DSX_API int dsx_moe_layer_set_weights(dsx_moe_layer* layer, const dsx_expert_store* routed,
                                      const dsx_expert_store* shared, const float* router_w, const float* router_bias);

/* x, out: DEVICE bf16 [T, hidden].  logits_in: optional DEVICE f32 [T, n_expert];
 * when given the router GEMV is skipped and these logits drive the routing
 * (the "pinned routing" of het/fidelity_tap.rs).  Asynchronous on `stream`.
 * Batches of 9..64 tokens route with one kernel whose n_expert/2 blocks meet at a barrier: they must all
 * be resident at once, so no other stream may occupy the device's SMs with long-running kernels while
 * this call runs.  If some blocks cannot start, the waiting ones give up after a bounded time, error
 * bit 8 is set (dsx_moe_layer_check returns DSX_ERR_DEVICE), the expert kernels of that call get an
 * empty work list and its output rows are undefined. */
DSX_API int dsx_moe_layer_forward(dsx_moe_layer* layer, const void* x_bf16, int64_t T, void* out_bf16,
                                  const float* logits_in, dsx_stream_t stream);
/* Same, with HOST buffers: copies x in, runs, copies out back, synchronises. */
DSX_API int dsx_moe_layer_forward_host(dsx_moe_layer* layer, const void* x_bf16_host, int64_t T,
                                       void* out_bf16_host, dsx_stream_t stream);

/* Expert-parallel form (what an owner of a subset of experts computes,
 * docs/v41/REMOTE_EXPERTS.md:204-229): the caller supplies the picks and
 * weights (ids outside [expert_lo, expert_lo + store slots) are skipped, as
 * NO_PICK is), and receives the weighted partial sum per token; with_shared
 * adds the shared expert. */
DSX_API int dsx_moe_layer_forward_picks(dsx_moe_layer* layer, const void* x_bf16, int64_t T,
                                        const int32_t* selected, const float* weights, int expert_lo,
                                        int with_shared, void* out_bf16, dsx_stream_t stream);
/* dsx_moe_layer_forward_picks with the result rows stored through a table instead of into one buffer: out_rows is a
 * device array of T row pointers (bf16 [hidden] each, 16-byte aligned, possibly in another GPU's mapped memory); a
 * NULL entry means the row is wanted nowhere and is not computed further.  hidden must be a multiple of 8. */
DSX_API int dsx_moe_layer_forward_picks_to(dsx_moe_layer* layer, const void* x_bf16, int64_t T, const int32_t* selected,
                                           const float* weights, int expert_lo, int with_shared, void* const* out_rows,
                                           dsx_stream_t stream);

/* The same with the reference's ownership table instead of a contiguous id range (encode_igpu_remap,
 * het/weights.rs:1357-1381; kernels/moe_group_builder.hip:53-123; docs/v41/REMOTE_EXPERTS.md:204-211):
 * remap is DEVICE int32 [n_expert]; remap[e] < 0 means this owner holds expert e in store slot -(remap[e] + 1),
 * remap[e] >= 0 means another device does (the value is its slot there and is not used here).  Picks < 0 or
 * >= n_expert (NO_PICK; the sentinel id n_expert that pads fixed-shape launches) belong to nobody.  Any placement
 * can be expressed: hot / cold splits, groups interleaved over GPUs.  Owners whose tables partition the experts
 * return partial sums that add up to the full layer. */
DSX_API int dsx_moe_layer_forward_remap(dsx_moe_layer* layer, const void* x_bf16, int64_t T, const int32_t* selected,
                                        const float* weights, const int32_t* remap, int n_expert, int with_shared,
                                        void* out_bf16, dsx_stream_t stream);

/* Device pointers into the layer's workspace holding the routing of the last
 * forward (valid until the next call): logits f32 [T,E], selected i32 [T,k],
 * weights f32 [T,k], hist i32 [E], offsets i32 [E+1], perm i32 [T*k].
 * Any output pointer may be NULL. */
DSX_API int dsx_moe_layer_routing(const dsx_moe_layer* layer, const float** logits, const int32_t** selected,
                                  const float** weights, const int32_t** hist, const int32_t** offsets,
                                  const int32_t** perm);
/* Reads (and clears) the device-side error word of the layer; synchronises
 * the stream.  Bits 1, 2, 4, 8: a bounded wait inside a kernel ran out (grouped
 * GEMV ring, tensor-core pipeline, router tile copy, wide-router grid barrier).
 * Bit 16: a value left the f16 range where a kernel multiplies in f16 (a token
 * value beyond +-65504 or not finite in a batch that takes the f16-operand
 * kernels, or a SwiGLU product beyond it with clamp = 0); the output rows it
 * feeds hold inf / NaN.  Returns DSX_ERR_DEVICE when the word is non-zero. */
DSX_API int dsx_moe_layer_check(dsx_moe_layer* layer, dsx_stream_t stream, uint32_t* error_word);
/* Per-stage device timing, the counterpart of EventPool::stage(name, stream)
 * (het/trace.rs:1-22): with profiling on, every forward brackets each stage with
 * a CUDA event pair on the caller's stream; dsx_moe_layer_stage_ms waits for the
 * last forward and returns DSX_STAGE_COUNT durations in ms (-1 = stage not run). */
enum dsx_stage {
    DSX_STAGE_ROUTER_LOGITS = 0, /* "dgpu.router" */
    DSX_STAGE_ROUTER_TOPK = 1,   /* "k.router.topk" */
    DSX_STAGE_GROUP_BUILD = 2,
    DSX_STAGE_GATE_UP = 3,       /* "igpu.pair_*" */
    DSX_STAGE_DOWN = 4,          /* "igpu.q2k_down" */
    DSX_STAGE_COMBINE = 5,
    DSX_STAGE_COUNT = 6
};
DSX_API int dsx_moe_layer_profile(dsx_moe_layer* layer, int enable);
DSX_API int dsx_moe_layer_stage_ms(dsx_moe_layer* layer, float* ms);
/* Kernel launches issued by this library on the calling thread since the last
 * reset (per-thread launch audit, crates/v4flash-hip/src/module.rs:97-131). */
DSX_API uint64_t dsx_launch_count(int reset);

/* --- The steps either side of the layer -------------------------------------
 * RmsNorm::launch_weighted_batched (src/rms_norm.rs:161-205; kernels/rms_norm.hip:48-84):
 *   out[t, i] = x[t, i] * (1 / sqrt(mean_i(x[t, i]^2) + eps)) * weight[i]
 * with the reference's summation order (thread j of 256 adds x[j + 256 m]^2 in double, the 256
 * partials are folded as f32 by a stride-128..1 tree).  Writes the bf16 rows the MoE layer reads
 * (out_bf16) and / or the f32 rows the reference writes (out_f32); either may be NULL. */
DSX_API int dsx_rms_norm_rows(const float* x, const float* weight, int64_t T, int64_t n, float eps, float* out_f32,
                              void* out_bf16, dsx_stream_t stream);
/* Reads (and clears) the device-side error word of the two kernels of this section on the current
 * device; synchronises the stream.  Non-zero (bit 1: a row copy inside dsx_rms_norm_rows never
 * arrived within its bounded wait, rows of that call are missing) returns DSX_ERR_DEVICE.
 * The reference has no such word: its kernels use no bounded waits. */
DSX_API int dsx_glue_check(dsx_stream_t stream, uint32_t* error_word);
/* hc_post_batched (kernels/hc_post.hip:36-68; src/head.rs:267-372; het/forward_layer.rs:3130-3152):
 *   out_hc[t, dst, d] = block_out[t, d] * post[t, dst] + sum_src comb[t, dst + src * n_hc] * residual_hc[t, src, d]
 * (one fused multiply-add per src, in src order).  block_out is the layer's bf16 output
 * (block_out_is_bf16 != 0) or f32 rows.  n_hc == 4 with 16-byte aligned rows takes a vectorised kernel;
 * other shapes are limited to 65535 tokens per call. */
DSX_API int dsx_hc_post(const void* block_out, int block_out_is_bf16, const float* residual_hc, const float* post,
                        const float* comb, int64_t T, int64_t n_embd, int n_hc, float* out_hc, dsx_stream_t stream);

/* --- Stand-alone operators of the expert path -------------------------------
 * For callers that drive the expert FFN step by step (the reference's
 * MoeExecutor hands Q8_K rows and runs matvec -> SwiGLU -> matvec -> add,
 * het/remote_experts.rs:7428-7442) instead of through dsx_moe_layer_forward.
 *
 * Q8KQuantize::launch / launch_with_offsets (src/q8_k.rs:33-104; kernels/q8_k_quantize.hip:23-90):
 * n_blocks blocks of 256 f32 values -> 292-byte block_q8_K records (f32 d | i8 qs[256] | i16 bsums[16]);
 *   max = the signed value of largest |x| (ties resolved as the reference kernel's stride-128..1 tree does),
 *   iscale = -127 / max, qs = clamp(rint(iscale * x), -128, 127), bsums[g] = sum of qs[16g .. 16g+15], d = 1 / iscale;
 * an all-zero block gives an all-zero record.  Offsets are applied by the caller to x (16-byte aligned) and
 * out (4-byte aligned: a record is 73 words).  Bit-exact. */
DSX_API int dsx_q8_k_quantize(const float* x, int64_t n_blocks, void* out, dsx_stream_t stream);
/* SwigluClampWeighted::launch (src/ffn.rs:91-114; kernels/swiglu_clamp_weighted.hip:16-37):
 *   mid[e, r] = silu(min(gate[e, r], clamp)) * min(max(up[e, r], -clamp), clamp) * expert_w[e]
 * (no clamping when clamp <= 1e-6), product taken left to right in f32.  The exponential inside silu is
 * evaluated from IEEE add / multiply / fma only (the routers' deterministic form), so results are
 * reproducible on a CPU bit for bit; they lie within 2 ulp of an expf-based evaluation.  ff_exp % 4 == 0,
 * rows 16-byte aligned. */
DSX_API int dsx_swiglu_clamp_weighted(float* mid, const float* gate, const float* up, const float* expert_w, float clamp,
                                      int64_t ff_exp, int64_t n_experts, dsx_stream_t stream);
/* VecAddInplace::launch (src/ffn.rs:135-151; kernels/vec_add.hip:6-13): out[i] += rhs[i], i < n. */
DSX_API int dsx_vec_add_inplace(float* out, const float* rhs, int64_t n, dsx_stream_t stream);
/* VecAddInplace::launch_gather (src/ffn.rs:155-177; kernels/vec_add.hip:18-27): out[i] = src[idx[i]] for
 * i < n; a negative index gives -inf. */
DSX_API int dsx_gather_f32(float* out, const float* src, const int32_t* idx, int64_t n, dsx_stream_t stream);

/* ------------------------------------------------------------------------
 * 3. Expert-parallel exchange over peer memory
 *
 * Replaces the transport of the reference's remote-expert path (TCP "DSXP",
 * het/remote_experts.rs: RemoteExpertClient::submit_dispatch :10060, the
 * executor's NO_PICK skipping :7428-7442; docs/v41/REMOTE_EXPERTS.md:163-164,
 * 196-229) for ranks that are processes on the GPUs of one node: what is sent
 * and returned is the same (a token row once per owning rank with all its
 * picks and weights; one weighted partial row back per received token; the
 * sender adds in rank order), but the rows are stored straight into the
 * owner's device memory, mapped through CUDA IPC, and nothing synchronises
 * with the host.  One step on one stream:
 *   dsx_ep_dispatch, dsx_ep_barrier, dsx_ep_prepare,
 *   dsx_moe_layer_forward_picks on the prepared rows (expert_lo = rank's first expert),
 *   dsx_ep_give_back, dsx_ep_barrier, dsx_ep_sum.
 * ---------------------------------------------------------------------- */
typedef struct dsx_ep_comm dsx_ep_comm;
/* cap: most tokens a rank dispatches in one step; at most 8 ranks. */
DSX_API int dsx_ep_create(int world, int rank, int64_t cap, int64_t hidden, int n_used, dsx_ep_comm** comm);
DSX_API int dsx_ep_destroy(dsx_ep_comm* comm);
/* 64-byte handle of this rank's receive slab; every rank passes all world handles, in rank order, to connect. */
DSX_API int dsx_ep_export(dsx_ep_comm* comm, uint8_t* handle64);
DSX_API int dsx_ep_connect(dsx_ep_comm* comm, const uint8_t* handles);
/* Ranks that live in one process on one device (tests): peers are plain pointers; the caller runs each
 * phase for every rank before the next phase and leaves the barriers out. */
DSX_API int dsx_ep_connect_local(dsx_ep_comm* comm, dsx_ep_comm* const* ranks);
/* Slots by exclusive scan over the tokens, rows + picks + weights stored into the owners' slabs. */
DSX_API int dsx_ep_dispatch(dsx_ep_comm* comm, const void* x_bf16, const int32_t* selected, const float* weights,
                            int64_t T, int n_expert, dsx_stream_t stream);
/* All ranks' earlier stores are visible after it.  The wait is bounded (error bit 1, see dsx_ep_check). */
DSX_API int dsx_ep_barrier(dsx_ep_comm* comm, dsx_stream_t stream);
/* How long a barrier waits for its peers before it gives up: `polls` polls of at least 100 ns each
 * (default 2^24, seconds).  A short limit lets a supervisor (or a test) see a missing rank as error
 * bit 1 within milliseconds; the kernel returns normally and the context stays usable.  The reference's
 * counterpart is the request timeout of its TCP transport (het/remote_experts.rs, RemoteExpertClient). */
DSX_API int dsx_ep_set_barrier_polls(dsx_ep_comm* comm, uint32_t polls);
/* Received rows [world*cap, hidden] bf16, their picks [world*cap, n_used] (-1 in unused slots) and weights. */
DSX_API int dsx_ep_prepare(dsx_ep_comm* comm, const void** x_rows, const int32_t** selected, const float** weights,
                           int64_t* n_slots, dsx_stream_t stream);
/* partial_rows [world*cap, hidden] bf16 (row i: weighted sum of slot i's owned picks) back to their sources. */
/* After dsx_ep_prepare: a device array of n_slots row pointers, entry i = where slot i's partial row belongs in its
 * source rank's slab (NULL for an unused slot).  An owner that lets its layer store the result rows through this table
 * (dsx_moe_layer_forward_picks_to) has handed them back -- the rows cross NVLink as the combine kernel produces them --
 * and skips dsx_ep_give_back.  (The reference's executor writes its partial rows into the reply frame it sends,
 * het/remote_experts.rs:7428-7442; there is no separate copy there either.) */
DSX_API int dsx_ep_back_rows(dsx_ep_comm* comm, void* const** rows);
DSX_API int dsx_ep_give_back(dsx_ep_comm* comm, const void* partial_rows_bf16, dsx_stream_t stream);
/* out[t] = shared[t] (or 0 when NULL) + the partial rows of token t in rank order, f32 adds, bf16 result. */
DSX_API int dsx_ep_sum(dsx_ep_comm* comm, const void* shared_bf16, int64_t T, void* out_bf16, dsx_stream_t stream);
/* Device array of `world` ints: rows received from every source this step (valid after the first barrier). */
DSX_API int dsx_ep_counts(dsx_ep_comm* comm, const int32_t** counts);
/* Reads and clears the error word (bit 1: a barrier gave up waiting); synchronises the stream.
 * Returns DSX_ERR_DEVICE when the word is non-zero, like dsx_moe_layer_check. */
DSX_API int dsx_ep_check(dsx_ep_comm* comm, dsx_stream_t stream, uint32_t* error_word);

#ifdef __cplusplus
}
#endif
#endif /* DSX_MOE_H */
