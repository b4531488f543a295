// Shared declarations of the B200 MoE library: error plumbing, the HBM tile
// layout of expert weights, and the device math every kernel agrees on.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/dsx_moe.h"

namespace dsx {

// ---------------------------------------------------------------- errors
int set_error(int code, const char* fmt, ...);
void count_launch();

#define DSX_CUDA(call)                                                                      \
    do {                                                                                    \
        cudaError_t _e = (call);                                                            \
        if (_e != cudaSuccess)                                                              \
            return ::dsx::set_error((int)_e, "%s failed: %s (%s:%d)", #call,                \
                                    cudaGetErrorString(_e), __FILE__, __LINE__);            \
    } while (0)

#define DSX_REQUIRE(cond, ...)                                                              \
    do {                                                                                    \
        if (!(cond)) return ::dsx::set_error(DSX_ERR_INVALID, __VA_ARGS__);                 \
    } while (0)

// Call right after a <<<>>> launch.
#define DSX_LAUNCHED()                                                                      \
    do {                                                                                    \
        ::dsx::count_launch();                                                              \
        DSX_CUDA(cudaGetLastError());                                                       \
    } while (0)

// Programmatic dependent launch: the decode chain (router -> gate/up -> down -> combine) is four
// short kernels, so each is launched with the stream-serialization attribute: its blocks may be
// scheduled while the previous kernel drains, do their set-up, and block in pdl_wait() until the
// previous grid has completed and its writes are visible.  Every kernel of the chain calls
// pdl_wait() before its first global access to data another kernel of the chain touches.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Error-word bit of a layer: a value did not fit f16 where a kernel multiplies in f16 (an activation beyond
// +-65504, an inf or a NaN; or an un-clamped SwiGLU product beyond it).  The result rows it feeds hold inf / NaN.
constexpr uint32_t kErrHalfRange = 16u;

// Two bf16 values (one 32-bit word) as f16x2.  `bad` collects a non-zero value when either result has all
// exponent bits set, i.e. the source was outside the f16 range or not finite.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w, uint32_t& bad) {
    const __half2 h = __floats2half2_rn(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    const uint32_t o = *reinterpret_cast<const uint32_t*>(&h);
    bad |= ((o & 0x7C007C00u) + 0x04000400u) & 0x80008000u;
    return o;
}
// f32 -> f16 with the same check
__device__ __forceinline__ __half f32_to_f16_checked(float v, uint32_t& bad) {
    const __half h = __float2half_rn(v);
    bad |= ((uint32_t)__half_as_ushort(h) & 0x7C00u) == 0x7C00u;
    return h;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// ------------------------------------------------------------ tile layout
// A weight matrix [rows, K] is stored as sub-tiles of 16 rows.  One sub-tile is
// what one warp feeds to mma.sync.m16n8k16 with a single 16-byte load per lane:
//   MXFP4: 16 rows x 64 columns = 512 B of 4-bit codes + 32 B of E8M0 scales
//   Q8_0 : 16 rows x 32 columns = 512 B of int8 (stored XOR 0x80) + 32 B of f16 scales
// Codes and scales live in two planes so every sub-tile starts 16-byte aligned
// (bulk-copy requirement).  Sub-tile order inside a plane: row tile major, then
// column tile; the gate/up plane interleaves [gate sub-tile][up sub-tile] per
// (row tile, column tile) so the fused kernel reads one contiguous stream.
//
// Lane l = 4*g + t of the warp owns bytes [16*l, 16*l+16) of a sub-tile.
// MXFP4 word s (s = 0..3, one per k16 step), column base c = 32*(s>>1) + 8*t + 4*(s&1):
//   byte0 = code(row g  , c+0) | code(row g  , c+1) << 4
//   byte1 = code(row g+8, c+0) | code(row g+8, c+1) << 4
//   byte2 = code(row g  , c+2) | code(row g  , c+3) << 4
//   byte3 = code(row g+8, c+2) | code(row g+8, c+3) << 4
// i.e. byte i converts (cvt.rn.f16x2.e2m1x2) straight into A-fragment register
// a_i of mma.m16n8k16.  Both 32-column scale blocks of the sub-tile map to two
// consecutive mma steps, and lane t reads 8 consecutive activation values per
// scale block.
// MXFP4 scales: bytes [4*g, 4*g+4) = {row g blk0, row g blk1, row g+8 blk0, row g+8 blk1}.
// Q8_0 word 2*s + h (s = k16 step, h = 0: row g, 1: row g+8): columns 8*t + 4*s + {0,1,2,3}.
// Q8_0 scales: halves [2*g, 2*g+2) = {row g, row g+8}.
constexpr int kTileRows = 16;
constexpr int kSubNibBytes = 512;
constexpr int kSubScBytes = 32;

__host__ __device__ inline int tile_k(int fmt) { return fmt == DSX_FMT_MXFP4 ? 64 : 32; }

struct MatrixView {       // one matrix (or gate/up pair) of one expert slot, tile layout
    const uint8_t* nib;   // sub-tile code plane
    const uint8_t* sc;    // sub-tile scale plane
};

// --------------------------------------------------- deterministic math
// exp / log1p from IEEE add, mul and fma only, so that a CPU restatement using
// fmaf() rounds identically.  Coefficients: Cephes expf / logf.
__device__ __forceinline__ float det_expf(float x) {
    x = fminf(fmaxf(x, -87.0f), 88.0f);
    const float n = floorf(__fmaf_rn(x, 1.44269504088896341f, 0.5f));
    float r = __fmaf_rn(n, -0.693359375f, x);
    r = __fmaf_rn(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    const float r2 = __fmul_rn(r, r);
    float y = __fmaf_rn(p, r2, r);
    y = __fadd_rn(y, 1.0f);
    return __fmul_rn(y, __uint_as_float((uint32_t)((int)n + 127) << 23));
}

__device__ __forceinline__ float det_logf(float u) {
    const uint32_t b = __float_as_uint(u);
    int e = (int)(b >> 23) - 126;
    float m = __uint_as_float((b & 0x007FFFFFu) | 0x3F000000u);
    if (m < 0.707106781186547524f) {
        e -= 1;
        m = __fadd_rn(__fadd_rn(m, m), -1.0f);
    } else {
        m = __fadd_rn(m, -1.0f);
    }
    const float z = __fmul_rn(m, m);
    float y = 7.0376836292e-2f;
    y = __fmaf_rn(y, m, -1.1514610310e-1f);
    y = __fmaf_rn(y, m, 1.1676998740e-1f);
    y = __fmaf_rn(y, m, -1.2420140846e-1f);
    y = __fmaf_rn(y, m, 1.4249322787e-1f);
    y = __fmaf_rn(y, m, -1.6668057665e-1f);
    y = __fmaf_rn(y, m, 2.0000714765e-1f);
    y = __fmaf_rn(y, m, -2.4999993993e-1f);
    y = __fmaf_rn(y, m, 3.3333331174e-1f);
    y = __fmul_rn(y, m);
    y = __fmul_rn(y, z);
    const float fe = (float)e;
    y = __fmaf_rn(fe, -2.12194440e-4f, y);
    y = __fmaf_rn(z, -0.5f, y);
    float r = __fadd_rn(m, y);
    r = __fmaf_rn(fe, 0.693359375f, r);
    return r;
}

__device__ __forceinline__ float det_log1pf(float y) {
    const float u = __fadd_rn(1.0f, y);
    if (u == 1.0f) return y;
    const float d = __fadd_rn(u, -1.0f);
    return __fmul_rn(det_logf(u), __fdiv_rn(y, d));
}

// Router probability, kernels/router_topk.hip:32-36,71 and laguna_ops.hip:59
// of the reference, on the deterministic exp/log above.
__device__ __forceinline__ float router_prob(float logit, int score_fn) {
    if (score_fn == DSX_SCORE_SIGMOID) return __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(-logit)));
    float sp;
    if (logit > 20.0f) sp = logit;
    else if (logit < -20.0f) sp = det_expf(logit);
    else sp = det_log1pf(det_expf(logit));
    return __fsqrt_rn(sp);
}

// One decode work item (an expert and up to 8 of its tokens) spelled out for the grouped GEMV:
// written by the decode router's group build, read with one coalesced load per item.
struct ItemRec {
    int32_t expert;       // local slot; n_expert means the shared expert
    int32_t n_tok;
    int32_t tok[8];       // token index (gate/up source row)
    int32_t mid_row[8];   // row of mid (expert-sorted order)
    int32_t out_row[8];   // row of partial (t*k+s, or P+t for the shared expert)
    float w[8];           // routing weight
    int32_t pad[2];
};
static_assert(sizeof(ItemRec) == 144, "ItemRec is 36 words");
constexpr int kItemRecWords = 34;   // words of an ItemRec that carry data

// ------------------------------------------------------- kernel launchers
// (defined in the .cu file named in the comment; all asynchronous on `stream`)

// repack.cu
int launch_repack(int fmt, int src_layout, const uint8_t* q, const uint8_t* s, int64_t rows, int64_t K,
                  uint8_t* nib, uint8_t* sc, int pair_stride, int pair_index, int n_mats, int64_t src_q_stride,
                  int64_t src_s_stride, int64_t dst_nib_stride, int64_t dst_sc_stride, cudaStream_t stream);
int launch_unpack(int fmt, const uint8_t* nib, const uint8_t* sc, int64_t rows, int64_t K, int pair_stride,
                  int pair_index, uint8_t* q_out, uint8_t* s_out, cudaStream_t stream);

// MXFP4 source layout -> the tensor-core planes (K-major codes + scale-factor chunks); pair_index 0 / 1 = gate / up,
// -1 = down (256-row tiles).
int launch_kmajor_mxfp4(int src_layout, const uint8_t* q, const uint8_t* s, int64_t rows, int64_t K, int pair_index, int n_mats,
                        int64_t src_q_stride, int64_t src_s_stride, uint8_t* km, int64_t km_stride, uint8_t* sf, int64_t sf_stride,
                        cudaStream_t stream);
int launch_max_byte(const uint8_t* p, int64_t bytes, uint32_t* out, cudaStream_t stream);

// router.cu
int launch_router_logits(const __nv_bfloat16* x, int64_t T, const float* W, int n_expert, int64_t H, float* logits,
                         cudaStream_t stream);
int launch_router_topk(const float* logits, const float* bias, int64_t T, const dsx_router_config& cfg,
                       int32_t* selected, float* weights, int n_alt, int32_t* alts, float* alt_w, float* range_out, cudaStream_t stream);
int launch_router_topk_prior(const float* logits, const float* bias, int64_t T, const dsx_router_config& cfg, int32_t* selected,
                             float* weights, int n_alt, int32_t* alts, float* alt_w, float* range_out, const float* prior, int n_protect,
                             int prior_dry, int32_t* orig_sel, cudaStream_t stream);
int router_configure();
bool router_fused_ok(int64_t T, const dsx_router_config& cfg, int64_t H);
int launch_router_fused(const __nv_bfloat16* x, int64_t T, const float* W, const float* bias, int64_t H, const dsx_router_config& cfg,
                        float* logits, int32_t* selected, float* weights, int chunk, int shared_T, int32_t* hist, int32_t* offsets,
                        int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap, ItemRec* item_recs,
                        unsigned int* counters, uint32_t* error_word, cudaStream_t stream);

// groups.cu
struct GroupScratch {      // device scratch for the multi-block counting sort
    int32_t* chunk_hist;   // [n_chunks, n_expert]
    int64_t capacity_chunks;
};
constexpr int kGroupChunk = 2048;  // picks per block of the counting sort
int launch_group_build(const int32_t* selected, int64_t T, int n_used, int n_expert, int expert_lo, int chunk,
                       int shared_items_for_T, int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items,
                       int32_t* n_work_items, int32_t work_cap, GroupScratch scratch, cudaStream_t stream);

int launch_expert_sel_count(unsigned int* counts, const int32_t* selected, unsigned int layer_off, unsigned int n_expert, int64_t total,
                            cudaStream_t stream);
int launch_group_build_static(const int32_t* selected, int64_t T, int n_used, int n_expert, int chunk, int32_t* hist,
                              int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap,
                              cudaStream_t stream);

// gemv.cu
struct GemvArgs {
    int fmt;                 // routed store format
    int shared_fmt;
    int n_expert;            // routed slots; item expert id == n_expert means "shared expert"
    int64_t K;               // reduction length (hidden for gate/up, ffn for down)
    int64_t rows;            // output rows per matrix (ffn for gate/up, hidden for down)
    const uint8_t* nib;      // plane base, routed
    const uint8_t* sc;
    int64_t nib_slot_stride; // bytes between expert slots
    int64_t sc_slot_stride;
    const uint8_t* sh_nib;   // shared expert planes (may be null)
    const uint8_t* sh_sc;
    int64_t sh_rows;
    const int32_t* work_items;   // (e<<16)|member_start, chunk 8
    const int32_t* n_work_items;
    const ItemRec* item_recs;    // one record per work item, or null (the kernel then derives them from offsets / perm / route_w)
    const int32_t* offsets;      // [n_expert+1]
    const int32_t* perm;         // [P]
    const float* route_w;        // [P] routing weights indexed by t*k+s
    int n_used;
    int64_t T;
    float clamp;
    const __nv_bfloat16* x;      // gate/up: [T, K] bf16
    __half* mid;                 // gate/up out / down in: [P + T, ffn] f16, permuted order
    int64_t mid_stride;          // elements per mid row
    float* partial;              // down out: [P + T, rows] f32, indexed t*k+s (shared: P+t)
    uint32_t* error_word;
};
int launch_gemv_gate_up(const GemvArgs& a, int sm_count, cudaStream_t stream);
int launch_gemv_down(const GemvArgs& a, int sm_count, cudaStream_t stream);
int gemv_configure();  // opt in to large dynamic shared memory (once per device)
bool gemv_fits(int64_t K);  // the kernels' shared memory holds a reduction of this length
bool gemv_small_batch_ok(int fmt, int64_t hidden, int64_t ffn, int64_t T);  // item records may be used for this chain

// combine.cu
int launch_combine(const float* partial, int64_t T, int n_used, int64_t H, int with_shared, const int32_t* selected,
                   int expert_lo, int n_local, __nv_bfloat16* out, cudaStream_t stream, __nv_bfloat16* const* out_rows = nullptr);

}  // namespace dsx
