// Router: logits GEMV and top-k selection.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   logits  crates/v4flash-kernels/kernels/f16_matvec.hip:26-45 (warp per row, f32 accumulate)
//   top-k   crates/v4flash-kernels/kernels/router_topk_par.hip:66-238 (k argmax passes, lower
//           index wins ties) and :294-434 (the 64-bit-key wave-reduction twin whose key
//           `(ord(score) << 32) | ~index` is reused here)
//   sigmoid crates/v4flash-kernels/kernels/laguna_ops.hip:55-62
#include <algorithm>

#include "groups.cuh"

namespace dsx {
namespace {

constexpr int kLogitWarps = 8;
constexpr int kLogitTokens = 8;  // tokens per warp pass

// One warp per (expert, tile of kLogitTokens tokens).  Lane l accumulates
// columns 4*l + 128*i in increasing i with one fma per element, then the warp
// folds with an xor butterfly: the f32 operation sequence of a (token, expert)
// pair is the same for every T, so decode and prefill route identically.
__global__ void __launch_bounds__(kLogitWarps * 32)
router_logits_kernel(const __nv_bfloat16* __restrict__ x, int64_t T, const float* __restrict__ W, int n_expert,
                     int64_t H, float* __restrict__ logits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * kLogitWarps + warp;
    if (e >= n_expert) return;
    const int64_t t0 = (int64_t)blockIdx.y * kLogitTokens;
    const int nt = (int)min((int64_t)kLogitTokens, T - t0);
    float acc[kLogitTokens];
    const uint2* xrow[kLogitTokens];
#pragma unroll
    for (int i = 0; i < kLogitTokens; i++) {
        acc[i] = 0.0f;
        // rows past the batch alias the last valid row: every load is legal, so the
        // compiler can issue all loads of an iteration before the first fma
        xrow[i] = reinterpret_cast<const uint2*>(x + min(t0 + i, T - 1) * H) + lane;
    }
    const float4* wrow = reinterpret_cast<const float4*>(W + (int64_t)e * H) + lane;
    const int n_iter = (int)(H >> 7);
#pragma unroll 2
    for (int i = 0; i < n_iter; i++) {
        const float4 w = __ldg(wrow + i * 32);
        uint2 xv[kLogitTokens];
#pragma unroll
        for (int tt = 0; tt < kLogitTokens; tt++) xv[tt] = __ldg(xrow[tt] + i * 32);
#pragma unroll
        for (int tt = 0; tt < kLogitTokens; tt++) {
            const float x0 = __uint_as_float(xv[tt].x << 16), x1 = __uint_as_float(xv[tt].x & 0xFFFF0000u);
            const float x2 = __uint_as_float(xv[tt].y << 16), x3 = __uint_as_float(xv[tt].y & 0xFFFF0000u);
            float a = acc[tt];
            a = __fmaf_rn(w.x, x0, a);
            a = __fmaf_rn(w.y, x1, a);
            a = __fmaf_rn(w.z, x2, a);
            a = __fmaf_rn(w.w, x3, a);
            acc[tt] = a;
        }
    }
#pragma unroll
    for (int tt = 0; tt < kLogitTokens; tt++) {
        float a = acc[tt];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, off));
        if (lane == 0 && tt < nt) logits[(t0 + tt) * n_expert + e] = a;
    }
}

__device__ __forceinline__ uint32_t ordered_bits(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

constexpr int kTopkWarps = 8;
constexpr int kMaxUsed = 16;

// Top-k of one token by one warp, VPL experts per lane (expert e = lane*VPL + j).
// s_score: E floats of shared memory private to the warp.
template <int VPL, typename LoadLogit>
__device__ __forceinline__ void topk_one_token(LoadLogit load_logit, const float* __restrict__ bias, const dsx_router_config& cfg,
                                               int32_t* __restrict__ sel_out, float* __restrict__ w_out, float* s_score) {
    const int lane = threadIdx.x & 31;
    const int E = VPL * 32;
    float p[VPL], s[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        const int e = lane * VPL + j;
        p[j] = router_prob(load_logit(e), cfg.score_fn);
        s[j] = bias ? __fadd_rn(p[j], bias[e]) : p[j];
    }
    if (cfg.n_group > 1) {
        // group score = sum of the two largest selection scores of the group;
        // keep the topk_group best groups (equal -> lower group index)
#pragma unroll
        for (int j = 0; j < VPL; j++) s_score[lane * VPL + j] = s[j];
        __syncwarp();
        const int per = E / cfg.n_group;
        float gs = -INFINITY;
        if (lane < cfg.n_group) {
            float m1 = -INFINITY, m2 = -INFINITY;
            for (int i = 0; i < per; i++) {
                const float v = s_score[lane * per + i];
                if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
            }
            gs = __fadd_rn(m1, m2);
        }
        int rank = 0;
        for (int h = 0; h < cfg.n_group; h++) {
            const float o = __shfl_sync(0xFFFFFFFFu, gs, h);
            if (o > gs || (o == gs && h < lane)) rank++;
        }
        const uint32_t keep = __ballot_sync(0xFFFFFFFFu, lane < cfg.n_group && rank < cfg.topk_group);
#pragma unroll
        for (int j = 0; j < VPL; j++) {
            const int grp = (lane * VPL + j) / per;
            if (!((keep >> grp) & 1u)) s[j] = -INFINITY;
        }
        __syncwarp();
    }
    unsigned long long key[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++)
        // adding +0 turns -0 into +0, so scores that compare equal get equal key prefixes
        key[j] = ((unsigned long long)ordered_bits(__fadd_rn(s[j], 0.0f)) << 32) |
                 (unsigned long long)(0xFFFFFFFFu - (uint32_t)(lane * VPL + j));
    float psel[kMaxUsed];
    int esel[kMaxUsed];
#pragma unroll
    for (int r = 0; r < kMaxUsed; r++) {
        if (r < cfg.n_used) {
            unsigned long long best = key[0];
#pragma unroll
            for (int j = 1; j < VPL; j++) best = key[j] > best ? key[j] : best;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const unsigned long long o = __shfl_xor_sync(0xFFFFFFFFu, best, off);
                best = o > best ? o : best;
            }
            const int e = (int)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull));
            const int owner = e / VPL, jj = e - owner * VPL;
            float pv = 0.0f;
#pragma unroll
            for (int j = 0; j < VPL; j++)
                if (lane == owner && j == jj) { pv = p[j]; key[j] = 0ull; }
            psel[r] = __shfl_sync(0xFFFFFFFFu, pv, owner);
            esel[r] = e;
        }
    }
    // weights from the unbiased probabilities, summed in slot order
    float sum = 0.0f;
#pragma unroll
    for (int r = 0; r < kMaxUsed; r++)
        if (r < cfg.n_used) sum = __fadd_rn(sum, psel[r]);
    if (sum < cfg.weight_eps) sum = cfg.weight_eps;
#pragma unroll
    for (int r = 0; r < kMaxUsed; r++)
        if (r < cfg.n_used && lane == (r & 31)) {
            sel_out[r] = esel[r];
            w_out[r] = __fmul_rn(__fdiv_rn(psel[r], sum), cfg.route_scale);
        }
}

template <int VPL>
__global__ void __launch_bounds__(kTopkWarps * 32)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T, dsx_router_config cfg,
                   int32_t* __restrict__ selected, float* __restrict__ weights) {
    __shared__ float s_score[kTopkWarps][VPL * 32];
    const int warp = threadIdx.x >> 5;
    const int64_t t = (int64_t)blockIdx.x * kTopkWarps + warp;
    if (t >= T) return;
    const float* row = logits + t * (VPL * 32);
    topk_one_token<VPL>([&](int e) { return row[e]; }, bias, cfg, selected + t * cfg.n_used, weights + t * cfg.n_used, s_score[warp]);
}

// ---- Decode router in ONE launch (T <= 64, E <= 256): logits, top-k and the group build.
// Grid (E/8, ceil(T/8)), 8 warps.  Each block stages its 8 token rows in shared memory and its warps
// stream one router row each (same f32 operation order as router_logits_kernel, so the logits
// are the same bits).  The last block of a token tile to finish (ticket counter) selects the
// experts of that tile's tokens, one warp per token; the last tile to finish builds histogram,
// offsets, permutation and work items.  The counters return to zero for the next launch.
template <int VPL>
__global__ void __launch_bounds__(kLogitWarps * 32)
router_fused_kernel(const __nv_bfloat16* __restrict__ x, int T, const float* __restrict__ W, const float* __restrict__ bias, int H,
                    dsx_router_config cfg, float* __restrict__ logits, int32_t* __restrict__ selected, float* __restrict__ weights,
                    int chunk, int shared_T, int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items,
                    int32_t* n_work_items, int32_t work_cap, unsigned int* counters /* [0]: tiles done, [1 + tile]: blocks done */) {
    extern __shared__ __align__(16) uint8_t fsm[];
    __shared__ int s_flag;
    __shared__ int s_warp[kLogitWarps + 1];
    constexpr int E = VPL * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.y, t0 = tile * kLogitTokens;
    const int nt = min(kLogitTokens, T - t0);
    // token rows of the tile -> shared memory (rows past the batch alias the last valid row)
    uint2* xs = reinterpret_cast<uint2*>(fsm);   // [8][H/4] of 4 x bf16
    const int vec = H >> 2;
    for (int i = threadIdx.x; i < kLogitTokens * vec; i += kLogitWarps * 32) {
        const int r = i / vec, c = i - r * vec;
        xs[i] = __ldg(reinterpret_cast<const uint2*>(x + (int64_t)min(t0 + r, T - 1) * H) + c);
    }
    __syncthreads();
    const int e = blockIdx.x * kLogitWarps + warp;
    {
        float acc[kLogitTokens];
#pragma unroll
        for (int i = 0; i < kLogitTokens; i++) acc[i] = 0.0f;
        const float4* wrow = reinterpret_cast<const float4*>(W + (int64_t)e * H) + lane;
        const int n_iter = H >> 7;
#pragma unroll 8
        for (int i = 0; i < n_iter; i++) {
            const float4 w = __ldg(wrow + i * 32);
#pragma unroll
            for (int tt = 0; tt < kLogitTokens; tt++) {
                const uint2 xv = xs[tt * vec + i * 32 + lane];
                const float x0 = __uint_as_float(xv.x << 16), x1 = __uint_as_float(xv.x & 0xFFFF0000u);
                const float x2 = __uint_as_float(xv.y << 16), x3 = __uint_as_float(xv.y & 0xFFFF0000u);
                float a = acc[tt];
                a = __fmaf_rn(w.x, x0, a);
                a = __fmaf_rn(w.y, x1, a);
                a = __fmaf_rn(w.z, x2, a);
                a = __fmaf_rn(w.w, x3, a);
                acc[tt] = a;
            }
        }
#pragma unroll
        for (int tt = 0; tt < kLogitTokens; tt++) {
            float a = acc[tt];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, off));
            if (lane == 0 && tt < nt) logits[(int64_t)(t0 + tt) * E + e] = a;
        }
    }
    // ---- last block of this token tile?
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_flag = (atomicAdd(&counters[1 + tile], 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (!s_flag) return;
    if (threadIdx.x == 0) counters[1 + tile] = 0u;
    __threadfence();
    float* s_score = reinterpret_cast<float*>(fsm);   // the token rows are no longer needed
    if (warp < nt) {
        const float* row = logits + (int64_t)(t0 + warp) * E;
        topk_one_token<VPL>([&](int ee) { return __ldcg(row + ee); }, bias, cfg, selected + (int64_t)(t0 + warp) * cfg.n_used,
                            weights + (int64_t)(t0 + warp) * cfg.n_used, s_score + warp * E);
    }
    // ---- last tile of the launch?
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_flag = (atomicAdd(&counters[0], 1u) == gridDim.y - 1) ? 1 : 0;
    __syncthreads();
    if (!s_flag) return;
    if (threadIdx.x == 0) counters[0] = 0u;
    __threadfence();
    int* wh = reinterpret_cast<int*>(fsm);
    groupdev::build_small<kLogitWarps * 32>(selected, (int64_t)T * cfg.n_used, E, 0, chunk, shared_T, hist, offsets, perm, work_items,
                                            n_work_items, work_cap, wh, s_warp);
}

}  // namespace

// Shapes the one-launch decode router covers (everything else takes the three separate kernels).
bool router_fused_ok(int64_t T, const dsx_router_config& cfg, int64_t H) {
    const int v = cfg.n_expert / 32;
    return T >= 1 && T <= 64 && cfg.n_expert % 32 == 0 && (v == 1 || v == 2 || v == 4 || v == 8) && H % 128 == 0 &&
           (size_t)kLogitTokens * H * 2 <= 96 * 1024 && T * cfg.n_used <= kGroupChunk && cfg.n_used <= kMaxUsed &&
           (cfg.n_group <= 1 || (cfg.n_group <= 32 && cfg.n_expert % cfg.n_group == 0));
}

int launch_router_logits(const __nv_bfloat16* x, int64_t T, const float* W, int n_expert, int64_t H, float* logits,
                         cudaStream_t stream) {
    DSX_REQUIRE(H % 128 == 0, "router_logits: hidden %lld must be a multiple of 128", (long long)H);
    if (T == 0) return DSX_OK;
    dim3 grid((unsigned)((n_expert + kLogitWarps - 1) / kLogitWarps), (unsigned)((T + kLogitTokens - 1) / kLogitTokens));
    router_logits_kernel<<<grid, kLogitWarps * 32, 0, stream>>>(x, T, W, n_expert, H, logits);
    DSX_LAUNCHED();
    return DSX_OK;
}

int launch_router_fused(const __nv_bfloat16* x, int64_t T, const float* W, const float* bias, int64_t H, const dsx_router_config& cfg,
                        float* logits, int32_t* selected, float* weights, int chunk, int shared_T, int32_t* hist, int32_t* offsets,
                        int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap, unsigned int* counters,
                        cudaStream_t stream) {
    DSX_REQUIRE(router_fused_ok(T, cfg, H), "router_fused: shape not covered");
    const size_t smem = std::max<size_t>((size_t)kLogitTokens * H * 2, (size_t)kLogitWarps * cfg.n_expert * 4);
    dim3 grid((unsigned)(cfg.n_expert / kLogitWarps), (unsigned)((T + kLogitTokens - 1) / kLogitTokens));
    switch (cfg.n_expert / 32) {
#define DSX_FUSED_CASE(V)                                                                                                     \
    case V:                                                                                                                   \
        router_fused_kernel<V><<<grid, kLogitWarps * 32, smem, stream>>>(x, (int)T, W, bias, (int)H, cfg, logits, selected, weights, \
                                                                        chunk, shared_T, hist, offsets, perm, work_items,     \
                                                                        n_work_items, work_cap, counters);                    \
        break;
        DSX_FUSED_CASE(1) DSX_FUSED_CASE(2) DSX_FUSED_CASE(4) DSX_FUSED_CASE(8)
#undef DSX_FUSED_CASE
        default:
            return set_error(DSX_ERR_UNSUPPORTED, "router_fused: n_expert %d not instantiated", cfg.n_expert);
    }
    DSX_LAUNCHED();
    return DSX_OK;
}

// Opt the fused router in to 96 KB of dynamic shared memory (once per device, at layer creation).
int router_configure() {
    DSX_CUDA(cudaFuncSetAttribute(router_fused_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    DSX_CUDA(cudaFuncSetAttribute(router_fused_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    DSX_CUDA(cudaFuncSetAttribute(router_fused_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    DSX_CUDA(cudaFuncSetAttribute(router_fused_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    return DSX_OK;
}

int launch_router_topk(const float* logits, const float* bias, int64_t T, const dsx_router_config& cfg,
                       int32_t* selected, float* weights, cudaStream_t stream) {
    DSX_REQUIRE(cfg.n_expert > 0 && cfg.n_expert % 32 == 0 && cfg.n_expert <= 512,
                "router_topk: n_expert %d must be a multiple of 32, at most 512", cfg.n_expert);
    DSX_REQUIRE(cfg.n_used >= 1 && cfg.n_used <= kMaxUsed && cfg.n_used <= cfg.n_expert, "router_topk: n_used %d out of range", cfg.n_used);
    if (cfg.n_group > 1) {
        DSX_REQUIRE(cfg.n_group <= 32 && cfg.n_expert % cfg.n_group == 0 && cfg.topk_group >= 1 && cfg.topk_group <= cfg.n_group,
                    "router_topk: bad group limit %d/%d", cfg.topk_group, cfg.n_group);
    }
    if (T == 0) return DSX_OK;
    const unsigned grid = (unsigned)((T + kTopkWarps - 1) / kTopkWarps);
    switch (cfg.n_expert / 32) {
#define DSX_TOPK_CASE(V)                                                                                   \
    case V:                                                                                                \
        router_topk_kernel<V><<<grid, kTopkWarps * 32, 0, stream>>>(logits, bias, T, cfg, selected, weights); \
        break;
        DSX_TOPK_CASE(1) DSX_TOPK_CASE(2) DSX_TOPK_CASE(3) DSX_TOPK_CASE(4) DSX_TOPK_CASE(6) DSX_TOPK_CASE(8)
        DSX_TOPK_CASE(12) DSX_TOPK_CASE(16)
#undef DSX_TOPK_CASE
        default:
            return set_error(DSX_ERR_UNSUPPORTED, "router_topk: n_expert %d not instantiated", cfg.n_expert);
    }
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace dsx
