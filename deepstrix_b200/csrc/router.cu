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
    for (int i0 = 0; i0 < n_iter; i0 += 4) {
        // four iterations' loads (router row and token rows) go out together, then the fmas
        float4 w4[4];
        uint2 xv[4][kLogitTokens];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = min(i0 + j, n_iter - 1);
            w4[j] = __ldg(wrow + i * 32);
#pragma unroll
            for (int tt = 0; tt < kLogitTokens; tt++) xv[j][tt] = __ldg(xrow[tt] + i * 32);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (i0 + j < n_iter) {
                const float4 w = w4[j];
#pragma unroll
                for (int tt = 0; tt < kLogitTokens; tt++) {
                    const float x0 = __uint_as_float(xv[j][tt].x << 16), x1 = __uint_as_float(xv[j][tt].x & 0xFFFF0000u);
                    const float x2 = __uint_as_float(xv[j][tt].y << 16), x3 = __uint_as_float(xv[j][tt].y & 0xFFFF0000u);
                    float a = acc[tt];
                    a = __fmaf_rn(w.x, x0, a);
                    a = __fmaf_rn(w.y, x1, a);
                    a = __fmaf_rn(w.z, x2, a);
                    a = __fmaf_rn(w.w, x3, a);
                    acc[tt] = a;
                }
            }
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
        const int per = E / cfg.n_group;
        const int lpg = per / VPL;   // lanes per group when a group is a whole number of lanes
        float gs = -INFINITY;        // score of group `lane` (lanes < n_group)
        if (per % VPL == 0 && (lpg & (lpg - 1)) == 0 && lpg >= 1 && lpg <= 32) {
            // top-2 of the lane's own values, then merged across the lanes of the group
            float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
            for (int j = 0; j < VPL; j++) {
                const float v = s[j];
                if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
            }
            for (int off = 1; off < lpg; off <<= 1) {
                const float o1 = __shfl_xor_sync(0xFFFFFFFFu, m1, off), o2 = __shfl_xor_sync(0xFFFFFFFFu, m2, off);
                const float lo = fminf(m1, o1);
                m1 = fmaxf(m1, o1);
                m2 = fmaxf(lo, fmaxf(m2, o2));
            }
            const float mine = __fadd_rn(m1, m2);                      // same in every lane of the group
            gs = __shfl_sync(0xFFFFFFFFu, mine, (lane * lpg) & 31);    // lane g reads group g's score
            if (lane >= cfg.n_group) gs = -INFINITY;
        } else {
#pragma unroll
            for (int j = 0; j < VPL; j++) s_score[lane * VPL + j] = s[j];
            __syncwarp();
            if (lane < cfg.n_group) {
                float m1 = -INFINITY, m2 = -INFINITY;
                for (int i = 0; i < per; i++) {
                    const float v = s_score[lane * per + i];
                    if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
                }
                gs = __fadd_rn(m1, m2);
            }
            __syncwarp();
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
    }
    // k selection rounds: warp-wide max of the ordered score bits (redux), then the lowest expert
    // index among the lanes that hold that score (redux min) -- equal scores go to the lower index.
    uint32_t ob[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++) ob[j] = ordered_bits(__fadd_rn(s[j], 0.0f));   // adding +0 turns -0 into +0
    // 0 marks "already taken": every non-NaN score maps to at least 0x007FFFFF (-inf)
    float psel[kMaxUsed];
    int esel[kMaxUsed];
#pragma unroll
    for (int r = 0; r < kMaxUsed; r++) {
        if (r < cfg.n_used) {
            uint32_t lb = 0u;
            int lj = 0;
#pragma unroll
            for (int j = VPL - 1; j >= 0; j--)
                if (ob[j] >= lb) { lb = ob[j]; lj = j; }   // ties inside the lane: lowest j
            const uint32_t mx = __reduce_max_sync(0xFFFFFFFFu, lb);
            const uint32_t cand = (lb == mx) ? (uint32_t)(lane * VPL + lj) : 0xFFFFFFFFu;
            const int e = (int)__reduce_min_sync(0xFFFFFFFFu, cand);
            const int owner = e / VPL, jj = e - owner * VPL;
            float pv = 0.0f;
#pragma unroll
            for (int j = 0; j < VPL; j++)
                if (lane == owner && j == jj) { pv = p[j]; ob[j] = 0u; }
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
    pdl_launch_dependents();
    pdl_wait();   // the routing buffers written below may still be read by the previous step's kernels
    // token rows of the tile -> shared memory (rows past the batch alias the last valid row)
    uint2* xs = reinterpret_cast<uint2*>(fsm);   // [8][H/4] of 4 x bf16
    const int vec = H >> 2;
    {   // warp r copies token row r: eight loads in flight per lane
        const uint2* src = reinterpret_cast<const uint2*>(x + (int64_t)min(t0 + warp, T - 1) * H);
        uint2* dst = xs + warp * vec;
        for (int c0 = lane; c0 < vec; c0 += 32 * 8) {
            uint2 v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = (c0 + 32 * j < vec) ? __ldg(src + c0 + 32 * j) : make_uint2(0u, 0u);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (c0 + 32 * j < vec) dst[c0 + 32 * j] = v[j];
        }
    }
    __syncthreads();
    const int e = blockIdx.x * kLogitWarps + warp;
    {
        float acc[kLogitTokens];
#pragma unroll
        for (int i = 0; i < kLogitTokens; i++) acc[i] = 0.0f;
        const float4* wrow = reinterpret_cast<const float4*>(W + (int64_t)e * H) + lane;
        const int n_iter = H >> 7;
        // router rows stream from HBM: fetch sixteen 512-byte pieces per round trip, then do the math
        for (int i0 = 0; i0 < n_iter; i0 += 16) {
            float4 w8[16];
#pragma unroll
            for (int j = 0; j < 16; j++) w8[j] = (i0 + j < n_iter) ? __ldg(wrow + (i0 + j) * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                if (i0 + j < n_iter) {
                    const float4 w = w8[j];
#pragma unroll
                    for (int tt = 0; tt < kLogitTokens; tt++) {
                        const uint2 xv = xs[tt * vec + (i0 + j) * 32 + lane];
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
        DSX_CUDA(launch_pdl(router_fused_kernel<V>, grid, dim3(kLogitWarps * 32), smem, stream, x, (int)T, W, bias, (int)H, cfg,     \
                            logits, selected, weights, chunk, shared_T, hist, offsets, perm, work_items, n_work_items, work_cap,  \
                            counters));                                                                                       \
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
