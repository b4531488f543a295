// Router: logits GEMV and top-k selection.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   logits  crates/v4flash-kernels/kernels/f16_matvec.hip:26-45 (warp per row, f32 accumulate)
//   top-k   crates/v4flash-kernels/kernels/router_topk_par.hip:66-238 (k argmax passes, lower
//           index wins ties) and :294-434 (the 64-bit-key wave-reduction twin whose key
//           `(ord(score) << 32) | ~index` is reused here)
//   sigmoid crates/v4flash-kernels/kernels/laguna_ops.hip:55-62
#include <algorithm>
#include <atomic>

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

// Same logits for prefill-size batches, tiled like a GEMM so that router rows and token rows are
// re-read from L2 16 and 32 times less: a block of 8 warps computes 16 router rows x 32 tokens,
// a warp 8 rows x 8 tokens (64 accumulators a lane; 0.75 bytes of shared memory read per FMA), two
// blocks to an SM.  The reduction runs in chunks of 128 columns, two per stage of shared memory
// filled by 16-byte async copies (three stages); lane l still owns columns 4l..4l+3 of every chunk and
// adds them in increasing column order, then the warp folds with the operand pairs of the xor
// butterfly: the f32 operation sequence of a (token, expert) pair is the one of router_logits_kernel,
// same bits.
constexpr int kTileRowsR = 16, kTileTok = 32, kTileStages = 3;
constexpr int kTileThreads = 256;
constexpr int kTileWarpRows = 8, kTileWarpTok = 8;
constexpr int kTileCols = 256;   // columns per stage: two 128-column chunks per block barrier
constexpr int kTileStageBytes = kTileRowsR * kTileCols * 4 + kTileTok * kTileCols * 2;   // 32 KB
static_assert((kTileRowsR / kTileWarpRows) * (kTileTok / kTileWarpTok) * 32 == kTileThreads, "warps must cover the block tile");

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
// (d.lo, d.hi) = (a.lo * b.lo + c.lo, a.hi * b.hi + c.hi), each half one IEEE fused multiply-add
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__global__ void __launch_bounds__(kTileThreads, 2)
router_logits_tiled_kernel(const __nv_bfloat16* __restrict__ x, int64_t T, const float* __restrict__ W, int n_expert, int64_t H,
                           float* __restrict__ logits) {
    extern __shared__ __align__(128) uint8_t tsm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rg = warp >> 2, tg = warp & 3;              // row group (8 rows), token group (8 tokens)
    const int e0 = blockIdx.x * kTileRowsR;
    const int64_t t0 = (int64_t)blockIdx.y * kTileTok;
    const int n_iter = (int)(H / kTileCols);
    // this thread's eight 16-byte pieces of every stage (rows past the batch alias the last valid row)
    const int wr = threadIdx.x >> 4, wc = threadIdx.x & 15;
    const float* wsrc = W + (int64_t)(e0 + wr) * H + wc * 4;
    const int xr = threadIdx.x >> 3, xc = threadIdx.x & 7;
    const __nv_bfloat16* xsrc = x + min(t0 + xr, T - 1) * H + xc * 8;
    auto stage_w = [&](int s) { return reinterpret_cast<float*>(tsm + (size_t)s * kTileStageBytes); };
    auto stage_x = [&](int s) { return reinterpret_cast<__nv_bfloat16*>(tsm + (size_t)s * kTileStageBytes + kTileRowsR * kTileCols * 4); };
    auto issue = [&](int i) {
        const int s = i % kTileStages;
#pragma unroll
        for (int j = 0; j < kTileCols / 64; j++) {
            cp_async16(stage_w(s) + wr * kTileCols + j * 64 + wc * 4, wsrc + (int64_t)i * kTileCols + j * 64);
            cp_async16(stage_x(s) + xr * kTileCols + j * 64 + xc * 8, xsrc + (int64_t)i * kTileCols + j * 64);
        }
    };
    // accumulators of token pairs (t, t + 1) share a 64-bit register: one packed instruction performs
    // the two round-to-nearest fused multiply-adds, each exactly the scalar one
    uint64_t acc[kTileWarpRows][kTileWarpTok / 2];
#pragma unroll
    for (int r = 0; r < kTileWarpRows; r++)
#pragma unroll
        for (int t = 0; t < kTileWarpTok / 2; t++) acc[r][t] = 0ull;
    issue(0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (n_iter > 1) issue(1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int i = 0; i < n_iter; i++) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();   // stage i has landed for every thread; everyone is done with stage i - 1
        if (i + 2 < n_iter) issue(i + 2);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int s = i % kTileStages;
#pragma unroll
        for (int h = 0; h < kTileCols / 128; h++) {   // 128-column chunks in increasing column order
            const float4* wp = reinterpret_cast<const float4*>(stage_w(s) + (rg * kTileWarpRows) * kTileCols + h * 128) + lane;
            const uint2* xp = reinterpret_cast<const uint2*>(stage_x(s) + (tg * kTileWarpTok) * kTileCols + h * 128) + lane;
            uint64_t xq[kTileWarpTok / 2][4];   // columns 4l..4l+3 of tokens (2p, 2p + 1), widened to f32
#pragma unroll
            for (int t = 0; t < kTileWarpTok / 2; t++) {
                const uint2 xa = xp[(2 * t) * (kTileCols / 4)], xb = xp[(2 * t + 1) * (kTileCols / 4)];
                xq[t][0] = pack2(xa.x << 16, xb.x << 16);
                xq[t][1] = pack2(xa.x & 0xFFFF0000u, xb.x & 0xFFFF0000u);
                xq[t][2] = pack2(xa.y << 16, xb.y << 16);
                xq[t][3] = pack2(xa.y & 0xFFFF0000u, xb.y & 0xFFFF0000u);
            }
#pragma unroll
            for (int r = 0; r < kTileWarpRows; r++) {
                const float4 w = wp[r * (kTileCols / 4)];
                const uint64_t w0 = pack2(__float_as_uint(w.x), __float_as_uint(w.x)), w1 = pack2(__float_as_uint(w.y), __float_as_uint(w.y));
                const uint64_t w2 = pack2(__float_as_uint(w.z), __float_as_uint(w.z)), w3 = pack2(__float_as_uint(w.w), __float_as_uint(w.w));
#pragma unroll
                for (int t = 0; t < kTileWarpTok / 2; t++) {
                    uint64_t a = acc[r][t];
                    a = fma2(w0, xq[t][0], a);
                    a = fma2(w1, xq[t][1], a);
                    a = fma2(w2, xq[t][2], a);
                    a = fma2(w3, xq[t][3], a);
                    acc[r][t] = a;
                }
            }
        }
    }
    // The butterfly of router_logits_kernel, folded: at the step with lane distance d a lane keeps the
    // half of its values its bit d selects and adds the partner's partial sums of the same values, so
    // every addition has the butterfly's two operands (f32 addition commutes) and each step halves the
    // work.  Value r * 8 + t ends, fully summed, in lane (r * 8 + t) / 2.
    float v[kTileWarpRows * kTileWarpTok];
#pragma unroll
    for (int r = 0; r < kTileWarpRows; r++)
#pragma unroll
        for (int t = 0; t < kTileWarpTok; t++) {
            const uint64_t q = acc[r][t >> 1];
            v[r * kTileWarpTok + t] = __uint_as_float((t & 1) ? (uint32_t)(q >> 32) : (uint32_t)q);
        }
#pragma unroll
    for (int half = kTileWarpRows * kTileWarpTok / 2, off = 16; off > 0; half >>= 1, off >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < half; j++) {
            const float keep = up ? v[j + half] : v[j];
            const float give = up ? v[j] : v[j + half];
            v[j] = __fadd_rn(keep, __shfl_xor_sync(0xFFFFFFFFu, give, off));
        }
    }
    static_assert(kTileWarpRows * kTileWarpTok == 64, "two finished values a lane");
    {
        const int r = lane >> 2;
        const int64_t tok = t0 + tg * kTileWarpTok + 2 * (lane & 3);
        float* out = logits + tok * n_expert + e0 + rg * kTileWarpRows + r;
        if (tok < T) out[0] = v[0];
        if (tok + 1 < T) out[n_expert] = v[1];
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
                                               int32_t* __restrict__ sel_out, float* __restrict__ w_out, float* s_score,
                                               int32_t* s_sel = nullptr, float* s_wsel = nullptr /* optional copies in shared memory */,
                                               int n_alt = 0, int32_t* __restrict__ alt_out = nullptr, float* __restrict__ altw_out = nullptr,
                                               float* __restrict__ range_out = nullptr) {
    const int lane = threadIdx.x & 31;
    const int E = VPL * 32;
    float p[VPL], s[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        const int e = lane * VPL + j;
        p[j] = router_prob(load_logit(e), cfg.score_fn);
        s[j] = bias ? __fadd_rn(p[j], bias[e]) : p[j];
    }
    if (range_out != nullptr) {   // max - min of the selection scores over all experts (router_topk_par.hip:140-160)
        float mx = s[0], mn = s[0];
#pragma unroll
        for (int j = 1; j < VPL; j++) { mx = fmaxf(mx, s[j]); mn = fminf(mn, s[j]); }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
            mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, off));
        }
        if (lane == 0) *range_out = __fsub_rn(mx, mn);
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
    // 0 marks "already taken": every non-NaN score maps to at least 0x007FFFFF (-inf).
    // The rounds run as a real loop: this code executes once per token on one warp, where fetching the
    // instructions of sixteen unrolled rounds costs more than running them.  Lane r keeps round r's
    // pick; the weights' sum is accumulated in slot order over the first n_used rounds.
    float sum = 0.0f, my_p = 0.0f;
    int my_e = 0;
    const int n_rounds = cfg.n_used + n_alt;   // rounds past n_used are the alternatives: they only mask further
#pragma unroll 1
    for (int r = 0; r < n_rounds; r++) {
        // the lane's best by a tournament (depth log2 VPL); `>` keeps the lower j on ties
        uint32_t v[VPL];
        int ix[VPL];
        float pp[VPL];
#pragma unroll
        for (int j = 0; j < VPL; j++) { v[j] = ob[j]; ix[j] = j; pp[j] = p[j]; }
#pragma unroll
        for (int lvl = 0; lvl < 5; lvl++) {
            const int w = 1 << lvl;
#pragma unroll
            for (int j = 0; j < VPL; j++) {
                if (w < VPL && (j & (2 * w - 1)) == 0 && j + w < VPL) {
                    const bool take = v[j + w] > v[j];
                    v[j] = take ? v[j + w] : v[j];
                    ix[j] = take ? ix[j + w] : ix[j];
                    pp[j] = take ? pp[j + w] : pp[j];
                }
            }
        }
        const uint32_t mx = __reduce_max_sync(0xFFFFFFFFu, v[0]);
        const uint32_t cand = (v[0] == mx) ? (uint32_t)(lane * VPL + ix[0]) : 0xFFFFFFFFu;
        const int e = (int)__reduce_min_sync(0xFFFFFFFFu, cand);
        const bool mine = cand == (uint32_t)e;
#pragma unroll
        for (int j = 0; j < VPL; j++)
            ob[j] = (mine && ix[0] == j) ? 0u : ob[j];
        const float pv = __shfl_sync(0xFFFFFFFFu, pp[0], e / VPL);
        if (r < cfg.n_used) sum = __fadd_rn(sum, pv);
        if (lane == r) { my_p = pv; my_e = e; }
    }
    if (sum < cfg.weight_eps) sum = cfg.weight_eps;
    if (lane >= cfg.n_used && lane < cfg.n_used + n_alt) {   // prob(alt) / (sum of the picks' probs) * scale
        alt_out[lane - cfg.n_used] = my_e;
        if (altw_out != nullptr) altw_out[lane - cfg.n_used] = __fmul_rn(__fdiv_rn(my_p, sum), cfg.route_scale);
    }
    if (lane < cfg.n_used) {
        const float wv = __fmul_rn(__fdiv_rn(my_p, sum), cfg.route_scale);
        sel_out[lane] = my_e;
        w_out[lane] = wv;
        if (s_sel != nullptr) { s_sel[lane] = my_e; s_wsel[lane] = wv; }
    }
}

template <int VPL>
__global__ void __launch_bounds__(kTopkWarps * 32)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T, dsx_router_config cfg,
                   int32_t* __restrict__ selected, float* __restrict__ weights, int n_alt, int32_t* __restrict__ alts,
                   float* __restrict__ alt_w, float* __restrict__ range_out) {
    __shared__ float s_score[kTopkWarps][VPL * 32];
    const int warp = threadIdx.x >> 5;
    const int64_t t = (int64_t)blockIdx.x * kTopkWarps + warp;
    if (t >= T) return;
    const float* row = logits + t * (VPL * 32);
    topk_one_token<VPL>([&](int e) { return row[e]; }, bias, cfg, selected + t * cfg.n_used, weights + t * cfg.n_used, s_score[warp], nullptr,
                        nullptr, n_alt, alts ? alts + t * n_alt : nullptr, alt_w ? alt_w + t * n_alt : nullptr,
                        range_out ? range_out + t : nullptr);
}

// ---- Top-k with the reference's cache prior (router_topk_par.hip:82-99,173-210): a per-expert prior is
// added to the SELECTION score; the first n_protect picks of the plain ranking are always kept, the
// remaining slots and the alternatives are the argmax of score + prior; weights still come from the
// unbiased probabilities of the emitted set.  orig_sel receives the plain top-n_used.  With
// prior_dry the roles swap: the plain picks are emitted (and weighted) and orig_sel carries what
// the prior would have chosen.  One warp per token; no group limit (the reference has none here).
template <int VPL>
__device__ __forceinline__ int prior_argmax_round(uint32_t (&ob)[VPL], int lane) {
    uint32_t best = ob[0];
    int bj = 0;
#pragma unroll
    for (int j = 1; j < VPL; j++)
        if (ob[j] > best) { best = ob[j]; bj = j; }   // `>` keeps the lower j on ties
    const uint32_t mx = __reduce_max_sync(0xFFFFFFFFu, best);
    const uint32_t cand = (best == mx) ? (uint32_t)(lane * VPL + bj) : 0xFFFFFFFFu;
    const int e = (int)__reduce_min_sync(0xFFFFFFFFu, cand);
#pragma unroll
    for (int j = 0; j < VPL; j++)
        ob[j] = (cand == (uint32_t)e && bj == j) ? 0u : ob[j];
    return e;
}

template <int VPL>
__global__ void __launch_bounds__(kTopkWarps * 32)
router_topk_prior_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T, dsx_router_config cfg,
                         int32_t* __restrict__ selected, float* __restrict__ weights, int n_alt, int32_t* __restrict__ alts,
                         float* __restrict__ alt_w, float* __restrict__ range_out, const float* __restrict__ prior, int n_protect,
                         int prior_dry, int32_t* __restrict__ orig_sel) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * kTopkWarps + warp;
    if (t >= T) return;
    const float* row = logits + t * (VPL * 32);
    float p[VPL], s[VPL];
    uint32_t ob[VPL], ob2[VPL];
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        const int e = lane * VPL + j;
        p[j] = router_prob(row[e], cfg.score_fn);
        s[j] = bias ? __fadd_rn(p[j], bias[e]) : p[j];
        ob[j] = ordered_bits(__fadd_rn(s[j], 0.0f));
        ob2[j] = ordered_bits(__fadd_rn(__fadd_rn(s[j], prior[e]), 0.0f));
    }
    if (range_out != nullptr) {
        float mx = s[0], mn = s[0];
#pragma unroll
        for (int j = 1; j < VPL; j++) { mx = fmaxf(mx, s[j]); mn = fminf(mn, s[j]); }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
            mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, off));
        }
        if (lane == 0) range_out[t] = __fsub_rn(mx, mn);
    }
    // lane r keeps rank r of both rankings
    int my_orig = -1, my_sel = -1;
#pragma unroll 1
    for (int r = 0; r < cfg.n_used; r++) {   // the ORIGINAL top-n_used, on the plain scores
        const int e = prior_argmax_round<VPL>(ob, lane);
        if (lane == r) my_orig = e;
    }
#pragma unroll 1
    for (int r = 0; r < n_protect; r++) {    // protected picks stay and leave the boosted pool
        const int e = __shfl_sync(0xFFFFFFFFu, my_orig, r);
        if (lane == r) my_sel = e;
#pragma unroll
        for (int j = 0; j < VPL; j++)
            ob2[j] = (lane * VPL + j == e) ? 0u : ob2[j];
    }
#pragma unroll 1
    for (int r = n_protect; r < cfg.n_used + n_alt; r++) {
        const int e = prior_argmax_round<VPL>(ob2, lane);
        if (lane == r) my_sel = e;
    }
    // dry run: emit the plain picks, report the prior's
    int emit = my_sel, other = my_orig;
    if (prior_dry && lane < cfg.n_used) { emit = my_orig; other = my_sel; }
    // unbiased probability of this lane's emitted expert: from the lane that owns it
    float my_p = 0.0f;
    for (int r = 0; r < cfg.n_used + n_alt; r++) {
        const int e = __shfl_sync(0xFFFFFFFFu, emit, r);
        float pv = 0.0f;
#pragma unroll
        for (int j = 0; j < VPL; j++)
            if (lane * VPL + j == e) pv = p[j];
        pv = __shfl_sync(0xFFFFFFFFu, pv, (e >= 0 ? e : 0) / VPL);
        if (lane == r) my_p = (e >= 0) ? pv : 0.0f;
    }
    float sum = 0.0f;
    for (int r = 0; r < cfg.n_used; r++) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, my_p, r));
    if (sum < cfg.weight_eps) sum = cfg.weight_eps;
    const float wv = __fmul_rn(__fdiv_rn(my_p, sum), cfg.route_scale);
    if (lane < cfg.n_used) {
        selected[t * cfg.n_used + lane] = emit;
        weights[t * cfg.n_used + lane] = wv;
        if (orig_sel != nullptr) orig_sel[t * cfg.n_used + lane] = other;
    } else if (lane < cfg.n_used + n_alt) {
        alts[t * n_alt + lane - cfg.n_used] = emit;
        if (alt_w != nullptr) alt_w[t * n_alt + lane - cfg.n_used] = wv;
    }
}

// ---- Decode router in ONE launch (T <= 64, E <= 256): logits, top-k and the group build.
//
// Grid (E/4, token tiles), 8 warps.  A tile is 2*NT tokens (NT = 1, 2 or 4, chosen from T).  The
// block's four router rows (f32) and the tile's token rows (bf16) come into shared memory as bulk
// async copies, all in flight at once, completing on mbarriers (a router row in two halves, so
// the arithmetic starts when the first half has landed).  Warp w works on row w/2 and on tokens
// (w%2)*NT .. +NT of the tile, in the f32 operation order of router_logits_kernel, so the logits
// are the same bits.  The last block of a token tile to finish (ticket counter) selects the
// experts of that tile's tokens, one warp per token; the last tile to finish builds histogram,
// offsets, permutation and work items.  The counters return to zero for the next launch.
constexpr int kFusedRows = 4;                 // router rows per block
constexpr int kFusedWarps = 2 * kFusedRows;   // two token halves per row
constexpr int kFusedMaxPicks = 512;           // T * n_used the in-kernel group build covers
constexpr int kFusedMaxItems = kFusedMaxPicks + 8;   // work items: at most one per pick, plus the shared expert's
constexpr size_t kFusedScratch = (size_t)(kFusedWarps * 256 + kFusedMaxPicks + kFusedMaxItems + 256 + 2) * 4;   // group-build scratch
constexpr uint32_t kRouterWaitSpins = 1u << 22;

__device__ __forceinline__ uint32_t r_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void r_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void r_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false when the phase did not complete in kRouterWaitSpins polls.
__device__ __forceinline__ bool r_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kRouterWaitSpins; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void r_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int VPL, int NT>
__global__ void __launch_bounds__(kFusedWarps * 32)
router_fused_kernel(const __nv_bfloat16* __restrict__ x, int T, const float* __restrict__ W, const float* __restrict__ bias, int H,
                    dsx_router_config cfg, float* __restrict__ logits, int32_t* __restrict__ selected, float* __restrict__ weights,
                    int chunk, int shared_T, int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items,
                    int32_t* n_work_items, int32_t work_cap, ItemRec* item_recs,
                    unsigned int* counters /* [0]: tiles done, [1 + tile]: blocks done */, uint32_t* error_word) {
    extern __shared__ __align__(128) uint8_t fsm[];
    __shared__ __align__(8) uint64_t s_bar[1 + 2 * kFusedRows];
    __shared__ int s_flag;
    __shared__ int s_warp[kFusedWarps + 1];
    __shared__ int32_t s_sel[kFusedMaxPicks];
    __shared__ float s_wsel[kFusedMaxPicks];
    constexpr int E = VPL * 32;
    constexpr int kTile = 2 * NT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.y, t0 = tile * kTile;
    const int nt = min(kTile, T - t0);
    const int row = warp >> 1, th = warp & 1;
    float* ws = reinterpret_cast<float*>(fsm);                              // [4][H] f32
    uint2* xs = reinterpret_cast<uint2*>(fsm + (size_t)kFusedRows * H * 4); // [kTile][H/4] of 4 x bf16
    const int vec = H >> 2;
    const uint32_t bar_x = r_smem_u32(&s_bar[0]);
    const uint32_t bar_w0 = r_smem_u32(&s_bar[1 + 2 * row]), bar_w1 = bar_w0 + 8;
    if (threadIdx.x == 0) {
        r_mbar_init(bar_x, (uint32_t)nt);
        for (int i = 0; i < 2 * kFusedRows; i++) r_mbar_init(r_smem_u32(&s_bar[1 + i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int e = blockIdx.x * kFusedRows + row;
    if (lane == 0) {
        // router weights are constants of the layer: their copies may start before the previous kernel ends
        const uint32_t half_bytes = (uint32_t)H * 2u;
        const uint32_t bw = th ? bar_w1 : bar_w0;
        r_mbar_expect_tx(bw, half_bytes);
        r_bulk_g2s(r_smem_u32(ws + (size_t)row * H) + th * half_bytes, reinterpret_cast<const uint8_t*>(W + (int64_t)e * H) + th * half_bytes,
                   half_bytes, bw);
    }
    pdl_wait();   // the token rows come from the previous kernel; the routing buffers written below may still be read by it
    // only now may the next kernel start: whatever it does before its own wait sees complete token rows
    pdl_launch_dependents();
    if (lane == 0 && warp < nt) {
        r_mbar_expect_tx(bar_x, (uint32_t)H * 2u);
        r_bulk_g2s(r_smem_u32(xs + (size_t)warp * vec), x + (int64_t)(t0 + warp) * H, (uint32_t)H * 2u, bar_x);
    }
    bool ok = true;
    if (th * NT < nt) {   // this warp has tokens (warp-uniform)
        float acc[NT];
        const uint2* xrow[NT];
#pragma unroll
        for (int i = 0; i < NT; i++) {
            acc[i] = 0.0f;
            xrow[i] = xs + (size_t)min(th * NT + i, nt - 1) * vec + lane;   // slots past the batch alias the last valid row
        }
        const float4* wrow = reinterpret_cast<const float4*>(ws + (size_t)row * H) + lane;
        const int n_iter = H >> 7, half_iter = n_iter >> 1;
        ok = r_mbar_wait(bar_x, 0) && r_mbar_wait(bar_w0, 0);
        for (int hlf = 0; hlf < 2 && ok; hlf++) {
            if (hlf == 1) ok = r_mbar_wait(bar_w1, 0);
            if (!ok) break;
#pragma unroll 4
            for (int i = hlf * half_iter; i < (hlf + 1) * half_iter; i++) {
                const float4 w = wrow[i * 32];
#pragma unroll
                for (int tt = 0; tt < NT; tt++) {
                    const uint2 xv = xrow[tt][i * 32];
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
#pragma unroll
        for (int tt = 0; tt < NT; tt++) {
            float a = acc[tt];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, off));
            if (lane == 0 && th * NT + tt < nt) logits[(int64_t)(t0 + th * NT + tt) * E + e] = a;
        }
    } else {
        // no tokens here, but no thread may leave while copies into this block's shared memory are in flight
        ok = r_mbar_wait(bar_x, 0) && r_mbar_wait(bar_w0, 0) && r_mbar_wait(bar_w1, 0);
    }
    if (!ok && lane == 0) atomicOr(error_word, 4u);
    // ---- last block of this token tile?
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_flag = (atomicAdd(&counters[1 + tile], 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (!s_flag) return;
    if (threadIdx.x == 0) counters[1 + tile] = 0u;
    __threadfence();
    float* s_score = reinterpret_cast<float*>(fsm);   // rows and tokens are no longer needed
    if (warp < nt) {
        const float* lrow = logits + (int64_t)(t0 + warp) * E;
        topk_one_token<VPL>([&](int ee) { return __ldcg(lrow + ee); }, bias, cfg, selected + (int64_t)(t0 + warp) * cfg.n_used,
                            weights + (int64_t)(t0 + warp) * cfg.n_used, s_score + warp * E, s_sel + (t0 + warp) * cfg.n_used,
                            s_wsel + (t0 + warp) * cfg.n_used);
    }
    const int P = T * cfg.n_used;
    if (gridDim.y > 1) {
        // ---- last tile of the launch?
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_flag = (atomicAdd(&counters[0], 1u) == gridDim.y - 1) ? 1 : 0;
        __syncthreads();
        if (!s_flag) return;
        if (threadIdx.x == 0) counters[0] = 0u;
        __threadfence();
        for (int i = threadIdx.x; i < P; i += kFusedWarps * 32) {   // the other tiles' picks
            s_sel[i] = __ldcg(selected + i);
            s_wsel[i] = __ldcg(weights + i);
        }
    }
    __syncthreads();
    if (item_recs != nullptr && P <= 32)
        groupdev::build_tiny_with_recs<kFusedWarps * 32>(s_sel, s_wsel, T, cfg.n_used, E, shared_T, hist, offsets, perm, work_items,
                                                         n_work_items, min(work_cap, kFusedMaxItems), item_recs, reinterpret_cast<int*>(fsm),
                                                         s_warp);
    else if (item_recs != nullptr)
        groupdev::build_small_with_recs<kFusedWarps * 32, kFusedMaxPicks>(s_sel, s_wsel, T, cfg.n_used, E, shared_T, hist, offsets, perm,
                                                                          work_items, n_work_items, min(work_cap, kFusedMaxItems),
                                                                          item_recs, reinterpret_cast<int*>(fsm), s_warp);
    else
        groupdev::build_small<kFusedWarps * 32, kFusedMaxPicks>(s_sel, P, E, 0, chunk, shared_T, hist, offsets, perm, work_items,
                                                                n_work_items, work_cap, reinterpret_cast<int*>(fsm), s_warp);
}


// ---- The same for 9..64 tokens: two router rows per block stay in shared memory while the token
// rows stream past them in tiles of 8 (double buffered bulk copies), so the grid is E/2 blocks
// whatever the batch size and the router weights are read once.  Warp w works on row w/4 and on
// tokens 2*(w%4), +1 of the tile, in the f32 operation order of router_logits_kernel.
// Then one barrier across the grid (every block is resident: the launcher checks E/2 against the
// SM count, and the next kernel of the chain cannot start before every block of this one has
// passed its release point; the wait is bounded and reports through error_word), the blocks share
// out the tokens' top-k, one warp per token, and the last block to finish (ticket) builds the groups.
// NI = H / 128 when the launcher knows it (0 otherwise): a warp then keeps its router row in NI x 4
// registers for the whole kernel and the tile loop reads only tokens from shared memory, whose
// bandwidth is what bounds this phase.
// counters[0]: barrier arrivals, counters[1]: ticket, counters[2]: a block gave up waiting; all return to zero.
constexpr int kWideRows = 2;
constexpr int kWideWarps = 8;
constexpr int kWideTile = 8;

template <int VPL, int NI>
__global__ void __launch_bounds__(kWideWarps * 32)
router_fused_wide_kernel(const __nv_bfloat16* __restrict__ x, int T, const float* __restrict__ W, const float* __restrict__ bias, int H,
                         dsx_router_config cfg, float* __restrict__ logits, int32_t* __restrict__ selected, float* __restrict__ weights,
                         int chunk, int shared_T, int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items,
                         int32_t* n_work_items, int32_t work_cap, unsigned int* counters, uint32_t* error_word) {
    extern __shared__ __align__(128) uint8_t fsm[];
    __shared__ __align__(8) uint64_t s_bar[3];   // router rows, token buffer 0, token buffer 1
    __shared__ int s_flag;
    __shared__ int s_warp[kWideWarps + 1];
    __shared__ int32_t s_sel[kFusedMaxPicks];
    constexpr int E = VPL * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = warp >> 2, q = warp & 3;
    const int vec = H >> 2;
    const int n_tiles = (T + kWideTile - 1) / kWideTile;
    float* ws = reinterpret_cast<float*>(fsm);                                   // [2][H] f32
    uint2* xs = reinterpret_cast<uint2*>(fsm + (size_t)kWideRows * H * 4);       // [2 buffers][8][H/4] of 4 x bf16
    const uint32_t bar_w = r_smem_u32(&s_bar[0]);
    if (threadIdx.x == 0) {
        for (int i = 0; i < 3; i++) r_mbar_init(r_smem_u32(&s_bar[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // router weights are constants of the layer: the copy may start before the previous kernel ends
        const uint32_t bytes = (uint32_t)kWideRows * (uint32_t)H * 4u;
        r_mbar_expect_tx(bar_w, bytes);
        r_bulk_g2s(r_smem_u32(ws), W + (int64_t)blockIdx.x * kWideRows * H, bytes, bar_w);
    }
    __syncthreads();
    pdl_wait();   // the token rows come from the previous kernel; the routing buffers written below may still be read by it
    pdl_launch_dependents();
    // blocks walk the tiles in rotated order, so that at any moment they read different token rows
    auto tile_of = [&](int i) { return (i + (int)blockIdx.x) % n_tiles; };
    auto load_tile = [&](int i) {   // thread 0: the i-th tile of this block into buffer i & 1 (a tile's rows are contiguous)
        const int t = tile_of(i);
        const int nt = min(kWideTile, T - t * kWideTile);
        const uint32_t bar = r_smem_u32(&s_bar[1 + (i & 1)]);
        r_mbar_expect_tx(bar, (uint32_t)nt * (uint32_t)H * 2u);
        r_bulk_g2s(r_smem_u32(xs + (size_t)(i & 1) * kWideTile * vec), x + (int64_t)t * kWideTile * H, (uint32_t)nt * (uint32_t)H * 2u, bar);
    };
    if (threadIdx.x == 0) {
        load_tile(0);
        if (n_tiles > 1) load_tile(1);
    }
    const int e = blockIdx.x * kWideRows + row;
    bool ok = r_mbar_wait(bar_w, 0);
    float4 wreg[NI > 0 ? NI : 1];
    if constexpr (NI > 0) {
        const float4* wsrc = reinterpret_cast<const float4*>(ws + (size_t)row * H) + lane;
#pragma unroll
        for (int c = 0; c < NI; c++) wreg[c] = wsrc[c * 32];
    }
    for (int i = 0; i < n_tiles; i++) {
        const int t = tile_of(i);
        const int nt = min(kWideTile, T - t * kWideTile);
        ok = ok && r_mbar_wait(r_smem_u32(&s_bar[1 + (i & 1)]), (uint32_t)((i >> 1) & 1));
        if (ok && 2 * q < nt) {
            const uint2* xb = xs + (size_t)(i & 1) * kWideTile * vec + lane;
            const uint2* x0p = xb + (size_t)(2 * q) * vec;
            const uint2* x1p = xb + (size_t)min(2 * q + 1, nt - 1) * vec;   // a slot past the batch aliases the last valid row
            const float4* wrow = reinterpret_cast<const float4*>(ws + (size_t)row * H) + lane;
            float a0 = 0.0f, a1 = 0.0f;
            auto step = [&](const float4& w, int c) {
                const uint2 u = x0p[c * 32], v = x1p[c * 32];
                a0 = __fmaf_rn(w.x, __uint_as_float(u.x << 16), a0);
                a0 = __fmaf_rn(w.y, __uint_as_float(u.x & 0xFFFF0000u), a0);
                a0 = __fmaf_rn(w.z, __uint_as_float(u.y << 16), a0);
                a0 = __fmaf_rn(w.w, __uint_as_float(u.y & 0xFFFF0000u), a0);
                a1 = __fmaf_rn(w.x, __uint_as_float(v.x << 16), a1);
                a1 = __fmaf_rn(w.y, __uint_as_float(v.x & 0xFFFF0000u), a1);
                a1 = __fmaf_rn(w.z, __uint_as_float(v.y << 16), a1);
                a1 = __fmaf_rn(w.w, __uint_as_float(v.y & 0xFFFF0000u), a1);
            };
            if constexpr (NI > 0) {
#pragma unroll
                for (int c = 0; c < NI; c++) step(wreg[c], c);
            } else {
                const int n_iter = H >> 7;
#pragma unroll 4
                for (int c = 0; c < n_iter; c++) step(wrow[c * 32], c);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                a0 = __fadd_rn(a0, __shfl_xor_sync(0xFFFFFFFFu, a0, off));
                a1 = __fadd_rn(a1, __shfl_xor_sync(0xFFFFFFFFu, a1, off));
            }
            if (lane == 0) {
                const int tok = t * kWideTile + 2 * q;
                logits[(int64_t)tok * E + e] = a0;
                if (2 * q + 1 < nt) logits[(int64_t)(tok + 1) * E + e] = a1;
            }
        }
        __syncthreads();   // every warp is done with this buffer
        if (threadIdx.x == 0 && i + 2 < n_tiles) load_tile(i + 2);
    }
    if (!ok && lane == 0) atomicOr(error_word, 4u);
    // ---- barrier across the grid: all logits are written
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd(&counters[0], 1u);
        bool arrived = false;
        for (uint32_t i = 0; i < kRouterWaitSpins && !arrived; i++) {
            arrived = __ldcg(&counters[0]) >= gridDim.x;
            if (!arrived) __nanosleep(64);
        }
        if (!arrived) {   // some blocks of the grid never became resident: the logits are incomplete
            atomicOr(error_word, 8u);
            atomicExch(&counters[2], 1u);
        }
        s_flag = arrived ? 1 : 0;
        __threadfence();
    }
    __syncthreads();
    float* s_score = reinterpret_cast<float*>(fsm);   // rows and tokens are no longer needed
    if (s_flag)
        for (int tok = blockIdx.x + warp * gridDim.x; tok < T; tok += kWideWarps * gridDim.x) {
            const float* lrow = logits + (int64_t)tok * E;
            topk_one_token<VPL>([&](int ee) { return __ldcg(lrow + ee); }, bias, cfg, selected + (int64_t)tok * cfg.n_used,
                                weights + (int64_t)tok * cfg.n_used, s_score + warp * E);
        }
    // ---- last block of the launch?
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_flag = (atomicAdd(&counters[1], 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (!s_flag) return;
    const bool failed = __ldcg(&counters[2]) != 0u;
    __syncthreads();
    if (threadIdx.x == 0) { counters[0] = 0u; counters[1] = 0u; counters[2] = 0u; }   // every block has left the barrier: it took a ticket
    __threadfence();
    if (failed) {
        // a barrier wait ran out: no picks are trustworthy, so the expert kernels get an empty work list
        // (the error word tells the host; the output rows of this call are undefined)
        for (int i = threadIdx.x; i <= E; i += kWideWarps * 32) {
            if (i < E) hist[i] = 0;
            offsets[i] = 0;
        }
        if (threadIdx.x == 0) n_work_items[0] = 0;
        return;
    }
    const int P = T * cfg.n_used;
    for (int i = threadIdx.x; i < P; i += kWideWarps * 32) s_sel[i] = __ldcg(selected + i);
    __syncthreads();
    groupdev::build_small<kWideWarps * 32, kFusedMaxPicks>(s_sel, P, E, 0, chunk, shared_T, hist, offsets, perm, work_items, n_work_items,
                                                           work_cap, reinterpret_cast<int*>(fsm), s_warp);
}

}  // namespace

// Shapes the one-launch decode router covers (everything else takes the three separate kernels).
bool router_fused_ok(int64_t T, const dsx_router_config& cfg, int64_t H) {
    const int v = cfg.n_expert / 32;
    return T >= 1 && T <= 64 && cfg.n_expert % 32 == 0 && (v == 1 || v == 2 || v == 4 || v == 8) && H % 256 == 0 &&
           (size_t)(kFusedRows * 4 + 8 * 2) * H <= 200 * 1024 && T * cfg.n_used <= kFusedMaxPicks && cfg.n_used <= kMaxUsed &&
           (cfg.n_group <= 1 || (cfg.n_group <= 32 && cfg.n_expert % cfg.n_group == 0));
}

int launch_router_logits(const __nv_bfloat16* x, int64_t T, const float* W, int n_expert, int64_t H, float* logits,
                         cudaStream_t stream) {
    DSX_REQUIRE(H % 128 == 0, "router_logits: hidden %lld must be a multiple of 128", (long long)H);
    if (T == 0) return DSX_OK;
    if (n_expert % kTileRowsR == 0 && T >= 128 && H % kTileCols == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0)) {   // a 16 x 32 tile finishes in about the time the warp-per-row kernel needs for 128 tokens
        // this entry point is also reached without a layer handle, so the opt-in to 96 KB of shared
        // memory is made here, once per device
        static std::atomic<uint64_t> opted_in{0};
        int dev = 0;
        DSX_CUDA(cudaGetDevice(&dev));
        if (!((opted_in.load(std::memory_order_relaxed) >> (dev & 63)) & 1)) {
            DSX_CUDA(cudaFuncSetAttribute(router_logits_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileStages * kTileStageBytes));
            opted_in.fetch_or(1ull << (dev & 63), std::memory_order_relaxed);
        }
        dim3 grid2((unsigned)(n_expert / kTileRowsR), (unsigned)((T + kTileTok - 1) / kTileTok));
        router_logits_tiled_kernel<<<grid2, kTileThreads, kTileStages * kTileStageBytes, stream>>>(x, T, W, n_expert, H, logits);
    } else {
        dim3 grid((unsigned)((n_expert + kLogitWarps - 1) / kLogitWarps), (unsigned)((T + kLogitTokens - 1) / kLogitTokens));
        router_logits_kernel<<<grid, kLogitWarps * 32, 0, stream>>>(x, T, W, n_expert, H, logits);
    }
    DSX_LAUNCHED();
    return DSX_OK;
}

namespace {
size_t fused_smem(int64_t H, int nt_per_warp, int n_expert) {
    return std::max<size_t>(std::max<size_t>((size_t)(kFusedRows * 4 + 2 * nt_per_warp * 2) * H, (size_t)kFusedWarps * n_expert * 4), kFusedScratch);
}
template <int V, int NT>
cudaError_t launch_fused_variant(dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16* x, int T, const float* W,
                                 const float* bias, int H, const dsx_router_config& cfg, float* logits, int32_t* selected,
                                 float* weights, int chunk, int shared_T, int32_t* hist, int32_t* offsets, int32_t* perm,
                                 int32_t* work_items, int32_t* n_work_items, int32_t work_cap, ItemRec* item_recs, unsigned int* counters,
                                 uint32_t* error_word) {
    return launch_pdl(router_fused_kernel<V, NT>, grid, dim3(kFusedWarps * 32), smem, stream, x, T, W, bias, H, cfg, logits, selected,
                      weights, chunk, shared_T, hist, offsets, perm, work_items, n_work_items, work_cap, item_recs, counters, error_word);
}
template <int V>
cudaError_t launch_fused_v(int nt_per_warp, dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16* x, int T, const float* W,
                           const float* bias, int H, const dsx_router_config& cfg, float* logits, int32_t* selected, float* weights,
                           int chunk, int shared_T, int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items,
                           int32_t* n_work_items, int32_t work_cap, ItemRec* item_recs, unsigned int* counters, uint32_t* error_word) {
#define DSX_FUSED_NT(N)                                                                                                         \
    case N:                                                                                                                      \
        return launch_fused_variant<V, N>(grid, smem, stream, x, T, W, bias, H, cfg, logits, selected, weights, chunk, shared_T, \
                                          hist, offsets, perm, work_items, n_work_items, work_cap, item_recs, counters, error_word);
    switch (nt_per_warp) {
        DSX_FUSED_NT(1) DSX_FUSED_NT(2) DSX_FUSED_NT(4)
    }
#undef DSX_FUSED_NT
    return cudaErrorInvalidValue;
}
template <int V, int NT>
cudaError_t configure_fused_variant() {
    return cudaFuncSetAttribute(router_fused_kernel<V, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}
size_t wide_smem(int64_t H, int n_expert) {
    return std::max<size_t>(std::max<size_t>((size_t)(kWideRows * 4 + 2 * kWideTile * 2) * H, (size_t)kWideWarps * n_expert * 4), kFusedScratch);
}
int g_sm_count = 0;   // of the device router_configure ran on
}  // namespace

int launch_router_fused(const __nv_bfloat16* x, int64_t T, const float* W, const float* bias, int64_t H, const dsx_router_config& cfg,
                        float* logits, int32_t* selected, float* weights, int chunk, int shared_T, int32_t* hist, int32_t* offsets,
                        int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap, ItemRec* item_recs,
                        unsigned int* counters, uint32_t* error_word, cudaStream_t stream) {
    DSX_REQUIRE(router_fused_ok(T, cfg, H) && chunk == 8, "router_fused: shape not covered");
    DSX_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0), "router_fused: token rows and router weights must be 16-byte aligned");
    if (T > kWideTile && cfg.n_expert / kWideRows <= g_sm_count && wide_smem(H, cfg.n_expert) <= 200 * 1024 && item_recs == nullptr) {
        // resident router rows, streamed tokens, one barrier across a grid that fits the device
        cudaError_t werr = cudaErrorInvalidValue;
        const dim3 wgrid((unsigned)(cfg.n_expert / kWideRows));
        const size_t wsmem = wide_smem(H, cfg.n_expert);
        const int ni = (H == 4096) ? 32 : (H == 2048 ? 16 : 0);   // widths whose router row lives in registers
#define DSX_WIDE_LAUNCH(V, N)                                                                                                     \
    werr = launch_pdl(router_fused_wide_kernel<V, N>, wgrid, dim3(kWideWarps * 32), wsmem, stream, x, (int)T, W, bias, (int)H, cfg,   \
                      logits, selected, weights, chunk, shared_T, hist, offsets, perm, work_items, n_work_items, work_cap,        \
                      counters, error_word)
#define DSX_WIDE_CASE(V)                                                  \
    case V:                                                               \
        if (ni == 32) DSX_WIDE_LAUNCH(V, 32);                             \
        else if (ni == 16) DSX_WIDE_LAUNCH(V, 16);                        \
        else DSX_WIDE_LAUNCH(V, 0);                                       \
        break;
        switch (cfg.n_expert / 32) {
            DSX_WIDE_CASE(1) DSX_WIDE_CASE(2) DSX_WIDE_CASE(4) DSX_WIDE_CASE(8)
            default:
                return set_error(DSX_ERR_UNSUPPORTED, "router_fused: n_expert %d not instantiated", cfg.n_expert);
        }
#undef DSX_WIDE_CASE
#undef DSX_WIDE_LAUNCH
        DSX_CUDA(werr);
        DSX_LAUNCHED();
        return DSX_OK;
    }
    const int nt_per_warp = T <= 2 ? 1 : (T <= 4 ? 2 : 4);
    const int tile = 2 * nt_per_warp;
    const size_t smem = fused_smem(H, nt_per_warp, cfg.n_expert);
    dim3 grid((unsigned)(cfg.n_expert / kFusedRows), (unsigned)((T + tile - 1) / tile));
    cudaError_t err = cudaErrorInvalidValue;
    switch (cfg.n_expert / 32) {
#define DSX_FUSED_CASE(V)                                                                                                      \
    case V:                                                                                                                    \
        err = launch_fused_v<V>(nt_per_warp, grid, smem, stream, x, (int)T, W, bias, (int)H, cfg, logits, selected, weights, chunk, \
                                shared_T, hist, offsets, perm, work_items, n_work_items, work_cap, item_recs, counters, error_word); \
        break;
        DSX_FUSED_CASE(1) DSX_FUSED_CASE(2) DSX_FUSED_CASE(4) DSX_FUSED_CASE(8)
#undef DSX_FUSED_CASE
        default:
            return set_error(DSX_ERR_UNSUPPORTED, "router_fused: n_expert %d not instantiated", cfg.n_expert);
    }
    DSX_CUDA(err);
    DSX_LAUNCHED();
    return DSX_OK;
}

// Opt the fused router in to its dynamic shared memory (once per device, at layer creation).
int router_configure() {
#define DSX_FUSED_CFG(V)                                  \
    DSX_CUDA((configure_fused_variant<V, 1>()));          \
    DSX_CUDA((configure_fused_variant<V, 2>()));          \
    DSX_CUDA((configure_fused_variant<V, 4>()));
    DSX_FUSED_CFG(1) DSX_FUSED_CFG(2) DSX_FUSED_CFG(4) DSX_FUSED_CFG(8)
#undef DSX_FUSED_CFG
#define DSX_WIDE_CFG(V)                                                                                                        \
    DSX_CUDA((cudaFuncSetAttribute(router_fused_wide_kernel<V, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));  \
    DSX_CUDA((cudaFuncSetAttribute(router_fused_wide_kernel<V, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024))); \
    DSX_CUDA((cudaFuncSetAttribute(router_fused_wide_kernel<V, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));
    DSX_WIDE_CFG(1) DSX_WIDE_CFG(2) DSX_WIDE_CFG(4) DSX_WIDE_CFG(8)
#undef DSX_WIDE_CFG
    int dev = 0;
    DSX_CUDA(cudaGetDevice(&dev));
    DSX_CUDA(cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev));
    return DSX_OK;
}

int launch_router_topk(const float* logits, const float* bias, int64_t T, const dsx_router_config& cfg,
                       int32_t* selected, float* weights, int n_alt, int32_t* alts, float* alt_w, float* range_out, cudaStream_t stream) {
    if (alts == nullptr) n_alt = 0;
    DSX_REQUIRE(n_alt >= 0 && cfg.n_used + n_alt <= kMaxUsed && cfg.n_used + n_alt <= cfg.n_expert,
                "router_topk: %d picks + %d alternatives (at most %d together)", cfg.n_used, n_alt, kMaxUsed);
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
        router_topk_kernel<V><<<grid, kTopkWarps * 32, 0, stream>>>(logits, bias, T, cfg, selected, weights, n_alt, alts, alt_w, range_out); \
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

int launch_router_topk_prior(const float* logits, const float* bias, int64_t T, const dsx_router_config& cfg, int32_t* selected,
                             float* weights, int n_alt, int32_t* alts, float* alt_w, float* range_out, const float* prior, int n_protect,
                             int prior_dry, int32_t* orig_sel, cudaStream_t stream) {
    if (alts == nullptr) n_alt = 0;
    DSX_REQUIRE(cfg.n_expert > 0 && cfg.n_expert % 32 == 0 && cfg.n_expert <= 512, "router_topk_prior: n_expert %d must be a multiple of 32, at most 512",
                cfg.n_expert);
    DSX_REQUIRE(cfg.n_used >= 1 && n_alt >= 0 && cfg.n_used + n_alt <= 32 && cfg.n_used + n_alt <= cfg.n_expert,
                "router_topk_prior: %d picks + %d alternatives", cfg.n_used, n_alt);
    DSX_REQUIRE(cfg.n_group <= 1, "router_topk_prior: the cache prior is defined without a group limit");
    DSX_REQUIRE(n_protect >= 0 && n_protect <= cfg.n_used, "router_topk_prior: n_protect %d of %d picks", n_protect, cfg.n_used);
    if (T == 0) return DSX_OK;
    const unsigned grid = (unsigned)((T + kTopkWarps - 1) / kTopkWarps);
    switch (cfg.n_expert / 32) {
#define DSX_PRIOR_CASE(V)                                                                                                         \
    case V:                                                                                                                       \
        router_topk_prior_kernel<V><<<grid, kTopkWarps * 32, 0, stream>>>(logits, bias, T, cfg, selected, weights, n_alt, alts, alt_w, \
                                                                          range_out, prior, n_protect, prior_dry, orig_sel);      \
        break;
        DSX_PRIOR_CASE(1) DSX_PRIOR_CASE(2) DSX_PRIOR_CASE(3) DSX_PRIOR_CASE(4) DSX_PRIOR_CASE(6) DSX_PRIOR_CASE(8)
        DSX_PRIOR_CASE(12) DSX_PRIOR_CASE(16)
#undef DSX_PRIOR_CASE
        default:
            return set_error(DSX_ERR_UNSUPPORTED, "router_topk_prior: n_expert %d not instantiated", cfg.n_expert);
    }
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace dsx
