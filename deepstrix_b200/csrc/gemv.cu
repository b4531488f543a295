// Decode-size grouped GEMV: gate/up + clamp + SwiGLU + routing weight, and down.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   gate/up  crates/v4flash-kernels/kernels/mxfp4_pair_matvec.hip:165-229 (decode, fused SwiGLU),
//            :566-640 (grouped by distinct expert: each expert read once)
//   down     crates/v4flash-kernels/kernels/mxfp4_matvec.hip:120-155, :534-600
//   Q8_0     crates/v4flash-kernels/kernels/q8_0_matvec.hip:64-91
//   SwiGLU   crates/v4flash-kernels/kernels/swiglu_clamp_weighted.hip:28-36
//
// Design (B200): one persistent block per SM.  A work item is (expert, up to 8
// tokens); a block takes a contiguous range of (item, 128-row block) units and
// each of its 8 warps owns one 16-row tile of the unit.  Weights are never
// touched by ordinary loads: lane 0 of every warp streams its row tile through a
// private 4-stage ring of shared memory with 1-D bulk copies (cp.async.bulk +
// mbarrier complete_tx), so each SM keeps ~140 KB of HBM reads in flight
// without spending registers on it, and every weight byte is read exactly once
// per item.  Lanes then read their 16 bytes per sub-tile from the ring, expand
// the 4-bit codes to f16 with the hardware converter (int8: byte permutes), and feed mma.sync.m16n8k16 with the item's (<= 8) tokens as the n dimension;
// the E8M0 / f16 block scale multiplies the f32 result of each 32-column block.
// Token columns are independent in the mma, so a token's result does not
// depend on which other tokens share its item.
#include <type_traits>

#include "dsx_common.cuh"

namespace dsx {
namespace {

constexpr int kRingStagesPerBlock = 32;  // ring stages per block: 8 warps x 4 deep, or 16 warps x 2 deep
constexpr int kSubPerStage = 8;  // sub-tiles per ring stage
constexpr int kStageNib = kSubPerStage * kSubNibBytes;
constexpr int kStageSc = kSubPerStage * kSubScBytes;
constexpr int kStageBytes = kStageNib + kStageSc;  // 4352
constexpr int kActPad = 32;                        // halves of padding per activation row (64 B: bank shift)
constexpr int kMaxTok = 8;
constexpr uint32_t kWaitSpins = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: returns false when the phase did not complete in kWaitSpins polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitSpins; i++) {
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
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Same with a zero accumulator input (first step of a scale block).
__device__ __forceinline__ void mma16816_zero(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

// Eight E2M1 codes -> the four f16x2 A-fragment registers of one k16 step: byte i
// of the word holds the two codes of register a_i, and the hardware converter
// (cvt.rn.f16x2.e2m1x2) expands a byte to two exact f16 values in one instruction.
__device__ __forceinline__ void mxfp4_frag(uint32_t q, uint32_t (&a)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
        : "r"(q));
}
// E8M0 byte number `b` of the packed scale word -> 2^(e-127) as f32 (mask, then
// shift into the exponent field; e = 0 gives 0 instead of the denormal 2^-127).
template <int B>
__device__ __forceinline__ float mxfp4_scale(uint32_t sw) {
    if constexpr (B == 3) return __uint_as_float((sw >> 1) & 0x7F800000u);
    else return __uint_as_float((sw & (0xFFu << (8 * B))) << (23 - 8 * B));
}

// Four offset-binary int8 (value ^ 0x80) -> two f16x2: 0x6400 | u is 1024 + u.
__device__ __forceinline__ uint32_t q8_pair(uint32_t w, uint32_t sel) {
    const uint32_t h = __byte_perm(w, 0x64646464u, sel);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&h), __half2half2(__ushort_as_half((unsigned short)0x6480)));
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int FMT>
__device__ __forceinline__ void compute_subtile(const uint8_t* nibp, const uint8_t* scp, int lane, const uint4* bf,
                                                float (&acc)[4]) {
    const uint4 wq = *reinterpret_cast<const uint4*>(nibp + lane * 16);
    const uint32_t sw = *reinterpret_cast<const uint32_t*>(scp + (lane >> 2) * 4);
    if (FMT == DSX_FMT_MXFP4) {
        uint32_t a[4];
        float c[4];
        // block 0: k16 steps 0 and 1
        mxfp4_frag(wq.x, a);
        mma16816_zero(c, a, bf[0].x, bf[0].y);
        mxfp4_frag(wq.y, a);
        mma16816(c, a, bf[0].z, bf[0].w);
        float s0 = mxfp4_scale<0>(sw), s1 = mxfp4_scale<2>(sw);
        acc[0] = fmaf(s0, c[0], acc[0]);
        acc[1] = fmaf(s0, c[1], acc[1]);
        acc[2] = fmaf(s1, c[2], acc[2]);
        acc[3] = fmaf(s1, c[3], acc[3]);
        // block 1: k16 steps 2 and 3
        mxfp4_frag(wq.z, a);
        mma16816_zero(c, a, bf[1].x, bf[1].y);
        mxfp4_frag(wq.w, a);
        mma16816(c, a, bf[1].z, bf[1].w);
        s0 = mxfp4_scale<1>(sw);
        s1 = mxfp4_scale<3>(sw);
        acc[0] = fmaf(s0, c[0], acc[0]);
        acc[1] = fmaf(s0, c[1], acc[1]);
        acc[2] = fmaf(s1, c[2], acc[2]);
        acc[3] = fmaf(s1, c[3], acc[3]);
    } else {
        float c[4];
        uint32_t a[4];
        a[0] = q8_pair(wq.x, 0x4140);
        a[2] = q8_pair(wq.x, 0x4342);
        a[1] = q8_pair(wq.y, 0x4140);
        a[3] = q8_pair(wq.y, 0x4342);
        mma16816_zero(c, a, bf[0].x, bf[0].y);
        a[0] = q8_pair(wq.z, 0x4140);
        a[2] = q8_pair(wq.z, 0x4342);
        a[1] = q8_pair(wq.w, 0x4140);
        a[3] = q8_pair(wq.w, 0x4342);
        mma16816(c, a, bf[0].z, bf[0].w);
        const __half2 sh = *reinterpret_cast<const __half2*>(&sw);
        const float s0 = __low2float(sh), s1 = __high2float(sh);
        acc[0] = fmaf(s0, c[0], acc[0]);
        acc[1] = fmaf(s0, c[1], acc[1]);
        acc[2] = fmaf(s1, c[2], acc[2]);
        acc[3] = fmaf(s1, c[3], acc[3]);
    }
}

// The current item of the block, in shared memory: derived in the kernel (ItemInfo), or an
// ItemRec copied from the decode router's records (small batches).
struct ItemInfo {
    int n_tok;
    int tok[kMaxTok];      // token index (gate/up source row)
    int mid_row[kMaxTok];  // row of mid (permuted order)
    int out_row[kMaxTok];  // row of partial (t*k+s, or P+t for the shared expert)
    float w[kMaxTok];
};

// FMT: routed format for routed items; shared items use SFMT.  The kernel is
// compiled for the (FMT, SFMT) pairs with FMT == SFMT only, which keeps one
// decode path per item.
// WARPS / KSPLIT: four warps per scheduler hide the cvt -> mma -> fma latencies that two cannot, so
// blocks have 16 warps (2 ring stages each) whenever the shape allows.  With >= 8 tokens there are
// enough (item, 256-row block) units for every SM (KSPLIT 1: one row tile per warp).  Below that,
// units stay 128 rows and two warps share a row tile, each taking one half of the reduction
// (KSPLIT 2); the halves are added through shared memory.  Every variant adds
// (first half of the columns) + (second half), so the bits do not depend on the variant.
//
// SMALL (batches below 8 tokens routed by the one-launch decode router, where the kernels' fixed
// costs are a large share): an item is one ready-made ItemRec, and what does not depend on the
// previous kernel of the chain runs before the wait for it: gate/up stages every token row once,
// as f16 (its predecessor releases it only after the token rows are complete); an item then only
// selects rows.  In every variant the down kernel reads the work list and requests its first weights
// before it waits for gate/up (gate/up releases it after its own wait, when the routing is complete;
// worth 3 us per layer step at every batch size).  Otherwise the kernel derives an
// item from offsets / perm / weights and stages its rows when the block reaches it; that code is
// kept apart at compile time because the streaming loop's schedule is sensitive to it.
template <int FMT, bool PAIR, int WARPS, int KSPLIT, bool SMALL>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_kernel(const GemvArgs a) {
    constexpr int kWarps = WARPS, kThreads = WARPS * 32, kStages = kRingStagesPerBlock / WARPS;
    constexpr int kRowWarps = WARPS / KSPLIT;   // row tiles per unit
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kTileK = (FMT == DSX_FMT_MXFP4) ? 64 : 32;
    constexpr int kBlocks = kTileK / 32;            // 32-column scale blocks per sub-tile
    constexpr int kSubPerCt = PAIR ? 2 : 1;          // sub-tiles per column tile
    constexpr int kCtPerStage = kSubPerStage / kSubPerCt;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int64_t K = a.K;
    const int act_stride = (int)K + kActPad;  // halves
    __half* act = reinterpret_cast<__half*>(smem);
    uint8_t* ring = smem + (((size_t)kMaxTok * act_stride * 2 + 127) & ~(size_t)127);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)kWarps * kStages * kStageBytes);
    using Info = typename std::conditional<SMALL, ItemRec, ItemInfo>::type;
    Info* info = reinterpret_cast<Info*>(bars + kWarps * kStages);
    float* halves = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(info) + ((sizeof(ItemRec) + 127) & ~(size_t)127));  // KSPLIT 2: [2][kRowWarps][32][8]
    const int rw = warp % kRowWarps, kh = warp / kRowWarps;   // row tile inside the unit, reduction half

    uint8_t* my_ring = ring + (size_t)warp * kStages * kStageBytes;
    const uint32_t my_bars = smem_u32(bars + warp * kStages);
    if (lane == 0)
        for (int s = 0; s < kStages; s++) mbar_init(my_bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    constexpr bool all_rows_staged = SMALL && PAIR;
    uint32_t bad = 0;   // a value that left the f16 range (reported once, when the block ends)
    if (all_rows_staged) {
        // loads that bypass L1: this runs while the previous kernel may still be executing
        const int vec_per_row = (int)(K >> 3);
        for (int v = threadIdx.x; v < (int)a.T * vec_per_row; v += kThreads) {
            const int r = v / vec_per_row, c8 = v - r * vec_per_row;
            const uint4 in = __ldcg(reinterpret_cast<const uint4*>(a.x + (int64_t)r * K) + c8);
            *reinterpret_cast<uint4*>(act + (size_t)r * act_stride + c8 * 8) =
                make_uint4(bf16x2_to_f16x2(in.x, bad), bf16x2_to_f16x2(in.y, bad), bf16x2_to_f16x2(in.z, bad), bf16x2_to_f16x2(in.w, bad));
        }
    }
    __syncthreads();
    if (PAIR) {
        pdl_wait();   // work items and routing come from the previous kernel of the chain
        // the next kernel (down) reads the routing before its own wait: release it only now
        pdl_launch_dependents();
    } else {
        // routing and weights are complete (the gate/up kernel released this one after its own wait):
        // everything up to the first weight requests runs beside the gate/up kernel's tail
        pdl_launch_dependents();
    }

    const int n_items = a.n_work_items[0];
    const int n_kt = (int)(K / kTileK);
    const int n_stage = (n_kt + kCtPerStage - 1) / kCtPerStage;
    const int bpi = (int)(a.rows / (kTileRows * kRowWarps));  // row blocks per item
    const int U = n_items * bpi;
    const int u0 = (int)((int64_t)U * blockIdx.x / gridDim.x), u1 = (int)((int64_t)U * (blockIdx.x + 1) / gridDim.x);
    const int n_half = n_stage / KSPLIT;    // stages of a unit this warp consumes (the launcher picks KSPLIT 2 only for even n_stage)
    const int hs = n_stage / 2;             // stages below hs form the "first half" sum in every variant
    const int total = (u1 - u0) * n_half;   // ring stages this warp will consume
    const int P = (int)(a.T * a.n_used);

    // ---- producer state (lane 0): next stage to request, tracked incrementally
    int p_item = u0 / bpi, p_rb = u0 - p_item * bpi, p_ls = 0, p_cnt = 0, p_cached = -1;
    const uint8_t* p_nib = nullptr;
    const uint8_t* p_sc = nullptr;
    auto issue = [&]() {
        if (p_item != p_cached) {
            const int e = SMALL ? __ldcg(&a.item_recs[p_item].expert) : (int)((uint32_t)a.work_items[p_item] >> 16);
            p_nib = (e == a.n_expert) ? a.sh_nib : a.nib + (int64_t)e * a.nib_slot_stride;
            p_sc = (e == a.n_expert) ? a.sh_sc : a.sc + (int64_t)e * a.sc_slot_stride;
            p_cached = p_item;
        }
        const int rt = p_rb * kRowWarps + rw;
        const int ct0 = (kh * n_half + p_ls) * kCtPerStage;
        const int n_ct = min(kCtPerStage, n_kt - ct0);
        const int64_t sub0 = ((int64_t)rt * n_kt + ct0) * kSubPerCt;
        const uint32_t nsub = (uint32_t)(n_ct * kSubPerCt);
        const int slot = p_cnt & (kStages - 1);
        const uint32_t bar = my_bars + 8 * slot;
        const uint32_t dst = smem_u32(my_ring + (size_t)slot * kStageBytes);
        mbar_expect_tx(bar, nsub * (kSubNibBytes + kSubScBytes));
        bulk_g2s(dst, p_nib + sub0 * kSubNibBytes, nsub * kSubNibBytes, bar);
        bulk_g2s(dst + kStageNib, p_sc + sub0 * kSubScBytes, nsub * kSubScBytes, bar);
        p_cnt++;
        if (++p_ls == n_half) {
            p_ls = 0;
            if (++p_rb == bpi) { p_rb = 0; p_item++; }
        }
    };

    if (lane == 0)
        for (int i = 0; i < total && i < kStages; i++) issue();
    if (!PAIR) pdl_wait();   // the rows of mid come from the gate/up kernel

    int item = u0 / bpi, rb = u0 - item * bpi, ls = 0;
    int cur_item = -1;
    bool dead = false;
    int unit_parity = 0;
    float acc0[4], acc1[4];     // running sums of the current half of the columns (gate / up, or single)
    float acc0a[4], acc1a[4];   // finished first half
    for (int cnt = 0; cnt < total; cnt++) {
        if (ls == 0) {
            if (item != cur_item) {
                // all warps of the block change item together (same unit sequence)
                __syncthreads();
                if constexpr (SMALL) {
                    if (threadIdx.x < kItemRecWords)
                        reinterpret_cast<int32_t*>(info)[threadIdx.x] = __ldcg(reinterpret_cast<const int32_t*>(a.item_recs + item) + threadIdx.x);
                } else if (threadIdx.x < kMaxTok) {
                    const uint32_t wi = (uint32_t)a.work_items[item];
                    const int e = (int)(wi >> 16), start = (int)(wi & 0xFFFFu), i = threadIdx.x;
                    if (e == a.n_expert) {  // shared expert: tokens start..start+7, weight 1
                        const int n = (int)min((int64_t)kMaxTok, a.T - start);
                        if (i == 0) info->n_tok = n;
                        info->tok[i] = start + i;
                        info->mid_row[i] = P + start + i;
                        info->out_row[i] = P + start + i;
                        info->w[i] = 1.0f;
                    } else {
                        const int seg0 = a.offsets[e], cntm = a.offsets[e + 1] - seg0;
                        const int n = min(kMaxTok, cntm - start);
                        if (i == 0) info->n_tok = n;
                        const int p = seg0 + start + min(i, n - 1);
                        const int ts = a.perm[p];
                        info->tok[i] = ts / a.n_used;
                        info->mid_row[i] = p;
                        info->out_row[i] = ts;
                        info->w[i] = a.route_w[ts];
                    }
                }
                __syncthreads();
                if (!all_rows_staged) {
                    // stage the item's activation rows as f16
                    const int n = info->n_tok;
                    const int vec_per_row = (int)(K >> 3);
                    for (int v = threadIdx.x; v < n * vec_per_row; v += kThreads) {
                        const int r = v / vec_per_row, c8 = v - r * vec_per_row;
                        uint4 out;
                        if (PAIR) {
                            const uint4 in = __ldg(reinterpret_cast<const uint4*>(a.x + (int64_t)info->tok[r] * K) + c8);
                            out = make_uint4(bf16x2_to_f16x2(in.x, bad), bf16x2_to_f16x2(in.y, bad), bf16x2_to_f16x2(in.z, bad),
                                             bf16x2_to_f16x2(in.w, bad));
                        } else {
                            out = *(reinterpret_cast<const uint4*>(a.mid + (int64_t)info->mid_row[r] * a.mid_stride) + c8);
                        }
                        *reinterpret_cast<uint4*>(act + (size_t)r * act_stride + c8 * 8) = out;
                    }
                    __syncthreads();
                }
                cur_item = item;
            }
#pragma unroll
            for (int i = 0; i < 4; i++) acc0[i] = acc1[i] = acc0a[i] = acc1a[i] = 0.f;
        }
        const int slot = cnt & (kStages - 1);
        if (!dead && !mbar_wait(my_bars + 8 * slot, (uint32_t)((cnt / kStages) & 1))) {
            dead = true;
            if (lane == 0) atomicOr(a.error_word, 1u);
        }
        if (!dead) {
            const uint8_t* st_nib = my_ring + (size_t)slot * kStageBytes;
            const uint8_t* st_sc = st_nib + kStageNib;
            const int ls_all = kh * n_half + ls;   // stage index inside the whole reduction
            const int ct0 = ls_all * kCtPerStage;
            const int n_ct = min(kCtPerStage, n_kt - ct0);
            if (ls_all == hs) {   // the second half starts: park the first half's sums
#pragma unroll
                for (int i = 0; i < 4; i++) { acc0a[i] = acc0[i]; acc1a[i] = acc1[i]; acc0[i] = acc1[i] = 0.f; }
            }
            const bool tok_ok = g < info->n_tok;
            const __half* arow = act + (size_t)(all_rows_staged ? (tok_ok ? info->tok[g] : 0) : g) * act_stride + (size_t)ct0 * kTileK + 8 * t4;
            auto col_tile = [&](int c) {
                uint4 bf[kBlocks];
#pragma unroll
                for (int b = 0; b < kBlocks; b++) {
                    bf[b] = make_uint4(0u, 0u, 0u, 0u);
                    if (tok_ok) bf[b] = *reinterpret_cast<const uint4*>(arow + c * kTileK + 32 * b);
                }
                compute_subtile<FMT>(st_nib + (size_t)(c * kSubPerCt) * kSubNibBytes, st_sc + (size_t)(c * kSubPerCt) * kSubScBytes, lane, bf, acc0);
                if (PAIR)
                    compute_subtile<FMT>(st_nib + (size_t)(c * 2 + 1) * kSubNibBytes, st_sc + (size_t)(c * 2 + 1) * kSubScBytes, lane, bf, acc1);
            };
            if (n_ct == kCtPerStage) {  // full stage: unrolled so independent sub-tiles overlap
#pragma unroll
                for (int c = 0; c < kCtPerStage; c++) col_tile(c);
            } else {
                for (int c = 0; c < n_ct; c++) col_tile(c);
            }
        }
        __syncwarp();
        if (lane == 0 && !dead && p_cnt < total) issue();

        if (KSPLIT == 2 && ls == n_half - 1) {
            // hand the second half's sums to the warp that owns the row tile
            float* slot = halves + ((size_t)(unit_parity * kRowWarps + rw) * 32 + lane) * 8;
            if (kh == 1) {   // this warp's running sums ARE the second half
#pragma unroll
                for (int i = 0; i < 4; i++) { slot[i] = acc0[i]; slot[4 + i] = acc1[i]; }
            }
            __syncthreads();
            if (kh == 0) {   // this warp's running sums are the first half
#pragma unroll
                for (int i = 0; i < 4; i++) { acc0a[i] = acc0[i]; acc1a[i] = acc1[i]; acc0[i] = slot[i]; acc1[i] = slot[4 + i]; }
            }
            unit_parity ^= 1;
        }
        if (ls == n_half - 1 && !dead && kh == 0) {
            const int row0 = (rb * kRowWarps + rw) * kTileRows + g;
#pragma unroll
            for (int i = 0; i < 4; i++) {   // (first half) + (second half), the same in every variant
                acc0[i] = acc0a[i] + acc0[i];
                acc1[i] = acc1a[i] + acc1[i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int n = 2 * t4 + (i & 1);
                const int row = row0 + ((i >> 1) ? 8 : 0);
                if (n < info->n_tok) {
                    if (PAIR) {
                        float gv = acc0[i], uv = acc1[i];
                        if (a.clamp > 1.0e-6f) {
                            gv = fminf(gv, a.clamp);
                            uv = fminf(fmaxf(uv, -a.clamp), a.clamp);
                        }
                        const float sig = 1.0f / (1.0f + __expf(-gv));
                        a.mid[(int64_t)info->mid_row[n] * a.mid_stride + row] = f32_to_f16_checked(gv * sig * uv * info->w[n], bad);
                    } else {
                        a.partial[(int64_t)info->out_row[n] * a.rows + row] = acc0[i];
                    }
                }
            }
        }
        if (++ls == n_half) {
            ls = 0;
            if (++rb == bpi) { rb = 0; item++; }
        }
    }
    if (bad) atomicOr(a.error_word, kErrHalfRange);
}

// Shared memory of one block: 8 activation rows, the rings, barriers, the item and (two warps per row
// tile only) the exchange buffer of the two halves.
size_t gemv_smem_bytes(int64_t K, bool with_halves) {
    const size_t act = (((size_t)kMaxTok * (size_t)(K + kActPad) * 2) + 127) & ~(size_t)127;
    return act + (size_t)kRingStagesPerBlock * kStageBytes + sizeof(uint64_t) * kRingStagesPerBlock + ((sizeof(ItemRec) + 127) & ~(size_t)127) +
           (with_halves ? (size_t)2 * 8 * 32 * 8 * sizeof(float) : 0) + 128;
}

constexpr size_t kMaxSmem = 227 * 1024;

#ifndef DSX_PAIR_WIDE_FROM
#define DSX_PAIR_WIDE_FROM 10
#endif

struct Variant {
    int warps, ksplit;   // 0 warps: nothing fits
    size_t smem;
};

// Which instantiation a launch takes.  256-row units (one row tile per warp) need enough (item, unit)
// pairs for every SM: the item count lives on the device, so the batch size decides (>= 8 tokens x
// top-k picks is plenty).  Below that two warps share a row tile when the stage count is even, else
// 8 warps own one each; a reduction too long for the exchange buffer falls back to 256-row units.
Variant pick_variant(int fmt, bool pair, int64_t K, int64_t rows, int64_t T) {
    const int tile_k = fmt == DSX_FMT_MXFP4 ? 64 : 32, ct_per_stage = pair ? kSubPerStage / 2 : kSubPerStage;
    const int n_stage = (int)((K / tile_k + ct_per_stage - 1) / ct_per_stage);
    const bool can_wide = rows % (kTileRows * 16) == 0;
    const size_t plain = gemv_smem_bytes(K, false), split = gemv_smem_bytes(K, true);
    // gate/up of 8 or 9 tokens: ~60 items x 8 wide units leave some blocks a fourth unit while most have
    // three; 128-row units halve that tail (a small gain at 8 tokens, a loss from 12 tokens on)
    const int64_t wide_from = (pair && n_stage % 2 == 0 && split <= kMaxSmem) ? DSX_PAIR_WIDE_FROM : 8;
    if (can_wide && T >= wide_from && plain <= kMaxSmem) return {16, 1, plain};
    if (n_stage % 2 == 0 && split <= kMaxSmem) return {16, 2, split};
    if (n_stage % 2 != 0 && plain <= kMaxSmem) return {8, 1, plain};
    if (can_wide && plain <= kMaxSmem) return {16, 1, plain};
    return {0, 0, plain};
}

template <int FMT, bool PAIR>
int launch_one(const GemvArgs& a, int sm_count, cudaStream_t stream) {
    const Variant v = pick_variant(FMT, PAIR, a.K, a.rows, a.T);
    DSX_REQUIRE(v.warps != 0, "gemv: reduction length %lld needs %zu B of shared memory (max %zu)", (long long)a.K, v.smem, kMaxSmem);
    const size_t smem = v.smem;
    const bool small = a.item_recs != nullptr && a.T < kMaxTok;
#define DSX_GEMV_LAUNCH(W, S, SM) DSX_CUDA(launch_pdl(gemv_kernel<FMT, PAIR, W, S, SM>, dim3(sm_count), dim3(W * 32), smem, stream, a))
    if (v.warps == 16 && v.ksplit == 1) {
        DSX_REQUIRE(!small, "gemv: item records need the small-batch kernels (see gemv_small_batch_ok)");
        DSX_GEMV_LAUNCH(16, 1, false);
    } else if (v.warps == 16) { if (small) DSX_GEMV_LAUNCH(16, 2, true); else DSX_GEMV_LAUNCH(16, 2, false); }
    else { if (small) DSX_GEMV_LAUNCH(8, 1, true); else DSX_GEMV_LAUNCH(8, 1, false); }
#undef DSX_GEMV_LAUNCH
    DSX_LAUNCHED();
    return DSX_OK;
}

int check_args(const GemvArgs& a) {
    DSX_REQUIRE(a.K % 256 == 0, "gemv: reduction length %lld must be a multiple of 256", (long long)a.K);
    DSX_REQUIRE(a.rows % (kTileRows * 8) == 0, "gemv: %lld rows must be a multiple of %d", (long long)a.rows, kTileRows * 8);
    DSX_REQUIRE(a.sh_nib == nullptr || (a.shared_fmt == a.fmt && a.sh_rows == a.rows),
                "gemv: the shared expert must have the routed experts' format and width");
    return DSX_OK;
}

}  // namespace

bool gemv_fits(int64_t K) { return K % 256 == 0 && gemv_smem_bytes(K, false) <= kMaxSmem; }

// Batches below 8 tokens may use item records only when both kernels of the chain take a small-batch
// instantiation (they rely on each other's release order).
bool gemv_small_batch_ok(int fmt, int64_t hidden, int64_t ffn, int64_t T) {
    const Variant gu = pick_variant(fmt, true, hidden, ffn, T), dn = pick_variant(fmt, false, ffn, hidden, T);
    return T < kMaxTok && gu.warps != 0 && dn.warps != 0 && !(gu.warps == 16 && gu.ksplit == 1) && !(dn.warps == 16 && dn.ksplit == 1);
}

int launch_gemv_gate_up(const GemvArgs& a, int sm_count, cudaStream_t stream) {
    if (int rc = check_args(a)) return rc;
    return a.fmt == DSX_FMT_MXFP4 ? launch_one<DSX_FMT_MXFP4, true>(a, sm_count, stream)
                                  : launch_one<DSX_FMT_Q8_0, true>(a, sm_count, stream);
}

int launch_gemv_down(const GemvArgs& a, int sm_count, cudaStream_t stream) {
    if (int rc = check_args(a)) return rc;
    return a.fmt == DSX_FMT_MXFP4 ? launch_one<DSX_FMT_MXFP4, false>(a, sm_count, stream)
                                  : launch_one<DSX_FMT_Q8_0, false>(a, sm_count, stream);
}

// Opt every instantiation in to the large dynamic shared-memory carve-out.  Done
// once per device at layer creation so that launches are plain stream work
// (capturable in a graph).
int gemv_configure() {
#define DSX_GEMV_ATTR(F, P, W, S, SM) DSX_CUDA(cudaFuncSetAttribute(gemv_kernel<F, P, W, S, SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem))
#define DSX_GEMV_ATTR3(F, P) DSX_GEMV_ATTR(F, P, 16, 1, false); DSX_GEMV_ATTR(F, P, 16, 2, false); DSX_GEMV_ATTR(F, P, 16, 2, true); \
                             DSX_GEMV_ATTR(F, P, 8, 1, false); DSX_GEMV_ATTR(F, P, 8, 1, true)
    DSX_GEMV_ATTR3(DSX_FMT_MXFP4, true); DSX_GEMV_ATTR3(DSX_FMT_MXFP4, false);
    DSX_GEMV_ATTR3(DSX_FMT_Q8_0, true); DSX_GEMV_ATTR3(DSX_FMT_Q8_0, false);
#undef DSX_GEMV_ATTR3
#undef DSX_GEMV_ATTR
    return DSX_OK;
}

}  // namespace dsx
