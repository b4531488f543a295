// Prefill-size grouped GEMM for MXFP4 experts on the block-scaled FP4 tensor cores
// (tcgen05.mma.kind::mxf4.block_scale), weights and scales consumed as stored.
//
// Reference counterparts (paths relative to the deepstrix repository): the by-expert prefill kernels
// and their matrix-core arms,
//   gate/up  crates/v4flash-kernels/kernels/mxfp4_pair_matvec.hip:293-564, mxfp4_moe_wmma.hip:137-368
//   down     crates/v4flash-kernels/kernels/mxfp4_matvec.hip:219-369,      mxfp4_moe_wmma.hip:370-388
//   activation quantiser  crates/v4flash-kernels/kernels/q8_k_quantize.hip:23-90 (the reference turns
//            activations into int8 blocks for its integer dot; here they become MXFP4 terms, see below)
//
// Operands.  The weights are E2M1 codes with one E8M0 scale per 32: exactly what kind::mxf4 multiplies,
// so they go from HBM to shared memory by TMA (K-major rows, 64-byte swizzle) and their scales to tensor
// memory, untouched.  The other operand of kind::mxf4 is FP4 too, and one FP4 value per
// activation is far too coarse (rel-L2 0.2 on the layer).  So an activation row x is written as a SUM of
// three MXFP4 rows, x ~ t1 + t2 + t3: t1 = x rounded to E2M1 with a power-of-two scale per 32, t2 the
// same rounding of the residual x - t1 with its own scales, t3 of x - t1 - t2 (mx_terms_of_block;
// every step exact in f32, so the CPU can restate it bit for bit).  Each term is one more MMA into the same
// accumulator.  Three terms leave a relative error of about 3e-3 on the layer output (two terms 2.5e-2,
// a single E4M3 term 4.6e-2), for 1.5 times the tensor-core time of one FP8 pass.
//
// Tiling.  Expert-sorted rows are cut into segments of at most 192 rows of one expert, and a tile = (segment, 256
// weight rows) = two M = 128 accumulators that share the segment's rows as N (first product: 128 gate rows and the
// 128 up rows of the same outputs, so that a tensor-memory lane holds gate and up of one output row).  Tensor
// memory: 2 x 192 accumulator columns and four scale slots of 32 columns, one per ring stage.  A pipeline stage is
// 128 reduction columns: 16 KB of weight codes (one TMA box), up to 3 x 12 KB of activation terms (one TMA box of
// 64, 128 or 192 rows x 3 terms), 1 KB + 3 KB of scale chunks, all arriving on one mbarrier; 4 stages.
// Warp roles (20 warps; register counts redistributed per warp group with setmaxnreg): one producer thread; two
// MMA threads, one accumulator each, 2 (k steps of 64) x 3 (terms) MMAs per stage; four scale warps, one per lane
// quarter of tensor memory, that move a landed stage's scale chunks from shared memory into the stage's scale slot
// (ld.shared + tcgen05.st -- the tensor core's own copy instruction, tcgen05.cp, runs in the MMA queue and held the
// MMAs up for 0.4 of 3.0 ms on the 8192-token layer); 12 epilogue warps that read the accumulators (tcgen05.ld), apply
// clamp + SwiGLU + routing weight and store mid (f16), or store the per-pick partial rows (f32): the second half of
// a warp's columns is read whole and tensor memory handed back before their arithmetic and stores run.
// CTA pairs.  From 96 rows per expert on (per call) the kernel runs as clusters of two CTAs with cta_group::2 MMAs:
// a pair takes two neighbouring tiles of one segment, every MMA spans both (M = 256), and each CTA loads only half
// of the segment's rows.  Each CTA's loads count on its own barrier; the scale warps of both report to the even CTA,
// whose two MMA threads issue for the pair; commits arrive in both.  No load is broadcast.
// Single CTAs (fewer rows per expert) cap their segments at 96 rows, which leaves tensor memory for two accumulator
// buffers that alternate per tile: a tile's read-out then runs under the next tile's MMAs.
// What bounds it.  (1) L2 -> shared-memory traffic, which a tall tile (many weight rows per activation row) and the
// pair's halved activation rows reduce.  (2) Shared memory's 128 bytes per clock, which the tensor core's operand
// reads share with those fills: an M = 128, K = 64 MMA over N rows reads 4 KB of weights and 32 N bytes of terms in
// N / 2 clocks, i.e. 8192 / N + 64 bytes per clock, which a wide N serves best.  The first shape of this kernel (512
// weight rows x 96 rows, four accumulators) needed 149 + 46 bytes per MMA clock: shared memory was 96 % busy, the
// tensor pipe 60 %.  (3) The tensor-core queue itself: MMAs, plus whatever else is put into it.  (4) The part of the
// epilogue that runs before tensor memory is handed back (the accumulators fill it: no double buffer): with the
// epilogue taken out the 8192-token layer is 0.46 ms shorter.
// Every wait is bounded; on a timeout the block raises an abort flag, all roles drain, tensor memory
// is freed and bit 2 of the layer's error word is set.
#include <algorithm>

#include "prefill.cuh"

namespace dsx {
namespace {

constexpr int kEpiWarps = 12;
constexpr int kMmaWarps = 2;                  // issuing warps: each owns one of the tile's two accumulators (one warp for both: 9 % slower)
constexpr int kScWarp0 = 4;                   // four warps (one per lane quarter of tensor memory) carry the scales
constexpr int kEpiWarp0 = 8;                  // warp 3 has no role: roles start on warp-group boundaries
constexpr int kThreads = (kEpiWarp0 + kEpiWarps) * 32;
static_assert(1 + kMmaWarps <= kScWarp0, "producer and issuing warps fit below the scale warps");
constexpr int kAccs = 2;                      // M = 128 accumulators per tile (256 weight rows), one per issuing warp
constexpr int kSegRows = 192;                 // most rows of a segment (MMA N)
constexpr int kBRows = 192;                   // rows of a term plane in shared memory
constexpr int kBoxRows = 64;                  // granularity of the token-tile copy: boxes of 64, 128 or 192 rows
constexpr int kTerms = 3;                     // MXFP4 terms per activation row
constexpr int kStageK = 128;                  // reduction columns per pipeline stage (4 scale blocks)
constexpr int kRowBytes = kStageK / 2;        // packed bytes per row and stage: one 64-byte swizzle row
constexpr int kStages = 4;
constexpr int kABytes = kAccs * 128 * kRowBytes;         // 16384
constexpr int kBTermBytes = kBRows * kRowBytes;          // 12288
constexpr int kBBytes = kTerms * kBTermBytes;            // 36864
constexpr int kSfChunk = 512;                            // 128 rows x 4 scale blocks
constexpr int kSfbChunks = (kSegRows + 127) / 128;       // chunks per term: rows 0..127, 128..191
constexpr int kSfaBytes = kAccs * kSfChunk;
constexpr int kSfbBytes = kTerms * kSfbChunks * kSfChunk;
constexpr int kSmemA = 0;
constexpr int kSmemB = kSmemA + kStages * kABytes;
constexpr int kSmemSfa = kSmemB + kStages * kBBytes;
constexpr int kSmemSfb = kSmemSfa + kStages * kSfaBytes;
constexpr int kSmemBar = kSmemSfb + kStages * kSfbBytes;
constexpr int kNumBars = 3 * kStages + 4;
constexpr int kSmemMisc = kSmemBar + kNumBars * 8;
constexpr int kSmemTotal = kSmemMisc + 16 + 1024;        // + alignment slack
static_assert(kSmemTotal <= 227 * 1024, "stage ring exceeds the shared memory of an SM");
// tensor-memory columns
constexpr uint32_t kSfaCol = kAccs * kSegRows;    // accumulator h at column h * kSegRows; then 4 columns of weight scales per accumulator
// scale slot of ring stage s: kScSlot columns at kSfaCol + s * kScSlot = 4 per accumulator (weight scales), then 4 per
// term and chunk of 128 rows (activation scales) -- the order in which a stage's chunks lie in shared memory
constexpr uint32_t kScSlot = 4 * kAccs + 4 * kSfbChunks * kTerms;
static_assert(kSfaCol + kStages * kScSlot <= 512, "tensor memory holds 512 columns");
static_assert(kScSlot == 32 && kSfaBytes + kSfbBytes == 32 * 128, "a scale warp moves a stage's scales as 32 registers per lane");
static_assert(kBTermBytes % 512 == 0, "a term plane must start on a swizzle-atom boundary");
static_assert(kAccs % kMmaWarps == 0, "accumulators divide evenly over the issuing warps");
constexpr uint32_t kSpinLimit = 1u << 22;
#ifndef DSX_MX_SMALL_MAX
#define DSX_MX_SMALL_MAX 8
#endif
constexpr int kMxSmallMax = DSX_MX_SMALL_MAX;
constexpr int kShortRows = 96;                // segment cap of the double-buffered form: 2 buffers x 2 accumulators x 96 columns
constexpr int kPairFromRows = 96;             // average rows per expert from which the GEMMs run as CTA pairs

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait that also gives up when another role of the block has aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1u;
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[128 x N] (+)= A[128 x 64] . B[N x 64]^T, E2M1 operands, one E8M0 scale per 32 columns of either operand;
// the descriptors are given as low words (the high word -- stride, version, swizzle -- is common to every
// operand tile): the issuing thread is bound by its own scalar instructions, a 32-bit add per operand is the least.
__device__ __forceinline__ void tc_mma_mxf4_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %7, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %4, [%5], [%6], p;\n\t}"
        ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// lane r of the warp writes 32 columns of its tensor-memory lane
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
          "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
          "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// ---- CTA pairs (cta_group::2): the even CTA of a cluster of two issues the MMAs for both
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t cta) {   // the same shared-memory offset in another CTA of the cluster
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(cta));
    return r;
}
// Arrival on a barrier of the other CTA of a pair.  Relaxed on purpose: what the arrival reports (tensor-memory stores
// this warp has waited for, TMA bytes whose barrier it has seen complete) is finished before the instruction issues, and
// the default .release form at cluster scope held the issuing thread for about a microsecond per arrival, which bounded
// a whole pipeline stage when one thread forwarded an arrival per stage.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {   // arrives on one barrier, of either CTA of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// D[256 x N] (+)= A[256 x 64] . B[N x 64]^T over a CTA pair: rows 0..127 of A and D belong to the even CTA, 128..255 to the
// odd one; each CTA holds N / 2 rows of B.
__device__ __forceinline__ void tc_mma_mxf4_lo_pair(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t sfa,
                                                    uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %7, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %4, [%5], [%6], p;\n\t}"
        ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}

// K-major operand tile with 64-byte rows and 64-byte swizzle: 8-row groups of 512 bytes.
__device__ __forceinline__ uint64_t operand_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);       // start address
    d |= (uint64_t)(512u >> 4) << 32;               // stride between 8-row groups
    d |= (uint64_t)1 << 46;                         // descriptor version (sm_100)
    d |= (uint64_t)4 << 61;                         // 64-byte swizzle
    return d;
}
// kind::mxf4: E2M1 x E2M1 -> f32, E8M0 scales, both operands K-major, M = 128, K = 64; sf = byte (0 or 2) of the
// 4-byte scale words that holds this k step's first block.
__device__ __forceinline__ uint32_t mxf4_idesc(int n, uint32_t sf, uint32_t m) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sf << 4) | (sf << 29);
}

struct MxGemmArgs {
    const PrefillSeg* segs;
    const int32_t* n_segs;
    int n_local;               // seg.expert == n_local -> shared expert
    int K;                     // reduction length (hidden for gate/up, ffn for down)
    int rows;                  // output rows of the matrix (ffn for gate/up, hidden for down)
    int n_used;
    int64_t P;                 // T * n_used: first row of the shared expert's rows
    const int32_t* perm;
    const float* route_w;
    float clamp;
    __half* mid;               // gate/up output [rows_total, ffn]
    int64_t mid_stride;
    float* partial;            // down output [rows_total, hidden]
    const uint8_t* sfa;        // weight scale chunks, routed: [slot][row tile][K/128][2][512]
    int64_t sfa_slot_stride;
    const uint8_t* sfa_shared;
    const uint8_t* sfb;        // activation scale chunks: [segment][K/128][term][2][512]
    uint32_t* error_word;
    int short_segments;        // every segment has at most kShortRows rows: two accumulator buffers, alternating per tile
};

// TWO: the kernel runs as clusters of two CTAs (cta_group::2).  A pair takes two neighbouring 256-row tiles of one
// segment, one per CTA; every MMA spans both CTAs (M = 256: 128 weight rows of each), so the segment's activation
// terms are split between them -- each CTA loads N / 2 rows of every term instead of all N, which is what the
// L2 -> shared-memory rate of this kernel is short of.  The even CTA issues all MMAs, scale copies and commits; each
// CTA loads its own operands (tile loads that count on the even CTA's barrier), reads its own accumulators and
// writes its own output rows.  The maps b32 / b64 / b96 then have boxes of 32 / 64 / 96 rows.
template <bool GATE_UP, bool TWO>
__global__ void __launch_bounds__(kThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_b32, const __grid_constant__ CUtensorMap tmap_b64,
               const __grid_constant__ CUtensorMap tmap_b96, const __grid_constant__ CUtensorMap tmap_w,
               const __grid_constant__ CUtensorMap tmap_w_shared, const MxGemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = sbase + kSmemBar;
    // FULL[s]: the stage's codes and scales have landed in this CTA (TMA bytes); SC_FULL[s]: the scale warps have moved the
    // stage's scales into tensor memory (a pair: those of both CTAs, all counted in the even CTA, so it also says that the
    // odd CTA's operands have landed); EMPTY[s]: the MMAs reading stage s have completed (one tcgen05.commit per issuing
    // warp); ACC_FULL[b] / ACC_EMPTY[b]: the accumulators of buffer b are complete / drained.  Buffer 1 exists only when every
    // segment is short (at most kShortRows rows; single CTAs): a tile's two accumulators then take 2 x 96 of the 384
    // accumulator columns, tiles alternate between the two halves, and a tile's read-out runs under the next tile's MMAs.
    constexpr int FULL = 0, EMPTY = FULL + kStages, ACC_FULL = EMPTY + kStages, ACC_EMPTY = ACC_FULL + 2, SC_FULL = ACC_EMPTY + 2;
    const bool dbl = !TWO && a.short_segments != 0;
    const uint32_t acc1_col = dbl ? (uint32_t)kShortRows : (uint32_t)kSegRows;   // column of the second accumulator inside a buffer
    auto acc_buf = [&](uint32_t t) { return dbl ? (t & 1u) : 0u; };             // buffer of this CTA's t-th tile
    auto acc_use = [&](uint32_t t) { return dbl ? (t >> 1) : t; };              // how often that buffer was used before
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    const uint32_t rank = TWO ? cluster_ctarank() : 0u;   // 0: issues the MMAs
    constexpr int kBoxRowsB = TWO ? kBoxRows / 2 : kBoxRows;         // granularity of the boxes that bring this CTA's rows of a term
    constexpr int kBBoxBytesB = kBoxRowsB * kRowBytes;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kSmemMisc);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; i++) {
            mbar_init(bar(FULL + i), 1);
            mbar_init(bar(EMPTY + i), kMmaWarps);
            mbar_init(bar(SC_FULL + i), TWO ? 8 : 4);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(bar(ACC_FULL + b), kMmaWarps);
            mbar_init(bar(ACC_EMPTY + b), (TWO && rank == 0) ? kEpiWarps + 1 : kEpiWarps);   // + one forwarded arrival for the odd CTA's twelve
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // all 512 columns of tensor memory (a pair: the same warp of both CTAs, the same columns in both)
        if (TWO) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32((const void*)tmem_slot)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32((const void*)tmem_slot)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (TWO) cluster_sync_all();   // both CTAs' barriers exist before either signals the other
    const uint32_t tmem_base = *tmem_slot;

    const int n_segs = a.n_segs[0];
    const int n_mb = a.rows / (GATE_UP ? 128 : 256);   // 256-row tiles (gate/up: 128 gate + 128 up)
    const int n_kc = a.K / kStageK;
    // work units: tiles, or pairs of neighbouring tiles; unit u of this CTA is tile (u / per_seg, (u % per_seg) * 2 + rank)
    const int per_seg = TWO ? n_mb / 2 : n_mb;
    const int n_tiles = n_segs * per_seg;
    const int unit0 = TWO ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, unit_step = TWO ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    auto unit_mb = [&](int u) { return TWO ? (u % per_seg) * 2 + (int)rank : u % per_seg; };

    // The kernel starts with 96 registers per thread (640 threads = a pool of 61440 that setmaxnreg only redistributes: the
    // three counts below add up to exactly that, and a larger request would wait for ever).  The epilogue warps need about
    // 120 for the columns they hold while tensor memory is handed back; the other two warp groups give theirs up.
    static_assert(128 * 64 + 128 * 56 + (kEpiWarps * 32) * 120 <= kThreads * 96, "register requests exceed the pool of the launch");
    if (warp < kScWarp0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;" ::: "memory");
    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t cnt = 0;
            bool ok = true;
            // weight map: gate/up = (bytes, row, matrix, slot) with a box of 64 x 128 x 2 (lands as 128 gate rows, then 128 up
            // rows); down = (bytes, row, 1, slot) with a box of 64 x 256 x 1
            auto w_row = [&](int mb) { return GATE_UP ? mb * 128 : mb * 256; };
            for (int tile = unit0; tile < n_tiles && ok; tile += unit_step) {
                const int si = tile / per_seg, mb = unit_mb(tile);
                const PrefillSeg seg = a.segs[si];
                const bool sh = seg.expert == a.n_local;
                const CUtensorMap* m_w = sh ? &tmap_w_shared : &tmap_w;
                const int slot = sh ? 0 : seg.expert;
                // weight scale chunks are stored per 256 gate/up (512 down) rows as [K/128][4][512] = (gate, up, gate, up) of two
                // 128-row halves (down: four 128-row quarters): this tile's two chunks are one half of such a group
                const uint8_t* sfa = (sh ? a.sfa_shared : a.sfa + (int64_t)slot * a.sfa_slot_stride) +
                                     ((int64_t)(mb >> 1) * n_kc * 4 + 2 * (mb & 1)) * kSfChunk;
                const uint8_t* sfb = a.sfb + (int64_t)si * n_kc * kSfbBytes;
                // one copy brings all three terms of the segment: boxes of 64, 128 or 192 rows x 3 terms (a term's rows land
                // box_rows * 64 bytes apart)
                const int n16 = max(16, (seg.n + 15) & ~15);
                const int n_mine = TWO ? n16 / 2 : n16;                     // rows of every term this CTA holds
                const int n_box = (n_mine + kBoxRowsB - 1) / kBoxRowsB;
                const CUtensorMap* m_b = n_box == 1 ? &tmap_b32 : (n_box == 2 ? &tmap_b64 : &tmap_b96);
                const int b_row0 = seg.row0 + (TWO ? (int)rank * n_mine : 0);
                const uint32_t tile_tx = (uint32_t)(kABytes + kTerms * n_box * kBBoxBytesB), sf_tx = (uint32_t)(kSfaBytes + kSfbBytes);
                // weights of this tile into L2 a few stages ahead of the ring
                constexpr int kAhead = 8;   // (4 was 7 % slower at 64 rows per expert, 16 slower everywhere)
                auto prefetch_w = [&](const CUtensorMap* m, int kc, int mb_, int slot_) { tma_prefetch_4d(m, kc * kRowBytes, w_row(mb_), 0, slot_); };
                if (tile == unit0)
                    for (int kc = 0; kc < kAhead && kc < n_kc; kc++) prefetch_w(m_w, kc, mb, slot);
                const int ntile = tile + unit_step;
                PrefillSeg nseg = seg;
                int nmb = mb;
                if (ntile < n_tiles) { nseg = a.segs[ntile / per_seg]; nmb = unit_mb(ntile); }
                const bool nsh = nseg.expert == a.n_local;
                for (int kc = 0; kc < n_kc && ok; kc++) {
                    const int pk = kc + kAhead;
                    if (pk < n_kc) prefetch_w(m_w, pk, mb, slot);
                    else if (ntile < n_tiles) prefetch_w(nsh ? &tmap_w_shared : &tmap_w, pk - n_kc, nmb, nsh ? 0 : nseg.expert);
                    const int s = cnt % kStages;
                    ok = mbar_wait(bar(EMPTY + s), ((cnt / kStages) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    const uint32_t a_dst = sbase + kSmemA + s * kABytes;
                    const uint32_t full = bar(FULL + s);   // every CTA's loads count on its own barrier
                    mbar_expect_tx(full, tile_tx + sf_tx);
                    tma_load_4d(a_dst, m_w, kc * kRowBytes, w_row(mb), 0, slot, full);
                    tma_load_3d(sbase + kSmemB + s * kBBytes, m_b, kc * kRowBytes, b_row0, 0, full);
                    bulk_load(sbase + kSmemSfa + s * kSfaBytes, sfa + (int64_t)kc * 4 * kSfChunk, kSfaBytes, full);
                    bulk_load(sbase + kSmemSfb + s * kSfbBytes, sfb + (int64_t)kc * kSfbBytes, kSfbBytes, full);
                    cnt++;
                }
            }
        }
    } else if (warp <= kMmaWarps) {
        // ----------------------------------------------------------- MMA issue
        // Two issuing warps, one accumulator each (first product: warp 1 the gate rows, warp 2 the up rows of the tile; a single
        // thread cannot issue a stage's MMAs and scale copies as fast as the tensor core retires them).  Each copies its
        // accumulator's weight scales and its own copy of the activation scales to tensor memory, so its MMAs depend only
        // on its own copies.
        if (TWO && rank != 0) {
            // odd CTA of a pair: nothing to issue.  One thread forwards "all twelve epilogue warps here have read tile t's
            // accumulators" to the even CTA.
            if (warp == 2 && lane == 0) {
                uint32_t t = 0;
                for (int tile = unit0; tile < n_tiles; tile += unit_step, t++) {
                    if (!mbar_wait(bar(ACC_EMPTY), t & 1u, abort_flag)) break;
                    mbar_arrive_cluster(map_to_cta(bar(ACC_EMPTY), 0u));
                }
            }
        } else if (lane == 0) {
            const int mw = warp - 1;
            constexpr int kAPW = kAccs / kMmaWarps;   // accumulators per issuing warp
            uint32_t tcnt = 0, s = 0, ph = 0;   // ring stage and its phase parity
            bool ok = true;
            const uint64_t d0 = operand_desc(sbase + kSmemA);
            const uint32_t hi = (uint32_t)(d0 >> 32);                       // same for every operand tile
            const uint32_t a_lo0 = (uint32_t)d0 + (uint32_t)((mw * kAPW * 128 * kRowBytes) >> 4), b_lo0 = (uint32_t)operand_desc(sbase + kSmemB);
            const uint32_t t_sfa0 = tmem_base + kSfaCol + 4u * (uint32_t)(mw * kAPW), t_sfb0 = tmem_base + kSfaCol + 4u * kAccs;
            const uint32_t t_acc0 = tmem_base + (uint32_t)(mw * kAPW) * acc1_col;
            // a pair: MMAs act in both CTAs; a commit arrives on this barrier of both, whose producers and epilogue warps each
            // wait on their own
            auto mma = [&](uint32_t d, uint32_t al, uint32_t bl, uint32_t h, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
                if (TWO) tc_mma_mxf4_lo_pair(d, al, bl, h, idesc, sfa, sfb, acc); else tc_mma_mxf4_lo(d, al, bl, h, idesc, sfa, sfb, acc);
            };
            auto commit = [&](uint32_t b) {
                if (TWO) { tc_commit_pair(b); tc_commit_pair(map_to_cta(b, 1u)); } else tc_commit(b);
            };
            for (int tile = unit0; tile < n_tiles && ok; tile += unit_step) {
                const PrefillSeg seg = a.segs[tile / per_seg];
                const int n16 = max(16, (seg.n + 15) & ~15);
                const uint32_t idesc0 = mxf4_idesc(n16, 0u, TWO ? 256u : 128u), idesc1 = mxf4_idesc(n16, 2u, TWO ? 256u : 128u);
                const int n_mine = TWO ? n16 / 2 : n16;
                const uint32_t term_step = (uint32_t)(((n_mine + kBoxRowsB - 1) / kBoxRowsB) * (kBBoxBytesB >> 4));   // a term's rows follow the previous term's box
                const uint32_t buf = acc_buf(tcnt), t_acc = t_acc0 + buf * (2u * kShortRows);
                ok = mbar_wait(bar(ACC_EMPTY) + 8u * buf, (acc_use(tcnt) & 1u) ^ 1u, abort_flag);   // the buffer's previous tile is read out
                if (!ok) break;
                tc_fence_after();
                for (int kc = 0; kc < n_kc; kc++) {
                    // the stage's operands have landed (in both CTAs of a pair) and its scales are in tensor memory
                    const uint32_t sc_full = bar(SC_FULL) + 8u * s, full = bar(FULL) + 8u * s;
                    if (!mbar_try(sc_full, ph) && !mbar_wait(sc_full, ph, abort_flag)) { ok = false; break; }
                    if (!mbar_try(full, ph) && !mbar_wait(full, ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t t_sfa = t_sfa0 + s * kScSlot, t_sfb = t_sfb0 + s * kScSlot;
                    const uint32_t a_lo = a_lo0 + s * (kABytes >> 4), b_lo = b_lo0 + s * (kBBytes >> 4);
                    const uint32_t first = kc != 0 ? 1u : 0u;
#pragma unroll
                    for (int ks = 0; ks < 2; ks++) {
                        const uint32_t idesc = ks ? idesc1 : idesc0;
#pragma unroll
                        for (int t = 0; t < kTerms; t++) {
                            const uint32_t bl = b_lo + (uint32_t)t * term_step + (uint32_t)(ks * 2);   // + 32 bytes per k step
                            const uint32_t acc = (ks | t) != 0 ? 1u : first;
#pragma unroll
                            for (int h = 0; h < kAPW; h++)
                                mma(t_acc + h * acc1_col, a_lo + (uint32_t)((h * 128 * kRowBytes) >> 4) + ks * 2, bl, hi, idesc, t_sfa + 4 * h,
                                    t_sfb + 4 * kSfbChunks * t, acc);
                        }
                    }
                    commit(bar(EMPTY) + 8u * s);   // arrives when the MMAs above have read their operands
                    if (++s == kStages) { s = 0; ph ^= 1u; }
                }
                if (ok) commit(bar(ACC_FULL) + 8u * buf);
                tcnt++;
            }
        }
    }
    } else if (warp < kEpiWarp0) {
        // -------------------------------------------------------- scale warps
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
        // A scale chunk (128 rows x 4 blocks) lies in shared memory as 32 rows of 16 bytes; the tensor core wants row r of it
        // in lane 32 q + r of every lane quarter q, 4 columns wide.  Warp q copies the stage's 8 chunks (2 of weight scales,
        // 3 terms x 2 of activation scales) into its quarter: lane r reads its 16 bytes of each chunk and stores them as 32
        // columns of the stage's scale slot.  (tcgen05.cp does the same inside the tensor-core queue, where every copy holds
        // up the MMAs behind it: 0.4 of 2.9 ms on the 8192-token layer.)
        const int q = warp & 3;
        uint32_t s = 0, ph = 0;
        const uint32_t t_slot0 = tmem_base + ((uint32_t)(q * 32) << 16) + kSfaCol;
        const uint32_t sc_bar0 = TWO ? map_to_cta(bar(SC_FULL), 0u) : bar(SC_FULL);
        bool ok = true;
        for (int tile = unit0; tile < n_tiles && ok; tile += unit_step) {
            for (int kc = 0; kc < n_kc; kc++) {
                if (!mbar_wait(bar(FULL) + 8u * s, ph, abort_flag)) { ok = false; break; }
                uint32_t v[32];
                const uint32_t src_a = sbase + kSmemSfa + s * kSfaBytes + (uint32_t)lane * 16u, src_b = sbase + kSmemSfb + s * kSfbBytes + (uint32_t)lane * 16u;
#pragma unroll
                for (int c = 0; c < kAccs; c++)
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[4 * c]), "=r"(v[4 * c + 1]), "=r"(v[4 * c + 2]), "=r"(v[4 * c + 3]) : "r"(src_a + c * kSfChunk));
#pragma unroll
                for (int c = 0; c < kSfbChunks * kTerms; c++)
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[4 * kAccs + 4 * c]), "=r"(v[4 * kAccs + 4 * c + 1]), "=r"(v[4 * kAccs + 4 * c + 2]), "=r"(v[4 * kAccs + 4 * c + 3]) : "r"(src_b + c * kSfChunk));
                tc_st32(t_slot0 + s * kScSlot, v);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (TWO && rank != 0) mbar_arrive_cluster(sc_bar0 + 8u * s); else mbar_arrive(bar(SC_FULL) + 8u * s);
                }
                if (++s == kStages) { s = 0; ph ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 120;" ::: "memory");
        // Warp w may read lanes 32 * (w % 4) .. + 31 of tensor memory; the three warps of a lane quarter take 64 columns of
        // the tile each, in blocks of 16.  A lane holds gate and up of one output row (first product), or rows r and r + 128.
        const int q = warp & 3, third = (warp - kEpiWarp0) >> 2;
        uint32_t tcnt = 0;
        bool ok = true;
        for (int tile = unit0; tile < n_tiles && ok; tile += unit_step) {
            const PrefillSeg seg = a.segs[tile / per_seg];
            const int mb = unit_mb(tile);
            const bool sh = seg.expert == a.n_local;
            const uint32_t buf = acc_buf(tcnt);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (2u * kShortRows);
            const int r_in = q * 32 + lane;           // row inside a 128-row accumulator
            const int c0 = (dbl ? 32 : 64) * third;   // short segments: 32 columns per warp cover the 96
            // lane j of the warp fetches the routing weight / output row of columns c0 + j and c0 + 32 + j (two dependent
            // loads: done while the tile's MMAs still run)
            float wv[2] = {0.f, 0.f};
            int orow[2] = {0, 0};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int c = c0 + 32 * h + lane;
                if (c < seg.n) {
                    if (sh) { wv[h] = 1.0f; orow[h] = seg.row0 + c; }
                    else { const int ts = a.perm[seg.row0 + c]; wv[h] = a.route_w[ts]; orow[h] = ts; }
                }
            }
            ok = mbar_wait(bar(ACC_FULL) + 8u * buf, acc_use(tcnt) & 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            // one 16-column block: v0 = accumulator 0, v1 = accumulator 1
            auto emit = [&](int cb, const uint32_t (&v0)[16], const uint32_t (&v1)[16]) {
                const int h = (cb - c0) >> 5, j0 = (cb - c0) & 31;
                if (GATE_UP) {
                    __half* dst = a.mid + (int64_t)(seg.row0 + cb) * a.mid_stride + mb * 128 + r_in;
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float wj = __shfl_sync(0xFFFFFFFFu, wv[h], j0 + j);
                        if (cb + j < seg.n) {
                            float gv = __uint_as_float(v0[j]), uv = __uint_as_float(v1[j]);
                            if (a.clamp > 1.0e-6f) {
                                gv = fminf(gv, a.clamp);
                                uv = fminf(fmaxf(uv, -a.clamp), a.clamp);
                            }
                            const float sig = __fdividef(1.0f, 1.0f + __expf(-gv));
                            dst[(int64_t)j * a.mid_stride] = __float2half_rn(gv * sig * uv * wj);
                        }
                    }
                } else {
                    const int hrow = mb * 256 + r_in;
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int rj = __shfl_sync(0xFFFFFFFFu, orow[h], j0 + j);
                        if (cb + j < seg.n) {
                            float* dst = a.partial + (int64_t)rj * a.rows + hrow;
                            dst[0] = __uint_as_float(v0[j]);
                            dst[128] = __uint_as_float(v1[j]);
                        }
                    }
                }
            };
            // Four blocks of 16 columns, read two at a time (a tcgen05.ld is asynchronous: nothing but the wait may stand between
            // it and the first use of its registers).  After the second pair has arrived the accumulators are handed back, and
            // its arithmetic and stores run while the next tile's MMAs have already started.
            uint32_t v0[16], v1[16], u0[16], u1[16];
            const bool b0 = c0 < seg.n, b1 = c0 + 16 < seg.n, b2 = !dbl && c0 + 32 < seg.n, b3 = !dbl && c0 + 48 < seg.n;
            auto ld_block = [&](int cb, uint32_t (&x0)[16], uint32_t (&x1)[16]) {
                tc_ld16(lane_addr + (uint32_t)cb, x0);
                tc_ld16(lane_addr + acc1_col + (uint32_t)cb, x1);
            };
            if (b0) {
                ld_block(c0, v0, v1);
                if (b1) ld_block(c0 + 16, u0, u1);
                tc_wait_ld();
                emit(c0, v0, v1);
                if (b1) emit(c0 + 16, u0, u1);
                if (b2) {
                    ld_block(c0 + 32, v0, v1);
                    if (b3) ld_block(c0 + 48, u0, u1);
                    tc_wait_ld();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ACC_EMPTY) + 8u * buf);   // (odd CTA of a pair: its own barrier; warp 2 forwards the completed phase)
            if (b2) {
                emit(c0 + 32, v0, v1);
                if (b3) emit(c0 + 48, u0, u1);
            }
            tcnt++;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(a.error_word, 2u);
    if (TWO) cluster_sync_all();   // neither CTA's shared or tensor memory goes away while the other may still use it
    if (warp == 1) {
        tc_fence_after();
        if (TWO) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// ------------------------------------------------------- activation terms
// E8M0 byte of the block scale for a block whose largest magnitude is amax: the smallest power of two 2^(e-127)
// with amax / 2^(e-127) <= 6 (the largest E2M1 value), kept inside [1, 253] so that the scale and its inverse are
// normal floats.  amax = m * 2^E with m in [1, 2): e - 127 = E - 2, one more when m > 1.5.
__device__ __forceinline__ uint32_t mx_scale_byte(float amax) {
    const uint32_t b = __float_as_uint(amax);
    const int e = (int)(b >> 23) - 2 + ((b & 0x7FFFFFu) > 0x400000u ? 1 : 0);
    return (uint32_t)min(max(e, 1), 253);
}
// Eight floats -> eight E2M1 codes (round to nearest even, saturating), element i in nibble i.
__device__ __forceinline__ uint32_t e2m1_pack8(const float (&v)[8]) {
    uint32_t out;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(out)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return out;
}
// The eight values a word of codes stands for (exact), element i from nibble i, by the hardware decoder.
__device__ __forceinline__ void e2m1_unpack8(uint32_t q, float (&d)[8]) {
    uint32_t h0, h1, h2, h3;
    asm volatile("{\n\t.reg .b8 c0, c1, c2, c3;\n\t"
                 "mov.b32 {c0, c1, c2, c3}, %4;\n\t"
                 "cvt.rn.f16x2.e2m1x2 %0, c0;\n\t"
                 "cvt.rn.f16x2.e2m1x2 %1, c1;\n\t"
                 "cvt.rn.f16x2.e2m1x2 %2, c2;\n\t"
                 "cvt.rn.f16x2.e2m1x2 %3, c3;\n\t}"
                 : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
                 : "r"(q));
    const uint32_t h[4] = {h0, h1, h2, h3};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
        d[2 * i] = f.x;
        d[2 * i + 1] = f.y;
    }
}

// The value of E2M1 code n (sign, two exponent bits, one mantissa bit): {0, .5, 1, 1.5, 2, 3, 4, 6}, exact.
// Plain integer arithmetic on the code.  (The hardware decoder, cvt.rn.f16x2.e2m1x2 followed by a widening to f32,
// gave wrong residuals inside this kernel on sm_100a with CUDA 12.9 although the same sequence is correct in
// isolation; the arithmetic form costs about 0.1 ms on the 8192-token layer and is kept.)
__device__ __forceinline__ float e2m1_value(uint32_t n) {
    const uint32_t mag = n & 7u;
    const uint32_t doubled = mag < 2u ? mag : ((2u | (mag & 1u)) << ((mag >> 1) - 1u));   // 0 1 2 3 4 6 8 12
    const float v = 0.5f * (float)doubled;
    return (n & 8u) ? -v : v;
}

// The segment holding expert-sorted row `row`, or -1 (a row of an expert the grouped GEMV takes): the last segment
// that starts at or before it (segments are sorted by first row).
__device__ __forceinline__ int find_segment(const PrefillSeg* __restrict__ segs, int n_segs, int64_t row, PrefillSeg* seg) {
    if (n_segs == 0) return -1;
    int lo = 0, hi = n_segs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((int64_t)segs[mid].row0 <= row) lo = mid; else hi = mid;
    }
    *seg = segs[lo];
    if (row < seg->row0 || row >= (int64_t)seg->row0 + seg->n) return -1;
    return lo;
}

// The kTerms MXFP4 terms of one 32-value block, all in one lane: codes[t] = the block's 32 E2M1 codes of term t (16
// bytes, element 2i in the low nibble of byte i), e[t] = its E8M0 scale byte.  No lane talks to another.
__device__ __forceinline__ void mx_terms_of_block(float (&v)[32], uint32_t opaque_zero, uint32_t* error_word, uint4 (&codes)[kTerms],
                                                  uint32_t (&e)[kTerms]) {
#pragma unroll
    for (int t = 0; t < kTerms; t++) {
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(v[j]));
        // an infinite value (an un-clamped SwiGLU product that left f16, or an infinite token value) has no terms
        if (t == 0 && amax > 3.0e38f) atomicOr(error_word, kErrHalfRange);
        e[t] = mx_scale_byte(amax);
        const float inv = __uint_as_float((254u - e[t]) << 23), scl = __uint_as_float(e[t] << 23);
        uint32_t w[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float sv[8];
#pragma unroll
            for (int j = 0; j < 8; j++) sv[j] = v[8 * g + j] * inv;
            w[g] = e2m1_pack8(sv);
            if (t + 1 < kTerms) {
                float d[8];
                if (opaque_zero == 0xFFFFFFFFu) {   // never: keeps the arithmetic decoder compiled for comparison
#pragma unroll
                    for (int j = 0; j < 8; j++) d[j] = e2m1_value(w[g] >> (4 * j));
                } else {
                    // the decoder must not see that its input comes straight from the encoder above: with the two chained,
                    // the compiled code produced wrong residuals (CUDA 12.9, sm_100a); an exclusive-or with a kernel
                    // argument that is always zero separates them
                    e2m1_unpack8(w[g] ^ opaque_zero, d);
                }
#pragma unroll
                for (int j = 0; j < 8; j++) v[8 * g + j] = __fmaf_rn(-d[j], scl, v[8 * g + j]);   // exact: the residual
            }
        }
        codes[t] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// The scale bytes of four consecutive blocks (lanes 4j .. 4j+3, one 128-column stage) as one word, valid in lane 4j.
__device__ __forceinline__ uint32_t mx_stage_scales(uint32_t e, int lane) {
    const int base = lane & ~3;
    return __shfl_sync(0xFFFFFFFFu, e, base) | (__shfl_sync(0xFFFFFFFFu, e, base + 1) << 8) | (__shfl_sync(0xFFFFFFFFu, e, base + 2) << 16) |
           (__shfl_sync(0xFFFFFFFFu, e, base + 3) << 24);
}

// Byte offset, inside the activation scale chunks, of row r of segment si (stage 0, term 0).
__device__ __forceinline__ int64_t mx_sf_offset(int si, int r, int n_kc) {
    return (int64_t)si * n_kc * kSfbBytes + (r >> 7) * kSfChunk + (r & 31) * 16 + ((r >> 5) & 3) * 4;   // chunk r / 128 of its term
}

// First product's operand.  One warp per (token, 1024 columns), a lane per 32-value block: the token row (bf16) becomes
// kTerms MXFP4 rows ONCE and is written to every expert-sorted row that holds a copy of it -- the sorted positions of its
// picks (inv_perm, -1 for picks that are not placed here) and row P + t of the shared expert -- codes to
// [term][row][K/2], scales into the row's segment's scale-factor chunks.  Rows outside every segment (experts handed to
// the grouped GEMV) get nothing.
__global__ void __launch_bounds__(256)
mx_quantize_tokens_kernel(const __nv_bfloat16* __restrict__ x, int64_t T, int K, const int32_t* __restrict__ inv_perm, int n_used, int64_t P,
                          int with_shared, const PrefillSeg* __restrict__ segs, const int32_t* __restrict__ n_segs_p, uint8_t* __restrict__ xq,
                          int64_t term_stride, uint8_t* __restrict__ sfb, uint32_t opaque_zero, uint32_t* __restrict__ error_word) {
    const int parts = (K + 1023) >> 10;
    const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t tok = w / parts;
    const int part = (int)(w - tok * parts);
    const int lane = threadIdx.x & 31;
    if (tok >= T) return;
    const int n_kc = K / kStageK;
    // lane d < n_used: pick d of the token; lane n_used: the shared expert's copy
    int64_t my_row = -1, my_sf = 0;
    if (lane < n_used) my_row = inv_perm[tok * n_used + lane];
    else if (lane == n_used && with_shared) my_row = P + tok;
    if (my_row >= 0) {
        PrefillSeg seg;
        const int si = find_segment(segs, n_segs_p[0], my_row, &seg);
        if (si < 0) my_row = -1;
        else my_sf = mx_sf_offset(si, (int)(my_row - seg.row0), n_kc);
    }
    const uint32_t dests = __ballot_sync(0xFFFFFFFFu, my_row >= 0);
    if (dests == 0u) return;
    const int blk = part * 32 + lane;            // 32-value block of the row
    const bool live = blk < (K >> 5);
    float v[32];
    if (live) {
        const uint4* in = reinterpret_cast<const uint4*>(x + tok * K + (int64_t)blk * 32);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint4 raw = __ldg(in + q);
            const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                v[8 * q + 2 * j] = __uint_as_float(wds[j] << 16);
                v[8 * q + 2 * j + 1] = __uint_as_float(wds[j] & 0xFFFF0000u);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = 0.0f;
    }
    uint4 codes[kTerms];
    uint32_t e[kTerms], sfw[kTerms];
    mx_terms_of_block(v, opaque_zero, error_word, codes, e);
#pragma unroll
    for (int t = 0; t < kTerms; t++) sfw[t] = mx_stage_scales(e[t], lane);
    for (uint32_t m = dests; m != 0u; m &= m - 1u) {
        const int d = __ffs(m) - 1;
        const int64_t row = __shfl_sync(0xFFFFFFFFu, my_row, d), sfo = __shfl_sync(0xFFFFFFFFu, my_sf, d);
        if (live) {
#pragma unroll
            for (int t = 0; t < kTerms; t++) {
                *reinterpret_cast<uint4*>(xq + (int64_t)t * term_stride + row * (K >> 1) + (int64_t)blk * 16) = codes[t];
                if ((lane & 3) == 0)
                    *reinterpret_cast<uint32_t*>(sfb + sfo + (int64_t)(blk >> 2) * kSfbBytes + (int64_t)t * kSfbChunks * kSfChunk) = sfw[t];
            }
        }
    }
}

// Second product's operand.  A warp per (expert-sorted row of mid, 1024 columns), a lane per block, over the rows that
// exist: the placed picks (offsets[n_local] of them, known on the device only -- in the expert-parallel form most of the
// P slots are empty) and the shared expert's rows P .. P + shared_rows - 1.  Rows outside every segment (experts handed
// to the grouped GEMV) are skipped.  Codes to [term][row][K/2], scales into the segment's scale-factor chunks.
__global__ void __launch_bounds__(256)
mx_quantize_mid_kernel(const __half* __restrict__ mid, const int32_t* __restrict__ offsets, int n_local, int64_t P, int64_t shared_rows, int K,
                       const PrefillSeg* __restrict__ segs, const int32_t* __restrict__ n_segs_p, uint8_t* __restrict__ xq, int64_t term_stride,
                       uint8_t* __restrict__ sfb, uint32_t opaque_zero, uint32_t* __restrict__ error_word) {
    const int parts = (K + 1023) >> 10;
    const int lane = threadIdx.x & 31;
    const int n_kc = K / kStageK;
    const int64_t placed = offsets[n_local], n_work = (placed + shared_rows) * parts;
    const int n_segs = n_segs_p[0];
    for (int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); w < n_work; w += (int64_t)gridDim.x * 8) {
        const int64_t idx = w / parts;
        const int part = (int)(w - idx * parts);
        const int64_t row = idx < placed ? idx : P + (idx - placed);
        PrefillSeg seg;
        const int si = find_segment(segs, n_segs, row, &seg);
        if (si < 0) continue;
        const int blk = part * 32 + lane;
        const bool live = blk < (K >> 5);
        float v[32];
        if (live) {
            const uint4* in = reinterpret_cast<const uint4*>(mid + row * K + (int64_t)blk * 32);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint4 raw = __ldg(in + q);
                const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wds[j]));
                    v[8 * q + 2 * j] = f.x;
                    v[8 * q + 2 * j + 1] = f.y;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = 0.0f;
        }
        uint4 codes[kTerms];
        uint32_t e[kTerms];
        mx_terms_of_block(v, opaque_zero, error_word, codes, e);
        uint8_t* sf_row = sfb + mx_sf_offset(si, (int)(row - seg.row0), n_kc);
#pragma unroll
        for (int t = 0; t < kTerms; t++) {
            const uint32_t sfw = mx_stage_scales(e[t], lane);
            if (live) {
                *reinterpret_cast<uint4*>(xq + (int64_t)t * term_stride + row * (K >> 1) + (int64_t)blk * 16) = codes[t];
                if ((lane & 3) == 0)
                    *reinterpret_cast<uint32_t*>(sf_row + (int64_t)(blk >> 2) * kSfbBytes + (int64_t)t * kSfbChunks * kSfChunk) = sfw;
            }
        }
    }
}

// inv_perm[pick] = expert-sorted position of the pick (the buffer is pre-set to -1: picks that are not placed here keep it).
__global__ void __launch_bounds__(256)
mx_invert_perm_kernel(const int32_t* __restrict__ perm, const int32_t* __restrict__ offsets, int n_local, int32_t* __restrict__ inv_perm) {
    const int64_t placed = offsets[n_local];
    for (int64_t p = (int64_t)blockIdx.x * 256 + threadIdx.x; p < placed; p += (int64_t)gridDim.x * 256) inv_perm[perm[p]] = (int32_t)p;
}

// (Re-)encode the weight maps when the layer points at other planes: gate/up as (bytes, row, matrix, slot)
// with a box of 64 bytes x 128 rows x both matrices, down as (bytes, row, 1, slot) with 64 x 256.
int map_weights(PrefillWorkspace* ws, int which, const uint8_t* km_gu, const uint8_t* km_dn, int64_t gu_stride, int64_t dn_stride,
                int n_slots) {
    if (ws->mapped_km_gu[which] == km_gu && ws->mapped_km_dn[which] == km_dn && ws->mapped_km_slots[which] == n_slots) return DSX_OK;
    const int64_t H = ws->H, F = ws->F;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)(H / 2), (cuuint64_t)F, 2, (cuuint64_t)n_slots};
        const cuuint64_t strides[3] = {(cuuint64_t)(H / 2), (cuuint64_t)(F * (H / 2)), (cuuint64_t)gu_stride};
        const cuuint32_t box[4] = {(cuuint32_t)kRowBytes, 128, 2, 1};
        if (int rc = tmap_encode(&ws->tmap_km_gu[which], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, km_gu, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B))
            return rc;
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)(F / 2), (cuuint64_t)H, 1, (cuuint64_t)n_slots};
        const cuuint64_t strides[3] = {(cuuint64_t)(F / 2), (cuuint64_t)(H * (F / 2)), (cuuint64_t)dn_stride};
        const cuuint32_t box[4] = {(cuuint32_t)kRowBytes, 256, 1, 1};
        if (int rc = tmap_encode(&ws->tmap_km_dn[which], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, km_dn, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B))
            return rc;
    }
    ws->mapped_km_gu[which] = km_gu;
    ws->mapped_km_dn[which] = km_dn;
    ws->mapped_km_slots[which] = n_slots;
    return DSX_OK;
}

template <bool GATE_UP>
int launch_mx_gemm(bool pair, const CUtensorMap* b_maps, const CUtensorMap& w_map, const CUtensorMap& w_shared_map, const MxGemmArgs& g, int sm_count,
                   cudaStream_t stream) {
    if (!pair) {
        mx_gemm_kernel<GATE_UP, false><<<sm_count, kThreads, kSmemTotal, stream>>>(b_maps[0], b_maps[1], b_maps[2], w_map, w_shared_map, g);
        DSX_LAUNCHED();
        return DSX_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sm_count & ~1));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    DSX_CUDA(cudaLaunchKernelEx(&cfg, mx_gemm_kernel<GATE_UP, true>, b_maps[0], b_maps[1], b_maps[2], w_map, w_shared_map, g));
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace

int prefill_mx_workspace_create(PrefillWorkspace* ws, const dsx_moe_config& cfg, int n_used) {
    ws->mx_ready = false;
    // shapes the tiles cover: 256 gate + 256 up rows per tile, 512 down rows per tile, 128-column stages
    if (cfg.ffn % 256 != 0 || cfg.hidden % 512 != 0 || (cfg.shared_ffn != 0 && cfg.shared_ffn != cfg.ffn)) return DSX_OK;
    const int64_t Kmax = std::max(cfg.hidden, cfg.ffn);
    ws->mx_seg_cap = cfg.router.n_expert + (int)((ws->cap_rows + kShortRows - 1) / kShortRows) + 8;   // every expert's last segment may be short
    ws->mx_term_stride = ws->cap_rows * (Kmax / 2);
    DSX_CUDA(cudaMalloc((void**)&ws->xq, (size_t)kTerms * (size_t)ws->mx_term_stride));
    DSX_CUDA(cudaMalloc((void**)&ws->sfb, (size_t)ws->mx_seg_cap * (size_t)(Kmax / kStageK) * kSfbBytes));
    DSX_CUDA(cudaMalloc((void**)&ws->mx_segs, sizeof(PrefillSeg) * (size_t)ws->mx_seg_cap));
    DSX_CUDA(cudaMalloc((void**)&ws->mx_inv_perm, sizeof(int32_t) * (size_t)cfg.max_tokens * (size_t)n_used));
    // activation terms as (bytes, row, term): boxes of 64 bytes x 64 / 128 / 192 rows x 3 terms
    for (int g = 0; g < 2; g++)
        for (int b = 0; b < 3; b++) {
            const int64_t K = g == 0 ? cfg.hidden : cfg.ffn;
            const cuuint64_t dims[3] = {(cuuint64_t)(K / 2), (cuuint64_t)ws->cap_rows, (cuuint64_t)kTerms};
            const cuuint64_t strides[2] = {(cuuint64_t)(K / 2), (cuuint64_t)ws->mx_term_stride};
            const cuuint32_t box[3] = {(cuuint32_t)kRowBytes, (cuuint32_t)((b + 1) * kBoxRows), (cuuint32_t)kTerms};
            if (int rc = tmap_encode(g == 0 ? &ws->tmap_xq[b] : &ws->tmap_mq[b], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, ws->xq, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_64B))
                return rc;
            // CTA pairs: each CTA fetches half of a segment's rows (boxes of 32 / 64 / 96 rows)
            const cuuint32_t box2[3] = {(cuuint32_t)kRowBytes, (cuuint32_t)((b + 1) * kBoxRows / 2), (cuuint32_t)kTerms};
            if (int rc = tmap_encode(g == 0 ? &ws->tmap_xq2[b] : &ws->tmap_mq2[b], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, ws->xq, dims, strides, box2,
                                     CU_TENSOR_MAP_SWIZZLE_64B))
                return rc;
        }
    DSX_CUDA(cudaFuncSetAttribute(mx_gemm_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    DSX_CUDA(cudaFuncSetAttribute(mx_gemm_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    DSX_CUDA(cudaFuncSetAttribute(mx_gemm_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    DSX_CUDA(cudaFuncSetAttribute(mx_gemm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    // CTA pairs need an even number of 256-row tiles per segment in both products (true of every shape this path takes)
    // DSX_MX_PAIR=0 / 1 pins the single-CTA or the CTA-pair form (tests compare the two bit for bit); otherwise per call
    const char* pair_env = std::getenv("DSX_MX_PAIR");
    ws->mx_pair_mode = pair_env == nullptr ? -1 : (pair_env[0] == '1' ? 1 : (pair_env[0] == '0' ? 0 : -1));
    {   // a device (or a partition of one) that cannot hold a cluster of two of these CTAs runs single CTAs only
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3(2);
        lc.blockDim = dim3(kThreads);
        lc.dynamicSmemBytes = kSmemTotal;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
        int n_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&n_clusters, mx_gemm_kernel<true, true>, &lc) != cudaSuccess || n_clusters < 1) {
            (void)cudaGetLastError();
            ws->mx_pair_mode = 0;
        }
    }
    ws->mx_ready = true;
    return DSX_OK;
}

void prefill_mx_workspace_free(PrefillWorkspace* ws) {
    cudaFree(ws->xq);
    cudaFree(ws->sfb);
    cudaFree(ws->mx_segs);
    cudaFree(ws->mx_inv_perm);
    ws->xq = nullptr; ws->sfb = nullptr; ws->mx_segs = nullptr; ws->mx_inv_perm = nullptr; ws->mx_ready = false;
}

int prefill_mx_forward(PrefillWorkspace* ws, const dsx_moe_config& cfg, const PrefillCall& c, cudaStream_t stream) {
    const int64_t P = c.T * c.n_used, rows = P + c.T;
    DSX_REQUIRE(rows <= ws->cap_rows, "prefill: %lld rows exceed the workspace (%lld)", (long long)rows, (long long)ws->cap_rows);
    if (int rc = launch_group_build(c.selected, c.T, c.n_used, c.n_local, c.expert_lo, 256, 0, c.hist, c.offsets, c.perm, nullptr, nullptr, 0,
                                    c.gs, stream))
        return rc;
    // Experts with at most kMxSmallMax rows go to the grouped GEMV: one 8-row item streams an expert's weights once at
    // HBM speed, which a tile pass (bound by the same bytes through L2) cannot beat; from 9 rows on the GEMV would
    // stream them twice.
    const int mx_small = ws->small_max > 0 ? kMxSmallMax : 0;
    // CTA pairs halve the activation rows a CTA loads per stage, which pays once segments are long: measured on the
    // 256-expert layer, pairs are 5 to 10 % faster from 128 rows per expert on and 2 to 9 % slower at 64 and fewer (a
    // stage is mostly weight bytes there, and a pair adds a hop to every hand-over).
    const bool pair = ws->mx_pair_mode >= 0 ? ws->mx_pair_mode == 1 : P >= (int64_t)kPairFromRows * c.n_local;
    // Below that, segments are capped at kShortRows rows, which leaves tensor memory for two accumulator buffers: a tile's
    // read-out then runs under the next tile's MMAs (tiles are short there, and the hand-over between them was a quarter
    // of their time).
    const bool short_segments = !pair;
    if (int rc = launch_build_segments(c.offsets, c.n_local, P, c.with_shared ? (int)c.T : 0, short_segments ? kShortRows : kSegRows, ws->mx_segs,
                                       ws->n_segs, ws->mx_seg_cap, mx_small, ws->small_items, ws->n_small, stream))
        return rc;
    if (int rc = map_weights(ws, 0, c.km_gu, c.km_dn, c.km_gu_stride, c.km_dn_stride, c.n_local)) return rc;
    const int shi = c.with_shared ? 1 : 0;   // without a shared expert the shared map aliases the routed one (never used)
    if (c.with_shared)
        if (int rc = map_weights(ws, 1, c.sh_km_gu, c.sh_km_dn, c.km_gu_stride, c.km_dn_stride, 1)) return rc;
    const int64_t quant_rows = c.with_shared ? rows : P;
    // experts with a handful of rows: the decode kernels, over the same sorted rows and partial rows
    GemvArgs v{};
    v.fmt = c.fmt; v.shared_fmt = c.fmt; v.n_expert = c.n_local;
    v.work_items = ws->small_items; v.n_work_items = ws->n_small; v.item_recs = nullptr; v.offsets = c.offsets; v.perm = c.perm;
    v.route_w = c.route_w; v.n_used = c.n_used; v.T = c.T; v.clamp = cfg.clamp; v.x = c.x; v.mid = c.mid; v.mid_stride = cfg.ffn;
    v.partial = c.partial; v.error_word = c.error_word;
    MxGemmArgs g{};
    g.segs = ws->mx_segs; g.n_segs = ws->n_segs; g.n_local = c.n_local; g.n_used = c.n_used; g.P = P; g.perm = c.perm;
    g.route_w = c.route_w; g.clamp = cfg.clamp; g.mid = c.mid; g.mid_stride = cfg.ffn; g.partial = c.partial; g.sfb = ws->sfb;
    g.error_word = c.error_word;
    g.short_segments = short_segments ? 1 : 0;

    // first product: K = hidden, rows = ffn
    DSX_CUDA(cudaMemsetAsync(ws->mx_inv_perm, 0xFF, sizeof(int32_t) * (size_t)P, stream));
    mx_invert_perm_kernel<<<(unsigned)std::min<int64_t>((P + 255) / 256, 4 * c.sm_count), 256, 0, stream>>>(c.perm, c.offsets, c.n_local, ws->mx_inv_perm);
    DSX_LAUNCHED();
    {
        const int64_t warps = c.T * ((cfg.hidden + 1023) >> 10);
        mx_quantize_tokens_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(c.x, c.T, (int)cfg.hidden, ws->mx_inv_perm, c.n_used, P,
                                                                                 c.with_shared ? 1 : 0, ws->mx_segs, ws->n_segs, ws->xq,
                                                                                 ws->mx_term_stride, ws->sfb, 0u, c.error_word);
        DSX_LAUNCHED();
    }
    g.K = cfg.hidden; g.rows = cfg.ffn;
    g.sfa = c.sf_gu; g.sfa_slot_stride = c.sf_gu_stride; g.sfa_shared = c.sh_sf_gu;
    if (int rc = launch_mx_gemm<true>(pair, pair ? ws->tmap_xq2 : ws->tmap_xq, ws->tmap_km_gu[0], ws->tmap_km_gu[shi], g, c.sm_count, stream))
        return rc;
    if (ws->small_max > 0) {
        v.K = cfg.hidden; v.rows = cfg.ffn; v.sh_rows = cfg.ffn;
        v.nib = c.gu_nib; v.sc = c.gu_sc; v.nib_slot_stride = c.gu_nib_stride; v.sc_slot_stride = c.gu_sc_stride;
        if (int rc = launch_gemv_gate_up(v, c.sm_count, stream)) return rc;
    }
    // second product: K = ffn, rows = hidden, over the terms of mid
    {
        const int64_t warps = quant_rows * ((cfg.ffn + 1023) >> 10);   // at most; the kernel walks the rows that exist
        const unsigned blocks = (unsigned)std::min<int64_t>((warps + 7) / 8, (int64_t)c.sm_count * 64);
        mx_quantize_mid_kernel<<<blocks, 256, 0, stream>>>(c.mid, c.offsets, c.n_local, P, c.with_shared ? c.T : 0, (int)cfg.ffn, ws->mx_segs,
                                                           ws->n_segs, ws->xq, ws->mx_term_stride, ws->sfb, 0u, c.error_word);
    }
    DSX_LAUNCHED();
    g.K = cfg.ffn; g.rows = cfg.hidden;
    g.sfa = c.sf_dn; g.sfa_slot_stride = c.sf_dn_stride; g.sfa_shared = c.sh_sf_dn;
    if (int rc = launch_mx_gemm<false>(pair, pair ? ws->tmap_mq2 : ws->tmap_mq, ws->tmap_km_dn[0], ws->tmap_km_dn[shi], g, c.sm_count, stream))
        return rc;
    if (ws->small_max > 0) {
        v.K = cfg.ffn; v.rows = cfg.hidden; v.sh_rows = cfg.hidden;
        v.nib = c.dn_nib; v.sc = c.dn_sc; v.nib_slot_stride = c.dn_nib_stride; v.sc_slot_stride = c.dn_sc_stride;
        if (int rc = launch_gemv_down(v, c.sm_count, stream)) return rc;
    }
    if (c.skip_combine) return DSX_OK;   // the caller adds another pass before it reduces the partial rows
    return launch_combine(c.partial, c.T, c.n_used, cfg.hidden, c.with_shared ? 1 : 0, c.filter_picks ? c.selected : nullptr, c.expert_lo,
                          c.n_local, c.out, stream, c.out_rows);
}

}  // namespace dsx
