// Prefill-size grouped GEMM on the 5th-generation tensor cores (tcgen05).
//
// Reference counterparts (paths relative to the deepstrix repository): the
// by-expert prefill kernels and their matrix-core arms,
//   gate/up  crates/v4flash-kernels/kernels/mxfp4_pair_matvec.hip:293-564, mxfp4_moe_wmma.hip:137-368
//   down     crates/v4flash-kernels/kernels/mxfp4_matvec.hip:219-369,      mxfp4_moe_wmma.hip:370-388
//   grouping crates/v4flash-kernels/kernels/moe_work_items_builder.hip:61-145 (work items sorted by expert)
//
// Design.  Expert-sorted token rows (the permutation of groups.cu) are cut into
// segments of <= 256 rows of one expert.  A tile = (segment, 256 weight rows).
// The weight rows are the M side of the MMA (two 128-row halves that share the
// token operand), the segment's tokens the N side (any multiple of 16 up to
// 256), so ragged expert sizes cost MMA time in proportion to their tokens.
// For gate/up the two halves are gate rows f0..f0+127 and up rows f0..f0+127: a
// TMEM lane then holds gate and up of the same output row and SwiGLU needs no
// exchange.  Per 64-column chunk of the reduction:
//   two producer threads  TMA-load the packed 4-bit sub-tiles (8.5 KB, a 4-D box) into a deep ring, and
//                     the token tile (256 x 64 f16, 128-byte swizzle) into its own ring
//   8 converter warps expand codes with cvt.rn.f16x2.e2m1x2, multiply by the E8M0
//                     block scale (exact in f16) and write the swizzled K-major A tile
//   MMA thread        8 x tcgen05.mma.kind::f16 (M128 x N x K16) into two TMEM accumulators
// and after the last chunk the 4 epilogue warps and the 8 converter warps read TMEM (tcgen05.ld), apply
// clamp + SwiGLU + routing weight (gate/up) and store mid (f16) or the per-pick
// partial rows (f32).  Every wait is bounded; on a timeout the block raises an
// abort flag, all roles drain, TMEM is freed and the layer's error word is set.
#include "prefill.cuh"

namespace dsx {
namespace {

constexpr int kThreads = 15 * 32;      // weight producer, MMA, 8 converters, 4 epilogue warps, token-tile producer
constexpr int kBProducerWarp = 14;
constexpr int kConvWarps = 8;
constexpr int kEpiWarp0 = 10;
constexpr int kSegRows = 256;          // max token rows per segment (MMA N)
constexpr int kTileM = 256;            // weight rows per tile (2 x M128)
constexpr int kChunkK = 64;            // reduction columns per pipeline step
constexpr int kPrefetchAhead = 8;     // chunks of packed weights requested into L2 ahead of the ring
constexpr int kABytes = kTileM * kChunkK * 2;        // 32768: converted weights of one chunk
constexpr int kBBytes = kSegRows * kChunkK * 2;      // 32768: token tile of one chunk

// Per-format pipeline shape.  A 64-column chunk of 256 weight rows is 16 MXFP4 sub-tiles
// (8.5 KB) or 32 Q8_0 sub-tiles (17 KB); Q8_0 pays for the larger raw stages with shallower rings.
template <int FMT>
struct Shape {
    static constexpr int kSubPerChunk = FMT == DSX_FMT_MXFP4 ? 16 : 32;
    static constexpr int kKtPerChunk = FMT == DSX_FMT_MXFP4 ? 1 : 2;       // column tiles per 64 columns
    static constexpr int kRawStages = 3;
    static constexpr int kAStages = FMT == DSX_FMT_MXFP4 ? 3 : 2;          // converted-weight ring (filled on chip: two stages cover it)
    static constexpr int kBStages = 3;                                     // token-tile ring (filled from L2, like the raw ring)
    static constexpr int kRawNib = kSubPerChunk * kSubNibBytes;
    static constexpr int kRawSc = kSubPerChunk * kSubScBytes;
    static constexpr int kRawBytes = kRawNib + kRawSc;
    static constexpr int kSmemA = 0;
    static constexpr int kSmemB = kSmemA + kAStages * kABytes;
    static constexpr int kSmemRaw = kSmemB + kBStages * kBBytes;
    static constexpr int kSmemBar = kSmemRaw + kRawStages * kRawBytes;
    static constexpr int kNumBars = 2 * kRawStages + 2 * kAStages + 2 * kBStages + 2;
    static constexpr int kSmemMisc = kSmemBar + kNumBars * 8;              // tmem base, abort flag
    static constexpr int kSmemTotal = kSmemMisc + 16 + 1024;               // + alignment slack
};
static_assert(Shape<DSX_FMT_MXFP4>::kSmemTotal <= 227 * 1024 && Shape<DSX_FMT_Q8_0>::kSmemTotal <= 227 * 1024, "rings exceed the shared memory of an SM");
constexpr uint32_t kSpinLimit = 1u << 22;

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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
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
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// The eight MMAs of one 64-column chunk (4 k16 steps x 2 row halves) in one block of PTX: the
// issuing thread is latency-bound on its own scalar instructions, so the descriptors are formed
// with one 32-bit add each (all operands of a stage share the high descriptor word).
// a_lo / b_lo: low descriptor words of the stage's A and B tiles; second row half = +1024 (16 KB).
__device__ __forceinline__ void tc_mma_chunk(uint32_t t0, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b32 t1, x, y;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "add.u32 t1, %0, 256;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
        "add.u32 x, %1, 1024;\n\t"
        "mov.b64 da, {x, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [t1], da, db, %4, p;\n\t"
        "setp.eq.b32 p, %4, %4;\n\t"
        "add.u32 x, %1, 2;\n\t"
        "add.u32 y, %2, 2;\n\t"
        "mov.b64 da, {x, %3};\n\t"
        "mov.b64 db, {y, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
        "add.u32 x, %1, 1026;\n\t"
        "mov.b64 da, {x, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [t1], da, db, %4, p;\n\t"
        "add.u32 x, %1, 4;\n\t"
        "add.u32 y, %2, 4;\n\t"
        "mov.b64 da, {x, %3};\n\t"
        "mov.b64 db, {y, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
        "add.u32 x, %1, 1028;\n\t"
        "mov.b64 da, {x, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [t1], da, db, %4, p;\n\t"
        "add.u32 x, %1, 6;\n\t"
        "add.u32 y, %2, 6;\n\t"
        "mov.b64 da, {x, %3};\n\t"
        "mov.b64 db, {y, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
        "add.u32 x, %1, 1030;\n\t"
        "mov.b64 da, {x, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [t1], da, db, %4, p;\n\t"
        "}"
        ::"r"(t0), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte-swizzled shared-memory operand: 8-row groups of 1024 B.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);       // start address
    d |= (uint64_t)(1024u >> 4) << 32;              // stride between 8-row groups
    d |= (uint64_t)1 << 46;                         // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                         // 128-byte swizzle
    return d;
}
// kind::f16, f16 x f16 -> f32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

// E8M0 byte -> f16x2 splat of 2^(e-127).  Normal f16 for e >= 113 (two integer
// ops); below that the multiplier is an f16 subnormal (2^-24 .. 2^-15) or zero.
__device__ __forceinline__ uint32_t scale_h2(uint32_t e) {
    uint32_t b = (e << 10) - (112u << 10);
    if (__builtin_expect(e < 113u, 0)) b = e >= 103u ? 1u << (e - 103u) : 0u;
    return b * 0x00010001u;
}
__device__ __forceinline__ void cvt4(uint32_t q, uint32_t (&h)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(q));
}
// Four offset-binary int8 (value ^ 0x80) -> two exact f16: 0x6400 | u is 1024 + u, minus 1152.
__device__ __forceinline__ uint32_t q8_pair(uint32_t w, uint32_t sel) {
    const uint32_t h = __byte_perm(w, 0x64646464u, sel);
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&h), __half2half2(__ushort_as_half((unsigned short)0x6480)));
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

struct GemmArgs {
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
    uint32_t* error_word;
};

template <int FMT, bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 1)
prefill_gemm_kernel(const __grid_constant__ CUtensorMap tmap_b64, const __grid_constant__ CUtensorMap tmap_b128,
                    const __grid_constant__ CUtensorMap tmap_b192, const __grid_constant__ CUtensorMap tmap_b256,
                    const __grid_constant__ CUtensorMap tmap_nib,
                    const __grid_constant__ CUtensorMap tmap_sc, const __grid_constant__ CUtensorMap tmap_sh_nib,
                    const __grid_constant__ CUtensorMap tmap_sh_sc, const GemmArgs a) {
    using C = Shape<FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
    const uint32_t bar0 = sbase + C::kSmemBar;
    // barrier indices
    // A_FULL[s]: the converted weights (8 converter warps) of stage s are in shared memory; B_FULL[s]: the token tile (TMA
    // bytes) of stage s; A_EMPTY / B_EMPTY[s]: the MMAs reading the stage have completed (one tcgen05.commit each).  The two
    // rings advance independently: the token tile comes from L2 and needs a deeper ring than the weights converted on chip.
    constexpr int RAW_FULL = 0, RAW_EMPTY = RAW_FULL + C::kRawStages, A_FULL = RAW_EMPTY + C::kRawStages, A_EMPTY = A_FULL + C::kAStages,
                  B_FULL = A_EMPTY + C::kAStages, B_EMPTY = B_FULL + C::kBStages, ACC_FULL = B_EMPTY + C::kBStages, ACC_EMPTY = ACC_FULL + 1;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::kSmemMisc);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    (void)bars;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::kRawStages; i++) { mbar_init(bar(RAW_FULL + i), 1); mbar_init(bar(RAW_EMPTY + i), kConvWarps); }
        for (int i = 0; i < C::kAStages; i++) { mbar_init(bar(A_FULL + i), kConvWarps); mbar_init(bar(A_EMPTY + i), 1); }
        for (int i = 0; i < C::kBStages; i++) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_EMPTY + i), 1); }
        mbar_init(bar(ACC_FULL), 1);
        mbar_init(bar(ACC_EMPTY), 4 + kConvWarps);
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM: all 512 columns (two 256-column accumulators)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32((const void*)tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_segs = a.n_segs[0];
    const int n_mb = a.rows / (GATE_UP ? 128 : 256);   // 256-row tiles (gate/up: 128 gate + 128 up)
    const int n_tiles = n_segs * n_mb;
    const int n_kc = a.K / kChunkK;

    // Accumulator read-out of one tile, shared by the 4 epilogue warps (rank 0) and the 8 converter
    // warps (ranks 1, 2), which are idle once a tile's last chunk is converted: warp w may read
    // TMEM lanes 32*(w%4)..+31, so each lane quarter has three warps that split the 32-column
    // chunks of the tile between them.
    auto epilogue = [&](int tile, int rank) {
        const PrefillSeg seg = a.segs[tile / n_mb];
        const int mb = tile % n_mb;
        const bool sh = seg.expert == a.n_local;
        const int q = warp & 3;
        tc_fence_after();
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const int r_in = q * 32 + lane;           // row inside a 128-row half
        uint32_t bad = 0;                         // an un-clamped SwiGLU product beyond the f16 range
        for (int c0 = 32 * rank; c0 < seg.n; c0 += 96) {
            // lane j of the warp fetches the routing weight / output row of column c0 + j
            float wv = 0.f;
            int orow = 0;
            if (c0 + lane < seg.n) {
                if (sh) { wv = 1.0f; orow = seg.row0 + c0 + lane; }
                else { const int ts = a.perm[seg.row0 + c0 + lane]; wv = a.route_w[ts]; orow = ts; }
            }
            uint32_t v0[32], v1[32];
            tc_ld32(lane_addr + (uint32_t)c0, v0);
            tc_ld32(lane_addr + 256u + (uint32_t)c0, v1);
            tc_wait_ld();
            if (GATE_UP) {
                __half* dst = a.mid + (int64_t)(seg.row0 + c0) * a.mid_stride + mb * 128 + r_in;
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const float wj = __shfl_sync(0xFFFFFFFFu, wv, j);
                    if (c0 + j < seg.n) {
                        float gv = __uint_as_float(v0[j]), uv = __uint_as_float(v1[j]);
                        if (a.clamp > 1.0e-6f) {
                            gv = fminf(gv, a.clamp);
                            uv = fminf(fmaxf(uv, -a.clamp), a.clamp);
                        }
                        const float sig = __fdividef(1.0f, 1.0f + __expf(-gv));
                        dst[(int64_t)j * a.mid_stride] = f32_to_f16_checked(gv * sig * uv * wj, bad);
                    }
                }
            } else {
                const int h = mb * 256 + r_in;
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int rj = __shfl_sync(0xFFFFFFFFu, orow, j);
                    if (c0 + j < seg.n) {
                        float* dst = a.partial + (int64_t)rj * a.rows + h;
                        dst[0] = __uint_as_float(v0[j]);
                        dst[128] = __uint_as_float(v1[j]);
                    }
                }
            }
        }
        if (bad) atomicOr(a.error_word, kErrHalfRange);
        tc_fence_before();
        __syncwarp();
    };

    if (warp == 0) {
        // ------------------------------------------------- packed-weight producer
        if (lane == 0) {
            uint32_t rcnt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const PrefillSeg seg = a.segs[tile / n_mb];
                const int mb = tile % n_mb;
                const bool sh = seg.expert == a.n_local;
                const CUtensorMap* m_nib = sh ? &tmap_sh_nib : &tmap_nib;
                const CUtensorMap* m_sc = sh ? &tmap_sh_sc : &tmap_sc;
                const int slot = sh ? 0 : seg.expert;
                constexpr int kRtPerTile = GATE_UP ? 8 : 16;   // 16-row tiles per stage (gate/up: each carries a gate and an up sub-tile)
                if (tile == (int)blockIdx.x)   // first tile: warm L2 with the first chunks
                    for (int kc = 0; kc < kPrefetchAhead && kc < n_kc; kc++) tma_prefetch_4d(m_nib, 0, kc * C::kKtPerChunk, mb * kRtPerTile, slot);
                // the tile this block runs next (its first chunks are prefetched while this one finishes)
                const int ntile = tile + gridDim.x;
                PrefillSeg nseg = seg;
                int nmb = mb;
                if (ntile < n_tiles) { nseg = a.segs[ntile / n_mb]; nmb = ntile % n_mb; }
                const bool nsh = nseg.expert == a.n_local;
                for (int kc = 0; kc < n_kc && ok; kc++) {
                    const int pk = kc + kPrefetchAhead;
                    if (pk < n_kc) tma_prefetch_4d(m_nib, 0, pk * C::kKtPerChunk, mb * kRtPerTile, slot);
                    else if (ntile < n_tiles)
                        tma_prefetch_4d(nsh ? &tmap_sh_nib : &tmap_nib, 0, (pk - n_kc) * C::kKtPerChunk, nmb * kRtPerTile, nsh ? 0 : nseg.expert);
                    // one box of codes, one of scales
                    const int s = rcnt % C::kRawStages;
                    ok = mbar_wait(bar(RAW_EMPTY + s), ((rcnt / C::kRawStages) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    const uint32_t dst = sbase + C::kSmemRaw + s * C::kRawBytes;
                    mbar_expect_tx(bar(RAW_FULL + s), C::kRawBytes);
                    tma_load_4d(dst, m_nib, 0, kc * C::kKtPerChunk, mb * kRtPerTile, slot, bar(RAW_FULL + s));
                    tma_load_4d(dst + C::kRawNib, m_sc, 0, kc * C::kKtPerChunk, mb * kRtPerTile, slot, bar(RAW_FULL + s));
                    rcnt++;
                }
            }
        }
    } else if (warp == kBProducerWarp) {
        // ---------------------------------------------------- token-tile producer
        if (lane == 0) {
            uint32_t bcnt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const PrefillSeg seg = a.segs[tile / n_mb];
                // only the rows the segment has, in boxes of 64 / 128 / 192 / 256 rows
                const int n_box = (max(16, (seg.n + 15) & ~15) + 63) >> 6;
                const CUtensorMap* m_b = n_box == 1 ? &tmap_b64 : (n_box == 2 ? &tmap_b128 : (n_box == 3 ? &tmap_b192 : &tmap_b256));
                for (int kc = 0; kc < n_kc && ok; kc++) {
                    const int s = bcnt % C::kBStages;
                    ok = mbar_wait(bar(B_EMPTY + s), ((bcnt / C::kBStages) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(bar(B_FULL + s), (uint32_t)(n_box * 64 * kChunkK * 2));
                    tma_load_2d(sbase + C::kSmemB + s * kBBytes, m_b, kc * kChunkK, seg.row0, bar(B_FULL + s));
                    bcnt++;
                }
            }
        }
    } else if (warp == 1) {
        // ----------------------------------------------------------- MMA issue
        if (lane == 0) {
            uint32_t tcnt = 0, sa = 0, ph = 0, sb = 0, phb = 0;   // ring stages and their phase parities
            bool ok = true;
            const uint64_t d0 = umma_desc(sbase + C::kSmemA);
            const uint32_t hi = (uint32_t)(d0 >> 32);                       // same for every operand tile
            const uint32_t a_lo0 = (uint32_t)d0, b_lo0 = (uint32_t)umma_desc(sbase + C::kSmemB);
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const PrefillSeg seg = a.segs[tile / n_mb];
                const int n16 = max(16, (seg.n + 15) & ~15);
                const uint32_t idesc = umma_idesc(n16);
                ok = mbar_wait(bar(ACC_EMPTY), (tcnt & 1u) ^ 1u, abort_flag);   // the previous tile's accumulators are drained
                if (!ok) break;
                tc_fence_after();
                for (int kc = 0; kc < n_kc; kc++) {
                    const uint32_t a_full = bar(A_FULL) + 8u * sa, b_full = bar(B_FULL) + 8u * sb;
                    if (!mbar_try(a_full, ph) && !mbar_wait(a_full, ph, abort_flag)) { ok = false; break; }
                    if (!mbar_try(b_full, phb) && !mbar_wait(b_full, phb, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    tc_mma_chunk(tmem_base, a_lo0 + sa * (kABytes >> 4), b_lo0 + sb * (kBBytes >> 4), hi, idesc, kc != 0 ? 1u : 0u);
                    tc_commit(bar(A_EMPTY) + 8u * sa);   // arrive when the MMAs above have read their operands
                    tc_commit(bar(B_EMPTY) + 8u * sb);
                    if (++sa == C::kAStages) { sa = 0; ph ^= 1u; }
                    if (++sb == C::kBStages) { sb = 0; phb ^= 1u; }
                }
                if (ok) tc_commit(bar(ACC_FULL));
                tcnt++;
            }
        }
    } else if (warp < 2 + kConvWarps) {
        // ---------------------------------------------------------- converters
        const int cw = warp - 2, g = lane >> 2, t = lane & 3;
        uint32_t rcnt = 0, acnt = 0, tcnt = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            for (int kc = 0; kc < n_kc && ok; kc++) {
                const int sr = rcnt % C::kRawStages, sa = acnt % C::kAStages;
                ok = mbar_wait(bar(RAW_FULL + sr), (rcnt / C::kRawStages) & 1u, abort_flag);
                ok = ok && mbar_wait(bar(A_EMPTY + sa), ((acnt / C::kAStages) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                const uint8_t* raw = smem + C::kSmemRaw + sr * C::kRawBytes;
                uint8_t* A = smem + C::kSmemA + sa * kABytes;
                if constexpr (FMT == DSX_FMT_MXFP4) {
                    // both sub-tiles of this warp: loads first, then the conversions
                    uint4 wq[2];
                    uint32_t sw[2];
    #pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const int st = cw + 8 * half;   // sub-tile of the raw stage
                        wq[half] = *reinterpret_cast<const uint4*>(raw + st * kSubNibBytes + lane * 16);
                        sw[half] = *reinterpret_cast<const uint32_t*>(raw + C::kRawNib + st * kSubScBytes + g * 4);
                    }
    #pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const int st = cw + 8 * half;
                        // gate/up stage order is [rt][gate, up]; A rows 0..127 = gate, 128..255 = up
                        const int row_base = GATE_UP ? ((st & 1) * 128 + (st >> 1) * 16) : st * 16;
                        const uint32_t w[4] = {wq[half].x, wq[half].y, wq[half].z, wq[half].w};
                        uint8_t* arow = A + (uint32_t)((row_base + g) >> 3) * 1024u + (uint32_t)g * 128u;
    #pragma unroll
                        for (int bi = 0; bi < 2; bi++) {
                            // odd row groups take the two scale blocks in the opposite order, so the eight
                            // lanes of a quarter warp store to eight different 16-byte bank groups
                            const int b = bi ^ (g & 1);
                            const uint32_t m0 = scale_h2((sw[half] >> (8 * b)) & 0xFFu), m1 = scale_h2((sw[half] >> (16 + 8 * b)) & 0xFFu);
                            uint32_t p[4], q[4];
                            cvt4(b ? w[2] : w[0], p);   // (g; c0,c1) (g+8; c0,c1) (g; c2,c3) (g+8; c2,c3)
                            cvt4(b ? w[3] : w[1], q);   // same for columns c4..c7
                            const uint4 r0 = make_uint4(hmul2(p[0], m0), hmul2(p[2], m0), hmul2(q[0], m0), hmul2(q[2], m0));
                            const uint4 r1 = make_uint4(hmul2(p[1], m1), hmul2(p[3], m1), hmul2(q[1], m1), hmul2(q[3], m1));
                            const uint32_t off = (uint32_t)(((4 * b + t) ^ g) << 4);   // 16-byte chunk 4b+t, swizzled by the row
                            *reinterpret_cast<uint4*>(arow + off) = r0;
                            *reinterpret_cast<uint4*>(arow + off + 1024u) = r1;   // row + 8: next 8-row group, same swizzle phase
                        }
                    }
                } else {
                    // Q8_0: 32 sub-tiles of 16 rows x 32 columns, stage order [row tile][column tile 0/1][gate, up]
                    // (down: [row tile][column tile]).  A warp takes two PAIRS of sub-tiles that differ in the column tile, in two
                    // rounds each: lanes of even row g convert column tile r, lanes of odd g column tile r ^ 1, so that the
                    // eight lanes of a quarter warp (two neighbouring g) store to eight different 16-byte bank groups of the
                    // swizzled operand tile (one column tile per round put them on four, every store a 2-way conflict).
                    // A lane's 16 bytes are rows g / g+8 x 8 consecutive columns: words {row g cols 0-3, row g+8 cols 0-3,
                    // row g cols 4-7, row g+8 cols 4-7}.
                    uint4 wq[4];
                    uint32_t sw[4];
                    constexpr int kColTileStep = GATE_UP ? 2 : 1;   // sub-tile index distance between the two column tiles
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int pr = cw + 8 * (i >> 1), kt2 = (i & 1) ^ (g & 1);
                        const int st = (GATE_UP ? (pr >> 1) * 4 + (pr & 1) : pr * 2) + kt2 * kColTileStep;
                        wq[i] = *reinterpret_cast<const uint4*>(raw + st * kSubNibBytes + lane * 16);
                        sw[i] = *reinterpret_cast<const uint32_t*>(raw + C::kRawNib + st * kSubScBytes + g * 4);
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int pr = cw + 8 * (i >> 1), kt2 = (i & 1) ^ (g & 1);
                        const int gu = GATE_UP ? (pr & 1) : 0, rt = GATE_UP ? (pr >> 1) : pr;
                        const int row_base = gu * 128 + rt * 16;
                        uint8_t* arow = A + (uint32_t)((row_base + g) >> 3) * 1024u + (uint32_t)g * 128u;
                        const uint32_t m0 = (sw[i] & 0xFFFFu) * 0x00010001u, m1 = (sw[i] >> 16) * 0x00010001u;   // f16 scale of row g / g+8
                        const uint4 r0 = make_uint4(hmul2(q8_pair(wq[i].x, 0x4140), m0), hmul2(q8_pair(wq[i].x, 0x4342), m0),
                                                    hmul2(q8_pair(wq[i].z, 0x4140), m0), hmul2(q8_pair(wq[i].z, 0x4342), m0));
                        const uint4 r1 = make_uint4(hmul2(q8_pair(wq[i].y, 0x4140), m1), hmul2(q8_pair(wq[i].y, 0x4342), m1),
                                                    hmul2(q8_pair(wq[i].w, 0x4140), m1), hmul2(q8_pair(wq[i].w, 0x4342), m1));
                        const uint32_t off = (uint32_t)(((4 * kt2 + t) ^ g) << 4);
                        *reinterpret_cast<uint4*>(arow + off) = r0;
                        *reinterpret_cast<uint4*>(arow + off + 1024u) = r1;
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar(A_FULL + sa));
                    mbar_arrive(bar(RAW_EMPTY + sr));
                }
                rcnt++;
                acnt++;
            }
            // the tile's operands are all converted: help drain its accumulators
            if (ok) ok = mbar_wait(bar(ACC_FULL), tcnt & 1u, abort_flag);
            if (!ok) break;
            epilogue(tile, 1 + (cw >> 2));
            if (lane == 0) mbar_arrive(bar(ACC_EMPTY));
            tcnt++;
        }
    } else if (warp < kEpiWarp0 + 4) {
        // ------------------------------------------------------------ epilogue
        uint32_t tcnt = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            ok = mbar_wait(bar(ACC_FULL), tcnt & 1u, abort_flag);
            if (!ok) break;
            epilogue(tile, 0);
            if (lane == 0) mbar_arrive(bar(ACC_EMPTY));
            tcnt++;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(a.error_word, 2u);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// ---------------------------------------------------------------- helpers
__device__ __forceinline__ int seg_size(int cnt, int seg_rows) {  // even split into segments of at most seg_rows rows, multiples of 16
    const int n = (cnt + seg_rows - 1) / seg_rows;
    return n == 0 ? 0 : min(seg_rows, (((cnt + n - 1) / n) + 15) & ~15);
}

// One block.  Segments sorted by expert; the shared expert's segments (expert id
// n_local) follow and cover rows P .. P+T-1.  Experts with at most small_max rows get no
// segment: a tile would spend a full pass of weight conversion on a handful of tokens, while the
// grouped GEMV streams the same weights at HBM speed, so they become GEMV work items instead.
#ifndef DSX_SMALL_MAX
#define DSX_SMALL_MAX 8
#endif
// One GEMV item (8 rows) streams an expert's weights once; from 9 rows on it would stream them again per item.  (With
// token-tile and converted-weight rings in lockstep a tile pass used to cost about three items, and the threshold was 24.)
constexpr int kSmallMax = DSX_SMALL_MAX;   // at most 32 (4 work items of 8 rows per expert)
static_assert(kSmallMax <= 32, "the work-item list holds 4 items per expert");

__global__ void __launch_bounds__(512)
build_segments_kernel(const int32_t* __restrict__ offsets, int n_local, int64_t P, int T_shared, int seg_rows,
                      PrefillSeg* __restrict__ segs, int32_t* __restrict__ n_segs, int cap, int small_max,
                      int32_t* __restrict__ small_items, int32_t* __restrict__ n_small) {
    // thread e = expert e (n_local <= 512): its segment count and GEMV item count, then an exclusive scan of both
    __shared__ int s_seg[512], s_small[512];
    const int e = threadIdx.x;
    int cnt = 0, sz = 0, nseg = 0, nsmall = 0;
    if (e < n_local) {
        cnt = offsets[e + 1] - offsets[e];
        if (cnt > 0 && cnt <= small_max) nsmall = (cnt + 7) >> 3;
        else { sz = seg_size(cnt, seg_rows); nseg = sz ? (cnt + sz - 1) / sz : 0; }
    }
    s_seg[e] = nseg;
    s_small[e] = nsmall;
    __syncthreads();
    for (int d = 1; d < 512; d <<= 1) {   // inclusive scan, 9 steps
        const int a = e >= d ? s_seg[e - d] : 0, b = e >= d ? s_small[e - d] : 0;
        __syncthreads();
        s_seg[e] += a;
        s_small[e] += b;
        __syncthreads();
    }
    const int seg_base = s_seg[e] - nseg, small_base = s_small[e] - nsmall;
    const int routed_segs = s_seg[511];
    if (e < n_local) {
        const int row0 = offsets[e];
        for (int i = 0; i < nsmall; i++) small_items[small_base + i] = (int32_t)(((uint32_t)e << 16) | (uint32_t)(8 * i));
        for (int i = 0, st = 0; i < nseg; i++, st += sz)
            if (seg_base + i < cap) segs[seg_base + i] = PrefillSeg{e, row0 + st, min(sz, cnt - st), 0};
    }
    // the shared expert's segments follow, over rows P .. P + T_shared - 1, spread over the threads
    const int ssz = seg_size(T_shared, seg_rows), sn = ssz ? (T_shared + ssz - 1) / ssz : 0;
    for (int i = e; i < sn; i += 512)
        if (routed_segs + i < cap) segs[routed_segs + i] = PrefillSeg{n_local, (int)P + i * ssz, min(ssz, T_shared - i * ssz), 0};
    if (e == 0) {
        n_segs[0] = min(cap, routed_segs + sn);
        if (n_small != nullptr) n_small[0] = s_small[511];
    }
}

// Token rows in expert-sorted order as f16 (row p < placed: token perm[p] / k),
// then every token once more for the shared expert (row P + t).
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ perm, const int32_t* __restrict__ offsets,
                   int n_local, int n_used, int64_t P, int64_t T, int shared_rows, int64_t H, __half* __restrict__ xperm,
                   uint32_t* __restrict__ error_word) {
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int64_t placed = offsets[n_local];
    int64_t src, dst;
    if (row < placed) { src = perm[row] / n_used; dst = row; }
    else if (row >= P && row < P + (shared_rows ? T : 0)) { src = row - P; dst = row; }
    else return;
    const uint4* in = reinterpret_cast<const uint4*>(x + src * H);
    uint4* out = reinterpret_cast<uint4*>(xperm + dst * H);
    uint32_t bad = 0;
    for (int64_t c = lane; c < H / 8; c += 32) {
        const uint4 v = __ldg(in + c);
        out[c] = make_uint4(bf16x2_to_f16x2(v.x, bad), bf16x2_to_f16x2(v.y, bad), bf16x2_to_f16x2(v.z, bad), bf16x2_to_f16x2(v.w, bad));
    }
    if (bad) atomicOr(error_word, kErrHalfRange);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library links no libcuda).
int tmap_encode(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
                const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        DSX_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !p) return set_error(DSX_ERR_UNSUPPORTED, "driver has no cuTensorMapEncodeTiled");
        fn = (EncodeTiledFn)p;
    }
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = fn(map, type, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(DSX_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return DSX_OK;
}

int launch_build_segments(const int32_t* offsets, int n_local, int64_t P, int T_shared, int seg_rows, PrefillSeg* segs, int32_t* n_segs,
                          int cap, int small_max, int32_t* small_items, int32_t* n_small, cudaStream_t stream) {
    build_segments_kernel<<<1, 512, 0, stream>>>(offsets, n_local, P, T_shared, seg_rows, segs, n_segs, cap, small_max, small_items, n_small);
    DSX_LAUNCHED();
    return DSX_OK;
}

namespace {

int encode_rows_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int box_rows) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        DSX_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !p) return set_error(DSX_ERR_UNSUPPORTED, "driver has no cuTensorMapEncodeTiled");
        fn = (EncodeTiledFn)p;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kChunkK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(DSX_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return DSX_OK;
}

// One plane of packed weights as [slot][row tile][column tile][inner bytes as u32]; the box is all
// `box_rt` row tiles x `box_kt` column tiles (one 64-column chunk), landing in shared memory as
// [row tile][column tile][inner bytes].
int encode_plane_map(CUtensorMap* map, const void* base, int inner_bytes, int64_t n_kt, int64_t n_rt, int64_t n_slots,
                     int64_t slot_stride, int box_kt, int box_rt) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        DSX_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !p) return set_error(DSX_ERR_UNSUPPORTED, "driver has no cuTensorMapEncodeTiled");
        fn = (EncodeTiledFn)p;
    }
    const cuuint64_t dims[4] = {(cuuint64_t)(inner_bytes / 4), (cuuint64_t)n_kt, (cuuint64_t)n_rt, (cuuint64_t)n_slots};
    const cuuint64_t strides[3] = {(cuuint64_t)inner_bytes, (cuuint64_t)(n_kt * inner_bytes), (cuuint64_t)slot_stride};
    const cuuint32_t box[4] = {(cuuint32_t)(inner_bytes / 4), (cuuint32_t)box_kt, (cuuint32_t)box_rt, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(DSX_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled (weights) failed with %d", (int)r);
    return DSX_OK;
}

// (Re-)encode the weight maps when the layer points at other planes.
int map_weights(PrefillWorkspace* ws, int which, const uint8_t* gu_nib, const uint8_t* gu_sc, const uint8_t* dn_nib,
                const uint8_t* dn_sc, int64_t gu_nib_stride, int64_t gu_sc_stride, int64_t dn_nib_stride, int64_t dn_sc_stride,
                int n_slots) {
    if (ws->mapped_gu_nib[which] == gu_nib && ws->mapped_dn_nib[which] == dn_nib) return DSX_OK;
    const int64_t H = ws->H, F = ws->F;
    const int tk = tile_k(ws->fmt), box_kt = 64 / tk;   // column tiles per 64-column chunk
    if (int rc = encode_plane_map(&ws->tmap_gu_nib[which], gu_nib, 2 * kSubNibBytes, H / tk, F / 16, n_slots, gu_nib_stride, box_kt, 8)) return rc;
    if (int rc = encode_plane_map(&ws->tmap_gu_sc[which], gu_sc, 2 * kSubScBytes, H / tk, F / 16, n_slots, gu_sc_stride, box_kt, 8)) return rc;
    if (int rc = encode_plane_map(&ws->tmap_dn_nib[which], dn_nib, kSubNibBytes, F / tk, H / 16, n_slots, dn_nib_stride, box_kt, 16)) return rc;
    if (int rc = encode_plane_map(&ws->tmap_dn_sc[which], dn_sc, kSubScBytes, F / tk, H / 16, n_slots, dn_sc_stride, box_kt, 16)) return rc;
    ws->mapped_gu_nib[which] = gu_nib;
    ws->mapped_dn_nib[which] = dn_nib;
    return DSX_OK;
}

}  // namespace

// The f16 copy of the sorted token rows (1 KB per row and 512 hidden columns) is only read by the f16-operand
// kernels: a layer whose stores take the block-scaled path never allocates it.
int prefill_f16_rows_ensure(PrefillWorkspace* ws) {
    if (!ws->ready || ws->xperm != nullptr) return DSX_OK;
    DSX_CUDA(cudaMalloc((void**)&ws->xperm, (size_t)ws->cap_rows * (size_t)ws->H * 2));
    for (int b = 0; b < 4; b++)
        if (int rc = encode_rows_map(&ws->tmap_x[b], ws->xperm, ws->cap_rows, ws->H, 64 * (b + 1))) return rc;
    return DSX_OK;
}

int prefill_workspace_create(PrefillWorkspace* ws, const dsx_moe_config& cfg, int n_used, __half* mid, bool f16_rows) {
    ws->ready = false;
    // shapes the tiles cover: 128 gate + 128 up rows per tile, 256 down rows per tile, 64-column chunks
    if (cfg.ffn % 128 != 0 || cfg.hidden % 256 != 0 || (cfg.shared_ffn != 0 && cfg.shared_ffn != cfg.ffn)) return DSX_OK;
    ws->H = cfg.hidden;
    ws->F = cfg.ffn;
    ws->cap_rows = (int64_t)cfg.max_tokens * n_used + cfg.max_tokens;
    ws->seg_cap = cfg.router.n_expert + (int)((ws->cap_rows + kSegRows - 1) / kSegRows) + 8;
    DSX_CUDA(cudaMalloc((void**)&ws->segs, sizeof(PrefillSeg) * (size_t)ws->seg_cap));
    DSX_CUDA(cudaMalloc((void**)&ws->n_segs, 256));
    DSX_CUDA(cudaMalloc((void**)&ws->small_items, sizeof(int32_t) * (size_t)(cfg.router.n_expert * 4 + 8)));   // up to 32 rows = 4 items per expert
    DSX_CUDA(cudaMalloc((void**)&ws->n_small, 256));
    DSX_CUDA(cudaMemset(ws->n_small, 0, 256));
    // a work item of the grouped GEMV holds at most 8 tokens; both reductions must fit its shared memory
    ws->small_max = (gemv_fits(cfg.hidden) && gemv_fits(cfg.ffn) && cfg.hidden % 128 == 0 && cfg.ffn % 128 == 0) ? kSmallMax : 0;
    for (int b = 0; b < 4; b++)
        if (int rc = encode_rows_map(&ws->tmap_mid[b], mid, ws->cap_rows, cfg.ffn, 64 * (b + 1))) return rc;
    DSX_CUDA(cudaFuncSetAttribute(prefill_gemm_kernel<DSX_FMT_MXFP4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<DSX_FMT_MXFP4>::kSmemTotal));
    DSX_CUDA(cudaFuncSetAttribute(prefill_gemm_kernel<DSX_FMT_MXFP4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<DSX_FMT_MXFP4>::kSmemTotal));
    DSX_CUDA(cudaFuncSetAttribute(prefill_gemm_kernel<DSX_FMT_Q8_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<DSX_FMT_Q8_0>::kSmemTotal));
    DSX_CUDA(cudaFuncSetAttribute(prefill_gemm_kernel<DSX_FMT_Q8_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<DSX_FMT_Q8_0>::kSmemTotal));
    ws->min_tokens = 65;
    ws->ready = true;
    return f16_rows ? prefill_f16_rows_ensure(ws) : DSX_OK;
}

void prefill_workspace_free(PrefillWorkspace* ws) {
    cudaFree(ws->xperm);
    cudaFree(ws->segs);
    cudaFree(ws->n_segs);
    cudaFree(ws->small_items);
    cudaFree(ws->n_small);
    ws->xperm = nullptr; ws->segs = nullptr; ws->n_segs = nullptr; ws->small_items = nullptr; ws->n_small = nullptr; ws->ready = false;
}

bool prefill_wanted(const PrefillWorkspace& ws, const dsx_moe_config&, int fmt, int64_t T) {
    (void)fmt;
    return ws.ready && T >= ws.min_tokens;
}

int prefill_forward(PrefillWorkspace* ws, const dsx_moe_config& cfg, const PrefillCall& c, cudaStream_t stream) {
    const int64_t P = c.T * c.n_used;
    DSX_REQUIRE(P + c.T <= ws->cap_rows, "prefill: %lld rows exceed the workspace (%lld)", (long long)(P + c.T), (long long)ws->cap_rows);
    if (int rc = launch_group_build(c.selected, c.T, c.n_used, c.n_local, c.expert_lo, kSegRows, 0, c.hist, c.offsets, c.perm,
                                    nullptr, nullptr, 0, c.gs, stream))
        return rc;
    if (int rc = launch_build_segments(c.offsets, c.n_local, P, c.with_shared ? (int)c.T : 0, kSegRows, ws->segs, ws->n_segs, ws->seg_cap,
                                       ws->small_max, ws->small_items, ws->n_small, stream))
        return rc;
    const int64_t rows = P + c.T;
    gather_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(c.x, c.perm, c.offsets, c.n_local, c.n_used, P, c.T,
                                                                      c.with_shared ? 1 : 0, cfg.hidden, ws->xperm, c.error_word);
    DSX_LAUNCHED();
    if (ws->fmt != c.fmt) { ws->fmt = c.fmt; ws->mapped_gu_nib[0] = ws->mapped_gu_nib[1] = nullptr; }
    if (int rc = map_weights(ws, 0, c.gu_nib, c.gu_sc, c.dn_nib, c.dn_sc, c.gu_nib_stride, c.gu_sc_stride, c.dn_nib_stride,
                             c.dn_sc_stride, c.n_local))
        return rc;
    const int shi = c.with_shared ? 1 : 0;   // without a shared expert the shared maps alias the routed ones (never used)
    if (c.with_shared)
        if (int rc = map_weights(ws, 1, c.sh_gu_nib, c.sh_gu_sc, c.sh_dn_nib, c.sh_dn_sc, c.gu_nib_stride, c.gu_sc_stride,
                                 c.dn_nib_stride, c.dn_sc_stride, 1))
            return rc;
    // experts with a handful of rows: the decode kernels, over the same sorted rows and partial rows
    GemvArgs v{};
    v.fmt = c.fmt; v.shared_fmt = c.fmt; v.n_expert = c.n_local;
    v.work_items = ws->small_items; v.n_work_items = ws->n_small; v.item_recs = nullptr; v.offsets = c.offsets; v.perm = c.perm;
    v.route_w = c.route_w; v.n_used = c.n_used; v.T = c.T; v.clamp = cfg.clamp; v.x = c.x; v.mid = c.mid; v.mid_stride = cfg.ffn;
    v.partial = c.partial; v.error_word = c.error_word;
    GemmArgs g{};
    g.segs = ws->segs; g.n_segs = ws->n_segs; g.n_local = c.n_local; g.n_used = c.n_used; g.P = P; g.perm = c.perm;
    g.route_w = c.route_w; g.clamp = cfg.clamp; g.mid = c.mid; g.mid_stride = cfg.ffn; g.partial = c.partial; g.error_word = c.error_word;
    // gate/up: K = hidden, rows = ffn
    g.K = cfg.hidden; g.rows = cfg.ffn;
    if (c.fmt == DSX_FMT_MXFP4)
        prefill_gemm_kernel<DSX_FMT_MXFP4, true><<<c.sm_count, kThreads, Shape<DSX_FMT_MXFP4>::kSmemTotal, stream>>>(
            ws->tmap_x[0], ws->tmap_x[1], ws->tmap_x[2], ws->tmap_x[3], ws->tmap_gu_nib[0], ws->tmap_gu_sc[0], ws->tmap_gu_nib[shi], ws->tmap_gu_sc[shi], g);
    else
        prefill_gemm_kernel<DSX_FMT_Q8_0, true><<<c.sm_count, kThreads, Shape<DSX_FMT_Q8_0>::kSmemTotal, stream>>>(
            ws->tmap_x[0], ws->tmap_x[1], ws->tmap_x[2], ws->tmap_x[3], ws->tmap_gu_nib[0], ws->tmap_gu_sc[0], ws->tmap_gu_nib[shi], ws->tmap_gu_sc[shi], g);
    DSX_LAUNCHED();
    if (ws->small_max > 0) {
        v.K = cfg.hidden; v.rows = cfg.ffn; v.sh_rows = cfg.ffn;
        v.nib = c.gu_nib; v.sc = c.gu_sc; v.nib_slot_stride = c.gu_nib_stride; v.sc_slot_stride = c.gu_sc_stride;
        if (int rc = launch_gemv_gate_up(v, c.sm_count, stream)) return rc;
    }
    // down: K = ffn, rows = hidden
    g.K = cfg.ffn; g.rows = cfg.hidden;
    if (c.fmt == DSX_FMT_MXFP4)
        prefill_gemm_kernel<DSX_FMT_MXFP4, false><<<c.sm_count, kThreads, Shape<DSX_FMT_MXFP4>::kSmemTotal, stream>>>(
            ws->tmap_mid[0], ws->tmap_mid[1], ws->tmap_mid[2], ws->tmap_mid[3], ws->tmap_dn_nib[0], ws->tmap_dn_sc[0], ws->tmap_dn_nib[shi], ws->tmap_dn_sc[shi], g);
    else
        prefill_gemm_kernel<DSX_FMT_Q8_0, false><<<c.sm_count, kThreads, Shape<DSX_FMT_Q8_0>::kSmemTotal, stream>>>(
            ws->tmap_mid[0], ws->tmap_mid[1], ws->tmap_mid[2], ws->tmap_mid[3], ws->tmap_dn_nib[0], ws->tmap_dn_sc[0], ws->tmap_dn_nib[shi], ws->tmap_dn_sc[shi], g);
    DSX_LAUNCHED();
    if (ws->small_max > 0) {
        v.K = cfg.ffn; v.rows = cfg.hidden; v.sh_rows = cfg.hidden;
        v.nib = c.dn_nib; v.sc = c.dn_sc; v.nib_slot_stride = c.dn_nib_stride; v.sc_slot_stride = c.dn_sc_stride;
        if (int rc = launch_gemv_down(v, c.sm_count, stream)) return rc;
    }
    if (c.skip_combine) return DSX_OK;   // the caller adds another pass before it reduces the partial rows
    return launch_combine(c.partial, c.T, c.n_used, cfg.hidden, c.with_shared ? 1 : 0, c.filter_picks ? c.selected : nullptr,
                          c.expert_lo, c.n_local, c.out, stream, c.out_rows);
}

}  // namespace dsx
