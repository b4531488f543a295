// Token -> expert histogram, offsets, stable permutation and work items.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   crates/v4flash-kernels/kernels/expert_sel_count.hip:17-28     histogram
//   crates/v4flash-kernels/kernels/moe_group_builder.hip:32-51     group inversion (atomic order)
//   crates/v4flash-kernels/kernels/moe_work_items_builder.hip:61-145  prefix sum + work items sorted by expert
//   crates/v4flash-kernels/kernels/b2_fast_chain.hip:46-128        fused single-block builder with the
//                                                                  deterministic (token, slot) member order
// The reference's atomic builder leaves member order unspecified; this one is a
// stable counting sort, so hist, offsets AND perm are reproducible bit for bit:
// warp ballots (match_any) rank equal experts inside a 32-pick step, per-warp
// and per-block prefix sums order the steps.
#include <mutex>

#include "dsx_common.cuh"

namespace dsx {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kPerWarp = kGroupChunk / kWarps;  // 128 picks per warp
constexpr int kMaxExperts = 512;

// wh[w*E + e] = picks of local expert e inside warp w's slice of the chunk.
__device__ void chunk_count(const int32_t* __restrict__ sel, int64_t P, int64_t chunk_base, int E, int lo, int* wh) {
    for (int i = threadIdx.x; i < kWarps * E; i += kThreads) wh[i] = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int it = 0; it < kPerWarp / 32; it++) {
        const int64_t idx = chunk_base + warp * kPerWarp + it * 32 + lane;
        if (idx < P) {
            const int e = sel[idx] - lo;
            if (e >= 0 && e < E) atomicAdd(&wh[warp * E + e], 1);
        }
    }
    __syncthreads();
}

// Exclusive scan of one value per thread over the block (kThreads threads).
__device__ int block_exclusive_scan(int v, int* total, int* s_warp /*[kWarps+1]*/) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xFFFFFFFFu, inc, off);
        if (lane >= off) inc += o;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < kWarps ? s_warp[lane] : 0;
        int winc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xFFFFFFFFu, winc, off);
            if (lane >= off) winc += o;
        }
        if (lane < kWarps) s_warp[lane] = winc - w;
        if (lane == kWarps - 1) s_warp[kWarps] = winc;
    }
    __syncthreads();
    const int res = s_warp[warp] + inc - v;
    *total = s_warp[kWarps];
    __syncthreads();
    return res;
}

// From hist (one expert per thread): offsets, work items (+ shared-expert items).
__device__ void write_offsets_and_items(int e, int E, int h, int chunk, int shared_T, int32_t* hist, int32_t* offsets,
                                        int32_t* work_items, int32_t* n_work_items, int32_t work_cap, int* s_warp) {
    int total;
    const int off = block_exclusive_scan(e < E ? h : 0, &total, s_warp);
    if (e < E) {
        hist[e] = h;
        offsets[e] = off;
    }
    if (threadIdx.x == 0) offsets[E] = total;
    if (work_items != nullptr) {
        const int ni = (e < E) ? (h + chunk - 1) / chunk : 0;
        int n_items;
        const int ibase = block_exclusive_scan(ni, &n_items, s_warp);
        for (int c = 0; c < ni; c++) {
            const int p = ibase + c;
            if (p < work_cap) work_items[p] = (int32_t)(((uint32_t)e << 16) | (((uint32_t)(c * chunk)) & 0xFFFFu));
        }
        // the shared expert is appended as pseudo expert id E over all tokens
        const int n_sh = (shared_T + chunk - 1) / chunk;
        for (int c = threadIdx.x; c < n_sh; c += kThreads) {
            const int p = n_items + c;
            if (p < work_cap) work_items[p] = (int32_t)(((uint32_t)E << 16) | (((uint32_t)(c * chunk)) & 0xFFFFu));
        }
        if (threadIdx.x == 0) n_work_items[0] = n_items + n_sh;
    }
}

// Stable placement of this block's chunk.  wh[w*E+e] holds the first free
// position of expert e for warp w; each warp walks its slice in order.
__device__ void chunk_place(const int32_t* __restrict__ sel, int64_t P, int64_t chunk_base, int E, int lo, int* wh,
                            int32_t* __restrict__ perm) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int it = 0; it < kPerWarp / 32; it++) {
        const int64_t idx = chunk_base + warp * kPerWarp + it * 32 + lane;
        int e = -1;
        if (idx < P) {
            e = sel[idx] - lo;
            if (e < 0 || e >= E) e = -1;
        }
        const int key = e >= 0 ? e : (0x40000000 | lane);
        const uint32_t mask = __match_any_sync(0xFFFFFFFFu, key);
        const int rank = __popc(mask & ((1u << lane) - 1u));
        if (e >= 0) perm[wh[warp * E + e] + rank] = (int32_t)idx;
        __syncwarp();
        if (e >= 0 && rank == 0) wh[warp * E + e] += __popc(mask);
        __syncwarp();
    }
}

// Single block: T*k <= kGroupChunk.
__global__ void __launch_bounds__(kThreads)
group_build_small_kernel(const int32_t* __restrict__ sel, int64_t P, int E, int lo, int chunk, int shared_T,
                         int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items,
                         int32_t work_cap) {
    extern __shared__ int wh[];
    __shared__ int s_warp[kWarps + 1];
    chunk_count(sel, P, 0, E, lo, wh);
    const int e = threadIdx.x;
    int h = 0;
    if (e < E)
        for (int w = 0; w < kWarps; w++) h += wh[w * E + e];
    write_offsets_and_items(e, E, h, chunk, shared_T, hist, offsets, work_items, n_work_items, work_cap, s_warp);
    if (e < E) {
        int run = offsets[e];
        for (int w = 0; w < kWarps; w++) {
            const int v = wh[w * E + e];
            wh[w * E + e] = run;
            run += v;
        }
    }
    __syncthreads();
    chunk_place(sel, P, 0, E, lo, wh, perm);
}

__global__ void __launch_bounds__(kThreads)
group_count_kernel(const int32_t* __restrict__ sel, int64_t P, int E, int lo, int32_t* __restrict__ chunk_hist) {
    extern __shared__ int wh[];
    chunk_count(sel, P, (int64_t)blockIdx.x * kGroupChunk, E, lo, wh);
    for (int e = threadIdx.x; e < E; e += kThreads) {
        int h = 0;
        for (int w = 0; w < kWarps; w++) h += wh[w * E + e];
        chunk_hist[(int64_t)blockIdx.x * E + e] = h;
    }
}

__global__ void __launch_bounds__(kThreads)
group_scan_kernel(int n_chunks, int E, int chunk, int shared_T, int32_t* chunk_hist, int32_t* hist, int32_t* offsets,
                  int32_t* work_items, int32_t* n_work_items, int32_t work_cap) {
    __shared__ int s_warp[kWarps + 1];
    const int e = threadIdx.x;
    int run = 0;
    if (e < E)
        for (int c = 0; c < n_chunks; c++) {
            const int v = chunk_hist[(int64_t)c * E + e];
            chunk_hist[(int64_t)c * E + e] = run;  // picks of e in earlier chunks
            run += v;
        }
    write_offsets_and_items(e, E, run, chunk, shared_T, hist, offsets, work_items, n_work_items, work_cap, s_warp);
}

__global__ void __launch_bounds__(kThreads)
group_place_kernel(const int32_t* __restrict__ sel, int64_t P, int E, int lo, const int32_t* __restrict__ chunk_hist,
                   const int32_t* __restrict__ offsets, int32_t* __restrict__ perm) {
    extern __shared__ int wh[];
    const int64_t base = (int64_t)blockIdx.x * kGroupChunk;
    chunk_count(sel, P, base, E, lo, wh);
    for (int e = threadIdx.x; e < E; e += kThreads) {
        int run = offsets[e] + chunk_hist[(int64_t)blockIdx.x * E + e];
        for (int w = 0; w < kWarps; w++) {
            const int v = wh[w * E + e];
            wh[w * E + e] = run;
            run += v;
        }
    }
    __syncthreads();
    chunk_place(sel, P, base, E, lo, wh, perm);
}

// Scratch of the allocation-free entry point: the per-chunk histograms of the
// multi-block counting sort, for at most kStaticMaxChunks chunks of kGroupChunk
// picks (131072 picks, e.g. 16384 tokens x top-8).  128 KiB of device memory on
// every GPU that loads the library, held until the process exits.
constexpr int kStaticMaxChunks = 64;
static __device__ __align__(256) int32_t g_static_chunk_hist[kStaticMaxChunks * kMaxExperts];

}  // namespace

// Device address of g_static_chunk_hist on the CURRENT device.  In host code the
// array's name is only a handle for cudaGetSymbolAddress, never a pointer a
// kernel may receive; the lookup is done once per device and cached.
static int static_scratch(int32_t** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int32_t* cache[kMaxDevices] = {};
    int dev = 0;
    DSX_CUDA(cudaGetDevice(&dev));
    DSX_REQUIRE(dev >= 0 && dev < kMaxDevices, "group_build_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        DSX_CUDA(cudaGetSymbolAddress(&p, g_static_chunk_hist));
        cache[dev] = static_cast<int32_t*>(p);
    }
    *out = cache[dev];
    return DSX_OK;
}

int launch_group_build_static(const int32_t* selected, int64_t T, int n_used, int n_expert, int chunk, int32_t* hist,
                              int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap,
                              cudaStream_t stream) {
    const int64_t P = T * n_used;
    const int64_t n_chunks = (P + kGroupChunk - 1) / kGroupChunk;
    if (n_chunks > kStaticMaxChunks)
        return set_error(DSX_ERR_UNSUPPORTED,
                         "group_build_static: %lld picks exceed the built-in scratch (at most %d picks); use dsx_moe_group_build",
                         (long long)P, kStaticMaxChunks * kGroupChunk);
    GroupScratch gs{};
    if (int rc = static_scratch(&gs.chunk_hist)) return rc;
    gs.capacity_chunks = kStaticMaxChunks;
    return launch_group_build(selected, T, n_used, n_expert, 0, chunk, 0, hist, offsets, perm, work_items, n_work_items, work_cap,
                              gs, stream);
}

int launch_group_build(const int32_t* selected, int64_t T, int n_used, int n_expert, int expert_lo, int chunk,
                       int shared_items_for_T, int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items,
                       int32_t* n_work_items, int32_t work_cap, GroupScratch scratch, cudaStream_t stream) {
    DSX_REQUIRE(n_expert >= 1 && n_expert <= kMaxExperts, "group_build: n_expert %d out of range (1..%d)", n_expert, kMaxExperts);
    DSX_REQUIRE(chunk >= 1, "group_build: chunk must be positive");
    DSX_REQUIRE(work_items == nullptr || T < 65536, "group_build: packed work items need fewer than 65536 tokens");
    const int64_t P = T * n_used;
    const size_t smem = sizeof(int) * (size_t)kWarps * (size_t)n_expert;
    if (P <= kGroupChunk) {
        group_build_small_kernel<<<1, kThreads, smem, stream>>>(selected, P, n_expert, expert_lo, chunk, shared_items_for_T,
                                                                hist, offsets, perm, work_items, n_work_items, work_cap);
        DSX_LAUNCHED();
        return DSX_OK;
    }
    const int64_t n_chunks = (P + kGroupChunk - 1) / kGroupChunk;
    DSX_REQUIRE(scratch.chunk_hist != nullptr && scratch.capacity_chunks >= n_chunks,
                "group_build: scratch holds %lld chunks, %lld needed", (long long)scratch.capacity_chunks, (long long)n_chunks);
    group_count_kernel<<<(unsigned)n_chunks, kThreads, smem, stream>>>(selected, P, n_expert, expert_lo, scratch.chunk_hist);
    DSX_LAUNCHED();
    group_scan_kernel<<<1, kThreads, 0, stream>>>((int)n_chunks, n_expert, chunk, shared_items_for_T, scratch.chunk_hist, hist,
                                                  offsets, work_items, n_work_items, work_cap);
    DSX_LAUNCHED();
    group_place_kernel<<<(unsigned)n_chunks, kThreads, smem, stream>>>(selected, P, n_expert, expert_lo, scratch.chunk_hist,
                                                                      offsets, perm);
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace dsx
