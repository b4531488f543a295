// Expert-parallel exchange over peer memory (NVLink / NVSwitch, plain loads and stores).
//
// What travels follows the reference's remote-expert protocol (paths relative to the deepstrix
// repository): docs/v41/REMOTE_EXPERTS.md:163-164,196-229 and het/remote_experts.rs:7428-7442 -- a
// token row is sent ONCE to every rank that owns at least one of its picks, with all its picks
// and weights; the owner skips the picks it does not own and returns one weighted partial row
// per received token; the sender adds the partials in rank order to its shared-expert output.
// The transport (TCP "DSXP" in the reference) is replaced: every rank owns one slab of device
// memory that its peers map (CUDA IPC) and write into directly.
//
// Slab of rank d (all offsets 256-byte aligned):
//   recv_x    [world][cap][H]   bf16   rows sent by source s land in region s, in token order
//   recv_meta [world][cap][2k]  i32    their picks, then their weights (bit-cast)
//   back      [world][cap][H]   bf16   partial rows returned by owner o land in region o, at the
//                                      slot the token had in the dispatch to o
//   counts    [world]           i32    rows sent by each source this step
//   flags     [world]           u32    barrier: the last epoch each peer has reached
//
// One step of a rank, all on one stream, no host synchronisation:
//   dispatch -> barrier -> prepare -> (owned experts on world*cap slots) -> give_back -> barrier -> sum
// A slot is fixed by an exclusive scan over the source's tokens, so the layout and the order of
// every addition are the same from run to run.  Buffer reuse between steps is safe because a
// rank passes the second barrier of step n only when every rank has finished reading step n's
// rows, and enters the first barrier of step n+1 only after its own sum of step n.
// The barrier is one small kernel: it publishes the epoch in every peer's flags with a
// system-scope release, then waits -- for a bounded number of polls, after which it records
// error bit 1 and returns -- until every peer has published the same epoch.
#include <algorithm>
#include <cstring>

#include "dsx_common.cuh"

namespace dsx {
namespace {

constexpr int kMaxWorld = 8;
constexpr uint32_t kBarrierPolls = 1u << 24;   // x >= 100 ns each: seconds

struct SlabLayout {
    size_t recv_x, recv_meta, back, counts, flags, total;
};

SlabLayout slab_layout(int world, int64_t cap, int64_t H, int k) {
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    SlabLayout l{};
    size_t o = 0;
    l.recv_x = o; o = up(o + (size_t)world * cap * H * 2);
    l.recv_meta = o; o = up(o + (size_t)world * cap * 2 * k * 4);
    l.back = o; o = up(o + (size_t)world * cap * H * 2);
    l.counts = o; o = up(o + (size_t)world * 4);
    l.flags = o; o = up(o + (size_t)world * 4);
    l.total = o;
    return l;
}

struct PeerTable {   // passed to kernels by value
    uint8_t* slab[kMaxWorld];
};

// ---- dispatch, step 1: one block per destination; slot of every token by an exclusive scan
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
ep_scan_kernel(const int32_t* __restrict__ selected, int T, int k, int per_rank, int cap, int32_t* __restrict__ slot_of /*[world][cap]*/,
               PeerTable peers, size_t counts_off, int rank) {
    __shared__ int s_warp[kScanThreads / 32 + 1];
    const int d = blockIdx.x;
    const int per_thread = (T + kScanThreads - 1) / kScanThreads;
    const int t0 = threadIdx.x * per_thread;
    // flags of this thread's run of tokens, as a bit mask (per_thread <= 32)
    uint32_t mine = 0;
    for (int i = 0; i < per_thread; i++) {
        const int t = t0 + i;
        if (t < T) {
            bool hit = false;
            for (int s = 0; s < k; s++) {
                const int e = selected[(int64_t)t * k + s];
                hit = hit || (e >= 0 && e / per_rank == d);
            }
            if (hit) mine |= 1u << i;
        }
    }
    const int cnt = __popc(mine);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int inc = cnt;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xFFFFFFFFu, inc, off);
        if (lane >= off) inc += o;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        const int w = s_warp[lane];
        int winc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xFFFFFFFFu, winc, off);
            if (lane >= off) winc += o;
        }
        s_warp[lane] = winc - w;
        if (lane == 31) s_warp[32] = winc;
    }
    __syncthreads();
    int pos = s_warp[warp] + inc - cnt;
    for (int i = 0; i < per_thread; i++) {
        const int t = t0 + i;
        if (t < T) {
            const bool hit = (mine >> i) & 1u;
            slot_of[(int64_t)d * cap + t] = hit ? pos : -1;
            pos += hit ? 1 : 0;
        }
    }
    if (threadIdx.x == 0) reinterpret_cast<int32_t*>(peers.slab[d] + counts_off)[rank] = s_warp[32];
}

// ---- dispatch, step 2: one block per token; the row is read once and stored to every owner
constexpr int kRowThreads = 256;
__global__ void __launch_bounds__(kRowThreads)
ep_send_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ selected, const float* __restrict__ weights, int T,
               int k, int64_t H, int cap, int world, int rank, const int32_t* __restrict__ slot_of, PeerTable peers, size_t recv_x_off,
               size_t recv_meta_off) {
    const int t = blockIdx.x;
    const int n16 = (int)(H >> 3);   // 16-byte pieces per row
    const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t * H);
    for (int d = 0; d < world; d++) {
        const int slot = slot_of[(int64_t)d * cap + t];
        if (slot < 0) continue;
        const int64_t row = (int64_t)rank * cap + slot;
        uint4* dst = reinterpret_cast<uint4*>(peers.slab[d] + recv_x_off) + row * n16;
        for (int c = threadIdx.x; c < n16; c += kRowThreads) dst[c] = __ldg(src + c);
        int32_t* meta = reinterpret_cast<int32_t*>(peers.slab[d] + recv_meta_off) + row * 2 * k;
        if (threadIdx.x < k) meta[threadIdx.x] = selected[(int64_t)t * k + threadIdx.x];
        else if (threadIdx.x < 2 * k) meta[threadIdx.x] = __float_as_int(weights[(int64_t)t * k + threadIdx.x - k]);
    }
}

// ---- barrier across the ranks
__global__ void ep_barrier_kernel(PeerTable peers, size_t flags_off, int world, int rank, uint32_t epoch, uint32_t polls,
                                  uint32_t* error_word) {
    const int p = threadIdx.x;
    if (p >= world) return;
    __threadfence_system();
    volatile uint32_t* theirs = reinterpret_cast<volatile uint32_t*>(peers.slab[p] + flags_off) + rank;
    *theirs = epoch;
    __threadfence_system();
    volatile uint32_t* mine = reinterpret_cast<volatile uint32_t*>(peers.slab[rank] + flags_off) + p;
    bool seen = false;
    for (uint32_t i = 0; i < polls && !seen; i++) {
        seen = (int32_t)(*mine - epoch) >= 0;
        if (!seen) __nanosleep(100);
    }
    if (!seen) atomicOr(error_word, 1u);
    __threadfence_system();
}

// ---- owner: dense picks / weights for all world*cap slots (-1 / 0 beyond each source's count)
// back_rows[slot]: where the owner's partial row of that slot belongs -- in the source rank's slab (null for unused slots):
// an owner that stores its result rows through this table needs no give-back pass.
__global__ void ep_prepare_kernel(const int32_t* __restrict__ meta, const int32_t* __restrict__ counts, int cap, int k, int64_t n_slots,
                                  int32_t* __restrict__ sel, float* __restrict__ w, PeerTable peers, size_t back_off, int rank, int64_t H,
                                  uint8_t** __restrict__ back_rows) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_slots * k) return;
    const int64_t slot = i / k;
    const int j = (int)(i - slot * k);
    const int s = (int)(slot / cap), r = (int)(slot - (int64_t)s * cap);
    const bool valid = r < counts[s];
    sel[i] = valid ? meta[slot * 2 * k + j] : -1;
    w[i] = valid ? __int_as_float(meta[slot * 2 * k + k + j]) : 0.0f;
    if (j == 0) back_rows[slot] = valid ? peers.slab[s] + back_off + ((size_t)rank * cap + r) * (size_t)H * 2 : nullptr;
}

// ---- owner: partial rows back to their sources
__global__ void __launch_bounds__(kRowThreads)
ep_give_back_kernel(const __nv_bfloat16* __restrict__ part, const int32_t* __restrict__ counts, int cap, int64_t H, int rank, int world,
                    PeerTable peers, size_t back_off) {
    // a fixed grid walks the rows that were actually received: block b takes rows b, b + grid, ... of every source
    const int n16 = (int)(H >> 3);
    for (int s = 0; s < world; s++) {
        const int n = counts[s];
        for (int r = blockIdx.x; r < n; r += gridDim.x) {
            const uint4* src = reinterpret_cast<const uint4*>(part + ((int64_t)s * cap + r) * H);
            uint4* dst = reinterpret_cast<uint4*>(peers.slab[s] + back_off) + ((int64_t)rank * cap + r) * n16;
            for (int c = threadIdx.x; c < n16; c += kRowThreads) dst[c] = __ldg(src + c);
        }
    }
}

// ---- source: out = shared + partials in rank order (f32), one thread per 8 columns
__global__ void __launch_bounds__(256)
ep_sum_kernel(const __nv_bfloat16* __restrict__ shared, const __nv_bfloat16* __restrict__ back, const int32_t* __restrict__ slot_of, int T,
              int64_t H, int cap, int world, __nv_bfloat16* __restrict__ out) {
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n16 = H >> 3;
    if (gid >= (int64_t)T * n16) return;
    const int64_t t = gid / n16, c = gid - t * n16;
    float acc[8];
    auto unpack = [](const uint4& v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    };
    if (shared != nullptr) unpack(*(reinterpret_cast<const uint4*>(shared + t * H) + c), acc);
    else
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = 0.0f;
    for (int d = 0; d < world; d++) {
        const int slot = slot_of[(int64_t)d * cap + t];
        if (slot < 0) continue;
        float f[8];
        unpack(__ldcg(reinterpret_cast<const uint4*>(back + ((int64_t)d * cap + slot) * H) + c), f);
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = __fadd_rn(acc[i], f[i]);
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        ow[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *(reinterpret_cast<uint4*>(out + t * H) + c) = o;
}

}  // namespace
}  // namespace dsx

using namespace dsx;

struct dsx_ep_comm {
    int world = 0, rank = 0, k = 0;
    int64_t cap = 0, H = 0;
    SlabLayout lay{};
    uint8_t* slab = nullptr;           // this rank's slab (cudaMalloc)
    PeerTable peers{};                 // every rank's slab as mapped here
    bool opened[kMaxWorld] = {};       // mapped through IPC (to close)
    int32_t* slot_of = nullptr;        // [world][cap]
    int32_t* sel = nullptr;            // [world*cap][k]
    float* w = nullptr;                // [world*cap][k]
    uint8_t** back_rows = nullptr;     // [world*cap]: destination of every slot's partial row in its source's slab (null: unused slot)
    uint32_t* error_word = nullptr;
    uint32_t epoch = 0;
    uint32_t barrier_polls = kBarrierPolls;   // polls (>= 100 ns each) before a barrier gives up
    bool connected = false;
};

extern "C" {

int dsx_ep_create(int world, int rank, int64_t cap, int64_t hidden, int n_used, dsx_ep_comm** out) {
    DSX_REQUIRE(out, "ep_create: null output");
    DSX_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "ep_create: rank %d of %d (at most %d ranks)", rank, world, kMaxWorld);
    DSX_REQUIRE(cap >= 1 && cap <= 32 * kScanThreads, "ep_create: %lld tokens per rank (at most %d)", (long long)cap, 32 * kScanThreads);
    DSX_REQUIRE(hidden >= 8 && hidden % 8 == 0 && n_used >= 1 && 2 * n_used <= kRowThreads, "ep_create: hidden %lld / n_used %d not supported",
                (long long)hidden, n_used);
    dsx_ep_comm* c = new dsx_ep_comm();
    c->world = world; c->rank = rank; c->k = n_used; c->cap = cap; c->H = hidden;
    c->lay = slab_layout(world, cap, hidden, n_used);
    cudaError_t e = cudaMalloc((void**)&c->slab, c->lay.total);
    if (e == cudaSuccess) e = cudaMemset(c->slab, 0, c->lay.total);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->slot_of, (size_t)world * cap * 4);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->sel, (size_t)world * cap * n_used * 4);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->w, (size_t)world * cap * n_used * 4);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->back_rows, (size_t)world * cap * sizeof(uint8_t*));
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->error_word, 256);
    if (e == cudaSuccess) e = cudaMemset(c->error_word, 0, 256);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(c->slab); cudaFree(c->slot_of); cudaFree(c->sel); cudaFree(c->w); cudaFree(c->back_rows); cudaFree(c->error_word);
        delete c;
        return set_error((int)e, "ep_create: allocation of %zu bytes failed: %s", slab_layout(world, cap, hidden, n_used).total, cudaGetErrorString(e));
    }
    c->peers.slab[rank] = c->slab;
    *out = c;
    return DSX_OK;
}

int dsx_ep_destroy(dsx_ep_comm* c) {
    if (!c) return DSX_OK;
    cudaDeviceSynchronize();
    for (int p = 0; p < c->world; p++)
        if (c->opened[p]) cudaIpcCloseMemHandle(c->peers.slab[p]);
    cudaFree(c->slab); cudaFree(c->slot_of); cudaFree(c->sel); cudaFree(c->w); cudaFree(c->back_rows); cudaFree(c->error_word);
    delete c;
    return DSX_OK;
}

// 64-byte handle of this rank's slab, to hand to the peers (they pass all of them to dsx_ep_connect).
int dsx_ep_export(dsx_ep_comm* c, uint8_t* handle64) {
    DSX_REQUIRE(c && handle64, "ep_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    DSX_CUDA(cudaIpcGetMemHandle(&h, c->slab));
    std::memcpy(handle64, &h, 64);
    return DSX_OK;
}

// handles: world x 64 bytes, in rank order (the own entry is ignored).  Ranks are processes on one node.
int dsx_ep_connect(dsx_ep_comm* c, const uint8_t* handles) {
    DSX_REQUIRE(c && handles, "ep_connect: null argument");
    DSX_REQUIRE(!c->connected, "ep_connect: already connected");
    for (int p = 0; p < c->world; p++) {
        if (p == c->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + (size_t)p * 64, 64);
        void* ptr = nullptr;
        DSX_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        c->peers.slab[p] = (uint8_t*)ptr;
        c->opened[p] = true;
    }
    c->connected = true;
    return DSX_OK;
}

// Several ranks inside one process on one device (tests): the peers' slabs are plain pointers.  The caller
// then runs every rank's phase before the next phase and leaves the barriers out.
int dsx_ep_connect_local(dsx_ep_comm* c, dsx_ep_comm* const* ranks) {
    DSX_REQUIRE(c && ranks, "ep_connect_local: null argument");
    for (int p = 0; p < c->world; p++) {
        DSX_REQUIRE(ranks[p] && ranks[p]->world == c->world && ranks[p]->cap == c->cap && ranks[p]->H == c->H && ranks[p]->k == c->k,
                    "ep_connect_local: rank %d does not match", p);
        c->peers.slab[p] = ranks[p]->slab;
    }
    c->connected = true;
    return DSX_OK;
}

int dsx_ep_dispatch(dsx_ep_comm* c, const void* x_bf16, const int32_t* selected, const float* weights, int64_t T, int n_expert,
                    dsx_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    DSX_REQUIRE(c, "ep_dispatch: null argument");
    DSX_REQUIRE(T == 0 || (x_bf16 && selected && weights), "ep_dispatch: null argument");
    DSX_REQUIRE(c->connected || c->world == 1, "ep_dispatch: not connected");
    DSX_REQUIRE(T >= 0 && T <= c->cap, "ep_dispatch: %lld tokens, capacity %lld", (long long)T, (long long)c->cap);
    DSX_REQUIRE(n_expert > 0 && n_expert % c->world == 0, "ep_dispatch: %d experts over %d ranks", n_expert, c->world);
    DSX_REQUIRE(((uintptr_t)x_bf16 & 15) == 0, "ep_dispatch: token rows must be 16-byte aligned");
    ep_scan_kernel<<<c->world, kScanThreads, 0, stream>>>(selected, (int)T, c->k, n_expert / c->world, (int)c->cap, c->slot_of, c->peers,
                                                          c->lay.counts, c->rank);
    DSX_LAUNCHED();
    if (T > 0) {
        ep_send_kernel<<<(unsigned)T, kRowThreads, 0, stream>>>((const __nv_bfloat16*)x_bf16, selected, weights, (int)T, c->k, c->H, (int)c->cap,
                                                                c->world, c->rank, c->slot_of, c->peers, c->lay.recv_x, c->lay.recv_meta);
        DSX_LAUNCHED();
    }
    return DSX_OK;
}

int dsx_ep_set_barrier_polls(dsx_ep_comm* c, uint32_t polls) {
    DSX_REQUIRE(c && polls >= 1, "ep_set_barrier_polls: bad argument");
    c->barrier_polls = polls;
    return DSX_OK;
}

int dsx_ep_barrier(dsx_ep_comm* c, dsx_stream_t stream_) {
    DSX_REQUIRE(c && c->connected, "ep_barrier: not connected");
    c->epoch++;
    ep_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream_>>>(c->peers, c->lay.flags, c->world, c->rank, c->epoch, c->barrier_polls,
                                                            c->error_word);
    DSX_LAUNCHED();
    return DSX_OK;
}

// After the barrier that follows the dispatches: picks and weights of all world*cap slots.
// Outputs: the received rows [world*cap, hidden] bf16, picks [world*cap, k] (-1 in unused slots), weights.
int dsx_ep_prepare(dsx_ep_comm* c, const void** x_rows, const int32_t** selected, const float** weights, int64_t* n_slots,
                   dsx_stream_t stream_) {
    DSX_REQUIRE(c, "ep_prepare: null argument");
    const int64_t slots = (int64_t)c->world * c->cap;
    const int64_t n = slots * c->k;
    ep_prepare_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream_>>>(
        reinterpret_cast<const int32_t*>(c->slab + c->lay.recv_meta), reinterpret_cast<const int32_t*>(c->slab + c->lay.counts), (int)c->cap,
        c->k, slots, c->sel, c->w, c->peers, c->lay.back, c->rank, c->H, c->back_rows);
    DSX_LAUNCHED();
    if (x_rows) *x_rows = c->slab + c->lay.recv_x;
    if (selected) *selected = c->sel;
    if (weights) *weights = c->w;
    if (n_slots) *n_slots = slots;
    return DSX_OK;
}

// After dsx_ep_prepare: [world*cap] row pointers, entry i = where slot i's partial row belongs in its source rank's slab (null
// for an unused slot).  An owner that writes its result rows through this table (dsx_moe_layer_forward_picks_to) has given
// them back already and skips dsx_ep_give_back.
int dsx_ep_back_rows(dsx_ep_comm* c, void* const** rows) {
    DSX_REQUIRE(c && rows, "ep_back_rows: null argument");
    *rows = reinterpret_cast<void* const*>(c->back_rows);
    return DSX_OK;
}

// partial_rows: [world*cap, hidden] bf16, row i the weighted sum of slot i's owned picks.
int dsx_ep_give_back(dsx_ep_comm* c, const void* partial_rows_bf16, dsx_stream_t stream_) {
    DSX_REQUIRE(c && partial_rows_bf16, "ep_give_back: null argument");
    DSX_REQUIRE(((uintptr_t)partial_rows_bf16 & 15) == 0, "ep_give_back: rows must be 16-byte aligned");
    const unsigned blocks = (unsigned)std::min<int64_t>(c->cap, 148 * 8);
    ep_give_back_kernel<<<blocks, kRowThreads, 0, (cudaStream_t)stream_>>>(
        (const __nv_bfloat16*)partial_rows_bf16, reinterpret_cast<const int32_t*>(c->slab + c->lay.counts), (int)c->cap, c->H, c->rank, c->world,
        c->peers, c->lay.back);
    DSX_LAUNCHED();
    return DSX_OK;
}

// After the barrier that follows give_back: out[t] = shared[t] + partials of token t in rank order.
int dsx_ep_sum(dsx_ep_comm* c, const void* shared_bf16, int64_t T, void* out_bf16, dsx_stream_t stream_) {
    DSX_REQUIRE(c && out_bf16, "ep_sum: null argument");
    DSX_REQUIRE(T >= 0 && T <= c->cap, "ep_sum: %lld tokens, capacity %lld", (long long)T, (long long)c->cap);
    if (T == 0) return DSX_OK;
    const int64_t n = T * (c->H >> 3);
    ep_sum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream_>>>(
        (const __nv_bfloat16*)shared_bf16, reinterpret_cast<const __nv_bfloat16*>(c->slab + c->lay.back), c->slot_of, (int)T, c->H, (int)c->cap,
        c->world, (__nv_bfloat16*)out_bf16);
    DSX_LAUNCHED();
    return DSX_OK;
}

// Rows sent by every source this step (device array of `world` ints, valid after the first barrier).
int dsx_ep_counts(dsx_ep_comm* c, const int32_t** counts) {
    DSX_REQUIRE(c && counts, "ep_counts: null argument");
    *counts = reinterpret_cast<const int32_t*>(c->slab + c->lay.counts);
    return DSX_OK;
}

// Reads (and clears) the error word: bit 1 = a barrier gave up waiting.  Synchronises the stream.
int dsx_ep_check(dsx_ep_comm* c, dsx_stream_t stream_, uint32_t* error_word) {
    DSX_REQUIRE(c, "ep_check: null argument");
    uint32_t w = 0;
    DSX_CUDA(cudaMemcpyAsync(&w, c->error_word, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream_));
    DSX_CUDA(cudaStreamSynchronize((cudaStream_t)stream_));
    if (w) DSX_CUDA(cudaMemsetAsync(c->error_word, 0, 4, (cudaStream_t)stream_));
    if (error_word) *error_word = w;
    if (w) return set_error(DSX_ERR_DEVICE, "an exchange kernel reported error word 0x%x (a bounded wait ran out)", w);
    return DSX_OK;
}

}  // extern "C"
