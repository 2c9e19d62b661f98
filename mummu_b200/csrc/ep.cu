// Expert-parallel exchange over peer memory (NVLink / NVSwitch): no host synchronisation, no
// staging copies, no library collective inside a step.  The reference has no collective for this
// path (its devices exchange through host memory: crates/mummu/src/backend.rs:128-143,
// nn/moe.rs:1219-1272).
//
// Every rank owns a contiguous block of experts, three peer-visible buffers and a private one:
//   recv_x [cap_rows, hidden]  rows routed to its experts, expert-major (sources in rank order)
//   back   [own_rows, hidden]  the expert outputs of ITS OWN (token, slot) pairs, in its sorted order
//   sync   flags, epochs and the gathered per-expert row counts (layout below)
//   ys     [cap_rows, hidden]  its experts' outputs for the received rows (private)
// Both directions PUSH: remote traffic is stores only (a store needs no round trip; loads over
// NVLink were three times slower here for the same bytes).
//
// One layer on one rank is four stages, each signalling the next ONE WAY: the producer's last
// block stores its epoch into a flag in every peer's sync block (system-scope release), and the
// consumer polls its own flags (system-scope acquire) in the head of a later kernel.  No kernel
// both signals and waits, so the stages of several ranks may also be issued one after another on
// a single stream (rank 0's stage, rank 1's stage, ..., then the next stage): nothing then waits
// for a kernel that has not run.  That is how the exchange is tested on one GPU.
//
//   post     : counts of this rank's rows per global expert -> counts_in[rank] of every rank; S1
//   dispatch : wait S1; plan from the gathered counts (where each sorted row lives in its owner's
//              buffers; rows, offsets and work order of the local experts); rows -> owners' recv_x
//              with 16-byte peer stores; S2
//   experts  : wait S2; the local experts over recv_x -> ys; every output row -> its source rank's
//              `back` buffer at the row's place in the source's sorted order, 16-byte peer stores; S3
//   combine  : wait S3; per token, ascending expert id, scaled = w * y; out += scaled, y read from
//              the own `back` buffer
// Plain peer loads and stores only.  Every wait is bounded: when it runs out the kernel raises
// the status word, skips its data movement and returns.
#include <cstring>

#include "common.cuh"

namespace mummu {

constexpr int EP_MAX_RANKS = 16;

struct PeerTable {
    void* ptr[EP_MAX_RANKS];
};

// sync block, 32-bit words (zeroed by its owner before the peers map it):
//   [0..3)    epoch of the owner's last signal per channel        (owner only)
//   [4..7)    epoch the owner last waited for per channel         (owner only)
//   [8..12)   arrival counters of multi-block kernels             (owner only)
//   [16 + 16*ch + s]  flag: last epoch rank s signalled to this rank on channel ch
//   [64 + s*E + e]    counts_in: rank s's rows for global expert e, this layer
// Epochs only grow; every rank issues the same sequence of stages, so "the next epoch" is the
// same number everywhere.
constexpr int EP_W_SIG = 0, EP_W_WAIT = 4, EP_W_DONE = 8, EP_W_FLAGS = 16, EP_W_COUNTS = 64;
constexpr int EP_CH_COUNTS = 0, EP_CH_ROWS = 1, EP_CH_OUT = 2;
constexpr uint32_t EP_WAIT_POLLS_DEFAULT = 1u << 24;   // x (0.2 us sleep + a load): a few seconds

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One warp of one block per kernel: everything this grid wrote before is visible to a rank that
// sees the new epoch.
__device__ void ep_signal(const PeerTable& sync, int rank, int world, int ch) {
    const int lane = threadIdx.x & 31;
    int32_t* own = reinterpret_cast<int32_t*>(sync.ptr[rank]);
    int32_t epoch = 0;
    if (lane == 0) {
        epoch = own[EP_W_SIG + ch] + 1;
        own[EP_W_SIG + ch] = epoch;
    }
    epoch = __shfl_sync(0xFFFFFFFFu, epoch, 0);
    __threadfence_system();
    if (lane < world) st_release_sys(reinterpret_cast<int32_t*>(sync.ptr[lane]) + EP_W_FLAGS + 16 * ch + rank, epoch);
}

// Threads 0..world-1 of a block poll this rank's own flags of channel ch until every rank has
// signalled the next epoch.  Returns false (and raises the status word) when the polls run out.
// Uniform over the block: ends with a block barrier.
__device__ bool ep_wait(const PeerTable& sync, int rank, int world, int ch, uint32_t limit, int32_t* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const int32_t* own = reinterpret_cast<const int32_t*>(sync.ptr[rank]);
        const int32_t target = *reinterpret_cast<const volatile int32_t*>(own + EP_W_WAIT + ch) + 1;
        const int32_t* flag = own + EP_W_FLAGS + 16 * ch + threadIdx.x;
        uint32_t polls = 0;
        while (ld_acquire_sys(flag) - target < 0) {
            if (++polls > 64) __nanosleep(200);
            if (polls > limit) {
                atomicOr(status, STATUS_TIMEOUT);
                s_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    __threadfence_system();
    return s_ok != 0;
}

// Arrival of one block of a multi-block kernel (call with the whole block, after the block's last
// global access).  Returns true in the block that arrived last, with the counter reset.
__device__ bool ep_last_block(int32_t* counter) {
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(counter, 1);
        s_last = (done == (int)(gridDim.x * gridDim.y) - 1);
        if (s_last) *counter = 0;
    }
    __syncthreads();
    if (s_last) __threadfence_system();
    return s_last != 0;
}

// ---- post -----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_post_counts_kernel(const int32_t* counts, PeerTable sync, int world, int rank,
                                                             int E) {
    for (int idx = threadIdx.x; idx < world * E; idx += blockDim.x) {
        const int s = idx / E, e = idx - s * E;
        reinterpret_cast<int32_t*>(sync.ptr[s])[EP_W_COUNTS + rank * E + e] = counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < 32) ep_signal(sync, rank, world, EP_CH_COUNTS);
}

// One warp copies one row of `vec` 16-byte pieces; up to eight loads are issued before the first store.
__device__ __forceinline__ void copy_row(const uint4* __restrict__ src, uint4* __restrict__ dst, int vec, int lane) {
    for (int i0 = lane; i0 < vec; i0 += 256) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (i0 + 32 * u < vec) v[u] = src[i0 + 32 * u];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (i0 + 32 * u < vec) dst[i0 + 32 * u] = v[u];
    }
}

// ---- dispatch ----------------------------------------------------------------------------------
struct DispatchArgs {
    const uint4* x;               // [tokens, hidden] 16-bit
    const int32_t* row_token;     // sorted row -> token
    const int32_t* offsets;       // [E + 1] first sorted row per global expert (this rank's rows)
    PeerTable sync, recv;
    int world, rank, E, EL, vec_per_row;
    int64_t rows, cap_rows;
    int32_t* dst_base;            // out [E]: first row, in the owner's buffers, of this rank's rows per expert
    int32_t* local_counts;        // out [EL]: rows per local expert over all sources
    int32_t* local_offsets;       // out [EL + 1]
    int32_t* active;              // out [EL]: local experts with rows, heaviest first
    int32_t* n_active;            // out [1]
    int32_t* ret_seg;             // out [EL * world + 1]: first local row of segment (local expert, source)
    int32_t* ret_dst;             // out [EL * world]: that segment's first row in the source's sorted order
    uint32_t wait_polls;
    int32_t* status;
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(DispatchArgs a) {
    extern __shared__ int32_t s_dyn[];
    int32_t* all_counts = s_dyn;                       // [world][E]
    int32_t* s_base = all_counts + a.world * a.E;      // [E]
    int32_t* s_lc = s_base + a.E;                      // [EL]
    int32_t* own = reinterpret_cast<int32_t*>(a.sync.ptr[a.rank]);
    const bool ok = ep_wait(a.sync, a.rank, a.world, EP_CH_COUNTS, a.wait_polls, a.status);
    if (ok) {
        const volatile int32_t* src = own + EP_W_COUNTS;
        for (int i = threadIdx.x; i < a.world * a.E; i += blockDim.x) all_counts[i] = src[i];
        __syncthreads();
        // buffers are expert-major with the sources in rank order inside an expert
        for (int le = threadIdx.x; le < a.EL; le += blockDim.x) {
            int c = 0;
            for (int s = 0; s < a.world; ++s) c += all_counts[s * a.E + a.rank * a.EL + le];
            s_lc[le] = c;
        }
        for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
            const int d = e / a.EL, le = e - d * a.EL;
            int base = 0;
            for (int l2 = 0; l2 < le; ++l2)
                for (int s = 0; s < a.world; ++s) base += all_counts[s * a.E + d * a.EL + l2];
            for (int s = 0; s < a.rank; ++s) base += all_counts[s * a.E + e];
            s_base[e] = base;
        }
        __syncthreads();
        if (blockIdx.x == 0) {
            for (int e = threadIdx.x; e < a.E; e += blockDim.x) a.dst_base[e] = s_base[e];
            // what the expert kernels need: rows, first row and work order (most rows first, then
            // lower id) of the local experts
            for (int le = threadIdx.x; le < a.EL; le += blockDim.x) {
                const int c = s_lc[le];
                int off = 0, before = 0;
                for (int i = 0; i < a.EL; ++i) {
                    const int ci = s_lc[i];
                    if (i < le) off += ci;
                    before += (ci > c || (ci == c && i < le)) && ci > 0;
                }
                a.local_counts[le] = c;
                a.local_offsets[le] = off;
                if (c > 0) a.active[before] = le;
                if (le == a.EL - 1) a.local_offsets[a.EL] = off + c;
            }
            if (threadIdx.x == 0) {
                int nz = 0;
                for (int i = 0; i < a.EL; ++i) nz += s_lc[i] > 0;
                *a.n_active = nz;
            }
            // the way back: local rows as segments (local expert, source rank), and where a
            // segment starts in its source's sorted order (the source's rows of earlier experts)
            for (int g = threadIdx.x; g < a.EL * a.world; g += blockDim.x) {
                const int le = g / a.world, s = g - le * a.world, e = a.rank * a.EL + le;
                int first = 0;
                for (int i = 0; i < le; ++i) first += s_lc[i];
                for (int s2 = 0; s2 < s; ++s2) first += all_counts[s2 * a.E + e];
                int before = 0;
                for (int e2 = 0; e2 < e; ++e2) before += all_counts[s * a.E + e2];
                a.ret_seg[g] = first;
                a.ret_dst[g] = before;
                if (g == a.EL * a.world - 1) a.ret_seg[g + 1] = first + all_counts[s * a.E + e];
            }
        }
        // a warp per row: the row's expert from the offsets (shared memory), then the row in
        // 16-byte pieces, eight in flight per lane
        int32_t* s_off = s_lc + a.EL;                            // [E + 1]
        for (int e = threadIdx.x; e <= a.E; e += blockDim.x) s_off[e] = a.offsets[e];
        __syncthreads();
        const int lane = threadIdx.x & 31;
        const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
        // Every rank walks its sorted rows starting at the rows of the NEXT rank's experts: at any
        // moment the ranks then write to different destinations instead of all to the same one
        // (whose ingress would carry the whole group's traffic while the other links idle).
        const int64_t rot = s_off[((a.rank + 1) % a.world) * a.EL];
        for (int64_t q = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); q < a.rows; q += warps) {
            const int64_t p = q + rot < a.rows ? q + rot : q + rot - a.rows;
            int lo = 0, hi = a.E;                                // last e with offsets[e] <= p
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (s_off[mid] <= p) lo = mid; else hi = mid;
            }
            const int e = lo;
            const int64_t drow = (int64_t)s_base[e] + (p - s_off[e]);
            if (drow >= 0 && drow < a.cap_rows) {
                const uint4* src = a.x + (size_t)a.row_token[p] * a.vec_per_row;
                uint4* dst = reinterpret_cast<uint4*>(a.recv.ptr[e / a.EL]) + (size_t)drow * a.vec_per_row;
                copy_row(src, dst, a.vec_per_row, lane);
            } else if (lane == 0) {
                atomicOr(a.status, STATUS_BOUNDS);               // the owner's buffer is too small: row dropped
            }
        }
    }
    if (ep_last_block(own + EP_W_DONE + 0)) {
        if (threadIdx.x == 0) own[EP_W_WAIT + EP_CH_COUNTS] += 1;
        if (ok && threadIdx.x < 32) ep_signal(a.sync, a.rank, a.world, EP_CH_ROWS);
    }
}

// ---- experts: a wait before, a signal after ----------------------------------------------------
__global__ void __launch_bounds__(32) ep_wait_kernel(PeerTable sync, int rank, int world, int ch, uint32_t wait_polls,
                                                     int32_t* status) {
    ep_wait(sync, rank, world, ch, wait_polls, status);
    if (threadIdx.x == 0) reinterpret_cast<int32_t*>(sync.ptr[rank])[EP_W_WAIT + ch] += 1;
}

__global__ void __launch_bounds__(32) ep_signal_kernel(PeerTable sync, int rank, int world, int ch) {
    ep_signal(sync, rank, world, ch);
}

// ---- return: expert outputs -> the ranks their tokens live on ----------------------------------
__global__ void __launch_bounds__(256) ep_return_kernel(const uint4* ys, PeerTable sync, PeerTable back, const int32_t* ret_seg,
                                                        const int32_t* ret_dst, int rank, int world, int EL,
                                                        int vec_per_row, int64_t ys_rows, int64_t back_rows, int32_t* status) {
    extern __shared__ int32_t s_dyn[];
    const int nseg = EL * world;
    int32_t* s_seg = s_dyn;                                      // [nseg + 1]
    int32_t* s_dst = s_seg + nseg + 1;                           // [nseg]
    for (int g = threadIdx.x; g <= nseg; g += blockDim.x) s_seg[g] = ret_seg[g];
    for (int g = threadIdx.x; g < nseg; g += blockDim.x) s_dst[g] = ret_dst[g];
    __syncthreads();
    const int64_t rows = min((int64_t)s_seg[nseg], ys_rows);
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        int lo = 0, hi = nseg;                                   // last segment that starts at or before r
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_seg[mid] <= r) lo = mid; else hi = mid;
        }
        const int s = lo % world;
        const int64_t drow = (int64_t)s_dst[lo] + (r - s_seg[lo]);
        if (drow >= 0 && drow < back_rows) {
            copy_row(ys + (size_t)r * vec_per_row, reinterpret_cast<uint4*>(back.ptr[s]) + (size_t)drow * vec_per_row,
                     vec_per_row, lane);
        } else if (lane == 0) {
            atomicOr(status, STATUS_BOUNDS);
        }
    }
    int32_t* own = reinterpret_cast<int32_t*>(sync.ptr[rank]);
    if (ep_last_block(own + EP_W_DONE + 2) && threadIdx.x < 32) ep_signal(sync, rank, world, EP_CH_OUT);
}

// ---- small-batch form: every rank gets every token ----------------------------------------------
// With few tokens per rank the three hops above (counts, rows, outputs) cost more than the rows
// they move.  Here every rank pushes its tokens to every rank (hop 1), routes ALL tokens itself -
// the router is replicated and bit-reproducible, so every rank computes the same plan and no
// counts are exchanged - runs its own experts on the rows the plan gives them, read in place
// from the gathered tokens, and pushes each output row to the rank its token lives on, at the
// row's position in the common sorted order (hop 2).
__global__ void __launch_bounds__(256) ep_gather_tokens_kernel(const uint4* x, PeerTable sync, PeerTable gx, int rank, int world,
                                                               int tokens, int vec_per_row) {
    const int lane = threadIdx.x & 31;
    const int64_t items = (int64_t)world * tokens;               // (destination rank, token)
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t it = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); it < items; it += warps) {
        // destinations in a different order on every rank, starting with the next one (no rank is
        // everybody's first target)
        const int dq = (int)(it / tokens), t = (int)(it - (int64_t)dq * tokens);
        const int d = (dq + rank + 1) % world;
        copy_row(x + (size_t)t * vec_per_row,
                 reinterpret_cast<uint4*>(gx.ptr[d]) + ((size_t)rank * tokens + t) * vec_per_row, vec_per_row, lane);
    }
    int32_t* own = reinterpret_cast<int32_t*>(sync.ptr[rank]);
    if (ep_last_block(own + EP_W_DONE + 0) && threadIdx.x < 32) ep_signal(sync, rank, world, EP_CH_COUNTS);
}

// local experts' view of the common plan: rows, first sorted row (absolute) and work order
__global__ void __launch_bounds__(256) ep_local_plan_kernel(const int32_t* counts, const int32_t* offsets, int first, int EL,
                                                            int32_t* l_counts, int32_t* l_offsets, int32_t* active,
                                                            int32_t* n_active) {
    extern __shared__ int32_t s_dyn[];
    for (int le = threadIdx.x; le < EL; le += blockDim.x) s_dyn[le] = counts[first + le];
    __syncthreads();
    for (int le = threadIdx.x; le < EL; le += blockDim.x) {
        const int c = s_dyn[le];
        int before = 0;
        for (int i = 0; i < EL; ++i) before += (s_dyn[i] > c || (s_dyn[i] == c && i < le)) && s_dyn[i] > 0;
        l_counts[le] = c;
        l_offsets[le] = offsets[first + le];
        if (c > 0) active[before] = le;
        if (le == EL - 1) l_offsets[EL] = offsets[first + le] + c;
    }
    if (threadIdx.x == 0) {
        int nz = 0;
        for (int i = 0; i < EL; ++i) nz += s_dyn[i] > 0;
        *n_active = nz;
    }
}

// expert outputs (f32, sorted order) of this rank's experts -> f16 rows in the buffer of the rank
// each row's token lives on, at the same sorted position
__global__ void __launch_bounds__(256) ep_return_gathered_kernel(const float* ys, const int32_t* row_token, const int32_t* l_offsets,
                                                                 int EL, PeerTable sync, PeerTable back, int rank, int world,
                                                                 int tokens_per_rank, int H, int64_t ys_rows, int64_t back_rows,
                                                                 int32_t* status) {
    const int lane = threadIdx.x & 31;
    const int64_t p0 = l_offsets[0], p1 = min((int64_t)l_offsets[EL], ys_rows);
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t p = p0 + (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < p1; p += warps) {
        const int d = row_token[p] / tokens_per_rank;
        if (d < 0 || d >= world || p >= back_rows) {
            if (lane == 0) atomicOr(status, STATUS_BOUNDS);
            continue;
        }
        const float* src = ys + (size_t)p * H;
        __half* dst = reinterpret_cast<__half*>(back.ptr[d]) + (size_t)p * H;
        for (int h = lane * 8; h < H; h += 256) {
            const float4 a = *reinterpret_cast<const float4*>(src + h), b = *reinterpret_cast<const float4*>(src + h + 4);
            uint4 o;
            __half2 t0 = __floats2half2_rn(a.x, a.y), t1 = __floats2half2_rn(a.z, a.w);
            __half2 t2 = __floats2half2_rn(b.x, b.y), t3 = __floats2half2_rn(b.z, b.w);
            o.x = *reinterpret_cast<uint32_t*>(&t0);
            o.y = *reinterpret_cast<uint32_t*>(&t1);
            o.z = *reinterpret_cast<uint32_t*>(&t2);
            o.w = *reinterpret_cast<uint32_t*>(&t3);
            *reinterpret_cast<uint4*>(dst + h) = o;
        }
    }
    int32_t* own = reinterpret_cast<int32_t*>(sync.ptr[rank]);
    if (ep_last_block(own + EP_W_DONE + 2) && threadIdx.x < 32) ep_signal(sync, rank, world, EP_CH_OUT);
}

// Placement: a routed expert id becomes the id of the bank slot that serves it for this rank's
// tokens.  An id outside the router's experts, or a table entry outside the slots, is reported
// (STATUS_BOUNDS) and sent to slot 0 so that nothing later indexes past a buffer.
__global__ void ep_place_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ table, int experts_real,
                                int slots, int64_t n, int32_t* __restrict__ out, int32_t* status) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = ids[i];
    int v = (e >= 0 && e < experts_real) ? table[e] : -1;
    if (v < 0 || v >= slots) {
        atomicOr(status, STATUS_BOUNDS);
        v = 0;
    }
    out[i] = v;
}

}  // namespace mummu

using namespace mummu;

extern "C" {

int32_t mummu_ep_alloc(int32_t device, size_t bytes, void** ptr, uint8_t* handle64) {
    MUMMU_REQUIRE(ptr && handle64 && bytes > 0, "mummu_ep_alloc: bad argument");
    int prev = -1;
    MUMMU_CUDA_TRY(cudaGetDevice(&prev));
    if (prev != device) MUMMU_CUDA_TRY(cudaSetDevice(device));
    cudaError_t err = cudaMalloc(ptr, bytes);
    if (err == cudaSuccess) err = cudaMemset(*ptr, 0, bytes);
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, *ptr);
    if (prev != device) cudaSetDevice(prev);
    if (err != cudaSuccess) {
        set_error("mummu_ep_alloc: %s", cudaGetErrorString(err));
        return MUMMU_ERR_DEVICE;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    return MUMMU_OK;
}

int32_t mummu_ep_open(int32_t device, const uint8_t* handle64, void** ptr) {
    MUMMU_REQUIRE(ptr && handle64, "mummu_ep_open: bad argument");
    int prev = -1;
    MUMMU_CUDA_TRY(cudaGetDevice(&prev));
    if (prev != device) MUMMU_CUDA_TRY(cudaSetDevice(device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t err = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (prev != device) cudaSetDevice(prev);
    if (err != cudaSuccess) {
        set_error("mummu_ep_open: %s", cudaGetErrorString(err));
        return MUMMU_ERR_DEVICE;
    }
    return MUMMU_OK;
}

int32_t mummu_ep_close(void* ptr) {
    if (ptr) MUMMU_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return MUMMU_OK;
}

int32_t mummu_ep_free(void* ptr) {
    if (ptr) MUMMU_CUDA_TRY(cudaFree(ptr));
    return MUMMU_OK;
}

size_t mummu_ep_sync_bytes(int32_t world, int32_t experts) {
    return (size_t)(EP_W_COUNTS + (size_t)world * experts) * 4;
}

int32_t mummu_ep_reset(int32_t device, void* own_sync, int32_t world, int32_t experts) {
    MUMMU_REQUIRE(own_sync && world >= 1 && experts >= 1, "mummu_ep_reset: bad argument");
    int prev = -1;
    MUMMU_CUDA_TRY(cudaGetDevice(&prev));
    if (prev != device) MUMMU_CUDA_TRY(cudaSetDevice(device));
    cudaError_t err = cudaDeviceSynchronize();
    if (err == cudaSuccess) err = cudaMemset(own_sync, 0, mummu_ep_sync_bytes(world, experts));
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (prev != device) cudaSetDevice(prev);
    if (err != cudaSuccess) {
        set_error("mummu_ep_reset: %s", cudaGetErrorString(err));
        return MUMMU_ERR_DEVICE;
    }
    return MUMMU_OK;
}

static int ep_check_ranks(MummuMoe* m, int32_t rank, int32_t world, const char* who) {
    MUMMU_REQUIRE(world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world &&
                      m->cfg.experts % world == 0 && m->cfg.experts_local == m->cfg.experts / world &&
                      m->cfg.expert_first == rank * m->cfg.experts_local,
                  "%s: rank %d of %d with local experts [%d, %d) of %d", who, rank, world, m->cfg.expert_first,
                  m->cfg.expert_first + m->cfg.experts_local, m->cfg.experts);
    return MUMMU_OK;
}

static PeerTable peer_table(void* const* ptrs, int world) {
    PeerTable t{};
    for (int i = 0; i < world; ++i) t.ptr[i] = ptrs[i];
    return t;
}

static uint32_t wait_polls_of(const MummuMoe* m) { return m->sw.wait_polls ? m->sw.wait_polls : EP_WAIT_POLLS_DEFAULT; }

int32_t mummu_ep_place(MummuMoe* m, const int32_t* ids, const int32_t* table, int32_t experts_real, int64_t n,
                       int32_t* ids_out, void* stream) {
    MUMMU_REQUIRE(m && ids && table && ids_out, "mummu_ep_place: null argument");
    MUMMU_REQUIRE(experts_real >= 1 && n >= 0, "mummu_ep_place: %d experts, %lld ids", experts_real, (long long)n);
    if (n == 0) return MUMMU_OK;
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    LaunchScope scope(m, s, "ep_place");
    ep_place_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(ids, table, experts_real, m->cfg.experts, n, ids_out, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_post_counts(MummuMoe* m, const int32_t* counts, void* const* peer_sync, int32_t rank,
                             int32_t world, void* stream) {
    MUMMU_REQUIRE(m && counts && peer_sync, "mummu_ep_post_counts: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_post_counts");
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    LaunchScope scope(m, s, "ep_post_counts");
    ep_post_counts_kernel<<<1, 256, 0, s>>>(counts, peer_table(peer_sync, world), world, rank, m->cfg.experts);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_dispatch(MummuMoe* m, const void* x, const int32_t* row_token, const int32_t* offsets,
                          void* const* peer_sync, void* const* peer_recv, int32_t rank, int32_t world,
                          int32_t rows, int64_t cap_rows, int32_t* dst_base, int32_t* local_counts, void* stream) {
    MUMMU_REQUIRE(m && x && row_token && offsets && peer_sync && peer_recv && dst_base && local_counts,
                  "mummu_ep_dispatch: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_dispatch");
    if (rc) return rc;
    MUMMU_REQUIRE(dtype_size(m->cfg.act_dtype) == 2 && m->cfg.hidden % 8 == 0,
                  "mummu_ep_dispatch: 16-bit activations with hidden %% 8 == 0 only");
    MUMMU_REQUIRE(rows >= 0 && cap_rows >= 0, "mummu_ep_dispatch: rows %d, cap_rows %lld", rows, (long long)cap_rows);
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    DispatchArgs a{};
    a.x = (const uint4*)x;
    a.row_token = row_token;
    a.offsets = offsets;
    a.sync = peer_table(peer_sync, world);
    a.recv = peer_table(peer_recv, world);
    a.world = world;
    a.rank = rank;
    a.E = m->cfg.experts;
    a.EL = m->cfg.experts_local;
    a.vec_per_row = m->cfg.hidden * 2 / 16;
    a.rows = rows;
    a.cap_rows = cap_rows;
    a.dst_base = dst_base;
    a.local_counts = local_counts;
    a.local_offsets = m->offsets;
    a.active = m->active;
    a.n_active = m->n_active;
    a.ret_seg = m->ret_seg;
    a.ret_dst = m->ret_dst;
    a.wait_polls = wait_polls_of(m);
    a.status = m->status;
    // even a rank without rows takes part: its block plans the local experts and signals
    const int64_t blocks = rows < 8 ? 1 : (rows / 8 < 148 * 8 ? rows / 8 : 148 * 8);     // a warp per row
    const size_t smem = ((size_t)world * a.E + a.E + a.EL + a.E + 1) * sizeof(int32_t);
    LaunchScope scope(m, s, "ep_dispatch");
    ep_dispatch_kernel<<<(unsigned)blocks, 256, smem, s>>>(a);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_experts(MummuMoe* m, void* const* peer_sync, void* const* peer_back, int32_t rank, int32_t world,
                         const void* recv_own, const int32_t* local_counts, int64_t rows_cap, void* ys_own,
                         int64_t back_rows, void* stream) {
    MUMMU_REQUIRE(m && peer_sync && peer_back && recv_own && local_counts && ys_own, "mummu_ep_experts: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_experts");
    if (rc) return rc;
    MUMMU_REQUIRE(rows_cap >= 0 && rows_cap <= INT32_MAX && back_rows >= 0, "mummu_ep_experts: rows_cap %lld, back_rows %lld",
                  (long long)rows_cap, (long long)back_rows);
    MUMMU_REQUIRE(dtype_size(m->cfg.act_dtype) == 2 && m->cfg.hidden % 8 == 0,
                  "mummu_ep_experts: 16-bit activations with hidden %% 8 == 0 only");
    cudaStream_t s;
    const PeerTable t = peer_table(peer_sync, world);
    {
        std::lock_guard<std::mutex> lock(m->mu);
        s = stream ? (cudaStream_t)stream : m->stream;
        LaunchScope scope(m, s, "ep_wait_rows");
        ep_wait_kernel<<<1, 32, 0, s>>>(t, rank, world, EP_CH_ROWS, wait_polls_of(m), m->status);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    // the dispatch stage left the local experts' offsets and work order in the handle; the down
    // projection is offered the peers' buffers and, where the tensor-core kernel runs, stores its
    // output rows there itself (the transfer then hides under the GEMM)
    m->scatter.offered = true;
    m->scatter.used = false;
    m->scatter.world = world;
    m->scatter.back_rows = back_rows;
    for (int r = 0; r < world; ++r) m->scatter.back[r] = peer_back[r];
    rc = mummu_moe_experts_planned(m, recv_own, local_counts, (int32_t)rows_cap, ys_own, s);
    m->scatter.offered = false;
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(m->mu);
    if (m->scatter.used) {
        LaunchScope scope(m, s, "ep_signal_out");
        ep_signal_kernel<<<1, 32, 0, s>>>(t, rank, world, EP_CH_OUT);
        MUMMU_CUDA_TRY(cudaGetLastError());
        return MUMMU_OK;
    }
    // even a rank whose experts got no rows takes part: its last block signals
    const int64_t blocks = rows_cap < 8 ? 1 : (rows_cap / 8 < 148 * 8 ? rows_cap / 8 : 148 * 8);
    const int nseg = m->cfg.experts_local * world;
    LaunchScope scope(m, s, "ep_return");
    ep_return_kernel<<<(unsigned)blocks, 256, (size_t)(2 * nseg + 1) * sizeof(int32_t), s>>>(
        (const uint4*)ys_own, t, peer_table(peer_back, world), m->ret_seg, m->ret_dst, rank, world, m->cfg.experts_local,
        m->cfg.hidden * 2 / 16, rows_cap, back_rows, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_gather_tokens(MummuMoe* m, const void* x, int32_t tokens, void* const* peer_sync, void* const* peer_gx,
                               int32_t rank, int32_t world, void* stream) {
    MUMMU_REQUIRE(m && peer_sync && peer_gx && (x || tokens == 0), "mummu_ep_gather_tokens: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_gather_tokens");
    if (rc) return rc;
    MUMMU_REQUIRE(dtype_size(m->cfg.act_dtype) == 2 && m->cfg.hidden % 8 == 0 && tokens >= 0,
                  "mummu_ep_gather_tokens: 16-bit activations with hidden %% 8 == 0 only");
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    const int64_t items = (int64_t)world * tokens;
    const int64_t blocks = items < 8 ? 1 : (items / 8 < 148 * 8 ? (items + 7) / 8 : 148 * 8);
    LaunchScope scope(m, s, "ep_gather_tokens");
    ep_gather_tokens_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint4*)x, peer_table(peer_sync, world),
                                                             peer_table(peer_gx, world), rank, world, tokens,
                                                             m->cfg.hidden * 2 / 16);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_wait(MummuMoe* m, void* const* peer_sync, int32_t rank, int32_t world, int32_t channel, void* stream) {
    MUMMU_REQUIRE(m && peer_sync && channel >= 0 && channel < 3, "mummu_ep_wait: bad argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_wait");
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    LaunchScope scope(m, s, "ep_wait");
    ep_wait_kernel<<<1, 32, 0, s>>>(peer_table(peer_sync, world), rank, world, channel, wait_polls_of(m), m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_experts_gathered(MummuMoe* m, void* const* peer_sync, void* const* peer_back, const void* gx_own,
                                  const int32_t* row_token, const int32_t* counts, const int32_t* offsets, int32_t rank,
                                  int32_t world, int32_t tokens_per_rank, int32_t top_k, int64_t back_rows, void* stream) {
    MUMMU_REQUIRE(m && peer_sync && peer_back && gx_own && row_token && counts && offsets,
                  "mummu_ep_experts_gathered: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_experts_gathered");
    if (rc) return rc;
    const MummuMoeConfig& c = m->cfg;
    const int64_t rows_total = (int64_t)world * tokens_per_rank * top_k;
    MUMMU_REQUIRE(tokens_per_rank >= 1 && top_k >= 1 && top_k <= c.top_k && back_rows >= 0,
                  "mummu_ep_experts_gathered: %d tokens per rank, top_k %d", tokens_per_rank, top_k);
    if (!(c.weight_dtype == MUMMU_Q4_K && c.act_dtype == MUMMU_F16 && c.hidden % 256 == 0 && c.inter % 256 == 0 &&
          c.hidden <= 8192 && c.inter <= 8192 && rows_total <= 8192 && (reinterpret_cast<uintptr_t>(gx_own) & 15) == 0)) {
        set_error("mummu_ep_experts_gathered: f16 activations on Q4_K experts, at most 8192 (token, slot) pairs over all ranks");
        return MUMMU_ERR_UNSUPPORTED;
    }
    MUMMU_REQUIRE(m->bank_set[0] && m->bank_set[1] && m->bank_set[2],
                  "MoE: expert banks were never set (mummu_moe_set_bank gate/up/down)");
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    if ((rc = ensure_scratch(m, (int64_t)world * tokens_per_rank))) return rc;
    const int EL = c.experts_local;
    {
        LaunchScope scope(m, s, "ep_local_plan");
        ep_local_plan_kernel<<<1, 256, (size_t)EL * sizeof(int32_t), s>>>(counts, offsets, c.expert_first, EL, m->counts,
                                                                           m->offsets, m->active, m->n_active);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    // this rank's experts see about rows_total / world rows; the kernels read them in place
    if ((rc = launch_decode_q4k_rows(m, gx_own, row_token, m->counts, m->offsets, (rows_total + world - 1) / world, (float*)m->ys, s)))
        return rc;
    const int64_t est = (rows_total + world - 1) / world;
    const int64_t blocks = est < 8 ? 1 : (est / 8 < 148 * 8 ? (est + 7) / 8 : 148 * 8);
    LaunchScope scope(m, s, "ep_return");
    ep_return_gathered_kernel<<<(unsigned)blocks, 256, 0, s>>>((const float*)m->ys, row_token, m->offsets, EL,
                                                               peer_table(peer_sync, world), peer_table(peer_back, world),
                                                               rank, world, tokens_per_rank, c.hidden, rows_total, back_rows,
                                                               m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_combine(MummuMoe* m, void* const* peer_sync, const void* back_own, const int32_t* ids,
                         const int32_t* order_ids, const float* w, const int32_t* pos, int32_t rank, int32_t world,
                         int32_t tokens, int32_t top_k, void* out, void* stream) {
    MUMMU_REQUIRE(m && peer_sync && back_own && ids && w && pos && out, "mummu_ep_combine: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_combine");
    if (rc) return rc;
    MUMMU_REQUIRE(dtype_size(m->cfg.act_dtype) == 2 && m->cfg.hidden % 8 == 0,
                  "mummu_ep_combine: 16-bit activations with hidden %% 8 == 0 only");
    MUMMU_REQUIRE(tokens >= 0 && top_k >= 1, "mummu_ep_combine: tokens %d, top_k %d", tokens, top_k);
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    {
        // a rank without tokens still consumes the epoch
        LaunchScope scope(m, s, "ep_wait_out");
        ep_wait_kernel<<<1, 32, 0, s>>>(peer_table(peer_sync, world), rank, world, EP_CH_OUT, wait_polls_of(m), m->status);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    // a token's terms in ascending EXPERT id (nn/moe.rs:296-328); with a placement `ids` are bank
    // slots and the expert ids come separately, so that the order does not follow the slots
    return launch_combine(m, back_own, m->cfg.act_dtype, order_ids ? order_ids : ids, w, pos, tokens, top_k, out, s);
}

}  // extern "C"
