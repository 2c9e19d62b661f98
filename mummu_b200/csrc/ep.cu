// Expert-parallel exchange over peer memory (NVLink / NVSwitch): no host synchronisation, no
// staging copies.  The reference has no collective for this path (its devices exchange through
// host memory: crates/mummu/src/backend.rs:128-143, nn/moe.rs:1219-1272).
//
// Every rank owns a contiguous block of experts and two peer-visible buffers:
//   recv_x [cap_rows, hidden]  rows routed to its experts, expert-major (sources in rank order)
//   ys     [cap_rows, hidden]  its experts' outputs for those rows
// From the all-gathered per-expert row counts every rank computes, on the device, where each of
// its sorted rows lives in the owner's buffers (ep_plan).  Dispatch is a gather from the layer
// input straight into the owners' recv_x with 16-byte peer stores (ep_dispatch); combine reads
// the expert outputs with peer loads, in ascending expert id with the reference's two roundings
// (ep_combine).  Plain peer loads and stores only.
#include <cstring>

#include "common.cuh"

namespace mummu {

constexpr int EP_MAX_RANKS = 16;

struct PeerTable {
    void* ptr[EP_MAX_RANKS];
};

// all_counts [world, E]: rows rank s routes to global expert e.
// dst_base[e]   : first row, in the owner's buffers, of THIS rank's rows for expert e
// local_counts[le], local_offsets[le] : rows / first row of local expert le, all sources together
__global__ void ep_plan_kernel(const int32_t* all_counts, int world, int rank, int E, int EL,
                               int32_t* dst_base, int32_t* local_counts) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int d = e / EL, le = e - d * EL;
        int base = 0;
        for (int l2 = 0; l2 < le; ++l2)                       // local experts of rank d before le: all sources
            for (int s = 0; s < world; ++s) base += all_counts[s * E + d * EL + l2];
        for (int s = 0; s < rank; ++s) base += all_counts[s * E + e];   // lower ranks' rows of this expert
        dst_base[e] = base;
    }
    for (int le = threadIdx.x; le < EL; le += blockDim.x) {
        int c = 0;
        for (int s = 0; s < world; ++s) c += all_counts[s * E + rank * EL + le];
        local_counts[le] = c;
    }
}

// ---------------------------------------------------------------------------------------------
// Device-side signalling between the ranks (one rank per GPU), so that a whole expert-parallel
// step holds no library collective and no host round trip and can be replayed from a CUDA graph.
// Every rank owns a peer-visible block of 32-bit words, zeroed by its owner before the peers map it:
//   [0]                  epoch of the owner's last signal (touched by the owner only)
//   [16 .. 16+R)         flag[s]: last epoch rank s has signalled to this rank
//   [64 .. 64+R*E)       counts_in[s][e]: rank s's per-expert row counts for the current layer
// A signal is a system-scope release store of the sender's epoch into flag[sender] of every rank;
// a wait polls the own flags with system-scope acquire loads until all have reached the epoch.
// Epochs only grow, so a rank that is already one signal ahead is harmless.  Polls are bounded
// (a second or two): when they run out the kernel raises the status word and returns.
// ---------------------------------------------------------------------------------------------
constexpr int EP_SYNC_FLAGS = 16, EP_SYNC_COUNTS = 64;
constexpr uint32_t EP_WAIT_LIMIT = 1u << 23;

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// one warp: lane s talks to rank s
__device__ void ep_signal_and_wait(const PeerTable& sync, int rank, int world, int32_t* status) {
    const int lane = threadIdx.x & 31;
    int32_t* own = reinterpret_cast<int32_t*>(sync.ptr[rank]);
    int32_t epoch = 0;
    if (lane == 0) {
        epoch = own[0] + 1;
        own[0] = epoch;
    }
    epoch = __shfl_sync(0xFFFFFFFFu, epoch, 0);
    __threadfence_system();
    if (lane < world) {
        st_release_sys(reinterpret_cast<int32_t*>(sync.ptr[lane]) + EP_SYNC_FLAGS + rank, epoch);
        const int32_t* flag = own + EP_SYNC_FLAGS + lane;
        uint32_t polls = 0;
        while (ld_acquire_sys(flag) - epoch < 0) {
            if (++polls > 64) __nanosleep(200);
            if (polls > EP_WAIT_LIMIT) {
                atomicOr(status, STATUS_TIMEOUT);
                break;
            }
        }
    }
    __syncwarp();
    __threadfence_system();
}

__global__ void __launch_bounds__(32) ep_barrier_kernel(PeerTable sync, int rank, int world, int32_t* status) {
    ep_signal_and_wait(sync, rank, world, status);
}

// counts all-gather + plan in one launch: every rank stores its counts into counts_in[rank] of
// every rank, signals, waits for the others' counts, then computes what ep_plan_kernel computes.
__global__ void __launch_bounds__(256) ep_exchange_plan_kernel(const int32_t* counts, PeerTable sync, int world,
                                                               int rank, int E, int EL, int32_t* dst_base,
                                                               int32_t* local_counts, int32_t* status) {
    for (int idx = threadIdx.x; idx < world * E; idx += blockDim.x) {
        const int s = idx / E, e = idx - s * E;
        reinterpret_cast<int32_t*>(sync.ptr[s])[EP_SYNC_COUNTS + rank * E + e] = counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < 32) ep_signal_and_wait(sync, rank, world, status);
    __syncthreads();
    // the gathered counts once into shared memory (coalesced), then the plan from there: read one
    // by one from global memory the dependent loads below cost tens of microseconds
    extern __shared__ int32_t all_counts[];                    // [world][E]
    {
        const volatile int32_t* src = reinterpret_cast<const volatile int32_t*>(sync.ptr[rank]) + EP_SYNC_COUNTS;
        for (int i = threadIdx.x; i < world * E; i += blockDim.x) all_counts[i] = src[i];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int d = e / EL, le = e - d * EL;
        int base = 0;
        for (int l2 = 0; l2 < le; ++l2)
            for (int s = 0; s < world; ++s) base += all_counts[s * E + d * EL + l2];
        for (int s = 0; s < rank; ++s) base += all_counts[s * E + e];
        dst_base[e] = base;
    }
    for (int le = threadIdx.x; le < EL; le += blockDim.x) {
        int c = 0;
        for (int s = 0; s < world; ++s) c += all_counts[s * E + rank * EL + le];
        local_counts[le] = c;
    }
}

// one block per sorted row p: recv_x[owner][dst_base[e] + (p - offsets[e])] = x[row_token[p]]
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const uint4* x, const int32_t* row_token,
                                                          const int32_t* offsets, const int32_t* dst_base,
                                                          PeerTable recv, int E, int EL, int vec_per_row,
                                                          int64_t rows) {
    __shared__ int s_e;
    for (int64_t p = blockIdx.x; p < rows; p += gridDim.x) {
        if (threadIdx.x == 0) {
            int lo = 0, hi = E;                               // last e with offsets[e] <= p
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (offsets[mid] <= p) lo = mid; else hi = mid;
            }
            s_e = lo;
        }
        __syncthreads();
        const int e = s_e;
        const int d = e / EL;
        const int64_t drow = (int64_t)dst_base[e] + (p - offsets[e]);
        const uint4* src = x + (size_t)row_token[p] * vec_per_row;
        uint4* dst = reinterpret_cast<uint4*>(recv.ptr[d]) + (size_t)drow * vec_per_row;
        for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
        __syncthreads();
    }
}

// per token: ascending expert id, scaled = w * y; out += scaled — y read from the owner's buffer
template <typename T>
__global__ void __launch_bounds__(256) ep_combine_kernel(PeerTable ys, const int32_t* ids, const float* w,
                                                         const int32_t* pos, const int32_t* offsets,
                                                         const int32_t* dst_base, int top_k, int H, int EL,
                                                         T* out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const T** s_row = reinterpret_cast<const T**>(smem_raw);
    float* s_w = reinterpret_cast<float*>(s_row + top_k);
    const int64_t t = blockIdx.x;
    for (int r = threadIdx.x; r < top_k; r += blockDim.x) {
        const int id = ids[t * top_k + r];
        int rank = 0;
        for (int q = 0; q < top_k; ++q) {
            const int other = ids[t * top_k + q];
            rank += (other < id || (other == id && q < r)) ? 1 : 0;
        }
        const int64_t drow = (int64_t)dst_base[id] + (pos[t * top_k + r] - offsets[id]);
        s_row[rank] = reinterpret_cast<const T*>(ys.ptr[id / EL]) + (size_t)drow * H;
        s_w[rank] = w[t * top_k + r];
    }
    __syncthreads();
    for (int h = (blockIdx.y * blockDim.x + threadIdx.x) * 8; h < H; h += gridDim.y * blockDim.x * 8) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r0 = 0; r0 < top_k; r0 += 4) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (r0 + u < top_k) raw[u] = *reinterpret_cast<const uint4*>(s_row[r0 + u] + h);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (r0 + u < top_k) {
                    const T* v = reinterpret_cast<const T*>(&raw[u]);
                    const float wv = s_w[r0 + u];
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(wv, to_f32(v[i])));
                }
        }
        uint4 o;
        T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) ov[i] = from_f32<T>(acc[i]);
        *reinterpret_cast<uint4*>(out + t * H + h) = o;
    }
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

int32_t mummu_ep_plan(MummuMoe* m, const int32_t* all_counts, int32_t rank, int32_t world,
                      int32_t* dst_base, int32_t* local_counts, void* stream) {
    MUMMU_REQUIRE(m && all_counts && dst_base && local_counts, "mummu_ep_plan: null argument");
    MUMMU_REQUIRE(world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world &&
                      m->cfg.experts % world == 0 && m->cfg.experts_local == m->cfg.experts / world,
                  "mummu_ep_plan: rank %d of %d with %d local experts of %d", rank, world,
                  m->cfg.experts_local, m->cfg.experts);
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    LaunchScope scope(m, s, "ep_plan");
    ep_plan_kernel<<<1, 256, 0, s>>>(all_counts, world, rank, m->cfg.experts, m->cfg.experts_local, dst_base,
                                     local_counts);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

static int ep_check_ranks(MummuMoe* m, int32_t rank, int32_t world, const char* who) {
    MUMMU_REQUIRE(world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world &&
                      m->cfg.experts % world == 0 && m->cfg.experts_local == m->cfg.experts / world,
                  "%s: rank %d of %d with %d local experts of %d", who, rank, world, m->cfg.experts_local,
                  m->cfg.experts);
    return MUMMU_OK;
}

size_t mummu_ep_sync_bytes(int32_t world, int32_t experts) {
    return (size_t)(EP_SYNC_COUNTS + (size_t)world * experts) * 4;
}

int32_t mummu_ep_exchange_plan(MummuMoe* m, const int32_t* counts, void* const* peer_sync, int32_t rank,
                               int32_t world, int32_t* dst_base, int32_t* local_counts, void* stream) {
    MUMMU_REQUIRE(m && counts && peer_sync && dst_base && local_counts, "mummu_ep_exchange_plan: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_exchange_plan");
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    PeerTable t{};
    for (int i = 0; i < world; ++i) t.ptr[i] = peer_sync[i];
    LaunchScope scope(m, s, "ep_exchange_plan");
    ep_exchange_plan_kernel<<<1, 256, (size_t)world * m->cfg.experts * sizeof(int32_t), s>>>(counts, t, world, rank, m->cfg.experts, m->cfg.experts_local, dst_base,
                                              local_counts, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_barrier(MummuMoe* m, void* const* peer_sync, int32_t rank, int32_t world, void* stream) {
    MUMMU_REQUIRE(m && peer_sync, "mummu_ep_barrier: null argument");
    int rc = ep_check_ranks(m, rank, world, "mummu_ep_barrier");
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    PeerTable t{};
    for (int i = 0; i < world; ++i) t.ptr[i] = peer_sync[i];
    LaunchScope scope(m, s, "ep_barrier");
    ep_barrier_kernel<<<1, 32, 0, s>>>(t, rank, world, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_dispatch(MummuMoe* m, const void* x, const int32_t* row_token, const int32_t* offsets,
                          const int32_t* dst_base, void* const* peer_recv, int32_t world, int32_t rows,
                          void* stream) {
    MUMMU_REQUIRE(m && x && row_token && offsets && dst_base && peer_recv, "mummu_ep_dispatch: null argument");
    MUMMU_REQUIRE(world >= 1 && world <= EP_MAX_RANKS, "mummu_ep_dispatch: %d ranks", world);
    MUMMU_REQUIRE(dtype_size(m->cfg.act_dtype) == 2 && m->cfg.hidden % 8 == 0,
                  "mummu_ep_dispatch: 16-bit activations with hidden %% 8 == 0 only");
    if (rows == 0) return MUMMU_OK;
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    PeerTable t{};
    for (int i = 0; i < world; ++i) t.ptr[i] = peer_recv[i];
    const int64_t blocks = rows < 148 * 16 ? rows : 148 * 16;
    LaunchScope scope(m, s, "ep_dispatch");
    ep_dispatch_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint4*)x, row_token, offsets, dst_base, t,
                                                        m->cfg.experts, m->cfg.experts_local,
                                                        m->cfg.hidden * 2 / 16, rows);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_ep_combine(MummuMoe* m, void* const* peer_ys, const int32_t* ids, const float* w,
                         const int32_t* pos, const int32_t* offsets, const int32_t* dst_base,
                         int32_t tokens, int32_t top_k, int32_t world, void* out, void* stream) {
    MUMMU_REQUIRE(m && peer_ys && ids && w && pos && offsets && dst_base && out, "mummu_ep_combine: null argument");
    MUMMU_REQUIRE(world >= 1 && world <= EP_MAX_RANKS, "mummu_ep_combine: %d ranks", world);
    MUMMU_REQUIRE(dtype_size(m->cfg.act_dtype) == 2 && m->cfg.hidden % 8 == 0,
                  "mummu_ep_combine: 16-bit activations with hidden %% 8 == 0 only");
    if (tokens == 0) return MUMMU_OK;
    std::lock_guard<std::mutex> lock(m->mu);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    PeerTable t{};
    for (int i = 0; i < world; ++i) t.ptr[i] = peer_ys[i];
    const int H = m->cfg.hidden;
    const dim3 grid((unsigned)tokens, tokens < 512 ? (unsigned)((H / 8 + 255) / 256) : 1u);
    const size_t smem = (size_t)top_k * (sizeof(void*) + sizeof(float));
    LaunchScope scope(m, s, "ep_combine");
    if (m->cfg.act_dtype == MUMMU_F16)
        ep_combine_kernel<__half><<<grid, 256, smem, s>>>(t, ids, w, pos, offsets, dst_base, top_k, H,
                                                         m->cfg.experts_local, (__half*)out);
    else
        ep_combine_kernel<__nv_bfloat16><<<grid, 256, smem, s>>>(t, ids, w, pos, offsets, dst_base, top_k, H,
                                                                m->cfg.experts_local, (__nv_bfloat16*)out);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

}  // extern "C"
