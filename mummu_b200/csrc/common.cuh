// Shared declarations of the mummu-cuda library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/mummu_cuda.h"

namespace mummu {

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);

#define MUMMU_CUDA_TRY(expr)                                                              \
    do {                                                                                  \
        cudaError_t err__ = (expr);                                                       \
        if (err__ != cudaSuccess) {                                                       \
            ::mummu::set_error("CUDA error %s at %s:%d: %s", cudaGetErrorName(err__),     \
                               __FILE__, __LINE__, cudaGetErrorString(err__));            \
            return MUMMU_ERR_DEVICE;                                                      \
        }                                                                                 \
    } while (0)

#define MUMMU_REQUIRE(cond, ...)              \
    do {                                      \
        if (!(cond)) {                        \
            ::mummu::set_error(__VA_ARGS__);  \
            return MUMMU_ERR_CONTRACT;        \
        }                                     \
    } while (0)

// device status word bits (sticky until mummu_moe_sync reads them)
constexpr int STATUS_NONFINITE = 1;
constexpr int STATUS_TIMEOUT = 2;
constexpr int STATUS_BOUNDS = 4;

// ---------------------------------------------------------------------------------------------
// dtype helpers
// ---------------------------------------------------------------------------------------------
inline size_t dtype_size(int dt) {
    switch (dt) {
        case MUMMU_F32: return 4;
        case MUMMU_F16: return 2;
        case MUMMU_BF16: return 2;
        default: return 0;
    }
}

constexpr int Q4K_BLOCK_ELEMS = 256;
constexpr int Q4K_BLOCK_BYTES = 144;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Tag type for Q4_K packed weights (rows of 144-byte super-blocks).
struct q4k_t { uint8_t b; };

// One Q4_K element, decoded exactly as the reference does (crates/mummu/src/gguf.rs:1685-1726):
// d*sc first, then *q, the min product on its own, one subtraction; every step rounded to f32.
__device__ __forceinline__ void q4k_scale_min(const uint8_t* scales, int j, float& sc, float& m) {
    uint32_t s, mn;
    if (j < 4) {
        s = scales[j] & 63u;
        mn = scales[j + 4] & 63u;
    } else {
        s = (scales[j + 4] & 0x0Fu) | ((uint32_t)(scales[j - 4] >> 6) << 4);
        mn = (uint32_t)(scales[j + 4] >> 4) | ((uint32_t)(scales[j] >> 6) << 4);
    }
    sc = (float)s;
    m = (float)mn;
}

__device__ __forceinline__ float q4k_decode_elem(const uint8_t* row, int k) {
    const uint8_t* blk = row + (size_t)(k >> 8) * Q4K_BLOCK_BYTES;
    int within = k & 255;
    int j = within >> 5;          // sub-block 0..7
    int chunk = j >> 1;
    int b = within & 31;
    float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
    float dmin = __half2float(__ushort_as_half((unsigned short)(blk[2] | (blk[3] << 8))));
    float sc, m;
    q4k_scale_min(blk + 4, j, sc, m);
    uint8_t byte = blk[16 + chunk * 32 + b];
    float q = (float)((j & 1) ? (byte >> 4) : (byte & 0x0F));
    float product = __fmul_rn(__fmul_rn(d, sc), q);
    return __fsub_rn(product, __fmul_rn(dmin, m));
}

// Sibling GGUF block formats, correctness path only (the SIMT bank decodes them element by
// element; the fast decode kernels take Q4_K).  Same operation order as the reference:
//   Q8_0 (crates/mummu/src/gguf.rs:1535-1543): 34 B = f16 d + 32 i8;            x = d*q
//   Q5_K (gguf.rs:1731-1765): 176 B = f16 d, f16 dmin, 12 B scales, 32 B fifth bits, 128 B nibbles;
//                              x = (d*sc)*(q + 16*bit) - dmin*m
//   Q6_K (gguf.rs:1769-1797): 210 B = 128 B low nibbles, 64 B high pairs, 16 i8 scales, f16 d;
//                              x = (d*s)*(q - 32)
struct q80_t { uint8_t b; };
struct q5k_t { uint8_t b; };
struct q6k_t { uint8_t b; };
constexpr int Q80_BLOCK_ELEMS = 32, Q80_BLOCK_BYTES = 34;
constexpr int Q5K_BLOCK_BYTES = 176, Q6K_BLOCK_BYTES = 210;   // 256 elements each

__device__ __forceinline__ float f16_at(const uint8_t* p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

__device__ __forceinline__ float q80_decode_elem(const uint8_t* row, int k) {
    const uint8_t* blk = row + (size_t)(k >> 5) * Q80_BLOCK_BYTES;
    return __fmul_rn(f16_at(blk), (float)(int8_t)blk[2 + (k & 31)]);
}

__device__ __forceinline__ float q5k_decode_elem(const uint8_t* row, int k) {
    const uint8_t* blk = row + (size_t)(k >> 8) * Q5K_BLOCK_BYTES;
    const int within = k & 255, j = within >> 5, chunk = j >> 1, b = within & 31;
    float sc, m;
    q4k_scale_min(blk + 4, j, sc, m);
    const uint8_t byte = blk[48 + chunk * 32 + b];
    const int top = (blk[16 + b] >> j) & 1;                   // bit-plane j of the shared 32 bytes
    const float q = (float)(((j & 1) ? (byte >> 4) : (byte & 0x0F)) + 16 * top);
    const float product = __fmul_rn(__fmul_rn(f16_at(blk), sc), q);
    return __fsub_rn(product, __fmul_rn(f16_at(blk + 2), m));
}

__device__ __forceinline__ float q6k_decode_elem(const uint8_t* row, int k) {
    const uint8_t* blk = row + (size_t)(k >> 8) * Q6K_BLOCK_BYTES;
    const int within = k & 255, half = within >> 7, r = within & 127, quarter = r >> 5, l = r & 31;
    const uint8_t lo = blk[half * 64 + l + ((quarter & 1) ? 32 : 0)];
    const uint8_t hi = blk[128 + half * 32 + l];
    const int low4 = (quarter & 2) ? (lo >> 4) : (lo & 0x0F);
    const int q = (low4 | (((hi >> (2 * quarter)) & 3) << 4)) - 32;
    const float s = (float)(int8_t)blk[192 + half * 8 + (l >> 4) + 2 * quarter];
    return __fmul_rn(__fmul_rn(f16_at(blk + 208), s), (float)q);
}

// ---------------------------------------------------------------------------------------------
// the handle
// ---------------------------------------------------------------------------------------------
struct KernelStat {
    int64_t launches = 0;
    double ms = 0.0;
};

struct Profiler {
    bool enabled = false;
    struct Pending { std::string name; cudaEvent_t a, b; };
    std::vector<Pending> pending;
    std::map<std::string, KernelStat> stats;
    std::vector<cudaEvent_t> pool;
};

}  // namespace mummu

// Kernel-variant switches of one handle.  Read once from the environment when the handle is
// created (MUMMU_CUDA_* variables, the way the reference reads its MUMMU_* switches once into
// OnceLocks, nn/packed_gemv.rs:85-92, 686-694); mummu_moe_set_switch changes one afterwards.
struct MummuSwitches {
    int no_tc = 0;            // MUMMU_CUDA_NO_TC: never take the tcgen05 grouped GEMM
    int no_host_graph = 0;    // MUMMU_CUDA_NO_HOST_GRAPH: host-pointer decode calls stay eager
    int router_plain = 0;     // MUMMU_CUDA_ROUTER_PLAIN: decode router without the bulk-copied slice image
    int decode_no_pdl = 0;    // MUMMU_CUDA_DECODE_NO_PDL: no programmatic dependent launch of the down kernel
    int decode_nt = 0;        // MUMMU_CUDA_DECODE_NT: 1 forces one 8-token tile per pass
    int decode_stream_min = 0;// MUMMU_CUDA_DECODE_STREAM_MIN: row tiles from which the streaming variant runs
    int decode_rb_gateup = 0; // MUMMU_CUDA_DECODE_RB_GATEUP / _DOWN: row tiles per CTA (0 = planned)
    int decode_rb_down = 0;
    int checked = 0;          // MUMMU_CUDA_CHECKED: kernels verify their indices and raise the status word
    uint32_t wait_polls = 0;  // bound of the device-side peer waits in polls (0 = the default, seconds)
};

struct MummuMoe {
    MummuMoeConfig cfg{};
    MummuSwitches sw{};
    std::mutex mu;
    cudaStream_t stream = nullptr;

    float* router_w = nullptr;      // f32 [hidden, experts]
    // the same weights as the decode router's shared-memory image: [experts/8][8 lanes j][8 experts]
    // [hidden/8 + 4] (value of row 8i+j at index i), present when hidden % 32 == 0, experts % 8 == 0
    float* router_wt = nullptr;
    float* router_bias = nullptr;   // f32 [experts] or null
    void* bank[3] = {nullptr, nullptr, nullptr};
    size_t bank_bytes[3] = {0, 0, 0};
    bool bank_set[3] = {false, false, false};
    bool router_set = false;

    // scratch, sized for cap_tokens tokens at cfg.top_k slots each
    int64_t cap_tokens = 0;
    bool scratch_borrowed = false;  // scratch belongs to another handle (mummu_moe_adopt_scratch)
    float* logits = nullptr;        // [tokens, experts]
    int32_t* tile_done = nullptr;   // router tile counters (self-resetting)
    int32_t* ids = nullptr;         // [tokens, k]
    float* wts = nullptr;           // [tokens, k]
    int32_t* counts = nullptr;      // [experts]
    int32_t* offsets = nullptr;     // [experts + 1]
    int32_t* active = nullptr;      // [experts] ids of experts with rows this call
    int32_t* n_active = nullptr;    // [1]
    int32_t* whist = nullptr;       // large-call grouping: per (warp of 256 pairs, expert) counts, then first rows
    int64_t whist_elems = 0;
    // expert-parallel return path: the local rows as segments (local expert, source rank)
    int32_t* ret_seg = nullptr;     // [experts_local * 16 + 1] first local row of every segment
    int32_t* ret_dst = nullptr;     // [experts_local * 16] the segment's first row in its source's buffer
    // set by the expert-parallel experts stage around its call of the expert kernels: where the
    // down projection may store its rows directly (peer buffers); `used` tells the stage whether
    // the kernel that ran took the offer
    // f16 image of a Q4_K bank for calls with too many rows for the packed-weight kernels: the
    // experts with rows are expanded per call and fed to the tensor-core GEMMs
    __half* wexp[3] = {nullptr, nullptr, nullptr};
    MummuMoe* scratch_donor = nullptr;      // the layer whose scratch (and expanded image) this one uses
    struct {
        bool offered = false, used = false;
        int world = 0;
        int64_t back_rows = 0;
        void* back[16] = {};
    } scatter;
    int32_t* row_token = nullptr;   // [tokens * k]
    int32_t* pos = nullptr;         // [tokens * k]
    void* xs = nullptr;             // gathered rows [tokens * k, hidden] act dtype (tensor path)
    void* hact = nullptr;           // [tokens * k, inter] f32 (or 16-bit, path dependent)
    void* ys = nullptr;             // [tokens * k, hidden] f32
    void* io_x = nullptr;           // device staging for host-pointer calls
    void* io_y = nullptr;
    float* ex_io = nullptr;         // f32 staging of the one-expert calls, grown on demand
    size_t ex_io_elems = 0;
    unsigned long long* hits = nullptr;  // [experts]
    int32_t* status = nullptr;      // device status word
    int32_t* status_host = nullptr; // pinned landing place for reads of the status word
    // cached tensor maps (CUtensorMap, 128 B each) of the Q4_K banks as [rows, row_bytes] byte views
    alignas(64) unsigned char q4k_map[3][128];
    const void* q4k_map_base[3] = {nullptr, nullptr, nullptr};
    int64_t launches = 0;
    mummu::Profiler prof;
    // host-pointer decode calls: the layer's launches captured once per (tokens, top_k, norm) and
    // replayed (every pointer inside is the handle's own); value null = capture failed, stay eager
    std::map<uint64_t, cudaGraphExec_t> host_graphs;
    std::map<uint64_t, int> host_calls;
};

namespace mummu {

size_t bank_row_bytes(const MummuMoeConfig& c, int which);
size_t bank_total_bytes(const MummuMoeConfig& c, int which);
int ensure_scratch(MummuMoe* m, int64_t tokens);
void clear_host_graphs(MummuMoe* m);

// Opt a kernel into the full 227 KB of dynamic shared memory, once per (kernel, device): the
// attribute call is kept out of the steady state so that a layer call can be stream-captured.
cudaError_t allow_big_smem_impl(const void* kernel, int device);
template <typename Kernel>
cudaError_t allow_big_smem(Kernel kernel, int device) {
    return allow_big_smem_impl(reinterpret_cast<const void*>(kernel), device);
}

// profiling-aware launch bracket
struct LaunchScope {
    MummuMoe* m;
    cudaStream_t s;
    const char* name;
    cudaEvent_t a = nullptr, b = nullptr;
    LaunchScope(MummuMoe* m_, cudaStream_t s_, const char* name_);
    ~LaunchScope();
};

// ---- kernels_basic.cu ----
// where the fused grouping of a decode-sized router call writes (null = the handle's own scratch)
struct GroupedOut {
    int32_t *counts, *offsets, *row_token, *pos;
};
int launch_router(MummuMoe* m, const void* x, int64_t tokens, int top_k, int norm, int32_t* ids,
                  float* wts, int32_t* counts, cudaStream_t s, bool fuse_permute = false,
                  const GroupedOut* grouped = nullptr);
int launch_count(MummuMoe* m, const int32_t* ids, int64_t n, int32_t* counts, cudaStream_t s);
int launch_permute(MummuMoe* m, const int32_t* ids, int64_t tokens, int top_k,
                   const int32_t* counts, int32_t* offsets, int32_t* row_token, int32_t* pos,
                   cudaStream_t s);
int launch_check_plan(MummuMoe* m, int32_t* ids, int32_t* pos, int32_t* row_token, const int32_t* counts,
                      const int32_t* offsets, int64_t tokens, int top_k, cudaStream_t s);
int launch_check_combine(MummuMoe* m, const int32_t* ids, const int32_t* pos, int32_t* ids_out, int32_t* pos_out,
                         int64_t pairs, cudaStream_t s);
int launch_check_counts(MummuMoe* m, const int32_t* counts, int32_t* counts_out, int n, int64_t rows, cudaStream_t s);
int launch_combine(MummuMoe* m, const void* ys, int ys_dtype, const int32_t* ids, const float* w,
                   const int32_t* pos, int64_t tokens, int top_k, void* out, cudaStream_t s);
int launch_offsets_from_counts(MummuMoe* m, const int32_t* counts, int n, int32_t* offsets,
                               cudaStream_t s);
// generic SIMT grouped SwiGLU (all dtypes); x_dtype is the dtype of `x`, rows come through
// row_index (may be null = identity); experts local ids 0..experts_local
int launch_experts_simt(MummuMoe* m, const void* x, int x_dtype, const int32_t* row_index,
                        const int32_t* counts, const int32_t* offsets, int64_t max_rows_per_expert,
                        int64_t total_rows, void* ys, int ys_dtype, int expert_only,
                        cudaStream_t s);
int launch_single_expert_plan(MummuMoe* m, int expert, int rows, cudaStream_t s);
int launch_gate_energy(MummuMoe* m, int expert, const float* x, int rows, float* energy, cudaStream_t s);
int launch_q4k_dequant(const void* src, float* dst, int64_t n_blocks, cudaStream_t s);
int launch_q4k_quantize(const float* src, void* dst, int64_t n_blocks, cudaStream_t s);
int launch_widen(const void* src, int dtype, float* dst, int64_t n, cudaStream_t s);
int launch_block_dequant(const void* src, int dtype, float* dst, int64_t rows, int64_t cols, size_t row_bytes,
                         cudaStream_t s);

// ---- prefill_tc.cu ----
bool prefill_tc_supported(const MummuMoeConfig& c, int64_t rows_total);
int launch_gather_rows(MummuMoe* m, const void* x, const int32_t* row_token, void* xs, int64_t rows,
                       cudaStream_t s);
int launch_block_expand_f16(MummuMoe* m, int which, __half* dst, const int32_t* counts, cudaStream_t s);
bool q4k_tc_supported(const MummuMoeConfig& c, int64_t rows_total);
int launch_experts_q4k_tc(MummuMoe* m, const void* xs, int64_t rows_cap, const int32_t* counts, const int32_t* offsets,
                          void* ys, int ys_dtype, cudaStream_t s);
int launch_experts_tc(MummuMoe* m, const void* xs, int64_t rows_cap, const int32_t* counts,
                      const int32_t* offsets, void* ys, int ys_dtype, cudaStream_t s);

// ---- decode_q4k.cu ----
bool decode_q4k_supported(const MummuMoeConfig& c, int64_t tokens);
int launch_decode_q4k(MummuMoe* m, const void* x, int64_t tokens, int top_k, cudaStream_t s);
int launch_decode_q4k_rows(MummuMoe* m, const void* x, const int32_t* row_token, const int32_t* counts,
                           const int32_t* offsets, int64_t rows_total, float* ys, cudaStream_t s);
int launch_narrow(const float* src, void* dst, int dtype, int64_t n, cudaStream_t s);
}  // namespace mummu
