// Prefill-regime expert bank on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 / f16.
//
// Two grouped GEMMs over rows already sorted by expert (reference math:
// crates/mummu/src/nn/moe.rs:312-316):
//   GEMM1  hact[p, n] = silu(xs[p,:] . Wg[e,n,:]) * (xs[p,:] . Wu[e,n,:])     (16-bit out)
//   GEMM2  ys[p, h]   = hact[p,:] . Wd[e,h,:]                                   (16-bit or f32 out)
// Every operand is K-major ("[rows, K]" with K contiguous), which is what tcgen05.mma wants.
//
// One persistent CTA per SM walks a tile list built on the device from the per-expert row counts:
// tile = (expert, 128 sorted rows, one N tile).  Each tile's accumulator is 128 TMEM lanes x 256
// f32 columns, written by two M=128,N=128,K=16 MMAs per K step: for GEMM1 the two halves are the
// gate and the up rows of the same 128 intermediate columns (so silu(g)*u happens in the
// epilogue, in registers), for GEMM2 they are two adjacent 128-column blocks of the output.
// Warp roles: warp 0 issues TMA loads (plain tiled loads, 128-byte swizzle) into a 4-stage
// shared-memory ring; warp 1 allocates TMEM and issues the MMAs from one elected thread,
// signalling stage reuse and accumulator completion with tcgen05.commit; warps 2-5 drain the
// accumulator (tcgen05.ld, one TMEM lane = one output row per thread) while the MMAs of the next
// tile fill the other accumulator stage (2 x 256 columns = all 512 TMEM columns).
// Ragged segments: a 128-row tile may run past its expert's rows; those rows are computed (they
// belong to the next expert or are zero fill) and masked at the store.
//
// Every wait on an mbarrier is bounded: when it runs out the CTA raises the handle's status word
// (MUMMU_ERR_TIMEOUT), stops issuing work, waits (bounded) for its own copies, frees its TMEM and
// returns.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace mummu {

constexpr int TC_BM = 128;           // rows per tile
constexpr int TC_BK = 64;            // K per stage: 64 x 2 B = one 128-byte swizzle row
constexpr int TC_STAGES = 4;
constexpr int TC_THREADS = 192;      // 6 warps
constexpr uint32_t TC_STAGE_BYTES = 3 * TC_BM * TC_BK * 2;   // A + B0 + B1 = 48 KiB
constexpr uint32_t TC_TMEM_COLS = 512;
constexpr uint32_t TC_SPIN_LIMIT = 4u << 20;                 // bounded waits (about a second)

struct TcArgs {
    const int32_t* counts;     // [E] rows per expert
    const int32_t* offsets;    // [E] first sorted row per expert
    int E;
    int K;                     // contraction width
    int n_tiles;               // N tiles per expert
    int b_rows_per_expert;     // rows of the weight view per expert
    int b_tile_rows;           // weight rows consumed by one tile in map B0 (GEMM1: 128, GEMM2: 256)
    int b1_row_offset;         // extra row offset of the second half in map B1 (GEMM1: 0, GEMM2: 128)
    void* out;
    int ld_out;
    int32_t* status;
    // GEMM2 with 16-bit output may send every output row somewhere else (expert parallelism: to
    // the rank the row came from).  Rows are segments (expert, source rank) in ret_seg order.
    const int32_t* ret_seg;    // [n_seg + 1] first row of every segment, or null: rows stay in `out`
    const int32_t* ret_dst;    // [n_seg] the segment's first row in its destination buffer
    int n_seg, world;
    int64_t back_rows;         // rows of a destination buffer
    void* back[16];            // destination buffer per rank (peer memory; plain stores)
};

constexpr uint32_t TC_EPI_STAGE_BYTES = 32 * 128;            // per epilogue warp: 32 rows x 64 values of 16 bits

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait_bounded(bar, parity, abort_flag, TC_SPIN_LIMIT);
}

__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// ------------------------------------------------------------------------------------------------
// tile list
// ------------------------------------------------------------------------------------------------
struct TileCursor {
    int e = 0;
    // tile index -> (expert, first sorted row, rows end of the expert, n tile)
    __device__ __forceinline__ void locate(const int* tile_start, const int32_t* counts, const int32_t* offsets,
                                           int tile, int n_tiles, int& expert, int& row0, int& row_end, int& nt) {
        while (tile >= tile_start[e + 1]) ++e;
        const int local = tile - tile_start[e];
        const int cnt = counts[e];
        const int m_tiles = (cnt + TC_BM - 1) / TC_BM;
        nt = local / m_tiles;
        const int mt = local - nt * m_tiles;
        expert = e;
        row0 = offsets[e] + mt * TC_BM;
        row_end = offsets[e] + cnt;
    }
};

// ------------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------------
// FUSED: GEMM1 (silu(D0)*D1 -> 128 output columns); otherwise GEMM2 (D0 | D1 -> 256 columns).
template <typename TIN, typename TOUT, bool FUSED>
__global__ void __launch_bounds__(TC_THREADS, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                       const __grid_constant__ CUtensorMap map_b1, TcArgs a) {
    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte alignment for the swizzled tiles
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* tiles = smem;                                           // TC_STAGES x 48 KiB
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);
    // bars: full[S], empty[S], tmem_full[2], tmem_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* tile_start = reinterpret_cast<int*>(tmem_slot + 2);               // [E + 1]
    // epilogue staging, 4 x 4 KiB, 16-byte aligned behind the tile list
    unsigned char* epi_stage = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tile_start + a.E + 1) + 15) & ~(uintptr_t)15);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + TC_STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * TC_STAGES), tempty0 = smem_u32(bars + 2 * TC_STAGES + 2);

    // tile prefix over experts (every CTA builds the same list)
    if (tid == 0) {
        int acc = 0;
        for (int e = 0; e < a.E; ++e) {
            tile_start[e] = acc;
            acc += ((a.counts[e] + TC_BM - 1) / TC_BM) * a.n_tiles;
        }
        tile_start[a.E] = acc;
        *abort_flag = 0;
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(tfull0 + 8 * s, 1);
            mbar_init(tempty0 + 8 * s, 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TC_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = tile_start[a.E];
    const int k_blocks = a.K / TC_BK;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            TileCursor cur;
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                int e, row0, row_end, nt;
                cur.locate(tile_start, a.counts, a.offsets, tile, a.n_tiles, e, row0, row_end, nt);
                const int brow0 = e * a.b_rows_per_expert + nt * a.b_tile_rows;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % TC_STAGES, ph = (it / TC_STAGES) & 1u;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t dst = smem_u32(tiles + s * TC_STAGE_BYTES);
                    mbar_expect_tx(full0 + 8 * s, TC_STAGE_BYTES);
                    tma_load_2d(dst, &map_a, kb * TC_BK, row0, full0 + 8 * s);
                    tma_load_2d(dst + TC_BM * TC_BK * 2, &map_b0, kb * TC_BK, brow0, full0 + 8 * s);
                    tma_load_2d(dst + 2 * TC_BM * TC_BK * 2, &map_b1, kb * TC_BK, brow0 + a.b1_row_offset, full0 + 8 * s);
                }
            }
            if (ok) {
                // tail: the commits that release the last stages arrive on this CTA's mbarriers
                // asynchronously; they must land before the shared memory goes to another CTA
                for (uint32_t back = 1; back <= TC_STAGES && back <= it; ++back) {
                    const uint32_t j = it - back, s = j % TC_STAGES, ph = (j / TC_STAGES) & 1u;
                    if (!mbar_wait(empty0 + 8 * s, ph, abort_flag)) break;
                }
            }
            if (!ok) {
                // gave up: let the copies already issued land before the CTA's shared memory goes away
                for (uint32_t back = 1; back <= TC_STAGES && back <= it; ++back) {
                    const uint32_t j = it - back, s = j % TC_STAGES, ph = (j / TC_STAGES) & 1u;
                    for (uint32_t spin = 0; spin < (1u << 16) && !mbar_test(full0 + 8 * s, ph); ++spin) __nanosleep(64);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t fmt = sizeof(TIN) == 2 && std::is_same<TIN, __nv_bfloat16>::value ? 1u : 0u;
            // one M=128, N=256, K=16 MMA per K step: the two 128-row weight tiles of a stage lie back
            // to back in shared memory (8-row groups 1024 bytes apart throughout), so one descriptor
            // covers both and the accumulator's two halves are columns 0..127 and 128..255
            const uint32_t idesc = make_idesc(fmt, 128, 256);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tcount) {
                const uint32_t as = tcount & 1u, aph = (tcount >> 1) & 1u;
                if (!mbar_wait(tempty0 + 8 * as, aph ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d0 = tmem_base + as * 256u;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % TC_STAGES, ph = (it / TC_STAGES) & 1u;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(tiles + s * TC_STAGE_BYTES);
                    const uint64_t da = smem_desc_sw128(sa);
                    const uint64_t db = smem_desc_sw128(sa + TC_BM * TC_BK * 2);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) umma_f16(d0, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);          // stage reusable once these MMAs have read it
                }
                if (ok) umma_commit(tfull0 + 8 * as);      // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----------------
        const uint32_t quarter = warp & 3u;
        TileCursor cur;
        uint32_t tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tcount) {
            int e, row0, row_end, nt;
            cur.locate(tile_start, a.counts, a.offsets, tile, a.n_tiles, e, row0, row_end, nt);
            const uint32_t as = tcount & 1u, aph = (tcount >> 1) & 1u;
            if (!mbar_wait(tfull0 + 8 * as, aph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = row0 + (int)quarter * 32 + lane;
            const bool valid = row < row_end;
            const uint32_t t0 = tmem_base + ((quarter * 32u) << 16) + as * 256u;
            if constexpr (FUSED) {
                TOUT* orow = reinterpret_cast<TOUT*>(a.out) + (size_t)row * a.ld_out + (size_t)nt * 128;
#pragma unroll 1
                for (int c = 0; c < 128; c += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld32(t0 + c, g);
                    tmem_ld32(t0 + 128 + c, u);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 v;
                            v.x = pack2<TOUT>(silu_fast(__uint_as_float(g[j + 0])) * __uint_as_float(u[j + 0]),
                                              silu_fast(__uint_as_float(g[j + 1])) * __uint_as_float(u[j + 1]));
                            v.y = pack2<TOUT>(silu_fast(__uint_as_float(g[j + 2])) * __uint_as_float(u[j + 2]),
                                              silu_fast(__uint_as_float(g[j + 3])) * __uint_as_float(u[j + 3]));
                            v.z = pack2<TOUT>(silu_fast(__uint_as_float(g[j + 4])) * __uint_as_float(u[j + 4]),
                                              silu_fast(__uint_as_float(g[j + 5])) * __uint_as_float(u[j + 5]));
                            v.w = pack2<TOUT>(silu_fast(__uint_as_float(g[j + 6])) * __uint_as_float(u[j + 6]),
                                              silu_fast(__uint_as_float(g[j + 7])) * __uint_as_float(u[j + 7]));
                            *reinterpret_cast<uint4*>(orow + c + j) = v;
                        }
                    }
                }
            } else if constexpr (sizeof(TOUT) == 4) {
                TOUT* orow = reinterpret_cast<TOUT*>(a.out) + (size_t)row * a.ld_out + (size_t)nt * 256;
#pragma unroll 1
                for (int c = 0; c < 256; c += 32) {
                    uint32_t d[32];
                    tmem_ld32(t0 + c, d);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<uint4*>(reinterpret_cast<float*>(orow) + c + j) =
                                make_uint4(d[j], d[j + 1], d[j + 2], d[j + 3]);
                    }
                }
            } else {
                // 16-bit output: where this lane's row goes (its own buffer, or the buffer of the
                // rank the row came from); then 64 columns at a time through shared memory, so that
                // a store instruction of the warp writes 128 contiguous bytes of each of 4 rows
                // instead of 16 bytes of each of 32 rows - what a store across NVLink needs
                unsigned char* dptr = nullptr;
                if (valid) {
                    if (a.ret_seg) {
                        int lo = 0, hi = a.n_seg;                // last segment that starts at or before row
                        while (hi - lo > 1) {
                            const int mid = (lo + hi) >> 1;
                            if (a.ret_seg[mid] <= row) lo = mid; else hi = mid;
                        }
                        const int64_t drow = (int64_t)a.ret_dst[lo] + (row - a.ret_seg[lo]);
                        if (drow >= 0 && drow < a.back_rows)
                            dptr = reinterpret_cast<unsigned char*>(a.back[lo % a.world]) + (size_t)drow * a.ld_out * 2;
                        else
                            atomicOr(a.status, STATUS_BOUNDS);
                    } else {
                        dptr = reinterpret_cast<unsigned char*>(a.out) + (size_t)row * a.ld_out * 2;
                    }
                    if (dptr) dptr += (size_t)nt * 256 * 2;
                }
                uint4* stg = reinterpret_cast<uint4*>(epi_stage + quarter * TC_EPI_STAGE_BYTES);
#pragma unroll 1
                for (int c = 0; c < 256; c += 64) {
                    uint32_t d0[32], d1[32];
                    tmem_ld32(t0 + c, d0);
                    tmem_ld32(t0 + c + 32, d1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 v, w;
                        v.x = pack2<TIN>(__uint_as_float(d0[8 * j + 0]), __uint_as_float(d0[8 * j + 1]));
                        v.y = pack2<TIN>(__uint_as_float(d0[8 * j + 2]), __uint_as_float(d0[8 * j + 3]));
                        v.z = pack2<TIN>(__uint_as_float(d0[8 * j + 4]), __uint_as_float(d0[8 * j + 5]));
                        v.w = pack2<TIN>(__uint_as_float(d0[8 * j + 6]), __uint_as_float(d0[8 * j + 7]));
                        w.x = pack2<TIN>(__uint_as_float(d1[8 * j + 0]), __uint_as_float(d1[8 * j + 1]));
                        w.y = pack2<TIN>(__uint_as_float(d1[8 * j + 2]), __uint_as_float(d1[8 * j + 3]));
                        w.z = pack2<TIN>(__uint_as_float(d1[8 * j + 4]), __uint_as_float(d1[8 * j + 5]));
                        w.w = pack2<TIN>(__uint_as_float(d1[8 * j + 6]), __uint_as_float(d1[8 * j + 7]));
                        // piece index swizzled by the row: the 32 lanes of a store hit 32 banks x 4
                        stg[lane * 8 + (j ^ (lane & 7))] = v;
                        stg[lane * 8 + ((j + 4) ^ (lane & 7))] = w;
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int idx = i * 32 + lane, r = idx >> 3, pc = idx & 7;
                        const uint4 v = stg[r * 8 + (pc ^ (r & 7))];
                        unsigned char* p = reinterpret_cast<unsigned char*>(
                            __shfl_sync(0xFFFFFFFFu, reinterpret_cast<unsigned long long>(dptr), r));
                        if (p) *reinterpret_cast<uint4*>(p + c * 2 + pc * 16) = v;
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            mbar_arrive(tempty0 + 8 * as);
        }
    }
    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicOr(a.status, STATUS_TIMEOUT);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TC_TMEM_COLS);
    }
}

// gather the routed rows in sorted order: xs[p, :] = x[row_token[p], :]   (16-bit rows).  A warp per
// row, up to eight 16-byte loads per lane issued before the first store.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ row_token,
                                                          uint4* __restrict__ xs, int64_t rows, int vec_per_row) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < rows; p += warps) {
        const uint4* src = x + (size_t)row_token[p] * vec_per_row;
        uint4* dst = xs + (size_t)p * vec_per_row;
        for (int i0 = lane; i0 < vec_per_row; i0 += 256) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + 32 * u < vec_per_row) v[u] = src[i0 + 32 * u];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (i0 + 32 * u < vec_per_row) dst[i0 + 32 * u] = v[u];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int encode_tiled_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, uint32_t elem_bytes,
                    uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                    CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return MUMMU_ERR_DEVICE;
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * elem_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed (%d) for a [%llu, %llu] view", (int)r, (unsigned long long)outer,
                  (unsigned long long)inner);
        return MUMMU_ERR_DEVICE;
    }
    return MUMMU_OK;
}

// [rows, K] 16-bit row-major view, box = 64 (K) x 128 (rows), 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t k) {
    return encode_tiled_2d(map, base,
                           dtype == MUMMU_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, k,
                           rows, TC_BK, TC_BM, CU_TENSOR_MAP_SWIZZLE_128B);
}

bool prefill_tc_supported(const MummuMoeConfig& c, int64_t rows_total) {
    return (c.weight_dtype == MUMMU_BF16 || c.weight_dtype == MUMMU_F16) && c.act_dtype == c.weight_dtype &&
           c.hidden % 256 == 0 && c.inter % 128 == 0 && rows_total >= 1;
}

static size_t tc_smem_bytes(int E) {
    return 1024 + (size_t)TC_STAGES * TC_STAGE_BYTES + (2 * TC_STAGES + 4) * 8 + 16 + (size_t)(E + 1) * 4 + 64 + 16 +
           4 * TC_EPI_STAGE_BYTES;
}

// banks: gate, up, down as [experts_local, out, in] in the activation's 16-bit type (the handle's
// own banks, or the expanded image of its Q4_K banks)
template <typename TIN>
static int launch_tc_typed(MummuMoe* m, const void* xs, int64_t rows_cap, const int32_t* counts,
                           const int32_t* offsets, void* ys, int ys_dtype, const void* const* banks, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    CUtensorMap map_x, map_h, map_g, map_u, map_d;
    int rc;
    if ((rc = make_map(&map_x, xs, c.act_dtype, (uint64_t)rows_cap, c.hidden))) return rc;
    if ((rc = make_map(&map_h, m->hact, c.act_dtype, (uint64_t)rows_cap, c.inter))) return rc;
    if ((rc = make_map(&map_g, banks[MUMMU_BANK_GATE], c.act_dtype, (uint64_t)c.experts_local * c.inter, c.hidden))) return rc;
    if ((rc = make_map(&map_u, banks[MUMMU_BANK_UP], c.act_dtype, (uint64_t)c.experts_local * c.inter, c.hidden))) return rc;
    if ((rc = make_map(&map_d, banks[MUMMU_BANK_DOWN], c.act_dtype, (uint64_t)c.experts_local * c.hidden, c.inter))) return rc;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c.device);
    const size_t smem = tc_smem_bytes(c.experts_local);

    TcArgs g{};
    g.counts = counts;
    g.offsets = offsets;
    g.E = c.experts_local;
    g.K = c.hidden;
    g.n_tiles = c.inter / 128;
    g.b_rows_per_expert = c.inter;
    g.b_tile_rows = 128;
    g.b1_row_offset = 0;
    g.out = m->hact;
    g.ld_out = c.inter;
    g.status = m->status;
    {
        MUMMU_CUDA_TRY(allow_big_smem(grouped_gemm_tc_kernel<TIN, TIN, true>, c.device));
        LaunchScope scope(m, s, "tc_gate_up");
        grouped_gemm_tc_kernel<TIN, TIN, true><<<sms, TC_THREADS, smem, s>>>(map_x, map_g, map_u, g);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    TcArgs d{};
    d.counts = counts;
    d.offsets = offsets;
    d.E = c.experts_local;
    d.K = c.inter;
    d.n_tiles = c.hidden / 256;
    d.b_rows_per_expert = c.hidden;
    d.b_tile_rows = 256;
    d.b1_row_offset = 128;
    d.out = ys;
    d.ld_out = c.hidden;
    d.status = m->status;
    if (m->scatter.offered && ys_dtype != MUMMU_F32) {
        d.ret_seg = m->ret_seg;
        d.ret_dst = m->ret_dst;
        d.n_seg = c.experts_local * m->scatter.world;
        d.world = m->scatter.world;
        d.back_rows = m->scatter.back_rows;
        for (int r = 0; r < m->scatter.world; ++r) d.back[r] = m->scatter.back[r];
        m->scatter.used = true;
    }
    LaunchScope scope(m, s, "tc_down");
    if (ys_dtype == MUMMU_F32) {
        MUMMU_CUDA_TRY(allow_big_smem(grouped_gemm_tc_kernel<TIN, float, false>, c.device));
        grouped_gemm_tc_kernel<TIN, float, false><<<sms, TC_THREADS, smem, s>>>(map_h, map_d, map_d, d);
    } else {
        MUMMU_CUDA_TRY(allow_big_smem(grouped_gemm_tc_kernel<TIN, TIN, false>, c.device));
        grouped_gemm_tc_kernel<TIN, TIN, false><<<sms, TC_THREADS, smem, s>>>(map_h, map_d, map_d, d);
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// xs: sorted rows [rows_cap, hidden] in the activation dtype (rows_cap = allocated rows, used as
// the tensor-map bound); ys: [rows, hidden] in ys_dtype (F32 or the activation dtype)
int launch_experts_tc(MummuMoe* m, const void* xs, int64_t rows_cap, const int32_t* counts,
                      const int32_t* offsets, void* ys, int ys_dtype, cudaStream_t s) {
    const void* banks[3] = {m->bank[0], m->bank[1], m->bank[2]};
    if (m->cfg.act_dtype == MUMMU_BF16)
        return launch_tc_typed<__nv_bfloat16>(m, xs, rows_cap, counts, offsets, ys, ys_dtype, banks, s);
    return launch_tc_typed<__half>(m, xs, rows_cap, counts, offsets, ys, ys_dtype, banks, s);
}

// ------------------------------------------------------------------------------------------------
// Q4_K banks on the tensor cores: experts with rows are expanded to f16 (one warp per 144-byte
// super-block: 8 values per lane, the reference's operation order of gguf.rs:1685-1726 in f32, one
// rounding to f16), then the same two grouped GEMMs.  For calls with more rows than the
// packed-weight kernels take (a prompt of more than 256 tokens).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) q4k_expand_f16_kernel(const uint8_t* __restrict__ src, __half* __restrict__ dst,
                                                             int64_t n_blocks, int64_t blocks_per_expert,
                                                             const int32_t* __restrict__ counts) {
    const int lane = threadIdx.x & 31;
    const int j = lane >> 2, chunk = j >> 1, b0 = (lane & 3) * 8;
    const int jm = j & 3;                                       // position inside the packed scale words
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < n_blocks; b += warps) {
        if (counts[b / blocks_per_expert] == 0) continue;        // nobody routed here this call
        const uint8_t* blk = src + (size_t)b * Q4K_BLOCK_BYTES;
        // the 16-byte head (d, dmin, 12 packed scale bytes) in one load - the same address for the
        // whole warp - and this lane's 8 quant bytes
        const uint4 head = *reinterpret_cast<const uint4*>(blk);
        const uint2 raw = *reinterpret_cast<const uint2*>(blk + 16 + chunk * 32 + b0);
        const float d = __half2float(__ushort_as_half((unsigned short)(head.x & 0xFFFFu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(head.x >> 16)));
        // 6-bit unpack (gguf.rs:1688-1695) on the words: scales[0..3] = head.y, [4..7] = head.z, [8..11] = head.w
        const uint32_t s0 = (head.y >> (8 * jm)) & 0xFFu, s1 = (head.z >> (8 * jm)) & 0xFFu, s2 = (head.w >> (8 * jm)) & 0xFFu;
        const uint32_t sc_i = j < 4 ? (s0 & 63u) : ((s2 & 0x0Fu) | ((s0 >> 6) << 4));
        const uint32_t mn_i = j < 4 ? (s1 & 63u) : ((s2 >> 4) | ((s1 >> 6) << 4));
        const float dsc = __fmul_rn(d, (float)sc_i), off = __fmul_rn(dmin, (float)mn_i);
        // the lane's 8 values are all low or all high nibbles of its 8 bytes
        const uint32_t w0 = (j & 1) ? (raw.x >> 4) & 0x0F0F0F0Fu : raw.x & 0x0F0F0F0Fu;
        const uint32_t w1 = (j & 1) ? (raw.y >> 4) & 0x0F0F0F0Fu : raw.y & 0x0F0F0F0Fu;
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = i < 2 ? w0 : w1;
            const float qa = (float)((w >> (16 * (i & 1))) & 0xFFu), qb = (float)((w >> (16 * (i & 1) + 8)) & 0xFFu);
            const __half2 h = __floats2half2_rn(__fsub_rn(__fmul_rn(dsc, qa), off), __fsub_rn(__fmul_rn(dsc, qb), off));
            o[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(dst + (size_t)b * 256 + lane * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Q4_K and, through the generic element decoders, its sibling block formats
bool q4k_tc_supported(const MummuMoeConfig& c, int64_t rows_total) {
    const bool packed = c.weight_dtype == MUMMU_Q4_K || c.weight_dtype == MUMMU_Q8_0 || c.weight_dtype == MUMMU_Q5_K ||
                        c.weight_dtype == MUMMU_Q6_K;
    return packed && c.act_dtype == MUMMU_F16 && c.hidden % 256 == 0 && c.inter % 256 == 0 && rows_total >= 1;
}

int launch_experts_q4k_tc(MummuMoe* m, const void* xs, int64_t rows_cap, const int32_t* counts, const int32_t* offsets,
                          void* ys, int ys_dtype, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    const int64_t per_bank = (int64_t)c.experts_local * c.inter * c.hidden;
    // the image is scratch: a stack of layers that shares scratch shares it too (it lives in the
    // layer the others adopted their scratch from, which must outlive them as for the rest)
    MummuMoe* owner = m->scratch_donor && m->scratch_donor->cfg.experts_local == c.experts_local ? m->scratch_donor : m;
    for (int b = 0; b < 3; ++b) {
        if (owner->wexp[b]) continue;
        MUMMU_CUDA_TRY(cudaMalloc((void**)&owner->wexp[b], (size_t)per_bank * sizeof(__half)));
    }
    const int64_t blocks_per_expert = (int64_t)c.inter * c.hidden / 256, n_blocks = blocks_per_expert * c.experts_local;
    if (c.weight_dtype != MUMMU_Q4_K) {
        LaunchScope scope(m, s, "block_expand");
        for (int b = 0; b < 3; ++b) {
            int rc = launch_block_expand_f16(m, b, owner->wexp[b], counts, s);
            if (rc) return rc;
        }
    } else {
        LaunchScope scope(m, s, "q4k_expand");
        for (int b = 0; b < 3; ++b) {
            q4k_expand_f16_kernel<<<148 * 16, 256, 0, s>>>((const uint8_t*)m->bank[b], owner->wexp[b], n_blocks,
                                                          blocks_per_expert, counts);
        }
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    const void* banks[3] = {owner->wexp[0], owner->wexp[1], owner->wexp[2]};
    return launch_tc_typed<__half>(m, xs, rows_cap, counts, offsets, ys, ys_dtype, banks, s);
}

int launch_gather_rows(MummuMoe* m, const void* x, const int32_t* row_token, void* xs, int64_t rows,
                       cudaStream_t s) {
    if (rows == 0) return MUMMU_OK;
    const int vec = m->cfg.hidden * 2 / 16;
    int64_t blocks = rows < 8 ? 1 : (rows / 8 < 148 * 8 ? (rows + 7) / 8 : 148 * 8);     // a warp per row
    LaunchScope scope(m, s, "gather_rows");
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint4*)x, row_token, (uint4*)xs, rows, vec);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

}  // namespace mummu
