// Decode-regime expert bank over GGUF Q4_K weights on the 5th-generation tensor cores.
//
// Same math as decode_q4k.cu (reference: crates/mummu/src/nn/moe.rs:314-316 over weights
// dequantised as in crates/mummu/src/gguf.rs:1701-1726), different machine mapping: the CUDA
// cores only turn nibbles into f16 operands; the products, the token tile and the accumulators
// live in the tensor core (tcgen05.mma, operands in shared memory, accumulators in TMEM), so a
// warp issues no MMA, holds no accumulator and reads no B fragment.
//
//   CTA = (active expert, 128 output rows of matrix 0 and of matrix 1)
//         gate/up: matrix 0 = gate rows, matrix 1 = the same rows of up      -> silu(g)*u, f16
//         down   : matrix 0 / 1 = two adjacent 128-row blocks of down        -> f32
//   per 256-value super-block sb, per matrix m:
//     TMA warp     : one box of 128 rows x 144 bytes (the raw super-blocks) into a raw ring
//     16 producers : thread = one weight row = one TMEM lane.  A row's 64-value chunk becomes 64
//                    exact f16 integers sc_j*q (LOP3 + HFMA2 as in decode_q4k.cu) written with
//                    ONE tcgen05.st into the A operand slot in TMEM (32 columns); the expanded
//                    weights never touch shared memory, which could not carry 4x the raw bytes
//                    in and out again at the rate HBM delivers them.  The row's eight 6-bit
//                    minimums (16 bytes) go to a small shared-memory A tile.
//     MMA thread   : acc[128 x 16 tokens] += A(TMEM) x token chunk(shared) (4 MMAs of K = 16 per
//                    slot) and mn = minimums(shared) x (sub-block sums of the tokens), one MMA of
//                    K = 16, into an accumulator block of its own
//     4 epilogue warps (thread = one TMEM lane = one row): y += d*acc - dmin*mn in f32 with the
//                    same three roundings as the other decode kernels, then the activation/store
// The token tile (up to 16 sorted rows, all of K) is staged once per pass in the same permuted K
// order the producers emit.  Every mbarrier wait is bounded; when one runs out the CTA raises the
// status word, every role stops at its next wait, TMEM is freed and the kernel returns.
#include <cstdlib>

#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace mummu {

constexpr int DU_PRODUCER_WARPS = 16;            // 2 matrices x 2 chunk halves x 4 row quarters
constexpr int DU_WARP_TMA = 16;
constexpr int DU_WARP_MMA = 17;
constexpr int DU_THREADS = 22 * 32;
constexpr uint32_t DU_RAW = 128 * Q4K_BLOCK_BYTES;   // 18432
constexpr uint32_t DU_CHUNK = 16 * 128;          // token chunk [16 tokens x 64 f16] = 2 KiB
constexpr uint32_t DU_TMEM_COLS = 512;
// TMEM columns, in blocks of 32.  Every accumulator (16 columns) has a 32-column block to
// itself: with a second accumulator, or an A operand, in the other half of a block, results were
// intermittently wrong whenever the MMAs touching the two halves were in flight together
// (measured on B200; the same kernel with exclusive blocks is bit-reproducible).
//   [0, 128)   main accumulators (matrix, buffer)
//   [128, 256) minimum accumulators (matrix, buffer)
//   [256, 512) A slots (matrix, chunk half, chunk): 32 columns = 64 halves per row
constexpr uint32_t DU_TM_ACC = 0, DU_TM_MN = 128, DU_TM_A = 256;
constexpr uint32_t DU_AMIN = 128 * 128;          // minimums tile [128 rows x 64 f16], 128-byte swizzle
constexpr uint32_t DU_SPIN_LIMIT = 2u << 20;

struct UmmaArgs {
    const __half* x;            // gate/up: layer input [tokens, K]; down: hact [rows, K]
    const int32_t* row_token;   // gate/up: sorted row -> token; down: null (identity)
    const int32_t* counts;
    const int32_t* offsets;
    const int32_t* active;
    const int32_t* n_active;
    const uint8_t* w0;          // bank of matrix 0 (gate, or down)
    const uint8_t* w1;          // bank of matrix 1 (up, or down again)
    int row_bytes;
    int K;
    int rows_per_expert;        // weight rows per expert
    int m_tiles;                // CTAs per expert
    int ld_out;
    void* out;
    int raw_stages;
    int32_t* status;
};

__device__ __forceinline__ uint32_t du_hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t du_hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t du_hsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// (w & mask) | bits in one logic op
__device__ __forceinline__ uint32_t du_and_or(uint32_t w, uint32_t mask, uint32_t bits) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(w), "r"(mask), "r"(bits));
    return d;
}
__device__ __forceinline__ uint4 du_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void du_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// this thread's TMEM lane, 32 consecutive 32-bit columns
__device__ __forceinline__ void du_tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void du_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// 16 consecutive f32 columns of this thread's TMEM lane
__device__ __forceinline__ void du_tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]^T: the A operand is 128 lanes x 8 columns (16 halves per row)
__device__ __forceinline__ void du_umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Stage one pass of the token tile: rows first_row .. first_row+npass-1 (zero beyond), every
// 64-value chunk as [16 tokens x 128 B] with the 128-byte swizzle, values inside each group of
// four in the order (e0, e2, e1, e3) that the nibble extraction produces; plus the f16 sums of x
// over each 32-value sub-block, laid out as the B operand of the minimum MMA: for super-block sb,
// unit 2*(sb%4) of chunk sb/4 in the variant for matrix 0, unit 2*(sb%4)+1 in the variant for
// matrix 1, zeros in the partner unit (where the A side holds the other matrix's minimums).
__device__ __forceinline__ void du_stage_tokens(const UmmaArgs& a, unsigned char* b_tile, unsigned char* b_min,
                                                int nb4, int first_row, int npass, int tid) {
    const int groups_per_row = a.K >> 3;
    for (int i = tid; i < 2 * nb4 * (int)(DU_CHUNK / 16); i += DU_THREADS)
        reinterpret_cast<uint4*>(b_min)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    for (int idx = tid; idx < 16 * groups_per_row; idx += DU_THREADS) {
        const int tok = idx / groups_per_row;
        const int q = idx - tok * groups_per_row;      // 8-value group along K
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < npass) {
            const int p = first_row + tok;
            const int64_t src = a.row_token ? a.row_token[p] : p;
            v = *reinterpret_cast<const uint4*>(a.x + src * a.K + (size_t)q * 8);
        }
        const int chunk = q >> 3, u = q & 7;
        uint4 o;
        o.x = __byte_perm(v.x, v.y, 0x5410);
        o.y = __byte_perm(v.x, v.y, 0x7632);
        o.z = __byte_perm(v.z, v.w, 0x5410);
        o.w = __byte_perm(v.z, v.w, 0x7632);
        *reinterpret_cast<uint4*>(b_tile + (size_t)chunk * DU_CHUNK + tok * 128 + ((u ^ (tok & 7)) << 4)) = o;
        const __half2* h2 = reinterpret_cast<const __half2*>(&v);
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 f2 = __half22float2(h2[k]);
            s += f2.x;
            s += f2.y;
        }
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
        if ((q & 3) == 0) {
            const int sb = q >> 5, j = (q >> 2) & 7;
            const __half hs = __float2half_rn(s);
            const int c4 = sb >> 2, unit = 2 * (sb & 3);
            unsigned char* row0 = b_min + (size_t)c4 * DU_CHUNK + tok * 128;
            unsigned char* row1 = row0 + (size_t)nb4 * DU_CHUNK;
            *reinterpret_cast<__half*>(row0 + ((unit ^ (tok & 7)) << 4) + j * 2) = hs;
            *reinterpret_cast<__half*>(row1 + (((unit + 1) ^ (tok & 7)) << 4) + j * 2) = hs;
        }
    }
}

template <bool GATEUP>
__global__ void __launch_bounds__(DU_THREADS, 1)
decode_q4k_umma_kernel(UmmaArgs a, const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ai = blockIdx.x / a.m_tiles;
    const int mt = blockIdx.x - ai * a.m_tiles;
    if (ai >= *a.n_active) return;
    const int e = a.active[ai];
    const int cnt = a.counts[e];
    const int base = a.offsets[e];
    const int npasses = (cnt + 15) >> 4;
    if (npasses == 0) return;

    const int nsb = a.K >> 8;
    const int nb4 = (nsb + 3) >> 2;
    const int R = a.raw_stages;
    const uint32_t s0 = smem_u32(smem);
    if (s0 & 1023u) {   // the swizzled tiles need 1024-byte alignment
        if (tid == 0) atomicOr(a.status, STATUS_TIMEOUT);
        return;
    }
    const uint32_t off_amin = 0;
    const uint32_t off_btile = DU_AMIN;
    const uint32_t off_bmin = off_btile + (uint32_t)(a.K >> 6) * DU_CHUNK;
    const uint32_t off_raw = off_bmin + 2u * (uint32_t)nb4 * DU_CHUNK;
    const uint32_t off_bars = off_raw + 2u * R * DU_RAW;
    const uint32_t bars = s0 + off_bars;
    // barrier indices: raw ring [m][stage]; A slots [m][th][c]; accumulators [m][buffer]
    const uint32_t RAW_FULL = 0, RAW_EMPTY = 2 * R, A_FULL = 4 * R, A_EMPTY = 4 * R + 8, ACC_FULL = 4 * R + 16,
                   ACC_EMPTY = 4 * R + 20, NBARS = 4 * R + 24;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + off_bars + NBARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
#define BAR(i) (bars + 8u * (uint32_t)(i))

    if (tid == 0) {
        *abort_flag = 0;
        for (int m = 0; m < 2; ++m) {
            for (int s = 0; s < R; ++s) {
                mbar_init(BAR(RAW_FULL + m * R + s), 1);
                mbar_init(BAR(RAW_EMPTY + m * R + s), 256);
            }
            for (int i = 0; i < 4; ++i) {
                mbar_init(BAR(A_FULL + m * 4 + i), 128);
                mbar_init(BAR(A_EMPTY + m * 4 + i), 1);
            }
            for (int i = 0; i < 2; ++i) {
                mbar_init(BAR(ACC_FULL + m * 2 + i), 1);
                mbar_init(BAR(ACC_EMPTY + m * 2 + i), 128);
            }
        }
        mbar_init_fence();
        fence_proxy_async_smem();
    }
    if (warp == DU_WARP_MMA) {
        tmem_alloc(smem_u32(tmem_slot), DU_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // first weight row of this CTA in matrix m
    const int wrow0 = GATEUP ? e * a.rows_per_expert + mt * 128 : e * a.rows_per_expert + mt * 256;
    const int wrow1 = GATEUP ? wrow0 : wrow0 + 128;

    // raw loads of the first super-blocks start before the tokens are staged
    uint32_t tma_it = 0;
    const uint32_t tma_total = (uint32_t)npasses * nsb;
    if (warp == DU_WARP_TMA && lane == 0) {
        for (; tma_it < (uint32_t)R && tma_it < tma_total; ++tma_it) {
            const int sb = tma_it % nsb;
            for (int m = 0; m < 2; ++m) {
                const uint32_t bar = BAR(RAW_FULL + m * R + tma_it);
                mbar_expect_tx(bar, DU_RAW);
                tma_load_2d(s0 + off_raw + (m * R + tma_it) * DU_RAW, m ? &map1 : &map0, sb * Q4K_BLOCK_BYTES,
                            m ? wrow1 : wrow0, bar);
            }
        }
    }
    // the minimums tile starts as zeros: a K step also covers the other matrix's unit, which meets
    // zeros on the token side and must therefore hold finite values from the start
    for (int i = tid; i < (int)(DU_AMIN / 16); i += DU_THREADS)
        reinterpret_cast<uint4*>(smem + off_amin)[i] = make_uint4(0, 0, 0, 0);
    du_stage_tokens(a, smem + off_btile, smem + off_bmin, nb4, base, min(16, cnt), tid);
    fence_proxy_async_smem();
    __syncthreads();

    for (int pass = 0; pass < npasses; ++pass) {
        const int npass = min(16, cnt - pass * 16);
        if (warp < DU_PRODUCER_WARPS) {
            // ---------------- producers: thread = weight row = TMEM lane ----------------
            const int m = warp >> 3, th = (warp >> 2) & 1, rq = warp & 3;
            const int row = rq * 32 + lane;
            const uint32_t lane_field = ((uint32_t)rq * 32u) << 16;
            const uint32_t k1024 = 0x64006400u, lo_mask = 0x000F000Fu, hi_mask = 0x00F000F0u;
            bool ok = true;
            for (int sb = 0; ok && sb < nsb; ++sb) {
                const uint32_t it = (uint32_t)(pass * nsb + sb);
                const uint32_t rs = it % R, rph = (it / R) & 1u;
                if (!mbar_wait_bounded(BAR(RAW_FULL + m * R + rs), rph, abort_flag, DU_SPIN_LIMIT)) break;
                const uint32_t rrow = s0 + off_raw + (m * R + rs) * DU_RAW + (uint32_t)row * Q4K_BLOCK_BYTES;
                const uint4 h = du_lds128(rrow);
                // 6-bit scales and minimums of the eight sub-blocks (gguf.rs:1685-1698)
                const uint32_t sc_a = h.y & 0x3F3F3F3Fu;                                      // sc 0..3
                const uint32_t sc_b = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);       // sc 4..7
                if (th == 0) {
                    const uint32_t mn_a = h.z & 0x3F3F3F3Fu;                                  // m 0..3
                    const uint32_t mn_b = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
                    // bytes (a, 0x64, b, 0x64) = halves (1024+a, 1024+b); minus 1024 -> the integers
                    const uint32_t m01 = du_hsub2(__byte_perm(mn_a, 0x64646464u, 0x4140), k1024);
                    const uint32_t m23 = du_hsub2(__byte_perm(mn_a, 0x64646464u, 0x4342), k1024);
                    const uint32_t m45 = du_hsub2(__byte_perm(mn_b, 0x64646464u, 0x4140), k1024);
                    const uint32_t m67 = du_hsub2(__byte_perm(mn_b, 0x64646464u, 0x4342), k1024);
                    // unit 2*(sb%4)+m of this row of the minimums tile (a four-deep ring over sb: the
                    // MMA that read this unit four super-blocks ago completed before the A slots of
                    // the super-blocks since were released to this thread)
                    du_sts128(s0 + off_amin + (uint32_t)row * 128u + ((((uint32_t)(2 * (sb & 3) + m)) ^ (uint32_t)(row & 7)) << 4),
                              m01, m23, m45, m67);
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    // chunk t = 2*th + c: sub-blocks 2t (low nibbles) and 2t+1 (high nibbles)
                    const uint32_t qoff = 16u + 32u * (uint32_t)(2 * th + c);
                    const uint4 qa = du_lds128(rrow + qoff);
                    const uint4 qb = du_lds128(rrow + qoff + 16u);
                    const uint32_t scw = th ? sc_b : sc_a;
                    const uint32_t pair = du_hsub2(__byte_perm(scw, 0x64646464u, c ? 0x4342 : 0x4140), k1024);
                    const uint32_t sc_lo = __byte_perm(pair, 0, 0x1010);
                    const uint32_t hi2 = __byte_perm(pair, 0, 0x3232);
                    const uint32_t c_lo = du_hmul2(sc_lo, 0xE400E400u);    // * -1024
                    const uint32_t sc_hi = du_hmul2(hi2, 0x2C002C00u);     // * 1/16
                    const uint32_t c_hi = du_hmul2(hi2, 0xD400D400u);      // * -64
                    const uint32_t wq[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    uint32_t v[32];   // columns 0..15: sub-block 2t, 16..31: sub-block 2t+1
#pragma unroll
                    for (int w = 0; w < 8; ++w) {
                        const uint32_t w0 = wq[w], sw = w0 >> 8;
                        v[2 * w] = du_hfma2(du_and_or(w0, lo_mask, k1024), sc_lo, c_lo);
                        v[2 * w + 1] = du_hfma2(du_and_or(sw, lo_mask, k1024), sc_lo, c_lo);
                        v[16 + 2 * w] = du_hfma2(du_and_or(w0, hi_mask, k1024), sc_hi, c_hi);
                        v[16 + 2 * w + 1] = du_hfma2(du_and_or(sw, hi_mask, k1024), sc_hi, c_hi);
                    }
                    // The raw stage is released only here, after instructions that consumed the loaded
                    // registers have issued: an arrive placed right after the loads could overtake
                    // them, and the copy engine refills the stage as soon as the last arrive lands.
                    if (c == 1) mbar_arrive(BAR(RAW_EMPTY + m * R + rs));
                    // slot (m, th, c) is used once per super-block
                    if (!mbar_wait_bounded(BAR(A_EMPTY + m * 4 + th * 2 + c), (it & 1u) ^ 1u, abort_flag, DU_SPIN_LIMIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    du_tmem_st32(tmem_base + lane_field + DU_TM_A + (uint32_t)((m * 2 + th) * 2 + c) * 32u, v);
                    du_tmem_st_wait();
                    tc_fence_before();
                    if (th == 0 && c == 0) fence_proxy_async_smem();   // the minimums written above
                    mbar_arrive(BAR(A_FULL + m * 4 + th * 2 + c));
                }
            }
        } else if (warp == DU_WARP_TMA) {
            // ---------------- raw super-blocks ----------------
            if (lane == 0) {
                const uint32_t end = (uint32_t)(pass + 1) * nsb;
                for (; tma_it < end; ++tma_it) {
                    const uint32_t rs = tma_it % R, rph = (tma_it / R) & 1u;
                    const int sb = tma_it % nsb;
                    bool ok = true;
                    for (int m = 0; m < 2 && ok; ++m) {
                        ok = mbar_wait_bounded(BAR(RAW_EMPTY + m * R + rs), rph ^ 1u, abort_flag, DU_SPIN_LIMIT);
                        if (!ok) break;
                        const uint32_t bar = BAR(RAW_FULL + m * R + rs);
                        mbar_expect_tx(bar, DU_RAW);
                        tma_load_2d(s0 + off_raw + (m * R + rs) * DU_RAW, m ? &map1 : &map0, sb * Q4K_BLOCK_BYTES,
                                    m ? wrow1 : wrow0, bar);
                    }
                    if (!ok) break;
                }
            }
        } else if (warp == DU_WARP_MMA) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                const uint32_t idesc = make_idesc(0u, 128, 16);
                bool ok = true;
                for (int sb = 0; ok && sb < nsb; ++sb) {
                    const uint32_t it = (uint32_t)(pass * nsb + sb);
                    const uint32_t buf = it & 1u, aph = (it >> 1) & 1u;
#pragma unroll
                    for (int g = 0; g < 8 && ok; ++g) {
                        const int m = g & 1, c = g >> 2, th = (g >> 1) & 1;
                        const int t = 2 * th + c;
                        const uint64_t db = smem_desc_sw128(s0 + off_btile + (uint32_t)(sb * 4 + t) * DU_CHUNK);
                        const uint32_t blk = (uint32_t)(m * 2 + buf) * 32u;
                        const uint32_t d_acc = tmem_base + DU_TM_ACC + blk;
                        if (!mbar_wait_bounded(BAR(A_FULL + m * 4 + th * 2 + c), it & 1u, abort_flag, DU_SPIN_LIMIT)) {
                            ok = false;
                            break;
                        }
                        if (g < 2) {
                            if (!mbar_wait_bounded(BAR(ACC_EMPTY + m * 2 + buf), aph ^ 1u, abort_flag, DU_SPIN_LIMIT)) {
                                ok = false;
                                break;
                            }
                        }
                        tc_fence_after();
                        if (g < 2) {
                            // minimums x sub-block sums: K step sb%4 of token-side chunk sb/4
                            const uint64_t dam = smem_desc_sw128(s0 + off_amin) + 2u * (uint32_t)(sb & 3);
                            const uint64_t dbm =
                                smem_desc_sw128(s0 + off_bmin + (uint32_t)(m * nb4 + (sb >> 2)) * DU_CHUNK) +
                                2u * (uint32_t)(sb & 3);
                            umma_f16(tmem_base + DU_TM_MN + blk, dam, dbm, idesc, 0u);
                        }
                        const uint32_t ta = tmem_base + DU_TM_A + (uint32_t)((m * 2 + th) * 2 + c) * 32u;
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            du_umma_ts(d_acc, ta + 8u * (uint32_t)k, db + 2 * k, idesc, (g >= 2 || k != 0) ? 1u : 0u);
                        umma_commit(BAR(A_EMPTY + m * 4 + th * 2 + c));
                        if (g >= 6) umma_commit(BAR(ACC_FULL + m * 2 + buf));
                    }
                }
            }
        } else {
            // ---------------- epilogue: thread = TMEM lane = weight row ----------------
            const uint32_t quarter = (uint32_t)warp & 3u;
            const int row = (int)quarter * 32 + lane;
            float y[2][16];
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int i = 0; i < 16; ++i) y[m][i] = 0.0f;
            const uint8_t* hp0 = a.w0 + (size_t)(wrow0 + row) * a.row_bytes;
            const uint8_t* hp1 = a.w1 + (size_t)(wrow1 + row) * a.row_bytes;
            uint32_t dd0 = __ldg(reinterpret_cast<const uint32_t*>(hp0));
            uint32_t dd1 = __ldg(reinterpret_cast<const uint32_t*>(hp1));
            bool ok = true;
            for (int sb = 0; ok && sb < nsb; ++sb) {
                const uint32_t it = (uint32_t)(pass * nsb + sb);
                const uint32_t buf = it & 1u, aph = (it >> 1) & 1u;
                const uint32_t cur0 = dd0, cur1 = dd1;
                if (sb + 1 < nsb) {
                    dd0 = __ldg(reinterpret_cast<const uint32_t*>(hp0 + (size_t)(sb + 1) * Q4K_BLOCK_BYTES));
                    dd1 = __ldg(reinterpret_cast<const uint32_t*>(hp1 + (size_t)(sb + 1) * Q4K_BLOCK_BYTES));
                }
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    if (!mbar_wait_bounded(BAR(ACC_FULL + m * 2 + buf), aph, abort_flag, DU_SPIN_LIMIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    uint32_t r[32];
                    du_tmem_ld16(tmem_base + ((quarter * 32u) << 16) + DU_TM_ACC + (uint32_t)(m * 2 + buf) * 32u, r);
                    du_tmem_ld16(tmem_base + ((quarter * 32u) << 16) + DU_TM_MN + (uint32_t)(m * 2 + buf) * 32u, r + 16);
                    tmem_ld_wait();
                    tc_fence_before();
                    mbar_arrive(BAR(ACC_EMPTY + m * 2 + buf));
                    const uint32_t dd = m ? cur1 : cur0;
                    const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFFu)));
                    const float dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        y[m][i] = __fadd_rn(y[m][i], __fmaf_rn(-dmin, __uint_as_float(r[16 + i]),
                                                               __fmul_rn(d, __uint_as_float(r[i]))));
                }
            }
            if (ok) {
                const int first_row = base + pass * 16;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (i < npass) {
                        const size_t orow = (size_t)(first_row + i);
                        if (GATEUP) {
                            const float g = y[0][i], u = y[1][i];
                            const float v = (g / (1.0f + expf(-g))) * u;
                            reinterpret_cast<__half*>(a.out)[orow * a.ld_out + mt * 128 + row] = __float2half_rn(v);
                        } else {
                            float* o32 = reinterpret_cast<float*>(a.out);
                            o32[orow * a.ld_out + mt * 256 + row] = y[0][i];
                            o32[orow * a.ld_out + mt * 256 + 128 + row] = y[1][i];
                        }
                    }
                }
            }
        }
        // pass boundary: every MMA of this pass has completed (the epilogue drained the last
        // accumulators), so the token tile may be replaced
        __syncthreads();
        if (pass + 1 < npasses && !*abort_flag) {
            du_stage_tokens(a, smem + off_btile, smem + off_bmin, nb4, base + (pass + 1) * 16,
                            min(16, cnt - (pass + 1) * 16), tid);
            fence_proxy_async_smem();
        }
        __syncthreads();
        if (*abort_flag) break;
    }
    // ---------------- teardown ----------------
    // Tail: the commits that release the A slots after their last use arrive on this CTA's
    // mbarriers asynchronously.  They must have landed before the shared memory is handed to the
    // next CTA on this SM, whose freshly initialised barriers they would otherwise hit.
    if (warp == DU_WARP_MMA && lane == 0 && !*abort_flag) {
        const uint32_t last = (uint32_t)(npasses * nsb - 1);
        for (int i = 0; i < 8; ++i) mbar_wait_bounded(BAR(A_EMPTY + i), last & 1u, abort_flag, DU_SPIN_LIMIT);
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicOr(a.status, STATUS_TIMEOUT);
    if (warp == DU_WARP_MMA) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, DU_TMEM_COLS);
    }
#undef BAR
}

static size_t du_smem_bytes(int K, int R) {
    const int nsb = K >> 8, nb4 = (nsb + 3) >> 2;
    return (size_t)DU_AMIN + (size_t)(K >> 6) * DU_CHUNK + (size_t)2 * nb4 * DU_CHUNK + (size_t)2 * R * DU_RAW +
           (size_t)(4 * R + 24) * 8 + 16;
}

bool decode_umma_supported(const MummuMoeConfig& c) {
    // Opt-in: measured on B200 at the decode benchmark's shape this variant is slower than the
    // mma.sync kernels of decode_q4k.cu (about 120 us against 60 us for gate/up: one CTA of 22 warps
    // per SM, token staging and pipeline fill paid per 128-row tile), so those stay the default.
    const char* env = getenv("MUMMU_CUDA_DECODE_UMMA");
    if (!env || atoi(env) == 0) return false;
    return c.weight_dtype == MUMMU_Q4_K && c.act_dtype == MUMMU_F16 && c.hidden % 256 == 0 && c.inter % 256 == 0 &&
           du_smem_bytes(c.hidden, 2) <= 227 * 1024 && du_smem_bytes(c.inter, 2) <= 227 * 1024;
}

// Tensor map of one Q4_K bank as a [rows, row_bytes] byte view with a 128-row x 144-byte box.
static int bank_map128(MummuMoe* m, int which, int row_bytes, int64_t rows, const CUtensorMap** out) {
    CUtensorMap* map = reinterpret_cast<CUtensorMap*>(m->q4k_map128[which]);
    if (m->q4k_map128_base[which] != m->bank[which]) {
        int rc = encode_tiled_2d(map, m->bank[which], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)row_bytes,
                                 (uint64_t)rows, Q4K_BLOCK_BYTES, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        m->q4k_map128_base[which] = m->bank[which];
    }
    *out = map;
    return MUMMU_OK;
}

// One projection of the decode bank.  x: input rows (f16); row_token: sorted row -> row of x or
// null; out: gate/up -> f16 [rows, inter], down -> f32 [rows, hidden].
int launch_decode_umma(MummuMoe* m, bool gateup, const void* x, const int32_t* row_token, const int32_t* counts,
                       const int32_t* offsets, int n_experts_max, void* out, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    UmmaArgs a{};
    a.x = (const __half*)x;
    a.row_token = row_token;
    a.counts = counts;
    a.offsets = offsets;
    a.active = m->active;
    a.n_active = m->n_active;
    a.status = m->status;
    a.out = out;
    const CUtensorMap *map0 = nullptr, *map1 = nullptr;
    int rc;
    if (gateup) {
        a.w0 = (const uint8_t*)m->bank[MUMMU_BANK_GATE];
        a.w1 = (const uint8_t*)m->bank[MUMMU_BANK_UP];
        a.row_bytes = (int)bank_row_bytes(c, MUMMU_BANK_GATE);
        a.K = c.hidden;
        a.rows_per_expert = c.inter;
        a.m_tiles = c.inter / 128;
        a.ld_out = c.inter;
        const int64_t rows = (int64_t)c.experts_local * c.inter;
        if ((rc = bank_map128(m, MUMMU_BANK_GATE, a.row_bytes, rows, &map0))) return rc;
        if ((rc = bank_map128(m, MUMMU_BANK_UP, a.row_bytes, rows, &map1))) return rc;
    } else {
        a.w0 = a.w1 = (const uint8_t*)m->bank[MUMMU_BANK_DOWN];
        a.row_bytes = (int)bank_row_bytes(c, MUMMU_BANK_DOWN);
        a.K = c.inter;
        a.rows_per_expert = c.hidden;
        a.m_tiles = c.hidden / 256;
        a.ld_out = c.hidden;
        const int64_t rows = (int64_t)c.experts_local * c.hidden;
        if ((rc = bank_map128(m, MUMMU_BANK_DOWN, a.row_bytes, rows, &map0))) return rc;
        map1 = map0;
    }
    int R = 4;   // raw stages per matrix
    while (R > 2 && du_smem_bytes(a.K, R) > 227 * 1024) --R;
    a.raw_stages = R;
    const size_t smem = du_smem_bytes(a.K, R);
    LaunchScope scope(m, s, gateup ? "q4k_gate_up" : "q4k_down");
    if (gateup) {
        MUMMU_CUDA_TRY(allow_big_smem(decode_q4k_umma_kernel<true>, c.device));
        decode_q4k_umma_kernel<true><<<n_experts_max * a.m_tiles, DU_THREADS, smem, s>>>(a, *map0, *map1);
    } else {
        MUMMU_CUDA_TRY(allow_big_smem(decode_q4k_umma_kernel<false>, c.device));
        decode_q4k_umma_kernel<false><<<n_experts_max * a.m_tiles, DU_THREADS, smem, s>>>(a, *map0, *map1);
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

}  // namespace mummu
