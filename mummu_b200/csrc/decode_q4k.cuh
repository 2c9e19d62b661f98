// Shared pieces of the Q4_K decode kernels: how a packed weight reaches the tensor core, the
// token-tile layout in shared memory, and the per-(super-block, 16 rows) arithmetic every variant
// uses, so that a token's result is bit-identical whichever kernel ran.
#pragma once
#include "common.cuh"
#include "tma.cuh"

namespace mummu {

constexpr int DQ_THREADS = 256;
constexpr int DQ_WARPS = 8;

struct DecodeArgs {
    const __half* x;            // gate/up: layer input [tokens, K]; down: hact [rows, K]
    const int32_t* row_token;   // gate/up: sorted row -> token; down: null (identity)
    const int32_t* counts;      // [E] rows per expert
    const int32_t* offsets;     // [E] first sorted row per expert
    const int32_t* active;      // [n_active] expert ids with rows
    const int32_t* n_active;
    const uint8_t* w0;          // gate bank (or down bank)
    const uint8_t* w1;          // up bank (gate/up only)
    size_t expert_stride;       // bytes per expert
    int row_bytes;              // bytes per weight row
    int K;                      // input width (multiple of 256)
    int n_rt;                   // row tiles per expert (gate/up: N/16, down: N/32)
    int rb;                     // row tiles per CTA
    int ctas_per_expert;
    int ld_out;                 // output row stride (elements)
    void* out;                  // gate/up: __half hact; down: float ys
    int rows_per_expert;        // weight rows per expert (TMA row coordinate)
    int ring_depth;             // TMA stages per warp
    int pdl;                    // this launch is one of a programmatically dependent pair
    int pass_split;             // CTAs sharing the passes of an expert (grid y)
    int32_t* status;            // handle's device status word
};

// D = A*B + C with C given separately (zero registers for the first MMA of a chain)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_1688_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
        "{%7,%7,%7,%7};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// two nibbles of a word -> half2 (1024+q) resp. (1024+16q)
// (one three-input logic op each: (w & mask) | 0x64006400)
__device__ __forceinline__ uint32_t and_or(uint32_t w, uint32_t mask, uint32_t bits) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(w), "r"(mask), "r"(bits));
    return d;
}
__device__ __forceinline__ uint32_t nib_lo(uint32_t w) { return and_or(w, 0x000F000Fu, 0x64006400u); }
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) { return and_or(w, 0x00F000F0u, 0x64006400u); }

// What one lane needs from the 16-byte super-block header (f16 d, f16 dmin, 12 packed scale
// bytes; crates/mummu/src/gguf.rs:1685-1698) for its two sub-blocks 2t and 2t+1.
struct LaneScales {
    uint32_t sc_lo, c_lo;   // half2 (sc_2t, sc_2t)        and (-1024*sc_2t) x2
    uint32_t sc_hi, c_hi;   // half2 (sc_2t+1/16) x2       and (-64*sc_2t+1) x2
    uint32_t m_h2;          // half2 (m_2t, m_2t+1)
    float d, dmin;
};

__device__ __forceinline__ void lane_scales(const uint4& h, bool upper, uint32_t sel, LaneScales& r) {
    r.d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu)));
    r.dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    const uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
    // upper (sub-blocks 4..7): sc = (s2 & 0xF) | ((s0 >> 6) << 4), m = (s2 >> 4) | ((s1 >> 6) << 4)
    const uint32_t scw = upper ? ((s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)) : (s0 & 0x3F3F3F3Fu);
    const uint32_t mw = upper ? (((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)) : (s1 & 0x3F3F3F3Fu);
    const uint32_t k1024 = 0x64006400u;
    // bytes (a, 0x64, b, 0x64) = half2 (1024+a, 1024+b); minus 1024 -> the integers as halves
    const uint32_t sc2 = hsub2_u32(__byte_perm(scw, 0x64646464u, sel), k1024);
    r.m_h2 = hsub2_u32(__byte_perm(mw, 0x64646464u, sel), k1024);
    r.sc_lo = __byte_perm(sc2, 0, 0x1010);
    const uint32_t hi2 = __byte_perm(sc2, 0, 0x3232);
    r.c_lo = hmul2_u32(r.sc_lo, 0xE400E400u);    // * -1024
    r.sc_hi = hmul2_u32(hi2, 0x2C002C00u);       // * 1/16
    r.c_hi = hmul2_u32(hi2, 0xD400D400u);        // * -64
}


// Stage one pass of a CTA's token tile in shared memory: the activations of up to 8*NT sorted
// rows, already in MMA B-fragment order, plus the f16 sums of x over each 32-value sub-block.
//   s_frag [nsb][NT][8 words][8 tokens][4 lanes-of-quad] x 16 B  (lo sub-block | hi sub-block)
//   s_sxh  [nsb][NT][8 tokens][8 sub-blocks]
template <int NT>
__device__ __forceinline__ void stage_token_tile(const DecodeArgs& a, uint4* s_frag, __half* s_sxh,
                                                 int first_row, int npass, int nt_count, int tid) {
    const int groups_per_row = a.K >> 3;   // 16-byte groups of 8 halves; a multiple of 32
    for (int idx = tid; idx < 8 * nt_count * groups_per_row; idx += DQ_THREADS) {
        const int i = idx / groups_per_row;          // token slot in this pass
        const int q = idx - i * groups_per_row;      // 8-value group along K
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i < npass) {
            const int p = first_row + i;
            const int64_t src = a.row_token ? a.row_token[p] : p;
            v = *reinterpret_cast<const uint4*>(a.x + src * a.K + (size_t)q * 8);
        }
        const int sb = q >> 5, j = (q >> 2) & 7, u = q & 3;
        const int nt = i >> 3, c = i & 7;
        // elements 8u..8u+7 of sub-block j: words 2u and 2u+1 of the owning lane (j>>1),
        // low (j even) or high (j odd) half of the 16-byte record; halves (e0,e2,e1,e3)
        uint2* dst = reinterpret_cast<uint2*>(
            s_frag + ((((size_t)sb * NT + nt) * 8 + 2 * u) * 8 + c) * 4 + (j >> 1)) + (j & 1);
        dst[0] = make_uint2(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632));
        dst[2 * 32] = make_uint2(__byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632));
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
        if (u == 0) s_sxh[(((size_t)sb * NT + nt) * 8 + c) * 8 + j] = __float2half_rn(s);
    }
}

// One (super-block, matrix) unit of a 16-row tile: the lane's two rows (g, g+8), each the
// 16-byte header and the lane's 32-byte quant chunk.
struct UnitRegs {
    uint4 hdr[2], qa[2], qb[2];
};

__device__ __forceinline__ void load_unit(UnitRegs& r, const uint8_t* row0, const uint8_t* row1, int t) {
    r.hdr[0] = __ldcs(reinterpret_cast<const uint4*>(row0));
    r.qa[0] = __ldcs(reinterpret_cast<const uint4*>(row0 + 16 + 32 * t));
    r.qb[0] = __ldcs(reinterpret_cast<const uint4*>(row0 + 32 + 32 * t));
    r.hdr[1] = __ldcs(reinterpret_cast<const uint4*>(row1));
    r.qa[1] = __ldcs(reinterpret_cast<const uint4*>(row1 + 16 + 32 * t));
    r.qb[1] = __ldcs(reinterpret_cast<const uint4*>(row1 + 32 + 32 * t));
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

// The unit's contribution to y: for each of the NTC token tiles in use,
// p = d*sum(sc*q*x) - dmin*sum(m*Sx) (rounded in that order), then y += p.  Every
// kernel variant adds the super-blocks in ascending order with exactly these roundings, so a
// token's result does not depend on its batch-mates or on which variant ran (the reference
// asserts this bit for bit, nn/moe.rs:2318-2338).
// frag_addr / sxh_addr: shared-space byte addresses of this lane's first B fragment of the
// super-block and of its sub-block sums.
// nt_frag / nt_sxh: byte distance between consecutive 8-token tiles in the two shared arrays.
template <int NTC>
__device__ __forceinline__ void unit_terms(const UnitRegs& r, bool upper, uint32_t sel, uint32_t frag_addr,
                                           uint32_t sxh_addr, uint32_t nt_frag, uint32_t nt_sxh, float (&y)[NTC][4]) {
    LaneScales r0, r1;
    lane_scales(r.hdr[0], upper, sel, r0);
    lane_scales(r.hdr[1], upper, sel, r1);
    float acc[NTC][4];
#pragma unroll
    for (int nt = 0; nt < NTC; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    const uint32_t wq0[8] = {r.qa[0].x, r.qa[0].y, r.qa[0].z, r.qa[0].w, r.qb[0].x, r.qb[0].y, r.qb[0].z, r.qb[0].w};
    const uint32_t wq1[8] = {r.qa[1].x, r.qa[1].y, r.qa[1].z, r.qa[1].w, r.qb[1].x, r.qb[1].y, r.qb[1].z, r.qb[1].w};
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const uint32_t u0 = wq0[w], u1 = wq1[w];
        const uint32_t a0 = hfma2_u32(nib_lo(u0), r0.sc_lo, r0.c_lo);
        const uint32_t a1 = hfma2_u32(nib_lo(u1), r1.sc_lo, r1.c_lo);
        const uint32_t a2 = hfma2_u32(nib_lo(u0 >> 8), r0.sc_lo, r0.c_lo);
        const uint32_t a3 = hfma2_u32(nib_lo(u1 >> 8), r1.sc_lo, r1.c_lo);
        const uint32_t h0 = hfma2_u32(nib_hi(u0), r0.sc_hi, r0.c_hi);
        const uint32_t h1 = hfma2_u32(nib_hi(u1), r1.sc_hi, r1.c_hi);
        const uint32_t h2 = hfma2_u32(nib_hi(u0 >> 8), r0.sc_hi, r0.c_hi);
        const uint32_t h3 = hfma2_u32(nib_hi(u1 >> 8), r1.sc_hi, r1.c_hi);
#pragma unroll
        for (int nt = 0; nt < NTC; ++nt) {
            const uint4 b = lds128(frag_addr + (uint32_t)nt * nt_frag + (uint32_t)(w * 32 * 16));
            mma_16816(acc[nt], a0, a1, a2, a3, b.x, b.y);
            mma_16816(acc[nt], h0, h1, h2, h3, b.z, b.w);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NTC; ++nt) {
        float mn[4];
        mma_1688_zero(mn, r0.m_h2, r1.m_h2, lds32(sxh_addr + (uint32_t)nt * nt_sxh));
        y[nt][0] = __fadd_rn(y[nt][0], __fmaf_rn(-r0.dmin, mn[0], __fmul_rn(r0.d, acc[nt][0])));
        y[nt][1] = __fadd_rn(y[nt][1], __fmaf_rn(-r0.dmin, mn[1], __fmul_rn(r0.d, acc[nt][1])));
        y[nt][2] = __fadd_rn(y[nt][2], __fmaf_rn(-r1.dmin, mn[2], __fmul_rn(r1.d, acc[nt][2])));
        y[nt][3] = __fadd_rn(y[nt][3], __fmaf_rn(-r1.dmin, mn[3], __fmul_rn(r1.d, acc[nt][3])));
    }
}


}  // namespace mummu
