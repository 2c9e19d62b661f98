// Decode-regime expert bank over GGUF Q4_K weights (tokens <= 64, f16 activations).
//
// HBM-bound: every routed expert's gate/up/down bytes are streamed once, the activations are tiny.
// Two kernels share one body:
//   gate/up : hact[row, n] = silu(gate[n,:] . x[row,:]) * (up[n,:] . x[row,:])      (f16 out)
//   down    : ys[row, h]   = down[h,:] . hact[row,:]                                 (f32 out)
// (reference math: crates/mummu/src/nn/moe.rs:314-316; from packed bytes:
//  models/qwen4exp/experts.rs:781-806, 401-457).
//
// How a weight reaches the tensor core.  A Q4_K value is d*sc_j*q - dmin*m_j with q a 4-bit
// integer and (sc_j, m_j) per 32-value sub-block.  A dot product over one sub-block is therefore
//     d*sc_j * sum(q*x)  -  dmin*m_j * sum(x).
// sum(q*x) is an m16n8k16 f16 MMA whose A operand is the raw nibbles turned into exact f16
// integers (one LOP3 per two values: 0x6400|q is the half 1024+q; the high nibble gives
// 1024+16q), whose B operand is the token tile, and whose C operand starts at -1024*sum(x) so
// the bias of that trick cancels.  The sub-block scale is applied in f32 after every 32-wide
// slice, so no weight is ever rounded to 16 bits.  The min term is one m16n8k8 MMA per
// super-block over (m_j) x (sub-block sums of x).
//
// Work split: one CTA = (active expert, a run of 16-row tiles); its 8 warps split K by
// super-block (and, when K has fewer than 8 super-blocks, take several row tiles at once); the
// token tile (fragments in MMA register order) and the sub-block sums of x sit in shared memory.
// A lane loads 8 contiguous bytes of each 32-byte quant chunk, so the four lanes that share a
// weight row read whole 32-byte sectors, and each 144-byte super-block is read exactly once.
#include "common.cuh"

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
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0));
}

// two nibbles of a word -> half2 of exact integers: (w & mask) | 0x6400 in each half
__device__ __forceinline__ uint32_t nib_lo(uint32_t w) { return (w & 0x000F000Fu) | 0x64006400u; }
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) { return (w & 0x00F000F0u) | 0x64006400u; }

struct RowScales {
    float dsc[8];     // even j: d*sc_j ; odd j: d*sc_j / 16 (the high-nibble MMA carries 16q)
    float dmin;
    uint32_t m_h2;    // half2 (m_{2t}, m_{2t+1})
};

// header = the first 16 bytes of a super-block: f16 d, f16 dmin, 12 packed scale bytes
// (crates/mummu/src/gguf.rs:1685-1698 unpacked four bytes at a time)
__device__ __forceinline__ void decode_scales(const uint4& h, int t, RowScales& r) {
    float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu)));
    r.dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    uint32_t s0 = h.y, s1 = h.z, s2 = h.w;
    uint32_t sc_lo = s0 & 0x3F3F3F3Fu;
    uint32_t m_lo = s1 & 0x3F3F3F3Fu;
    uint32_t sc_hi = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    uint32_t m_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
    const float d16 = d * 0.0625f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float a = (float)((sc_lo >> (8 * i)) & 0xFFu);
        float b = (float)((sc_hi >> (8 * i)) & 0xFFu);
        r.dsc[i] = (i & 1) ? d16 * a : d * a;
        r.dsc[4 + i] = (i & 1) ? d16 * b : d * b;
    }
    uint32_t msel = (t < 2) ? m_lo : m_hi;
    uint32_t pair = (msel >> (16 * (t & 1))) & 0xFFFFu;
    uint32_t spread = (pair & 0xFFu) | ((pair & 0xFF00u) << 8);
    uint32_t bits = spread | 0x64006400u;   // half2 (1024 + m_a, 1024 + m_b)
    __half2 mh = __hsub2(*reinterpret_cast<__half2*>(&bits),
                         __half2half2(__ushort_as_half((unsigned short)0x6400)));
    r.m_h2 = *reinterpret_cast<uint32_t*>(&mh);
}

// shared-memory carve-up for one CTA
struct SmemLayout {
    uint4* frag;      // [nsb*8][NT][8 tok][4 t]  B fragments (16 B each)
    float* negs;      // [nsb*8][NT][8 tok]       -1024 * sub-block sum of x
    __half* sxh;      // [nsb][NT][8 tok][8 j]    sub-block sums of x, f16
    float4* part;     // [2][8 warps][2 mats][NT][32 lanes]
};

template <int NT>
__host__ __device__ inline size_t dq_smem_bytes(int nsb) {
    return (size_t)nsb * 8 * NT * 8 * 4 * 16 + (size_t)nsb * 8 * NT * 8 * 4 + (size_t)nsb * NT * 8 * 8 * 2 +
           (size_t)2 * DQ_WARPS * 2 * NT * 32 * 16;
}

template <int NT, bool GATEUP>
__global__ void __launch_bounds__(DQ_THREADS, 2) decode_q4k_kernel(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int nsb = a.K >> 8;
    SmemLayout sm;
    sm.frag = reinterpret_cast<uint4*>(smem_raw);
    sm.negs = reinterpret_cast<float*>(sm.frag + (size_t)nsb * 8 * NT * 32);
    sm.sxh = reinterpret_cast<__half*>(sm.negs + (size_t)nsb * 8 * NT * 8);
    sm.part = reinterpret_cast<float4*>(sm.sxh + (size_t)nsb * NT * 64);

    const int ai = blockIdx.x / a.ctas_per_expert;
    const int cb = blockIdx.x - ai * a.ctas_per_expert;
    if (ai >= *a.n_active) return;
    const int e = a.active[ai];
    const int cnt = a.counts[e];
    const int base = a.offsets[e];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int KS = nsb < DQ_WARPS ? nsb : DQ_WARPS;   // K slices (warps per row tile)
    const int RG = DQ_WARPS / KS;                     // row tiles in flight per CTA
    const int ks = warp % KS, rg = warp / KS;
    const bool warp_active = warp < KS * RG;
    const int rt_begin = cb * a.rb;
    const int rt_end = min(a.n_rt, rt_begin + a.rb);
    const uint8_t* w0e = a.w0 + (size_t)e * a.expert_stride;
    const uint8_t* w1e = GATEUP ? a.w1 + (size_t)e * a.expert_stride : w0e;
    const int groups_per_row = a.K >> 3;   // 16-byte groups of 8 halves

    for (int pass0 = 0; pass0 < cnt; pass0 += 8 * NT) {
        const int npass = min(8 * NT, cnt - pass0);
        __syncthreads();   // previous pass finished reading the token tile
        // ---- stage the token tile: fragments in MMA order + sub-block sums ----
        for (int idx = tid; idx < 8 * NT * groups_per_row; idx += DQ_THREADS) {
            int i = idx / groups_per_row;          // token slot in this pass
            int q = idx - i * groups_per_row;      // 8-value group along K
            uint4 v = make_uint4(0, 0, 0, 0);
            if (i < npass) {
                int p = base + pass0 + i;
                int64_t src = a.row_token ? a.row_token[p] : p;
                v = *reinterpret_cast<const uint4*>(a.x + src * a.K + (size_t)q * 8);
            }
            // halves e0..e7 -> [e0,e2,e1,e3 | e4,e6,e5,e7]
            uint4 f;
            f.x = __byte_perm(v.x, v.y, 0x5410);
            f.y = __byte_perm(v.x, v.y, 0x7632);
            f.z = __byte_perm(v.z, v.w, 0x5410);
            f.w = __byte_perm(v.z, v.w, 0x7632);
            int sb = q >> 5, j = (q >> 2) & 7, tt = q & 3;
            int nt = i >> 3, c = i & 7;
            sm.frag[(((size_t)(sb * 8 + j) * NT + nt) * 8 + c) * 4 + tt] = f;
            const __half2* h2 = reinterpret_cast<const __half2*>(&v);
            float s = 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float2 f2 = __half22float2(h2[u]);
                s += f2.x;
                s += f2.y;
            }
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            if (tt == 0) {
                sm.negs[((size_t)(sb * 8 + j) * NT + nt) * 8 + c] = -1024.0f * s;
                sm.sxh[(((size_t)sb * NT + nt) * 8 + c) * 8 + j] = __float2half_rn(s);
            }
        }
        __syncthreads();

        int it = 0;
        for (int rt0 = rt_begin; rt0 < rt_end; rt0 += RG, ++it) {
            const int rt = rt0 + rg;
            float y[2][NT][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) y[mt][nt][i] = 0.0f;

            if (warp_active && rt < rt_end) {
                for (int sb = ks; sb < nsb; sb += KS) {
                    // rows of this lane: (mat, half) -> weight row pointer at this super-block
                    const uint8_t* rowp[2][2];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            int row = GATEUP ? rt * 16 + g + 8 * hf : rt * 32 + 16 * mt + g + 8 * hf;
                            const uint8_t* bank = mt == 0 ? w0e : w1e;
                            rowp[mt][hf] = bank + (size_t)row * a.row_bytes + (size_t)sb * Q4K_BLOCK_BYTES;
                        }
                    uint4 hdr[2][2];
                    uint2 qw[2][2][4];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            hdr[mt][hf] = __ldcs(reinterpret_cast<const uint4*>(rowp[mt][hf]));
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                qw[mt][hf][c] = __ldcs(reinterpret_cast<const uint2*>(rowp[mt][hf] + 16 + 32 * c + 8 * t));
                        }
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        RowScales rs[2];
                        decode_scales(hdr[mt][0], t, rs[0]);
                        decode_scales(hdr[mt][1], t, rs[1]);
                        // min term: (m_j) x (sum x over sub-block j)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            float mn[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            uint32_t b = *reinterpret_cast<const uint32_t*>(
                                sm.sxh + (((size_t)sb * NT + nt) * 8 + g) * 8 + 2 * t);
                            mma_1688(mn, rs[0].m_h2, rs[1].m_h2, b);
                            y[mt][nt][0] -= rs[0].dmin * mn[0];
                            y[mt][nt][1] -= rs[0].dmin * mn[1];
                            y[mt][nt][2] -= rs[1].dmin * mn[2];
                            y[mt][nt][3] -= rs[1].dmin * mn[3];
                        }
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t w00 = qw[mt][0][c].x, w01 = qw[mt][0][c].y;   // row g
                            const uint32_t w10 = qw[mt][1][c].x, w11 = qw[mt][1][c].y;   // row g+8
#pragma unroll
                            for (int hi = 0; hi < 2; ++hi) {
                                const int j = 2 * c + hi;
                                uint32_t a0, a1, a2, a3, a4, a5, a6, a7;
                                if (hi == 0) {
                                    a0 = nib_lo(w00); a1 = nib_lo(w10); a2 = nib_lo(w00 >> 8); a3 = nib_lo(w10 >> 8);
                                    a4 = nib_lo(w01); a5 = nib_lo(w11); a6 = nib_lo(w01 >> 8); a7 = nib_lo(w11 >> 8);
                                } else {
                                    a0 = nib_hi(w00); a1 = nib_hi(w10); a2 = nib_hi(w00 >> 8); a3 = nib_hi(w10 >> 8);
                                    a4 = nib_hi(w01); a5 = nib_hi(w11); a6 = nib_hi(w01 >> 8); a7 = nib_hi(w11 >> 8);
                                }
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt) {
                                    const size_t rec = ((size_t)(sb * 8 + j) * NT + nt) * 8;
                                    const uint4 b = sm.frag[(rec + g) * 4 + t];
                                    const float2 ns = *reinterpret_cast<const float2*>(sm.negs + rec + 2 * t);
                                    float acc[4] = {ns.x, ns.y, ns.x, ns.y};
                                    mma_16816(acc, a0, a1, a2, a3, b.x, b.y);
                                    mma_16816(acc, a4, a5, a6, a7, b.z, b.w);
                                    y[mt][nt][0] = fmaf(rs[0].dsc[j], acc[0], y[mt][nt][0]);
                                    y[mt][nt][1] = fmaf(rs[0].dsc[j], acc[1], y[mt][nt][1]);
                                    y[mt][nt][2] = fmaf(rs[1].dsc[j], acc[2], y[mt][nt][2]);
                                    y[mt][nt][3] = fmaf(rs[1].dsc[j], acc[3], y[mt][nt][3]);
                                }
                            }
                        }
                    }
                }
            }
            // ---- fold the K slices and write out ----
            float4* part = sm.part + (size_t)(it & 1) * DQ_WARPS * 2 * NT * 32;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    part[((warp * 2 + mt) * NT + nt) * 32 + lane] =
                        make_float4(y[mt][nt][0], y[mt][nt][1], y[mt][nt][2], y[mt][nt][3]);
            __syncthreads();
            const float* pf = reinterpret_cast<const float*>(part);
            for (int o = tid; o < RG * NT * 128; o += DQ_THREADS) {
                int rgo = o / (NT * 128);
                int rem = o - rgo * NT * 128;
                int nt = rem >> 7;
                int li = rem & 127;          // lane*4 + i
                int ln = li >> 2, i = li & 3;
                int rto = rt0 + rgo;
                if (rto >= rt_end) continue;
                int col = (ln & 3) * 2 + (i & 1);          // token within the n-tile
                int row = (ln >> 2) + ((i >> 1) << 3);     // weight row within the 16-row tile
                int slot = nt * 8 + col;
                if (slot >= npass) continue;
                float s0 = 0.0f, s1 = 0.0f;
                for (int w = 0; w < KS; ++w) {
                    int wp = rgo * KS + w;
                    s0 += pf[(((size_t)(wp * 2 + 0) * NT + nt) * 32 + ln) * 4 + i];
                    s1 += pf[(((size_t)(wp * 2 + 1) * NT + nt) * 32 + ln) * 4 + i];
                }
                size_t orow = (size_t)(base + pass0 + slot);
                if (GATEUP) {
                    float v = (s0 / (1.0f + expf(-s0))) * s1;
                    reinterpret_cast<__half*>(a.out)[orow * a.ld_out + rto * 16 + row] = __float2half_rn(v);
                } else {
                    float* o32 = reinterpret_cast<float*>(a.out);
                    o32[orow * a.ld_out + rto * 32 + row] = s0;
                    o32[orow * a.ld_out + rto * 32 + 16 + row] = s1;
                }
            }
        }
    }
}

// active-expert list: experts with at least one row, ascending id
__global__ void active_list_kernel(const int32_t* counts, int E, int32_t* active, int32_t* n_active) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int n = 0;
        for (int e = 0; e < E; ++e)
            if (counts[e] > 0) active[n++] = e;
        *n_active = n;
    }
}

bool decode_q4k_supported(const MummuMoeConfig& c, int64_t tokens) {
    return c.weight_dtype == MUMMU_Q4_K && c.act_dtype == MUMMU_F16 && tokens >= 1 && tokens <= 64 &&
           c.hidden % 256 == 0 && c.inter % 256 == 0 && c.hidden <= 8192 && c.inter <= 8192;
}

template <int NT, bool GATEUP>
static int launch_one(MummuMoe* m, DecodeArgs& a, int n_experts_max, cudaStream_t s, const char* name) {
    size_t smem = dq_smem_bytes<NT>(a.K >> 8);
    if (smem > 200 * 1024) {
        set_error("decode_q4k: %zu bytes of shared memory needed for K=%d", smem, a.K);
        return MUMMU_ERR_UNSUPPORTED;
    }
    MUMMU_CUDA_TRY(cudaFuncSetAttribute(decode_q4k_kernel<NT, GATEUP>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(m, s, name);
    decode_q4k_kernel<NT, GATEUP><<<n_experts_max * a.ctas_per_expert, DQ_THREADS, smem, s>>>(a);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

static int pick_rb(int n_rt, int rg, int experts_est) {
    // aim for ~4 CTAs per SM over the active experts, but keep each CTA's weight stream long
    int rb = rg;
    while (rb * 2 <= n_rt && (int64_t)experts_est * (n_rt / (rb * 2)) >= 148 * 3) rb *= 2;
    return rb;
}

int launch_decode_q4k(MummuMoe* m, const void* x, int64_t tokens, int top_k, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    int32_t* active = m->active;
    int32_t* n_active = m->n_active;
    {
        LaunchScope scope(m, s, "active_list");
        active_list_kernel<<<1, 32, 0, s>>>(m->counts, c.experts, active, n_active);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    int experts_est = (int)std::min<int64_t>(c.experts, tokens * top_k);
    const bool nt2 = tokens > 8;

    DecodeArgs g{};
    g.x = (const __half*)x;
    g.row_token = m->row_token;
    g.counts = m->counts;
    g.offsets = m->offsets;
    g.active = active;
    g.n_active = n_active;
    g.w0 = (const uint8_t*)m->bank[MUMMU_BANK_GATE];
    g.w1 = (const uint8_t*)m->bank[MUMMU_BANK_UP];
    g.row_bytes = (int)bank_row_bytes(c, MUMMU_BANK_GATE);
    g.expert_stride = (size_t)g.row_bytes * c.inter;
    g.K = c.hidden;
    g.n_rt = c.inter / 16;
    {
        int nsb = g.K >> 8, ks = nsb < DQ_WARPS ? nsb : DQ_WARPS, rg = DQ_WARPS / ks;
        g.rb = pick_rb(g.n_rt, rg, experts_est);
    }
    g.ctas_per_expert = (g.n_rt + g.rb - 1) / g.rb;
    g.ld_out = c.inter;
    g.out = m->hact;
    int rc = nt2 ? launch_one<2, true>(m, g, experts_est, s, "q4k_gate_up")
                 : launch_one<1, true>(m, g, experts_est, s, "q4k_gate_up");
    if (rc) return rc;

    DecodeArgs d{};
    d.x = (const __half*)m->hact;
    d.row_token = nullptr;
    d.counts = m->counts;
    d.offsets = m->offsets;
    d.active = active;
    d.n_active = n_active;
    d.w0 = (const uint8_t*)m->bank[MUMMU_BANK_DOWN];
    d.w1 = nullptr;
    d.row_bytes = (int)bank_row_bytes(c, MUMMU_BANK_DOWN);
    d.expert_stride = (size_t)d.row_bytes * c.hidden;
    d.K = c.inter;
    d.n_rt = c.hidden / 32;
    {
        int nsb = d.K >> 8, ks = nsb < DQ_WARPS ? nsb : DQ_WARPS, rg = DQ_WARPS / ks;
        d.rb = pick_rb(d.n_rt, rg, experts_est);
    }
    d.ctas_per_expert = (d.n_rt + d.rb - 1) / d.rb;
    d.ld_out = c.hidden;
    d.out = m->ys;
    return nt2 ? launch_one<2, false>(m, d, experts_est, s, "q4k_down")
               : launch_one<1, false>(m, d, experts_est, s, "q4k_down");
}

}  // namespace mummu
