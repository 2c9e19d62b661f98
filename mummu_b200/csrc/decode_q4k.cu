// Decode-regime expert bank over GGUF Q4_K weights (tokens <= 256, f16 activations).
//
// HBM-bound: every routed expert's gate/up/down bytes are streamed once, the activations are tiny.
// Two kernels share one body:
//   gate/up : hact[row, n] = silu(gate[n,:] . x[row,:]) * (up[n,:] . x[row,:])      (f16 out)
//   down    : ys[row, h]   = down[h,:] . hact[row,:]                                 (f32 out)
// (reference math: crates/mummu/src/nn/moe.rs:314-316; from packed bytes:
//  models/qwen4exp/experts.rs:781-806, 401-457).
//
// How a weight reaches the tensor core.  A Q4_K value is d*sc_j*q - dmin*m_j with q a 4-bit
// integer and (sc_j, m_j) 6-bit integers per 32-value sub-block, so over one 256-value super-block
//     dot = d * sum_j sum_k (sc_j*q_k) x_k  -  dmin * sum_j m_j * (sum of x over sub-block j).
// sc_j*q_k <= 945 is an integer an f16 holds exactly.  One LOP3 turns two nibbles of a word into
// the halves 1024+q (low nibble: 0x6400|q) or 1024+16q (high nibble), and one HFMA2 with the
// lane's (sc, -1024*sc) or (sc/16, -64*sc) turns those into sc*q with no rounding at all.  These
// feed m16n8k16 f16 MMAs against the token tile with f32 accumulation over the whole super-block;
// d and dmin are applied in f32 once per super-block.  No weight is rounded to 16 bits.  The min
// term is one m16n8k8 MMA per super-block over (m_j) x (sub-block sums of x).
//
// Lane mapping: the four lanes that share a weight row (the MMA "quad") each own one 32-byte
// quant chunk = two whole sub-blocks, so a lane needs only its own two (sc, m) pairs, loads its
// chunk with two 128-bit loads, and the quad reads one whole 144-byte super-block contiguously.
// Work split: one CTA = (active expert, a run of 16-row tiles); its 8 warps split K by
// super-block (and, when K has fewer than 8 super-blocks, take several row tiles at once); the
// token tile sits in shared memory already in MMA fragment order.
#include "decode_q4k.cuh"

namespace mummu {

template <int NT>
__host__ __device__ inline size_t dq_smem_bytes(int nsb) {
    return (size_t)nsb * NT * 4096 + (size_t)nsb * NT * 128 + (size_t)2 * DQ_WARPS * 2 * NT * 32 * 16;
}

template <int NT, bool GATEUP>
__global__ void __launch_bounds__(DQ_THREADS, 2) decode_q4k_kernel(DecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nsb = a.K >> 8;
    // [nsb][NT][8 words][8 tokens][4 lanes-of-quad] x 16 B: (lo sub-block 4 halves | hi sub-block 4 halves)
    uint4* s_frag = reinterpret_cast<uint4*>(smem_raw);
    // [nsb][NT][8 tokens][8 sub-blocks] f16 sums of x
    __half* s_sxh = reinterpret_cast<__half*>(s_frag + (size_t)nsb * NT * 256);
    float4* s_part = reinterpret_cast<float4*>(s_sxh + (size_t)nsb * NT * 64);
    const uint32_t frag_base = (uint32_t)__cvta_generic_to_shared(s_frag);
    const uint32_t sxh_base = (uint32_t)__cvta_generic_to_shared(s_sxh);

    const int ai = blockIdx.x / a.ctas_per_expert;
    const int cb = blockIdx.x - ai * a.ctas_per_expert;
    if (ai >= *a.n_active) return;
    const int e = a.active[ai];
    const int cnt = a.counts[e];
    const int base = a.offsets[e];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool upper = t >= 2;
    const uint32_t sel = (t & 1) ? 0x4342u : 0x4140u;
    const int KS = nsb < DQ_WARPS ? nsb : DQ_WARPS;   // K slices (warps per row tile)
    const int RG = DQ_WARPS / KS;                     // row tiles in flight per CTA
    const int ks = warp % KS, rg = warp / KS;
    const bool warp_active = warp < KS * RG;
    const int rt_begin = cb * a.rb;
    const int rt_end = min(a.n_rt, rt_begin + a.rb);
    const uint8_t* w0e = a.w0 + (size_t)e * a.expert_stride;
    const uint8_t* w1e = GATEUP ? a.w1 + (size_t)e * a.expert_stride : w0e;

    for (int pass0 = 0; pass0 < cnt; pass0 += 8 * NT) {
        const int npass = min(8 * NT, cnt - pass0);
        const int nt_count = (npass + 7) >> 3;
        __syncthreads();   // previous pass finished reading the token tile
        stage_token_tile<NT>(a, s_frag, s_sxh, base + pass0, npass, nt_count, tid);
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
                    UnitRegs un[2];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        const int row = GATEUP ? rt * 16 + g : rt * 32 + 16 * mt + g;
                        const uint8_t* row0 = (mt == 0 ? w0e : w1e) + (size_t)row * a.row_bytes +
                                              (size_t)sb * Q4K_BLOCK_BYTES;
                        load_unit(un[mt], row0, row0 + (size_t)8 * a.row_bytes, t);
                    }
                    const uint32_t frag_addr = frag_base + (uint32_t)(((sb * NT * 64 + g) * 4 + t) * 16);
                    const uint32_t sxh_addr = sxh_base + (uint32_t)((((sb * NT * 8 + g) * 8) + 2 * t) * 2);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        if (NT == 1 || nt_count == 1)
                            unit_terms<1>(un[mt], upper, sel, frag_addr, sxh_addr, 4096u, 128u,
                                              *reinterpret_cast<float(*)[1][4]>(&y[mt][0][0]));
                        else
                            unit_terms<NT>(un[mt], upper, sel, frag_addr, sxh_addr, 4096u, 128u, y[mt]);
                    }
                }
            }
            // ---- fold the K slices and write out ----
            float4* part = s_part + (size_t)(it & 1) * DQ_WARPS * 2 * NT * 32;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    part[((warp * 2 + mt) * NT + nt) * 32 + lane] =
                        make_float4(y[mt][nt][0], y[mt][nt][1], y[mt][nt][2], y[mt][nt][3]);
            __syncthreads();
            const float* pf = reinterpret_cast<const float*>(part);
            for (int o = tid; o < RG * NT * 128; o += DQ_THREADS) {
                const int rgo = o / (NT * 128);
                const int rem = o - rgo * NT * 128;
                const int nt = rem >> 7;
                const int li = rem & 127;          // lane*4 + i
                const int ln = li >> 2, i = li & 3;
                const int rto = rt0 + rgo;
                if (rto >= rt_end) continue;
                const int col = (ln & 3) * 2 + (i & 1);          // token within the n-tile
                const int row = (ln >> 2) + ((i >> 1) << 3);     // weight row within the 16-row tile
                const int slot = nt * 8 + col;
                if (slot >= npass) continue;
                float s0 = 0.0f, s1 = 0.0f;     // ascending super-block order (see unit_terms)
                for (int w = 0; w < KS; ++w) {
                    const int wp = rgo * KS + w;
                    s0 = __fadd_rn(s0, pf[(((size_t)(wp * 2 + 0) * NT + nt) * 32 + ln) * 4 + i]);
                    s1 = __fadd_rn(s1, pf[(((size_t)(wp * 2 + 1) * NT + nt) * 32 + ln) * 4 + i]);
                }
                const size_t orow = (size_t)(base + pass0 + slot);
                if (GATEUP) {
                    const float v = (s0 / (1.0f + expf(-s0))) * s1;
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


// ------------------------------------------------------------------------------------------------
// Streaming variant with the weights staged by the copy engine.
//
// The banks are described to TMA as 2-D byte tensors [expert*rows, row_bytes]; one
// (super-block, matrix) unit of a 16-row tile is then ONE box of 16 rows x 144 bytes = 2304 B,
// fetched by one instruction from one lane into the warp's private ring (ring_depth stages, one
// mbarrier each), instead of six per-lane copies with their address arithmetic.  The 144-byte
// row pitch in shared memory makes the lanes' 16-byte reads conflict free.  Each warp is its own
// producer: after copying a stage into registers it refills that stage, so up to ring_depth
// units are in flight per warp while one is multiplied.  The first units are requested before
// the token tile is staged (weights do not depend on the tokens).  Waits are bounded: when one
// runs out the warp raises the status word, stops waiting and finishes with whatever it has.
// ------------------------------------------------------------------------------------------------
constexpr uint32_t DQ_UNIT_BYTES = 16 * Q4K_BLOCK_BYTES;   // 2304
constexpr uint32_t DQ_WAIT_LIMIT = 1u << 21;

struct UnitRing {
    uint32_t data;       // shared address of this warp's first stage
    uint32_t bars;       // shared address of this warp's first mbarrier
    int depth;
    // consumer
    int c_stage;
    uint32_t c_phase;
    bool dead;           // a wait ran out
    // producer cursor (uniform over the warp)
    int p_rt, p_sb, p_m, p_pass;
    bool p_valid;
};

template <bool GATEUP>
__device__ __forceinline__ void ring_issue(UnitRing& r, int stage, const CUtensorMap* map0, const CUtensorMap* map1,
                                           int row_base, int rt_first, int rt_end, int nsb, int npasses, int lane) {
    if (lane == 0) {
        const int row = GATEUP ? row_base + r.p_rt * 16 : row_base + r.p_rt * 32 + 16 * r.p_m;
        const uint32_t bar = r.bars + (uint32_t)stage * 8u;
        mbar_expect_tx(bar, DQ_UNIT_BYTES);
        tma_load_2d(r.data + (uint32_t)stage * DQ_UNIT_BYTES, (GATEUP && r.p_m) ? map1 : map0,
                    r.p_sb * Q4K_BLOCK_BYTES, row, bar);
    }
    r.p_m ^= 1;
    if (r.p_m == 0 && ++r.p_sb == nsb) {
        r.p_sb = 0;
        r.p_rt += DQ_WARPS;
        if (r.p_rt >= rt_end) {
            r.p_rt = rt_first;
            if (++r.p_pass >= npasses) r.p_valid = false;
        }
    }
}

__device__ __forceinline__ void ring_take(UnitRing& r, UnitRegs& u, int g, int t, int32_t* status) {
    const uint32_t bar = r.bars + (uint32_t)r.c_stage * 8u;
    if (!r.dead) {
        uint32_t i = 0;
        while (!mbar_test(bar, r.c_phase)) {
            if (++i > 64) __nanosleep(32);
            if (i >= DQ_WAIT_LIMIT) {
                r.dead = true;
                atomicOr(status, STATUS_TIMEOUT);
                break;
            }
        }
    }
    const uint32_t row0 = r.data + (uint32_t)r.c_stage * DQ_UNIT_BYTES + (uint32_t)(g * Q4K_BLOCK_BYTES);
    const uint32_t row1 = row0 + 8u * Q4K_BLOCK_BYTES;
    u.hdr[0] = lds128(row0);
    u.qa[0] = lds128(row0 + 16 + 32 * t);
    u.qb[0] = lds128(row0 + 32 + 32 * t);
    u.hdr[1] = lds128(row1);
    u.qa[1] = lds128(row1 + 16 + 32 * t);
    u.qb[1] = lds128(row1 + 32 + 32 * t);
    __syncwarp();   // every lane holds its copy: the stage may be refilled
}

template <int NT, int NTC, bool GATEUP>
__device__ __forceinline__ void ring_rows(const DecodeArgs& a, UnitRing& r, const CUtensorMap* map0,
                                          const CUtensorMap* map1, uint32_t frag_base, uint32_t sxh_base, int row_base,
                                          int rt_first, int rt_end, int nsb, int npasses, int g, int t, int lane,
                                          bool upper, uint32_t sel, int first_row, int npass) {
    for (int rt = rt_first; rt < rt_end; rt += DQ_WARPS) {
        float y[2][NTC][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTC; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) y[mt][nt][i] = 0.0f;
        uint32_t frag_addr = frag_base + (uint32_t)((g * 4 + t) * 16);
        uint32_t sxh_addr = sxh_base + (uint32_t)((g * 8 + 2 * t) * 2);
        for (int sb = 0; sb < nsb; ++sb) {
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                UnitRegs un;
                ring_take(r, un, g, t, a.status);
                if (r.p_valid) ring_issue<GATEUP>(r, r.c_stage, map0, map1, row_base, rt_first, rt_end, nsb, npasses, lane);
                if (++r.c_stage == r.depth) {
                    r.c_stage = 0;
                    r.c_phase ^= 1u;
                }
                unit_terms<NTC>(un, upper, sel, frag_addr, sxh_addr, 4096u, 128u, y[mt]);
            }
            frag_addr += (uint32_t)(NT * 64 * 4 * 16);
            sxh_addr += (uint32_t)(NT * 8 * 8 * 2);
        }
        // epilogue from registers: lane (g, t) holds rows g, g+8 x tokens 2t, 2t+1
#pragma unroll
        for (int nt = 0; nt < NTC; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int slot = nt * 8 + 2 * t + (i & 1);
                const int row = g + ((i >> 1) << 3);
                if (slot < npass) {
                    const size_t orow = (size_t)(first_row + slot);
                    if (GATEUP) {
                        const float s0 = y[0][nt][i], s1 = y[1][nt][i];
                        const float v = (s0 / (1.0f + expf(-s0))) * s1;
                        reinterpret_cast<__half*>(a.out)[orow * a.ld_out + rt * 16 + row] = __float2half_rn(v);
                    } else {
                        float* o32 = reinterpret_cast<float*>(a.out);
                        o32[orow * a.ld_out + rt * 32 + row] = y[0][nt][i];
                        o32[orow * a.ld_out + rt * 32 + 16 + row] = y[1][nt][i];
                    }
                }
            }
    }
}

template <int NT>
__host__ __device__ inline size_t dq_ring_smem_bytes(int nsb, int depth) {
    return (size_t)nsb * NT * 4096 + (size_t)nsb * NT * 128 + 128 + (size_t)DQ_WARPS * depth * (DQ_UNIT_BYTES + 8);
}

template <int NT, bool GATEUP>
__global__ void __launch_bounds__(DQ_THREADS, 2)
decode_q4k_tma_kernel(DecodeArgs a, const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int nsb = a.K >> 8;
    uint4* s_frag = reinterpret_cast<uint4*>(smem_raw);
    __half* s_sxh = reinterpret_cast<__half*>(s_frag + (size_t)nsb * NT * 256);
    const uint32_t frag_base = smem_u32(s_frag);
    const uint32_t sxh_base = smem_u32(s_sxh);

    const int ai = blockIdx.x / a.ctas_per_expert;
    const int cb = blockIdx.x - ai * a.ctas_per_expert;
    if (ai >= *a.n_active) return;
    const int e = a.active[ai];
    const int cnt = a.counts[e];
    const int base = a.offsets[e];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool upper = t >= 2;
    const uint32_t sel = (t & 1) ? 0x4342u : 0x4140u;
    const int rt_begin = cb * a.rb;
    const int rt_end = min(a.n_rt, rt_begin + a.rb);
    const int rt_first = rt_begin + warp;
    // An expert with more rows than one token tile holds needs several passes over its weights;
    // gridDim.y CTAs share them (pass p goes to CTA p % gridDim.y), each streaming the weights again
    // (from L2 after the first), instead of one CTA looping while SMs stand idle.
    const int pass_first = (int)blockIdx.y * 8 * NT, pass_step = (int)gridDim.y * 8 * NT;
    if (pass_first >= cnt) return;
    const int npasses = (cnt - pass_first + pass_step - 1) / pass_step;
    const int row_base = e * a.rows_per_expert;

    UnitRing r;
    r.depth = a.ring_depth;
    const uint32_t ring_base = (sxh_base + (uint32_t)(nsb * NT * 128) + 127u) & ~127u;
    r.data = ring_base + (uint32_t)(warp * r.depth) * DQ_UNIT_BYTES;
    r.bars = ring_base + (uint32_t)(DQ_WARPS * r.depth) * DQ_UNIT_BYTES + (uint32_t)(warp * r.depth) * 8u;
    r.c_stage = 0;
    r.c_phase = 0;
    r.dead = false;
    r.p_rt = rt_first;
    r.p_sb = 0;
    r.p_m = 0;
    r.p_pass = 0;
    r.p_valid = rt_first < rt_end && npasses > 0;
    if (lane == 0) {
        for (int i = 0; i < r.depth; ++i) mbar_init(r.bars + (uint32_t)i * 8u, 1);
        mbar_init_fence();
    }
    __syncwarp();
    // request the first units before the tokens are staged
    for (int i = 0; i < r.depth; ++i)
        if (r.p_valid) ring_issue<GATEUP>(r, i, &map0, &map1, row_base, rt_first, rt_end, nsb, npasses, lane);
    if (!a.pdl) {
    } else if (GATEUP) {
        // programmatic dependent launch: the down kernel's CTAs may take the SMs this grid leaves
        // idle in its tail and request their first weights there
        asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    } else {
        // launched early (see above): the weights requested so far do not depend on the previous
        // grid, the activations staged next do.  Returns at once after an ordinary launch.
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
    }

    for (int pass0 = pass_first; pass0 < cnt; pass0 += pass_step) {
        const int npass = min(8 * NT, cnt - pass0);
        const int nt_count = (npass + 7) >> 3;
        __syncthreads();
        stage_token_tile<NT>(a, s_frag, s_sxh, base + pass0, npass, nt_count, tid);
        __syncthreads();

        if (NT == 1 || nt_count == 1)
            ring_rows<NT, 1, GATEUP>(a, r, &map0, &map1, frag_base, sxh_base, row_base, rt_first, rt_end, nsb, npasses,
                                     g, t, lane, upper, sel, base + pass0, npass);
        else
            ring_rows<NT, NT, GATEUP>(a, r, &map0, &map1, frag_base, sxh_base, row_base, rt_first, rt_end, nsb, npasses,
                                      g, t, lane, upper, sel, base + pass0, npass);
    }
}

bool decode_q4k_supported(const MummuMoeConfig& c, int64_t tokens) {
    // up to 256 tokens: beyond one 16-row token tile per expert the kernels make several passes
    // (shared between CTAs), still far ahead of the generic bank
    return c.weight_dtype == MUMMU_Q4_K && c.act_dtype == MUMMU_F16 && tokens >= 1 && tokens <= 256 &&
           c.hidden % 256 == 0 && c.inter % 256 == 0 && c.hidden <= 8192 && c.inter <= 8192;
}

// Tensor map of one Q4_K bank as a [rows, row_bytes] byte view with a 16-row x 144-byte box,
// encoded once per bank pointer and kept in the handle.
static int bank_map(MummuMoe* m, int which, int row_bytes, int64_t rows, const CUtensorMap** out) {
    CUtensorMap* map = reinterpret_cast<CUtensorMap*>(m->q4k_map[which]);
    if (m->q4k_map_base[which] != m->bank[which]) {
        int rc = encode_tiled_2d(map, m->bank[which], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)row_bytes,
                                 (uint64_t)rows, Q4K_BLOCK_BYTES, 16, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        m->q4k_map_base[which] = m->bank[which];
    }
    *out = map;
    return MUMMU_OK;
}

template <int NT, bool GATEUP>
static int launch_one(MummuMoe* m, DecodeArgs& a, int n_experts_max, bool stream, cudaStream_t s,
                      const char* name, bool pdl = false, bool* used_tma = nullptr) {
    const int nsb = a.K >> 8;
    if (stream) {
        // deepest ring (2..4 stages per warp) that still lets two CTAs share an SM
        int depth = 4;
        while (depth > 2 && 2 * (dq_ring_smem_bytes<NT>(nsb, depth) + 1024) > 227 * 1024) --depth;
        const size_t smem = dq_ring_smem_bytes<NT>(nsb, depth);
        if (smem <= 200 * 1024) {
            const CUtensorMap *map0 = nullptr, *map1 = nullptr;
            const int64_t rows = (int64_t)m->cfg.experts_local * a.rows_per_expert;
            int rc = bank_map(m, GATEUP ? MUMMU_BANK_GATE : MUMMU_BANK_DOWN, a.row_bytes, rows, &map0);
            if (!rc && GATEUP) rc = bank_map(m, MUMMU_BANK_UP, a.row_bytes, rows, &map1);
            if (rc) return rc;
            if (!GATEUP) map1 = map0;
            a.ring_depth = depth;
            LaunchScope scope(m, s, name);
            MUMMU_CUDA_TRY(allow_big_smem(decode_q4k_tma_kernel<NT, GATEUP>, m->cfg.device));
            if (!GATEUP && pdl) {
                // may start while the gate/up grid drains (it waits on the device before it reads hact)
                cudaLaunchConfig_t cfg{};
                cfg.gridDim = dim3((unsigned)(n_experts_max * a.ctas_per_expert), (unsigned)a.pass_split);
                cfg.blockDim = dim3(DQ_THREADS);
                cfg.dynamicSmemBytes = smem;
                cfg.stream = s;
                cudaLaunchAttribute attr[1];
                attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[0].val.programmaticStreamSerializationAllowed = 1;
                cfg.attrs = attr;
                cfg.numAttrs = 1;
                MUMMU_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_q4k_tma_kernel<NT, GATEUP>, a, *map0, *map1));
            } else {
                decode_q4k_tma_kernel<NT, GATEUP><<<dim3((unsigned)(n_experts_max * a.ctas_per_expert), (unsigned)a.pass_split), DQ_THREADS, smem, s>>>(a, *map0, *map1);
            }
            MUMMU_CUDA_TRY(cudaGetLastError());
            if (used_tma) *used_tma = true;
            return MUMMU_OK;
        }
    }
    // (a token tile too wide to share the SM with a weight ring: the split-K kernel takes the call)
    const size_t smem = dq_smem_bytes<NT>(nsb);
    if (smem > 200 * 1024) {
        set_error("decode_q4k: %zu bytes of shared memory needed for K=%d", smem, a.K);
        return MUMMU_ERR_UNSUPPORTED;
    }
    LaunchScope scope(m, s, name);
    MUMMU_CUDA_TRY(allow_big_smem(decode_q4k_kernel<NT, GATEUP>, m->cfg.device));
    decode_q4k_kernel<NT, GATEUP><<<n_experts_max * a.ctas_per_expert, DQ_THREADS, smem, s>>>(a);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// Work split for one projection.  Streaming (one warp per row tile over all of K) needs row
// tiles for a fair share of the 148 SMs x 16 resident warps (measured at the OLMoE shape: 36.9 us
// against 35.3 us for split-K with 8 experts, 39 against 51 with 15, 48 against 72 with 27);
// below that the split-K variant spreads each row tile over up to 8 warps.
static void plan(const MummuSwitches& sw, DecodeArgs& a, int experts_est, int64_t rows_total, int nt, bool& stream) {
    const int nsb = a.K >> 8;
    // expected passes per expert from the row bound the caller gave (1 in plain decode calls)
    int64_t per_expert = (rows_total + experts_est - 1) / experts_est;
    a.pass_split = (int)std::min<int64_t>(4, std::max<int64_t>(1, (per_expert + 8 * nt - 1) / (8 * nt)));
    // measured: streaming wins from about 15 experts' row tiles on
    const int stream_min = sw.decode_stream_min > 0 ? sw.decode_stream_min : 148 * 5;
    stream = (int64_t)experts_est * a.n_rt * a.pass_split >= stream_min;
    if (stream) {
        a.rb = DQ_WARPS;                       // one row tile per warp
        // two row tiles per warp as long as the CTAs still cover the SMs one and a half times:
        // the token tile is then staged half as often (measured: 2 % on the layer)
        while (a.rb * 2 <= a.n_rt && (int64_t)experts_est * (a.n_rt / (a.rb * 2)) * a.pass_split * 2 >= 148 * 3) a.rb *= 2;
    } else {
        const int ks = nsb < DQ_WARPS ? nsb : DQ_WARPS, rg = DQ_WARPS / ks;
        a.rb = rg;
        while (a.rb * 2 <= a.n_rt && (int64_t)experts_est * (a.n_rt / (a.rb * 2)) >= 148 * 3) a.rb *= 2;
    }
    const int forced_rb = a.w1 ? sw.decode_rb_gateup : sw.decode_rb_down;
    if (forced_rb >= 1 && forced_rb <= a.n_rt) a.rb = forced_rb;
    a.ctas_per_expert = (a.n_rt + a.rb - 1) / a.rb;
}

// x: gate/up input rows (f16); row_token: sorted row -> row of x, or null when x is already sorted;
// counts/offsets/active/n_active: per local expert; rows_total bounds the number of sorted rows.
// Writes m->hact (f16) and ys (f32, [rows, hidden]).
int launch_decode_q4k_rows(MummuMoe* m, const void* x, const int32_t* row_token, const int32_t* counts,
                           const int32_t* offsets, int64_t rows_total, float* ys, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    int32_t* active = m->active;
    int32_t* n_active = m->n_active;
    int experts_est = (int)std::min<int64_t>(c.experts_local, rows_total);
    bool nt2 = rows_total > 8;
    if (m->sw.decode_nt == 1) nt2 = false;

    DecodeArgs g{};
    g.x = (const __half*)x;
    g.row_token = row_token;
    g.counts = counts;
    g.offsets = offsets;
    g.active = active;
    g.n_active = n_active;
    g.w0 = (const uint8_t*)m->bank[MUMMU_BANK_GATE];
    g.w1 = (const uint8_t*)m->bank[MUMMU_BANK_UP];
    g.row_bytes = (int)bank_row_bytes(c, MUMMU_BANK_GATE);
    g.expert_stride = (size_t)g.row_bytes * c.inter;
    g.K = c.hidden;
    g.n_rt = c.inter / 16;
    bool g_stream;
    plan(m->sw, g, experts_est, rows_total, nt2 ? 2 : 1, g_stream);
    g.ld_out = c.inter;
    g.out = m->hact;
    g.rows_per_expert = c.inter;
    g.status = m->status;
    // Programmatic dependent launch of the down kernel behind gate/up (measured: 2 % of the layer
    // at T=64, 6-8 % at T=8..32; MUMMU_CUDA_DECODE_NO_PDL=1 turns it off); profiling brackets
    // every launch with events, which would serialise the pair anyway.
    const bool want_pdl = !m->sw.decode_no_pdl && !m->prof.enabled;
    g.pdl = want_pdl ? 1 : 0;
    bool g_tma = false;
    int rc = nt2 ? launch_one<2, true>(m, g, experts_est, g_stream, s, "q4k_gate_up", false, &g_tma)
                 : launch_one<1, true>(m, g, experts_est, g_stream, s, "q4k_gate_up", false, &g_tma);
    if (rc) return rc;
    // profiling brackets every launch with events, which would serialise the pair anyway
    const bool pdl = g_tma && want_pdl;

    DecodeArgs d{};
    d.x = (const __half*)m->hact;
    d.row_token = nullptr;
    d.counts = counts;
    d.offsets = offsets;
    d.active = active;
    d.n_active = n_active;
    d.w0 = (const uint8_t*)m->bank[MUMMU_BANK_DOWN];
    d.w1 = nullptr;
    d.row_bytes = (int)bank_row_bytes(c, MUMMU_BANK_DOWN);
    d.expert_stride = (size_t)d.row_bytes * c.hidden;
    d.K = c.inter;
    d.n_rt = c.hidden / 32;
    bool d_stream;
    plan(m->sw, d, experts_est, rows_total, nt2 ? 2 : 1, d_stream);
    d.pdl = pdl ? 1 : 0;
    d.ld_out = c.hidden;
    d.out = ys;
    d.rows_per_expert = c.hidden;
    d.status = m->status;
    return nt2 ? launch_one<2, false>(m, d, experts_est, d_stream, s, "q4k_down", pdl)
               : launch_one<1, false>(m, d, experts_est, d_stream, s, "q4k_down", pdl);
}

int launch_decode_q4k(MummuMoe* m, const void* x, int64_t tokens, int top_k, cudaStream_t s) {
    return launch_decode_q4k_rows(m, x, m->row_token, m->counts, m->offsets, tokens * top_k, (float*)m->ys, s);
}

}  // namespace mummu
