// Streaming form of the Q4_K decode bank for calls that route to many experts (tokens <= 256 per
// call, f16 activations; reference math: crates/mummu/src/nn/moe.rs:314-316 over weights decoded
// as in gguf.rs:1701-1726, from packed bytes as models/qwen4exp/experts.rs:401-457).
//
// Three launches per layer call:
//   stage_rows     the routed rows of x, gathered and rewritten once into MMA-fragment order
//                  ("token tiles" of 8 rows, with the f16 sums of x over every 32-value sub-block),
//                  plus the work list of the two kernels below
//   gate/up        hact = silu(Wg x) * (Wu x), written as token tiles for the next kernel
//   down           ys = Wd hact
// Both expert kernels are persistent: 2 CTAs per SM pull work items (expert, token pass, run of
// jobs) from a counter, most loaded experts first, so every SM stays busy until the list is empty.
// A job is what one warp streams over all of K: for gate/up 8 gate rows + the same 8 up rows (one
// 16-row MMA tile holds both, so silu(g)*u happens in the lane that holds them), for down 16 rows.
// The token tile of an item arrives with one bulk copy (no per-CTA gather or permutation); the
// weights arrive as TMA boxes of 8 or 16 rows x 144 bytes into a private ring per warp.  Per
// (super-block, job) the arithmetic is unit_terms of decode_q4k.cuh, super-blocks in ascending
// order: bit-identical to the split-K kernel, so a token's result does not depend on its
// batch-mates (the reference asserts this, nn/moe.rs:2318-2338).
#include "decode_q4k.cuh"

namespace mummu {

constexpr int DS_THREADS = 256;
constexpr int DS_WARPS = 8;
constexpr uint32_t DS_UNIT_BYTES = 16 * Q4K_BLOCK_BYTES;   // one ring stage: 16 rows x 144 B
constexpr uint32_t DS_WAIT_LIMIT = 1u << 21;

// ------------------------------------------------------------------------------------------------
// stage_rows: x -> token tiles, sub-block sums, tile and item prefixes, counters reset
// ------------------------------------------------------------------------------------------------
struct StageArgs {
    const __half* x;            // [*, K]
    const int32_t* row_token;   // sorted row -> row of x, or null (identity)
    const int32_t* counts;      // [E]
    const int32_t* offsets;     // [E + 1]
    const int32_t* active;      // [n_active] experts with rows, most rows first
    const int32_t* n_active;
    int E, K, nt;               // nt: 8-row tiles per pass (1 or 2)
    int chunks_gu, chunks_dn;   // items per (expert, pass) of the two kernels
    uint4* tiles;               // [tile][K/256][8 words][8 rows][4 lanes-of-quad] x 16 B
    __half* sums;               // [tile][K/256][8 rows][8 sub-blocks]
    int32_t* tile_base;         // out [E]: first tile of each expert
    int32_t* item_gu;           // out [n_active + 1]: first gate/up item of each active expert
    int32_t* item_dn;           // out [n_active + 1]
    int32_t* work;              // out [2]: the two kernels' item counters, zeroed
};

__global__ void __launch_bounds__(256) stage_rows_kernel(StageArgs a) {
    __shared__ int32_t s_tile_base[257];
    __shared__ int s_e;
    const int tid = threadIdx.x;
    // tiles before each expert: every block needs its own row's; block 0 publishes all of them
    if (tid < 32) {
        int acc = 0;
        for (int e0 = 0; e0 < a.E; e0 += 32) {
            const int e = e0 + tid;
            const int c = e < a.E ? (a.counts[e] + 7) >> 3 : 0;
            int incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int up = __shfl_up_sync(0xFFFFFFFFu, incl, off);
                if (tid >= off) incl += up;
            }
            if (e < a.E) s_tile_base[e] = acc + incl - c;
            acc += __shfl_sync(0xFFFFFFFFu, incl, 31);
        }
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        for (int e = tid; e < a.E; e += blockDim.x) a.tile_base[e] = s_tile_base[e];
        if (tid == 0) {
            const int na = *a.n_active;
            int gu = 0, dn = 0;
            for (int i = 0; i < na; ++i) {
                a.item_gu[i] = gu;
                a.item_dn[i] = dn;
                const int passes = (a.counts[a.active[i]] + 8 * a.nt - 1) / (8 * a.nt);
                gu += passes * a.chunks_gu;
                dn += passes * a.chunks_dn;
            }
            a.item_gu[na] = gu;
            a.item_dn[na] = dn;
            a.work[0] = 0;
            a.work[1] = 0;
        }
    }
    const int total = a.offsets[a.E];
    const int nsb = a.K >> 8;
    const int groups = a.K >> 3;                      // 16-byte groups of 8 halves per row
    for (int p = blockIdx.x; p < total; p += gridDim.x) {
        __syncthreads();
        for (int e = tid; e < a.E; e += blockDim.x)
            if (a.offsets[e] <= p && p < a.offsets[e + 1]) s_e = e;
        __syncthreads();
        const int e = s_e;
        const int i = p - a.offsets[e];
        const int tile = s_tile_base[e] + (i >> 3), c = i & 7;
        const int64_t src = a.row_token ? a.row_token[p] : p;
        const uint4* xrow = reinterpret_cast<const uint4*>(a.x + src * a.K);
        for (int q = tid; q < groups; q += blockDim.x) {
            const uint4 v = xrow[q];
            const int sb = q >> 5, j = (q >> 2) & 7, u = q & 3;
            // elements 8u..8u+7 of sub-block j: words 2u and 2u+1 of the owning lane (j >> 1), low
            // (j even) or high (j odd) half of the 16-byte record; halves in the order (e0,e2,e1,e3)
            uint2* dst = reinterpret_cast<uint2*>(a.tiles + ((((size_t)tile * nsb + sb) * 8 + 2 * u) * 8 + c) * 4 + (j >> 1)) + (j & 1);
            dst[0] = make_uint2(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632));
            dst[2 * 32] = make_uint2(__byte_perm(v.z, v.w, 0x5410), __byte_perm(v.z, v.w, 0x7632));
            const __half2* h2 = reinterpret_cast<const __half2*>(&v);
            float s = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f2 = __half22float2(h2[k]);
                s += f2.x;
                s += f2.y;
            }
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            if (u == 0) a.sums[(((size_t)tile * nsb + sb) * 8 + c) * 8 + j] = __float2half_rn(s);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// the persistent expert kernel
// ------------------------------------------------------------------------------------------------
struct StreamArgs {
    const uint4* tiles;         // token tiles of this kernel's input
    const __half* sums;         // their sub-block sums (gate/up) or null (down: derived from the tile)
    const int32_t* counts;
    const int32_t* offsets;
    const int32_t* active;
    const int32_t* n_active;
    const int32_t* tile_base;
    const int32_t* item_base;   // [n_active + 1]
    int32_t* work;              // next item
    int nsb;                    // super-blocks per weight row
    int rows_per_expert;        // weight rows per expert in each bank view
    int jobs_per_expert;        // gate/up: inter / 8; down: hidden / 16
    int chunk_jobs;             // jobs per item
    int chunks;                 // items per (expert, pass)
    int depth;                  // ring stages per warp
    uint4* out_tiles;           // gate/up: hact as token tiles of the down kernel
    int out_nsb;                //          their super-blocks per row (inter / 256)
    float* ys;                  // down: [rows, ld_out] f32
    int ld_out;
    int pdl;
    int32_t* status;
};

struct ItemInfo {
    int e, cnt, base, pass0, tile0, job0, jobs;
};

template <int NT>
__host__ __device__ inline size_t ds_smem_bytes(int nsb, int depth) {
    return (size_t)NT * nsb * (4096 + 128) + 128 + (size_t)DS_WARPS * depth * (DS_UNIT_BYTES + 8) + 64;
}

template <int NT, bool GATEUP>
__global__ void __launch_bounds__(DS_THREADS, 2)
decode_stream_kernel(StreamArgs a, const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ ItemInfo s_item;
    __shared__ __align__(8) unsigned long long s_tok_bar;
    __shared__ int s_dead;
    const int nsb = a.nsb;
    uint4* s_frag = reinterpret_cast<uint4*>(smem_raw);                        // [NT][nsb][8][8][4]
    __half* s_sxh = reinterpret_cast<__half*>(s_frag + (size_t)NT * nsb * 256); // [NT][nsb][8][8]
    const uint32_t frag_base = smem_u32(s_frag), sxh_base = smem_u32(s_sxh);
    const uint32_t nt_frag = (uint32_t)nsb * 4096u, nt_sxh = (uint32_t)nsb * 128u;
    const uint32_t ring_base = (sxh_base + (uint32_t)NT * nt_sxh + 127u) & ~127u;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool upper = t >= 2;
    const uint32_t sel = (t & 1) ? 0x4342u : 0x4140u;
    const int depth = a.depth;
    const uint32_t ring_data = ring_base + (uint32_t)(warp * depth) * DS_UNIT_BYTES;
    const uint32_t ring_bars = ring_base + (uint32_t)(DS_WARPS * depth) * DS_UNIT_BYTES + (uint32_t)(warp * depth) * 8u;
    const uint32_t tok_bar = smem_u32(&s_tok_bar);

    if (tid == 0) {
        mbar_init(tok_bar, 1);
        s_dead = 0;
    }
    if (lane == 0)
        for (int i = 0; i < depth; ++i) mbar_init(ring_bars + (uint32_t)i * 8u, 1);
    mbar_init_fence();
    if (a.pdl && GATEUP) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    int c_stage = 0;
    uint32_t c_phase = 0, tok_phase = 0;
    bool dead = false, first = true;
    const int n_act = *a.n_active;
    const int total = a.item_base[n_act];

    while (true) {
        __syncthreads();                        // every warp is done with the token tile and with s_item
        if (tid == 0) {
            const int item = atomicAdd(a.work, 1);
            ItemInfo it;
            it.e = -1;
            if (item < total && !s_dead) {
                int lo = 0, hi = n_act;         // last active expert whose first item is <= item
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (a.item_base[mid] <= item) lo = mid; else hi = mid;
                }
                const int local = item - a.item_base[lo];
                const int pass = local / a.chunks, chunk = local - pass * a.chunks;
                it.e = a.active[lo];
                it.cnt = a.counts[it.e];
                it.base = a.offsets[it.e];
                it.pass0 = pass * 8 * NT;
                it.tile0 = a.tile_base[it.e] + pass * NT;
                it.job0 = chunk * a.chunk_jobs;
                it.jobs = min(a.chunk_jobs, a.jobs_per_expert - it.job0);
            }
            s_item = it;
        }
        __syncthreads();
        const ItemInfo it = s_item;
        if (it.e < 0) break;
        const int npass = min(8 * NT, it.cnt - it.pass0);
        const int nt_count = (npass + 7) >> 3;
        const int row_base = it.e * a.rows_per_expert;
        const int job_end = it.job0 + it.jobs;

        // ---- weights: this warp's units in the order it will consume them ----
        int p_job = it.job0 + warp, p_sb = 0;
        bool p_valid = p_job < job_end;
        auto issue = [&](int stage) {
            if (lane == 0) {
                const uint32_t bar = ring_bars + (uint32_t)stage * 8u;
                const uint32_t dst = ring_data + (uint32_t)stage * DS_UNIT_BYTES;
                mbar_expect_tx(bar, DS_UNIT_BYTES);
                if (GATEUP) {
                    const int row = row_base + p_job * 8;
                    tma_load_2d(dst, &map0, p_sb * Q4K_BLOCK_BYTES, row, bar);                      // 8 gate rows
                    tma_load_2d(dst + 8u * Q4K_BLOCK_BYTES, &map1, p_sb * Q4K_BLOCK_BYTES, row, bar);   // the same 8 up rows
                } else {
                    tma_load_2d(dst, &map0, p_sb * Q4K_BLOCK_BYTES, row_base + p_job * 16, bar);
                }
            }
            if (++p_sb == nsb) {
                p_sb = 0;
                p_job += DS_WARPS;
                p_valid = p_job < job_end;
            }
        };
        {
            int st = c_stage;
            for (int i = 0; i < depth && p_valid; ++i) {
                issue(st);
                if (++st == depth) st = 0;
            }
        }
        // ---- tokens: one bulk copy of the pass's tiles (and their sums) ----
        if (first && a.pdl && !GATEUP) asm volatile("griddepcontrol.wait;\n" ::: "memory");   // hact is complete
        first = false;
        if (tid == 0) {
            const uint32_t tile_bytes = (uint32_t)nt_count * nt_frag;
            const uint32_t sum_bytes = GATEUP ? (uint32_t)nt_count * nt_sxh : 0u;
            mbar_expect_tx(tok_bar, tile_bytes + sum_bytes);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(frag_base),
                         "l"(a.tiles + (size_t)it.tile0 * nsb * 256), "r"(tile_bytes), "r"(tok_bar)
                         : "memory");
            if (GATEUP)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(sxh_base),
                             "l"(a.sums + (size_t)it.tile0 * nsb * 64), "r"(sum_bytes), "r"(tok_bar)
                             : "memory");
        }
        if (!dead) {
            uint32_t i = 0;
            while (!mbar_test(tok_bar, tok_phase)) {
                if (++i > 64) __nanosleep(32);
                if (i >= DS_WAIT_LIMIT) {
                    dead = true;
                    s_dead = 1;
                    atomicOr(a.status, STATUS_TIMEOUT);
                    break;
                }
            }
        }
        tok_phase ^= 1u;
        if (!GATEUP) {
            // f16 sums of the activations over each 32-value sub-block, added in the order the
            // staging kernel uses: 8 values left to right, then (s0 + s1) + (s2 + s3)
            for (int idx = tid; idx < nt_count * nsb * 64; idx += DS_THREADS) {
                const int nt = idx / (nsb * 64), rem = idx - nt * nsb * 64;
                const int sb = rem >> 6, c = (rem >> 3) & 7, j = rem & 7;
                const unsigned char* rec = reinterpret_cast<const unsigned char*>(s_frag) + (size_t)nt * nt_frag +
                                           ((size_t)((sb * 8) * 8 + c) * 4 + (j >> 1)) * 16 + (j & 1) * 8;
                float su[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float s = 0.0f;
#pragma unroll
                    for (int w2 = 0; w2 < 2; ++w2) {
                        const uint2 v = *reinterpret_cast<const uint2*>(rec + (size_t)(2 * u + w2) * 8 * 4 * 16);
                        const float2 a02 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));   // (e0, e2)
                        const float2 a13 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));   // (e1, e3)
                        s += a02.x;
                        s += a13.x;
                        s += a02.y;
                        s += a13.y;
                    }
                    su[u] = s;
                }
                s_sxh[(size_t)nt * (nt_sxh / 2) + ((sb * 8 + c) * 8) + j] = __float2half_rn((su[0] + su[1]) + (su[2] + su[3]));
            }
            __syncthreads();
        }

        // ---- jobs ----
        auto run_jobs = [&](auto ntc_tag) {
            constexpr int NTC = decltype(ntc_tag)::value;
            for (int job = it.job0 + warp; job < job_end; job += DS_WARPS) {
                float y[NTC][4];
#pragma unroll
                for (int nt = 0; nt < NTC; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) y[nt][i] = 0.0f;
                uint32_t frag_addr = frag_base + (uint32_t)((g * 4 + t) * 16);
                uint32_t sxh_addr = sxh_base + (uint32_t)((g * 8 + 2 * t) * 2);
                for (int sb = 0; sb < nsb; ++sb) {
                    UnitRegs un;
                    const uint32_t bar = ring_bars + (uint32_t)c_stage * 8u;
                    if (!dead) {
                        uint32_t i = 0;
                        while (!mbar_test(bar, c_phase)) {
                            if (++i > 64) __nanosleep(32);
                            if (i >= DS_WAIT_LIMIT) {
                                dead = true;
                                s_dead = 1;
                                atomicOr(a.status, STATUS_TIMEOUT);
                                break;
                            }
                        }
                    }
                    const uint32_t row0 = ring_data + (uint32_t)c_stage * DS_UNIT_BYTES + (uint32_t)(g * Q4K_BLOCK_BYTES);
                    const uint32_t row1 = row0 + 8u * Q4K_BLOCK_BYTES;     // gate/up: the up row; down: row g + 8
                    un.hdr[0] = lds128(row0);
                    un.qa[0] = lds128(row0 + 16 + 32 * t);
                    un.qb[0] = lds128(row0 + 32 + 32 * t);
                    un.hdr[1] = lds128(row1);
                    un.qa[1] = lds128(row1 + 16 + 32 * t);
                    un.qb[1] = lds128(row1 + 32 + 32 * t);
                    __syncwarp();                   // every lane holds its copy: the stage may be refilled
                    if (p_valid) issue(c_stage);
                    if (++c_stage == depth) {
                        c_stage = 0;
                        c_phase ^= 1u;
                    }
                    unit_terms<NTC>(un, upper, sel, frag_addr, sxh_addr, nt_frag, nt_sxh, y);
                    frag_addr += 4096u;
                    sxh_addr += 128u;
                }
                // ---- epilogue from registers ----
#pragma unroll
                for (int nt = 0; nt < NTC; ++nt) {
                    if (GATEUP) {
                        // lane (g, t): gate row and up row `job*8 + g` for the tokens 2t and 2t+1 of the tile
                        const int n = job * 8 + g;
                        const int osb = n >> 8, rr = n & 255;
                        const int tq = rr >> 6, hf = (rr >> 5) & 1, w = (rr & 31) >> 2, ii = rr & 3;
                        const int pos = hf * 4 + ((ii & 1) << 1) + (ii >> 1);      // halves sit as (e0, e2, e1, e3)
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const int c = 2 * t + i;
                            if (nt * 8 + c < npass) {
                                const float s0 = y[nt][i], s1 = y[nt][i + 2];
                                const float v = (s0 / (1.0f + expf(-s0))) * s1;
                                __half* rec = reinterpret_cast<__half*>(
                                    a.out_tiles + ((((size_t)(it.tile0 + nt) * a.out_nsb + osb) * 8 + w) * 8 + c) * 4 + tq);
                                rec[pos] = __float2half_rn(v);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int slot = nt * 8 + 2 * t + (i & 1);
                            const int row = g + ((i >> 1) << 3);
                            if (slot < npass)
                                a.ys[(size_t)(it.base + it.pass0 + slot) * a.ld_out + job * 16 + row] = y[nt][i];
                        }
                    }
                }
            }
        };
        if (NT == 1 || nt_count == 1) run_jobs(std::integral_constant<int, 1>{});
        else run_jobs(std::integral_constant<int, NT>{});
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
// Tensor map of one Q4_K bank as a [rows, row_bytes] byte view with a box of `box_rows` x 144 B.
static int bank_box_map(MummuMoe* m, int slot, int which, int row_bytes, int64_t rows, int box_rows,
                        const CUtensorMap** out) {
    CUtensorMap* map = reinterpret_cast<CUtensorMap*>(m->q4k_map[slot]);
    if (m->q4k_map_base[slot] != m->bank[which]) {
        int rc = encode_tiled_2d(map, m->bank[which], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)row_bytes,
                                 (uint64_t)rows, Q4K_BLOCK_BYTES, (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        m->q4k_map_base[slot] = m->bank[which];
    }
    *out = map;
    return MUMMU_OK;
}

bool decode_stream_supported(const MummuMoe* m) {
    const MummuMoeConfig& c = m->cfg;
    return m->xt != nullptr && c.inter % 256 == 0 && c.hidden % 256 == 0 && c.experts_local <= 256 &&
           ds_smem_bytes<2>(c.hidden >> 8, 2) <= 112 * 1024 && ds_smem_bytes<2>(c.inter >> 8, 2) <= 112 * 1024;
}

template <int NT, bool GATEUP>
static int launch_stream(MummuMoe* m, StreamArgs& a, cudaStream_t s, const char* name, bool pdl_attr) {
    const MummuMoeConfig& c = m->cfg;
    int depth = 4;
    while (depth > 2 && 2 * (ds_smem_bytes<NT>(a.nsb, depth) + 1024) > 227 * 1024) --depth;
    a.depth = depth;
    const size_t smem = ds_smem_bytes<NT>(a.nsb, depth);
    const CUtensorMap *map0 = nullptr, *map1 = nullptr;
    const int64_t rows = (int64_t)c.experts_local * a.rows_per_expert;
    const int row_bytes = a.nsb * Q4K_BLOCK_BYTES;
    int rc;
    if (GATEUP) {
        if ((rc = bank_box_map(m, 3, MUMMU_BANK_GATE, row_bytes, rows, 8, &map0))) return rc;
        if ((rc = bank_box_map(m, 4, MUMMU_BANK_UP, row_bytes, rows, 8, &map1))) return rc;
    } else {
        if ((rc = bank_box_map(m, MUMMU_BANK_DOWN, MUMMU_BANK_DOWN, row_bytes, rows, 16, &map0))) return rc;
        map1 = map0;
    }
    LaunchScope scope(m, s, name);
    MUMMU_CUDA_TRY(allow_big_smem(decode_stream_kernel<NT, GATEUP>, c.device));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * 148);
    cfg.blockDim = dim3(DS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_attr ? 1 : 0;
    MUMMU_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_stream_kernel<NT, GATEUP>, a, *map0, *map1));
    return MUMMU_OK;
}

// x: input rows (f16); row_token: sorted row -> row of x, or null when x is already sorted;
// counts / offsets / the handle's active list: per local expert; rows_bound bounds the sorted rows.
// Writes ys (f32, [rows, hidden]).
int launch_decode_stream(MummuMoe* m, const void* x, const int32_t* row_token, const int32_t* counts,
                         const int32_t* offsets, int64_t rows_bound, float* ys, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    const bool nt2 = rows_bound > 8 && m->sw.decode_nt != 1;
    const int r = m->sw.decode_rb_gateup > 0 ? m->sw.decode_rb_gateup : 2;      // jobs per warp per item
    const int r_dn = m->sw.decode_rb_down > 0 ? m->sw.decode_rb_down : 2 * r;
    const int jobs_gu = c.inter / 8, jobs_dn = c.hidden / 16;
    const int chunk_gu = std::min(jobs_gu, DS_WARPS * r), chunk_dn = std::min(jobs_dn, DS_WARPS * r_dn);

    StageArgs st{};
    st.x = (const __half*)x;
    st.row_token = row_token;
    st.counts = counts;
    st.offsets = offsets;
    st.active = m->active;
    st.n_active = m->n_active;
    st.E = c.experts_local;
    st.K = c.hidden;
    st.nt = nt2 ? 2 : 1;
    st.chunks_gu = (jobs_gu + chunk_gu - 1) / chunk_gu;
    st.chunks_dn = (jobs_dn + chunk_dn - 1) / chunk_dn;
    st.tiles = (uint4*)m->xt;
    st.sums = (__half*)m->xsum;
    st.tile_base = m->tile_base;
    st.item_gu = m->item_gu;
    st.item_dn = m->item_dn;
    st.work = m->work;
    {
        LaunchScope scope(m, s, "q4k_stage_rows");
        const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(rows_bound, 148 * 8));
        stage_rows_kernel<<<blocks, 256, 0, s>>>(st);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    const bool pdl = !m->sw.decode_no_pdl && !m->prof.enabled;

    StreamArgs g{};
    g.tiles = (const uint4*)m->xt;
    g.sums = (const __half*)m->xsum;
    g.counts = counts;
    g.offsets = offsets;
    g.active = m->active;
    g.n_active = m->n_active;
    g.tile_base = m->tile_base;
    g.item_base = m->item_gu;
    g.work = m->work;
    g.nsb = c.hidden >> 8;
    g.rows_per_expert = c.inter;
    g.jobs_per_expert = jobs_gu;
    g.chunk_jobs = chunk_gu;
    g.chunks = st.chunks_gu;
    g.out_tiles = (uint4*)m->ht;
    g.out_nsb = c.inter >> 8;
    g.pdl = pdl ? 1 : 0;
    g.status = m->status;
    int rc = nt2 ? launch_stream<2, true>(m, g, s, "q4k_gate_up", false) : launch_stream<1, true>(m, g, s, "q4k_gate_up", false);
    if (rc) return rc;

    StreamArgs d{};
    d.tiles = (const uint4*)m->ht;
    d.sums = nullptr;
    d.counts = counts;
    d.offsets = offsets;
    d.active = m->active;
    d.n_active = m->n_active;
    d.tile_base = m->tile_base;
    d.item_base = m->item_dn;
    d.work = m->work + 1;
    d.nsb = c.inter >> 8;
    d.rows_per_expert = c.hidden;
    d.jobs_per_expert = jobs_dn;
    d.chunk_jobs = chunk_dn;
    d.chunks = st.chunks_dn;
    d.ys = ys;
    d.ld_out = c.hidden;
    d.pdl = pdl ? 1 : 0;
    d.status = m->status;
    return nt2 ? launch_stream<2, false>(m, d, s, "q4k_down", pdl) : launch_stream<1, false>(m, d, s, "q4k_down", pdl);
}

}  // namespace mummu
