// Router, permute, combine, the all-format SIMT expert bank and the Q4_K encode/decode kernels.
//
// The router reproduces, operation for operation, the CPU oracle's arithmetic so that routing ids
// and weights can be compared bit for bit:
//   logit  = 8-lane dot product: lane l accumulates elements l, l+8, ... with one fused
//            multiply-add per step; lanes fold as ((a0+a4)+(a1+a5))+((a2+a6)+(a3+a7)); leftover
//            elements are fused in one by one (lane order of the reference's
//            models/qwen4exp/experts.rs:463-478, fused steps like the gemm crate behind burn's Linear)
//   p      = exp_det(logit - max) / (left-to-right sum)           (nn/moe.rs:2138-2141)
//   top-k  = descending p, equal p in ascending expert id         (experts.rs:532-535, 562-574)
//   weight = p, or p / (sum of the picked p in slot order)        (nn/moe.rs:146-150, 2146-2152)
#include <cfloat>
#include <climits>
#include <cstdlib>

#include "common.cuh"
#include "tma.cuh"

namespace mummu {

// ---------------------------------------------------------------------------------------------
// deterministic e^x: the same IEEE operation sequence as the oracle's orc_exp
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float exp_det(float x) {
    if (x != x) return x;
    if (x > 88.7f) return __int_as_float(0x7F800000);
    if (x < -104.0f) return 0.0f;
    const float LOG2E = 1.4426950216293335f;
    const float LN2_HI = 0.693145751953125f;
    const float LN2_LO = 1.4286068203094172e-06f;
    const float MAGIC = 12582912.0f;
    float t = __fmaf_rn(x, LOG2E, MAGIC);
    float n = __fsub_rn(t, MAGIC);
    float r = __fmaf_rn(-n, LN2_HI, x);
    r = __fmaf_rn(-n, LN2_LO, r);
    float p = 1.0f / 5040.0f;
    p = __fmaf_rn(p, r, 1.0f / 720.0f);
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    int ni = (int)n;
    int a = ni / 2;
    int b = ni - a;
    float fa = __int_as_float((a + 127) << 23);
    float fb = __int_as_float((b + 127) << 23);
    return __fmul_rn(__fmul_rn(p, fa), fb);
}

// ---------------------------------------------------------------------------------------------
// router
// ---------------------------------------------------------------------------------------------
constexpr int R_ES = 8;          // experts per block
constexpr int R_THREADS = 256;   // 8 experts x 8 lanes x 4 token groups
constexpr int R_MAXV = 8;        // probabilities per lane in the top-k stage: experts <= 256

struct RouterArgs {
    const void* x;
    const float* w;      // [H, E]
    const float* wt;     // shared-memory image of the 8-expert slices, or null
    const float* bias;   // [E] or null
    float* logits;       // [T, E] scratch
    int32_t* tile_done;  // [tiles] zero on entry, zero on exit
    int32_t* ids;        // [T, k]
    float* wts;          // [T, k]
    int32_t* counts;     // [E] or null
    unsigned long long* hits;  // [E] or null
    int32_t* status;
    int T, H, E, k, norm;
    // decode-sized calls: the block that finishes last also groups the (token, slot) pairs by
    // expert, so the layer needs no separate permute launch (see fused_permute)
    int fuse;
    int32_t* p_counts;
    int32_t* p_offsets;
    int32_t* p_row_token;
    int32_t* p_pos;
    int32_t* p_active;
    int32_t* p_n_active;
};

// One warp: softmax over one token's logits, then top-k.  sm_v: E floats, sm_vals: k floats,
// sm_ids: k ints (all private to the warp).
template <int NV = R_MAXV>   // probabilities per lane: experts <= 32 * NV
__device__ void warp_softmax_topk(const RouterArgs& a, int t, float* sm_v, float* sm_vals,
                                  int32_t* sm_ids) {
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xFFFFFFFFu;
    const float* lrow = a.logits + (size_t)t * a.E;
    float l[NV], p[NV];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        int e = lane + 32 * i;
        l[i] = e < a.E ? __ldcg(lrow + e) : -FLT_MAX;
        if (e < a.E && !isfinite(l[i])) bad = true;
    }
    bad = __any_sync(full, bad);
    if (bad) {
        // the reference's host router refuses non-finite logits (experts.rs:553-560); here the
        // token gets experts 0..k-1 with zero weight and the sticky status word records it
        if (lane == 0) atomicOr(a.status, STATUS_NONFINITE);
        for (int r = lane; r < a.k; r += 32) {
            a.ids[(size_t)t * a.k + r] = r;
            a.wts[(size_t)t * a.k + r] = 0.0f;
            if (a.counts) atomicAdd(a.counts + r, 1);
            if (a.hits) atomicAdd(a.hits + r, 1ull);
        }
        return;
    }
    float mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < NV; ++i) mx = fmaxf(mx, l[i]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(full, mx, off));
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        int e = lane + 32 * i;
        if (e < a.E) {
            p[i] = exp_det(__fsub_rn(l[i], mx));
            sm_v[e] = p[i];
        }
    }
    __syncwarp();
    float total = 0.0f;
#pragma unroll 8
    for (int e = 0; e < a.E; ++e) total = __fadd_rn(total, sm_v[e]);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        int e = lane + 32 * i;
        p[i] = e < a.E ? __fdiv_rn(p[i], total) : -1.0f;
    }
    float denom = 0.0f;
    for (int r = 0; r < a.k; ++r) {
        float bp = -2.0f;
        int be = INT_MAX;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (p[i] > bp) {
                bp = p[i];
                be = lane + 32 * i;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            float op = __shfl_xor_sync(full, bp, off);
            int oe = __shfl_xor_sync(full, be, off);
            if (op > bp || (op == bp && oe < be)) {
                bp = op;
                be = oe;
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (be == lane + 32 * i) p[i] = -1.0f;
        denom = __fadd_rn(denom, bp);
        if (lane == 0) {
            sm_vals[r] = bp;
            sm_ids[r] = be;
        }
    }
    __syncwarp();
    for (int r = lane; r < a.k; r += 32) {
        float wv = sm_vals[r];
        if (a.norm) wv = __fdiv_rn(wv, denom);
        int e = sm_ids[r];
        a.ids[(size_t)t * a.k + r] = e;
        a.wts[(size_t)t * a.k + r] = wv;
        if (a.counts) atomicAdd(a.counts + e, 1);
        if (a.hits) atomicAdd(a.hits + e, 1ull);
    }
    __syncwarp();
}


// One block (256 threads) builds, for at most 1024 (token, slot) pairs, everything permute_kernel
// builds: counts, offsets, the heaviest-first active list, row_token and pos (stable: ascending
// token inside an expert).  Called by the last block of router_kernel; scratch is that block's
// dynamic shared memory, free by then.  Counting sort in three parallel steps: per 32-pair chunk
// a histogram by expert (warp match), an exclusive prefix over the chunks per expert, then
// pos = offset[expert] + pairs of that expert in earlier chunks + rank inside the chunk.
__device__ void fused_permute(const RouterArgs& a, unsigned char* smem_raw) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = a.T * a.k, E = a.E;
    const int chunks = (n + 31) >> 5;
    int32_t* ids_s = reinterpret_cast<int32_t*>(smem_raw);      // [chunks * 32]
    int32_t* cnt_s = ids_s + chunks * 32;                        // [E]
    int32_t* off_s = cnt_s + E;                                  // [E + 1]
    int32_t* hist = off_s + E + 1;                               // [chunks][E] -> exclusive prefix over chunks
    for (int i = tid; i < chunks * E; i += R_THREADS) hist[i] = 0;
    __syncthreads();
    for (int c = warp; c < chunks; c += R_THREADS / 32) {
        const int i = c * 32 + lane;
        const int e = i < n ? __ldcg(a.ids + i) : -1;
        ids_s[i] = e;
        const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
        if (e >= 0 && (same & ((1u << lane) - 1u)) == 0) hist[c * E + e] = __popc(same);   // group leader
    }
    __syncthreads();
    for (int e = tid; e < E; e += R_THREADS) {
        int run = 0;
        for (int c = 0; c < chunks; ++c) {
            const int h = hist[c * E + e];
            hist[c * E + e] = run;
            run += h;
        }
        cnt_s[e] = run;
    }
    __syncthreads();
    if (warp == 0) {
        int acc = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < E ? cnt_s[e] : 0;
            int incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int up = __shfl_up_sync(0xFFFFFFFFu, incl, off);
                if (lane >= off) incl += up;
            }
            if (e < E) off_s[e] = acc + incl - c;
            acc += __shfl_sync(0xFFFFFFFFu, incl, 31);
        }
        if (lane == 0) off_s[E] = acc;
    }
    __syncthreads();
    // heaviest-first order: rank of expert e = experts that come before it; four threads per expert
    // each compare against a quarter of the others
    for (int q0 = 0; q0 < 4 * E; q0 += R_THREADS) {       // every thread makes every trip (shuffles)
        const int q = q0 + tid;
        const bool valid = q < 4 * E;
        const int e = valid ? q >> 2 : 0, part = q & 3;
        const int c = cnt_s[e];
        int rank = 0;
        for (int i = part; i < E; i += 4) {
            const int ci = cnt_s[i];
            rank += (ci > c || (ci == c && i < e)) ? 1 : 0;
        }
        rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 1);
        rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 2);
        if (valid && part == 0) {
            a.p_counts[e] = c;
            a.p_offsets[e] = off_s[e];
            if (c > 0) a.p_active[rank] = e;
        }
    }
    if (warp == 1) {
        int nz = 0;
        for (int e = lane; e < E; e += 32) nz += cnt_s[e] > 0;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) nz += __shfl_xor_sync(0xFFFFFFFFu, nz, off);
        if (lane == 0) {
            a.p_offsets[E] = off_s[E];
            *a.p_n_active = nz;
        }
    }
    for (int c = warp; c < chunks; c += R_THREADS / 32) {
        const int i = c * 32 + lane;
        const int e = ids_s[i];
        const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
        if (e >= 0) {
            const int p = off_s[e] + hist[c * E + e] + __popc(same & ((1u << lane) - 1u));
            a.p_row_token[p] = i / a.k;
            a.p_pos[i] = p;
        }
    }
}

// grid (expert slices, token tiles).  Each block stages its 8-expert slice of W and its token
// tile of x in shared memory, computes the logits in the fixed lane order, and the block that
// finishes a token tile last runs softmax + top-k for that tile.
// TR (hidden % 32 == 0, experts % 8 == 0, 16-byte aligned 16-bit activations): W and x sit in
// shared memory transposed, one padded row per (lane j, expert) resp. (token, lane j), so that a
// thread's chain reads four consecutive steps with one 128-bit load; same sums in the same order.
template <typename TX, int TPT, bool TR>
__global__ void __launch_bounds__(R_THREADS) router_kernel(RouterArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long w_bar;         // TR: completion of the W bulk copy
    constexpr int TT = 4 * TPT;
    const int H = a.H, E = a.E;
    const int H8 = H & ~7;
    const int S = (H >> 3) + 4;                                // padded row of the transposed layout
    float* Ws = reinterpret_cast<float*>(smem_raw);           // [H8][8]        | TR: [8 j][8 e][S]
    float* xs = Ws + (TR ? (size_t)64 * S : (size_t)H8 * R_ES);   // [TT][H]    | TR: [TT][8 j][S]
    float* parts = xs + (TR ? (size_t)TT * 8 * S : (size_t)TT * H);   // [TT][8][8]
    float* tk = parts + TT * 64;                               // top-k scratch, 8 warps
    const int tid = threadIdx.x;
    const int e0 = blockIdx.x * R_ES;
    const int t0 = blockIdx.y * TT;
    const TX* x = reinterpret_cast<const TX*>(a.x);

    if constexpr (TR) {
        const int steps = H >> 3;                              // i = 0 .. steps-1, row h = 8 i + j
        // x first (kept in registers while W streams in), then W eight rows per thread at a time
        // with all loads issued before the first store: the block's critical path is L2 latency
        constexpr int XU = TT;                                // 16-byte groups per thread up to H = 2048
        uint4 xv[XU];
        const int xgroups = TT * steps;
#pragma unroll
        for (int u = 0; u < XU; ++u) {
            const int idx = tid + u * R_THREADS;
            xv[u] = make_uint4(0, 0, 0, 0);
            if (idx < xgroups && idx < XU * R_THREADS) {
                const int tt = idx / steps, i = idx - tt * steps;
                if (t0 + tt < a.T) xv[u] = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + tt) * H + (size_t)i * 8);
            }
        }
        // W: the slice's image lies contiguous in global memory; one bulk copy by the copy engine
        // (issued first, above the x loads would be even better, but x needs no barrier)
        const uint32_t bar = smem_u32(&w_bar);
        const uint32_t w_bytes = (uint32_t)(64 * S * 4);
        if (tid == 0) {
            mbar_init(bar, 1);
            mbar_init_fence();
            mbar_expect_tx(bar, w_bytes);
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                    smem_u32(Ws)),
                "l"(a.wt + (size_t)blockIdx.x * 64 * S), "r"(w_bytes), "r"(bar)
                : "memory");
        }
#pragma unroll
        for (int u = 0; u < XU; ++u) {
            const int idx = tid + u * R_THREADS;
            if (idx < xgroups && idx < XU * R_THREADS) {
                const int tt = idx / steps, i = idx - tt * steps;
                const TX* hv = reinterpret_cast<const TX*>(&xv[u]);
                float* dst = xs + (size_t)(tt * 8) * S + i;
#pragma unroll
                for (int q = 0; q < 8; ++q) dst[q * S] = to_f32(hv[q]);
            }
        }
        // wider rows than the registers above cover (hidden > 2048): the rest, plainly
        for (int idx = tid + XU * R_THREADS; idx < xgroups; idx += R_THREADS) {
            const int tt = idx / steps, i = idx - tt * steps;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t0 + tt < a.T) v = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + tt) * H + (size_t)i * 8);
            const TX* hv = reinterpret_cast<const TX*>(&v);
            float* dst = xs + (size_t)(tt * 8) * S + i;
#pragma unroll
            for (int q = 0; q < 8; ++q) dst[q * S] = to_f32(hv[q]);
        }
    } else if ((E & 3) == 0 && e0 + R_ES <= E) {
        // 8 experts of one row = two aligned float4
        const float4* w4 = reinterpret_cast<const float4*>(a.w);
        float4* Ws4 = reinterpret_cast<float4*>(Ws);
        const int e4 = E >> 2, o4 = e0 >> 2;
#pragma unroll 8
        for (int idx = tid; idx < H8 * 2; idx += R_THREADS)
            Ws4[idx] = __ldg(w4 + (size_t)(idx >> 1) * e4 + o4 + (idx & 1));
    } else {
        for (int idx = tid; idx < H8 * R_ES; idx += R_THREADS) {
            int i = idx >> 3, el = idx & 7;
            int e = e0 + el;
            Ws[idx] = e < E ? a.w[(size_t)i * E + e] : 0.0f;
        }
    }
    if constexpr (TR) {
    } else if (sizeof(TX) == 2 && (H & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const int groups = H >> 3;
#pragma unroll 4
        for (int idx = tid; idx < TT * groups; idx += R_THREADS) {
            int tt = idx / groups, q = idx - tt * groups;
            int t = t0 + tt;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t < a.T) v = *reinterpret_cast<const uint4*>(x + (size_t)t * H + (size_t)q * 8);
            const TX* hv = reinterpret_cast<const TX*>(&v);
            float* dst = xs + (size_t)tt * H + (size_t)q * 8;
#pragma unroll
            for (int u = 0; u < 8; ++u) dst[u] = to_f32(hv[u]);
        }
    } else {
        for (int idx = tid; idx < TT * H; idx += R_THREADS) {
            int tt = idx / H, h = idx - tt * H;
            int t = t0 + tt;
            xs[idx] = t < a.T ? to_f32(x[(size_t)t * H + h]) : 0.0f;
        }
    }
    if constexpr (TR) {
        __syncthreads();                       // the barrier initialised by thread 0 is visible
        uint32_t polls = 0;
        while (!mbar_try_wait(smem_u32(&w_bar), 0, 1000u)) {
            if (++polls > (1u << 20)) {        // a bulk copy from valid memory always lands; bounded anyway
                if (tid == 0) atomicOr(a.status, STATUS_TIMEOUT);
                break;
            }
        }
    }
    __syncthreads();

    const int el = tid & 7, j = (tid >> 3) & 7, tg = tid >> 6;
    float acc[TPT];
#pragma unroll
    for (int u = 0; u < TPT; ++u) acc[u] = 0.0f;
    const int iters = H8 >> 3;
    if constexpr (TR) {
        const float4* wrow = reinterpret_cast<const float4*>(Ws + (size_t)(j * 8 + el) * S);
#pragma unroll 4
        for (int i4 = 0; i4 < (iters >> 2); ++i4) {
            const float4 wv = wrow[i4];
#pragma unroll
            for (int u = 0; u < TPT; ++u) {
                const float4 xv = reinterpret_cast<const float4*>(xs + (size_t)((tg + 4 * u) * 8 + j) * S)[i4];
                acc[u] = __fmaf_rn(xv.x, wv.x, acc[u]);
                acc[u] = __fmaf_rn(xv.y, wv.y, acc[u]);
                acc[u] = __fmaf_rn(xv.z, wv.z, acc[u]);
                acc[u] = __fmaf_rn(xv.w, wv.w, acc[u]);
            }
        }
    } else {
#pragma unroll 4
        for (int i = 0; i < iters; ++i) {
            float wv = Ws[(i * 8 + j) * R_ES + el];
#pragma unroll
            for (int u = 0; u < TPT; ++u) {
                float xv = xs[(size_t)(tg + 4 * u) * H + i * 8 + j];
                acc[u] = __fmaf_rn(xv, wv, acc[u]);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < TPT; ++u) parts[((tg + 4 * u) * 8 + el) * 8 + j] = acc[u];
    __syncthreads();
    if (tid < TT * 8) {
        int tt = tid >> 3, el2 = tid & 7;
        int t = t0 + tt, e = e0 + el2;
        if (t < a.T && e < E) {
            const float* q = parts + (tt * 8 + el2) * 8;
            float s = __fadd_rn(__fadd_rn(__fadd_rn(q[0], q[4]), __fadd_rn(q[1], q[5])),
                                __fadd_rn(__fadd_rn(q[2], q[6]), __fadd_rn(q[3], q[7])));
            for (int i = H8; i < H; ++i)
                s = __fmaf_rn(xs[(size_t)tt * H + i], a.w[(size_t)i * E + e], s);
            if (a.bias) s = __fadd_rn(s, a.bias[e]);
            a.logits[(size_t)t * E + e] = s;
        }
    }
    // last block of this token tile does the selection
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int done = atomicAdd(a.tile_done + blockIdx.y, 1);
        is_last = (done == (int)gridDim.x - 1);
        if (is_last) a.tile_done[blockIdx.y] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const int warp = tid >> 5;
    const int per_warp = E + 2 * a.k;
    float* sm_v = tk + (size_t)warp * per_warp;
    float* sm_vals = sm_v + E;
    int32_t* sm_ids = reinterpret_cast<int32_t*>(sm_vals + a.k);
    for (int tt = warp; tt < TT; tt += R_THREADS / 32) {
        int t = t0 + tt;
        if (t < a.T) {
            if (E <= 64) warp_softmax_topk<2>(a, t, sm_v, sm_vals, sm_ids);
            else warp_softmax_topk<R_MAXV>(a, t, sm_v, sm_vals, sm_ids);
        }
    }
    if (!a.fuse) return;
    // the block that finishes the last token tile groups the pairs by expert
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int32_t* all_done = a.tile_done + gridDim.y;
        int done = atomicAdd(all_done, 1);
        is_last = (done == (int)gridDim.y - 1);
        if (is_last) *all_done = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    fused_permute(a, smem_raw);
}


// Large-T router: one block owns ALL experts of a tile of 16 tokens (thread = (expert, lane) of the
// 8-lane dot), so the router weight is read once per 16 tokens, the logits never leave shared memory
// and the selection runs in the same block.  Same arithmetic, same order as router_kernel.
// SPLIT groups of e_pad*8 threads share the staged tokens; group g owns tokens g*RW_TT/SPLIT ... of the tile,
// which doubles the resident warps (latency hiding) at the same shared-memory footprint.
template <typename TX, int e_pad, int RW_TT, int SPLIT>
__global__ void __launch_bounds__(e_pad * 8 * SPLIT) router_wide_kernel(RouterArgs a) {
    constexpr int TPG = RW_TT / SPLIT;   // tokens per thread group
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, E = a.E;
    const int H8 = H & ~7;
    const int row = (H8 >> 3) + 4;                               // padded length of one (token, lane) row
    float* xs = reinterpret_cast<float*>(smem_raw);              // [TT][8][row]: element k = 8i+j at [j][i]
    float* parts = xs + (size_t)RW_TT * 8 * row;                 // [TT][e_pad][8]
    float* logit_s = parts + (size_t)RW_TT * e_pad * 8;          // [TT][E]
    float* tk = logit_s + (size_t)RW_TT * E;                     // top-k scratch per warp
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int t0 = blockIdx.x * RW_TT;
    const TX* x = reinterpret_cast<const TX*>(a.x);
    for (int tt = 0; tt < RW_TT; ++tt) {
        const int t = t0 + tt;
        for (int k = tid; k < H8; k += nthreads)
            xs[((size_t)tt * 8 + (k & 7)) * row + (k >> 3)] = t < a.T ? to_f32(x[(size_t)t * H + k]) : 0.0f;
    }
    __syncthreads();
    const int grp = tid / (e_pad * 8), lt = tid - grp * (e_pad * 8);
    const int e = lt % e_pad, j = lt / e_pad;                    // a warp = 32 experts of one lane j
    const int tt0 = grp * TPG;
    float acc[TPG];
#pragma unroll
    for (int tt = 0; tt < TPG; ++tt) acc[tt] = 0.0f;
    if (e < E) {
        const float* wcol = a.w + e;
        const int quads = H8 >> 5;                               // 4 lane-steps (32 k) per iteration
        // the weight stream runs 3 iterations ahead of the arithmetic through a 4-slot register ring
        // (slot index is a compile-time constant after the 4x unroll)
        float ring[4][4];
#pragma unroll
        for (int d = 0; d < 3; ++d)
#pragma unroll
            for (int u = 0; u < 4; ++u) ring[d][u] = d < quads ? __ldg(wcol + (size_t)(8 * (4 * d + u) + j) * E) : 0.0f;
        int q = 0;
        for (; q + 4 <= quads; q += 4) {
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                const int qq = q + d;
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    ring[(d + 3) & 3][u] = qq + 3 < quads ? __ldg(wcol + (size_t)(8 * (4 * (qq + 3) + u) + j) * E) : 0.0f;
#pragma unroll
                for (int tt = 0; tt < TPG; ++tt) {
                    const float4 xv = *reinterpret_cast<const float4*>(xs + ((size_t)(tt0 + tt) * 8 + j) * row + 4 * qq);
                    acc[tt] = __fmaf_rn(xv.x, ring[d][0], acc[tt]);
                    acc[tt] = __fmaf_rn(xv.y, ring[d][1], acc[tt]);
                    acc[tt] = __fmaf_rn(xv.z, ring[d][2], acc[tt]);
                    acc[tt] = __fmaf_rn(xv.w, ring[d][3], acc[tt]);
                }
            }
        }
        for (; q < quads; ++q) {                                 // fewer than 4 iterations left
            float w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = __ldg(wcol + (size_t)(8 * (4 * q + u) + j) * E);
#pragma unroll
            for (int tt = 0; tt < TPG; ++tt) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + ((size_t)(tt0 + tt) * 8 + j) * row + 4 * q);
                acc[tt] = __fmaf_rn(xv.x, w[0], acc[tt]);
                acc[tt] = __fmaf_rn(xv.y, w[1], acc[tt]);
                acc[tt] = __fmaf_rn(xv.z, w[2], acc[tt]);
                acc[tt] = __fmaf_rn(xv.w, w[3], acc[tt]);
            }
        }
        for (int i = quads * 4; i < (H8 >> 3); ++i) {            // lane-steps left when H8 % 32 != 0
            const float wv = __ldg(wcol + (size_t)(8 * i + j) * E);
#pragma unroll
            for (int tt = 0; tt < TPG; ++tt)
                acc[tt] = __fmaf_rn(xs[((size_t)(tt0 + tt) * 8 + j) * row + i], wv, acc[tt]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < TPG; ++tt) parts[((size_t)(tt0 + tt) * e_pad + e) * 8 + j] = acc[tt];
    __syncthreads();
    for (int o = tid; o < RW_TT * E; o += nthreads) {
        const int tt = o / E, e2 = o - tt * E;
        const int t = t0 + tt;
        if (t < a.T) {
            const float* q = parts + ((size_t)tt * e_pad + e2) * 8;
            float sacc = __fadd_rn(__fadd_rn(__fadd_rn(q[0], q[4]), __fadd_rn(q[1], q[5])),
                                   __fadd_rn(__fadd_rn(q[2], q[6]), __fadd_rn(q[3], q[7])));
            for (int i = H8; i < H; ++i)
                sacc = __fmaf_rn(to_f32(x[(size_t)t * H + i]), a.w[(size_t)i * E + e2], sacc);
            if (a.bias) sacc = __fadd_rn(sacc, a.bias[e2]);
            a.logits[(size_t)t * E + e2] = sacc;                 // selection below reads them back (L1 bypass)
        }
    }
    __threadfence_block();
    __syncthreads();
    const int warp = tid >> 5, nwarps = nthreads >> 5;
    const int per_warp = E + 2 * a.k;
    for (int tt = warp; tt < RW_TT; tt += nwarps) {
        const int t = t0 + tt;
        float* sm_v = tk + (size_t)warp * per_warp;
        if (t < a.T) warp_softmax_topk(a, t, sm_v, sm_v + E, reinterpret_cast<int32_t*>(sm_v + E + a.k));
    }
}

// Register-tiled large-T router.  The oracle's dot is 8 independent FMA chains per (token, expert),
// chain j over k = j, 8 + j, 16 + j, ... in ascending order: eight K = H / 8 matrix products whose
// inner loop may be tiled freely as long as each chain stays in one thread, in order.  Here warp j
// of a block owns chain j for a tile of TM * 4 tokens x 64 experts; a thread keeps TM x 8
// accumulators, so a k-step costs (TM + 8) / 4 shared-memory loads of 16 bytes for TM * 8 FMAs, and
// the router weight is read from L2 once per TM * 4 tokens instead of once per 8.  Chunks of 64 k
// are staged three deep (weights by cp.async, tokens converted to f32 and laid out per chain on
// the way in).  Experts beyond the first 64 take further passes over the same tokens; logits,
// selection and counters are the same code as in the other router kernels.
constexpr int RT_KC = 64;                  // k per stage: 8 steps of every chain
constexpr int RT_XROW = 36;                // floats per (chain, step) row of tokens: 32 + 4 against bank conflicts
constexpr int RT_XSTAGES = 2;

__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Two independent IEEE f32 FMAs in one instruction (sm_100): halves the issue slots of the k loop.
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// a token's 8 consecutive values as they sit in memory (converted when they are stored)
template <typename TX> struct OctetRaw { uint4 r; };
template <> struct OctetRaw<float> { uint4 r, r2; };
template <typename TX> __device__ __forceinline__ void load_raw(const TX* p, OctetRaw<TX>& o) {
    o.r = *reinterpret_cast<const uint4*>(p);
}
template <> __device__ __forceinline__ void load_raw<float>(const float* p, OctetRaw<float>& o) {
    o.r = *reinterpret_cast<const uint4*>(p);
    o.r2 = *reinterpret_cast<const uint4*>(p + 4);
}
__device__ __forceinline__ void octet_f32(const OctetRaw<float>& o, float (&v)[8]) {
    v[0] = __uint_as_float(o.r.x); v[1] = __uint_as_float(o.r.y); v[2] = __uint_as_float(o.r.z); v[3] = __uint_as_float(o.r.w);
    v[4] = __uint_as_float(o.r2.x); v[5] = __uint_as_float(o.r2.y); v[6] = __uint_as_float(o.r2.z); v[7] = __uint_as_float(o.r2.w);
}
__device__ __forceinline__ void octet_f32(const OctetRaw<__half>& o, float (&v)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&o.r);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const float2 f = __half22float2(h[u]);
        v[2 * u] = f.x;
        v[2 * u + 1] = f.y;
    }
}
__device__ __forceinline__ void octet_f32(const OctetRaw<__nv_bfloat16>& o, float (&v)[8]) {
    // bf16 -> f32 is a shift: no conversion instruction
    const uint32_t w[4] = {o.r.x, o.r.y, o.r.z, o.r.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        v[2 * u] = __uint_as_float(w[u] << 16);
        v[2 * u + 1] = __uint_as_float(w[u] & 0xFFFF0000u);
    }
}

template <typename TX> __device__ __forceinline__ void load_octet(const TX* p, float (&v)[8]);
template <> __device__ __forceinline__ void load_octet<float>(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load_octet<__half>(const __half* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const float2 f = __half22float2(h[u]);
        v[2 * u] = f.x;
        v[2 * u + 1] = f.y;
    }
}
template <> __device__ __forceinline__ void load_octet<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const float2 f = __bfloat1622float2(h[u]);
        v[2 * u] = f.x;
        v[2 * u + 1] = f.y;
    }
}

// stages of the asynchronous copies: a 16-token tile spends so little time on a chunk that it needs
// more chunks in flight to cover the latency of L2
constexpr int rt_stages(int TM) { return TM == 4 ? 5 : 3; }

static size_t router_tile_smem(int E, int k, int TM, size_t x_size) {
    const size_t S = rt_stages(TM);
    const size_t stage = S * RT_KC * 64 * 4 + (size_t)RT_XSTAGES * 8 * 8 * RT_XROW * 4 + S * (TM * 4) * RT_KC * x_size;
    const size_t parts = (size_t)8 * (TM * 4) * 68 * 4;
    return (stage > parts ? stage : parts) + (size_t)8 * (E + 2 * k) * 4;
}

template <typename TX, int TM>
__global__ void __launch_bounds__(256, 2) router_tile_kernel(RouterArgs a) {
    constexpr int S = rt_stages(TM);                             // copies in flight: S - 1 chunks ahead
    constexpr int TT = TM * 4;                                   // tokens per block
    constexpr int NH = TM / 4;                                   // 4-token groups per thread
    constexpr int OCT = 8 * (int)sizeof(TX);                     // bytes of 8 consecutive values of a token
    constexpr size_t STAGE_B = (size_t)S * RT_KC * 64 * 4 + (size_t)RT_XSTAGES * 8 * 8 * RT_XROW * 4 +
                               (size_t)S * TT * RT_KC * sizeof(TX);
    constexpr size_t PARTS_B = (size_t)8 * TT * 68 * 4;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* ws = reinterpret_cast<float*>(smem_raw);              // [S][8 chains][8 steps][64 experts]
    float* xs = ws + S * RT_KC * 64;                    // [2][8 chains][8 steps][RT_XROW tokens]
    unsigned char* raws = reinterpret_cast<unsigned char*>(xs + RT_XSTAGES * 8 * 8 * RT_XROW);   // [S][TT][64 k] as stored
    float* parts = reinterpret_cast<float*>(smem_raw);           // after the k loop: [8 chains][TT][68]
    float* tk = reinterpret_cast<float*>(smem_raw + (STAGE_B > PARTS_B ? STAGE_B : PARTS_B));
    const int tid = threadIdx.x, lane = tid & 31, j = tid >> 5;
    const int tg = lane >> 3, eg = lane & 7;
    const int H = a.H, E = a.E, H8 = H & ~7;
    const int t0 = blockIdx.x * TT;
    const TX* x = reinterpret_cast<const TX*>(a.x);
    const int chunks = H8 / RT_KC;
    // staging roles: thread -> (token, octet of the chunk) for x; four 16-byte pieces of the weights
    const int x_oc = tid & 7, x_t = tid >> 3;
    const bool x_role = x_t < TT;
    const bool x_valid = x_role && t0 + x_t < a.T;
    const TX* x_src = x + (size_t)(t0 + (x_valid ? x_t : 0)) * H + x_oc * 8;
    unsigned char* x_raw = raws + ((size_t)x_t * 8 + x_oc) * OCT;

    for (int e0 = 0; e0 < E; e0 += 64) {
        unsigned long long acc[TM][4];                           // [token][expert pair]
#pragma unroll
        for (int m = 0; m < TM; ++m)
#pragma unroll
            for (int n = 0; n < 4; ++n) acc[m][n] = 0ull;
        // group g of the asynchronous copies: weights of chunk g, tokens (as stored) of chunk g + 1
        auto stage = [&](int g) {
            if (g < chunks) {
                float* dst = ws + (size_t)(g % S) * RT_KC * 64;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int idx = tid + 256 * r, kk = idx >> 4, e4 = (idx & 15) * 4;
                    const bool ok = e0 + e4 < E;                 // E % 4 == 0: a piece is inside or outside
                    cp_async16_zfill(dst + ((kk & 7) * 8 + (kk >> 3)) * 64 + e4,
                                     a.w + (size_t)(g * RT_KC + kk) * E + (ok ? e0 + e4 : 0), ok);
                }
            }
            if (g + 1 < chunks && x_role) {
                unsigned char* dst = x_raw + (size_t)((g + 1) % S) * TT * RT_KC * sizeof(TX);
                const TX* src = x_src + (size_t)(g + 1) * RT_KC;
                cp_async16_zfill(dst, src, x_valid);
                if (sizeof(TX) == 4) cp_async16_zfill(dst + 16, src + 4, x_valid);
            }
            cp_async_commit();
        };
        auto store_x = [&](int c, const OctetRaw<TX>& raw) {     // chunk c: converted, one row per (chain, step)
            float v[8];
            octet_f32(raw, v);
            float* dst = xs + (size_t)(c % RT_XSTAGES) * 8 * 8 * RT_XROW;
#pragma unroll
            for (int u = 0; u < 8; ++u) dst[(u * 8 + x_oc) * RT_XROW + x_t] = v[u];
        };
        OctetRaw<TX> xraw;
        __syncthreads();                                         // the previous pass is done with the buffers
#pragma unroll
        for (int g = 0; g < S - 1; ++g) stage(g);
        if (x_role) {
            load_raw<TX>(x_src, xraw);
            if (!x_valid) xraw = OctetRaw<TX>{};
            store_x(0, xraw);
        }
        cp_async_wait<S - 2>();
        __syncthreads();
        for (int c = 0; c < chunks; ++c) {
            stage(c + S - 1);
            if (c + 1 < chunks && x_role) {                      // landed with group c
                const unsigned char* src = x_raw + (size_t)((c + 1) % S) * TT * RT_KC * sizeof(TX);
                xraw.r = *reinterpret_cast<const uint4*>(src);
                if constexpr (sizeof(TX) == 4) xraw.r2 = *reinterpret_cast<const uint4*>(src + 16);
                store_x(c + 1, xraw);
            }
            const float* wj = ws + (size_t)(c % S) * RT_KC * 64 + (size_t)j * 8 * 64;
            const float* xj = xs + (size_t)(c % RT_XSTAGES) * 8 * 8 * RT_XROW + (size_t)j * 8 * RT_XROW;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const ulonglong2 w0 = *reinterpret_cast<const ulonglong2*>(wj + i * 64 + eg * 4);
                const ulonglong2 w1 = *reinterpret_cast<const ulonglong2*>(wj + i * 64 + 32 + eg * 4);
                const unsigned long long wp[4] = {w0.x, w0.y, w1.x, w1.y};
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    const float4 xq = *reinterpret_cast<const float4*>(xj + i * RT_XROW + h * 16 + tg * 4);
                    const unsigned long long xp[4] = {pack2(xq.x, xq.x), pack2(xq.y, xq.y), pack2(xq.z, xq.z), pack2(xq.w, xq.w)};
#pragma unroll
                    for (int m = 0; m < 4; ++m)
#pragma unroll
                        for (int n = 0; n < 4; ++n) acc[h * 4 + m][n] = fma2(xp[m], wp[n], acc[h * 4 + m][n]);
                }
            }
            cp_async_wait<S - 2>();
            __syncthreads();
        }
        cp_async_wait<0>();
        __syncthreads();
        // chain partials -> shared memory (over the staging buffers), then the fixed tree
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                float* dst = parts + ((size_t)j * TT + h * 16 + tg * 4 + m) * 68;
                *reinterpret_cast<ulonglong2*>(dst + eg * 4) = make_ulonglong2(acc[h * 4 + m][0], acc[h * 4 + m][1]);
                *reinterpret_cast<ulonglong2*>(dst + 32 + eg * 4) = make_ulonglong2(acc[h * 4 + m][2], acc[h * 4 + m][3]);
            }
        __syncthreads();
        for (int o = tid; o < TT * 64; o += 256) {
            const int tt = o >> 6, el = o & 63, e2 = e0 + el, t = t0 + tt;
            if (t < a.T && e2 < E) {
                float q[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) q[jj] = parts[((size_t)jj * TT + tt) * 68 + el];
                float sacc = __fadd_rn(__fadd_rn(__fadd_rn(q[0], q[4]), __fadd_rn(q[1], q[5])),
                                       __fadd_rn(__fadd_rn(q[2], q[6]), __fadd_rn(q[3], q[7])));
                for (int i = H8; i < H; ++i)
                    sacc = __fmaf_rn(to_f32(x[(size_t)t * H + i]), a.w[(size_t)i * E + e2], sacc);
                if (a.bias) sacc = __fadd_rn(sacc, a.bias[e2]);
                a.logits[(size_t)t * E + e2] = sacc;             // the selection reads them back (L1 bypass)
            }
        }
    }
    __threadfence_block();
    __syncthreads();
    const int per_warp = E + 2 * a.k;
    for (int tt = j; tt < TT; tt += 8) {
        const int t = t0 + tt;
        float* sm_v = tk + (size_t)j * per_warp;
        if (t < a.T) {
            if (E <= 64) warp_softmax_topk<2>(a, t, sm_v, sm_v + E, reinterpret_cast<int32_t*>(sm_v + E + a.k));
            else if (E <= 128) warp_softmax_topk<4>(a, t, sm_v, sm_v + E, reinterpret_cast<int32_t*>(sm_v + E + a.k));
            else warp_softmax_topk<R_MAXV>(a, t, sm_v, sm_v + E, reinterpret_cast<int32_t*>(sm_v + E + a.k));
        }
    }
}

static size_t router_wide_smem(int H, int E, int e_pad, int k, int nwarps, int RW_TT) {
    const size_t row = (size_t)((H & ~7) >> 3) + 4;
    return (RW_TT * 8 * row + (size_t)RW_TT * e_pad * 8 + (size_t)RW_TT * E + (size_t)nwarps * (E + 2 * k)) * 4;
}


static size_t router_smem(int H, int E, int k, int TT) {
    size_t H8 = (size_t)(H & ~7);
    return (H8 * R_ES + (size_t)TT * H + (size_t)TT * 64 + (size_t)8 * (E + 2 * k)) * 4;
}

template <typename TX>
static int launch_router_t(MummuMoe* m, RouterArgs& a, cudaStream_t s) {
    const int e_pad = (a.E + 31) & ~31;
    if (a.T >= 256 && a.E > 32 && a.E % 4 == 0 && (a.H & ~7) % RT_KC == 0 && a.H >= RT_KC && !m->sw.router_plain &&
        (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (a.H * sizeof(TX)) % 16 == 0) {
        // 32-token tiles while they still give every SM two blocks; 16-token tiles below that
        const bool big = (a.T + 31) / 32 >= 2 * 148;
        const size_t smem = router_tile_smem(a.E, a.k, big ? 8 : 4, sizeof(TX));
        LaunchScope scope(m, s, "router");
        if (big) {
            MUMMU_CUDA_TRY(allow_big_smem(router_tile_kernel<TX, 8>, m->cfg.device));
            router_tile_kernel<TX, 8><<<(a.T + 31) / 32, 256, smem, s>>>(a);
        } else {
            MUMMU_CUDA_TRY(allow_big_smem(router_tile_kernel<TX, 4>, m->cfg.device));
            router_tile_kernel<TX, 4><<<(a.T + 15) / 16, 256, smem, s>>>(a);
        }
        MUMMU_CUDA_TRY(cudaGetLastError());
        return MUMMU_OK;
    }
    if (a.T >= 256 && e_pad <= 128) {
        // up to 64 experts: 512 threads with 128 registers each take 16 tokens per block; wider
        // routers run 1024 threads (64 registers) and take 8
        const int threads = e_pad * 8;
        const int tt = e_pad <= 64 ? 16 : 8;
        const size_t smem = router_wide_smem(a.H, a.E, e_pad, a.k, threads / 32, tt);
        if (smem <= 200 * 1024) {
            LaunchScope scope(m, s, "router");
            const unsigned blocks = (a.T + tt - 1) / tt;
            switch (e_pad) {
                case 32:
                    MUMMU_CUDA_TRY(allow_big_smem(router_wide_kernel<TX, 32, 16, 1>, m->cfg.device));
                    router_wide_kernel<TX, 32, 16, 1><<<blocks, threads, smem, s>>>(a);
                    break;
                case 64:
                    MUMMU_CUDA_TRY(allow_big_smem(router_wide_kernel<TX, 64, 16, 1>, m->cfg.device));
                    router_wide_kernel<TX, 64, 16, 1><<<blocks, threads, smem, s>>>(a);
                    break;
                case 96:
                    MUMMU_CUDA_TRY(allow_big_smem(router_wide_kernel<TX, 96, 8, 1>, m->cfg.device));
                    router_wide_kernel<TX, 96, 8, 1><<<blocks, threads, smem, s>>>(a);
                    break;
                default:
                    MUMMU_CUDA_TRY(allow_big_smem(router_wide_kernel<TX, 128, 8, 1>, m->cfg.device));
                    router_wide_kernel<TX, 128, 8, 1><<<blocks, threads, smem, s>>>(a);
                    break;
            }
            MUMMU_CUDA_TRY(cudaGetLastError());
            return MUMMU_OK;
        }
    }
    int tpt = a.T >= 2048 ? 4 : (a.T >= 256 ? 2 : 1);
    while (tpt > 1 && router_smem(a.H, a.E, a.k, 4 * tpt) > 200 * 1024) tpt >>= 1;
    if (tpt == 1 && sizeof(TX) == 2 && a.H % 32 == 0 && a.E % R_ES == 0 &&
        a.wt != nullptr && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && !m->sw.router_plain) {
        const int S = a.H / 8 + 4;
        const size_t smem_t = ((size_t)64 * S + (size_t)4 * 8 * S + 4 * 64 + (size_t)8 * (a.E + 2 * a.k)) * 4;
        if (smem_t <= 200 * 1024) {
            dim3 grid_t(a.E / R_ES, (a.T + 3) / 4);
            LaunchScope scope(m, s, "router");
            MUMMU_CUDA_TRY(allow_big_smem(router_kernel<TX, 1, true>, m->cfg.device));
            router_kernel<TX, 1, true><<<grid_t, R_THREADS, smem_t, s>>>(a);
            MUMMU_CUDA_TRY(cudaGetLastError());
            return MUMMU_OK;
        }
    }
    size_t smem = router_smem(a.H, a.E, a.k, 4 * tpt);
    if (smem > 220 * 1024) {
        set_error("router: hidden %d too wide for the shared-memory staged router", a.H);
        return MUMMU_ERR_UNSUPPORTED;
    }
    dim3 grid((a.E + R_ES - 1) / R_ES, (a.T + 4 * tpt - 1) / (4 * tpt));
    LaunchScope scope(m, s, "router");
    switch (tpt) {
        case 4:
            MUMMU_CUDA_TRY(allow_big_smem(router_kernel<TX, 4, false>, m->cfg.device));
            router_kernel<TX, 4, false><<<grid, R_THREADS, smem, s>>>(a);
            break;
        case 2:
            MUMMU_CUDA_TRY(allow_big_smem(router_kernel<TX, 2, false>, m->cfg.device));
            router_kernel<TX, 2, false><<<grid, R_THREADS, smem, s>>>(a);
            break;
        default:
            MUMMU_CUDA_TRY(allow_big_smem(router_kernel<TX, 1, false>, m->cfg.device));
            router_kernel<TX, 1, false><<<grid, R_THREADS, smem, s>>>(a);
            break;
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int launch_router(MummuMoe* m, const void* x, int64_t tokens, int top_k, int norm, int32_t* ids,
                  float* wts, int32_t* counts, cudaStream_t s, bool fuse_permute, const GroupedOut* grouped) {
    const MummuMoeConfig& c = m->cfg;
    if (c.experts > 32 * R_MAXV) {
        set_error("router: %d experts exceed the %d this build selects over", c.experts, 32 * R_MAXV);
        return MUMMU_ERR_UNSUPPORTED;
    }
    // fused grouping: one block sorts up to 1024 pairs in the narrow kernel's shared memory
    const int64_t pairs = tokens * top_k, pair_chunks = (pairs + 31) / 32;
    const bool fuse = fuse_permute && (counts == m->counts || grouped) && tokens < 256 && pairs <= 1024 &&
                      (size_t)(pair_chunks * 32 + 2 * c.experts + 2 + pair_chunks * c.experts) * 4 <=
                          router_smem(c.hidden, c.experts, top_k, 4);
    if (fuse_permute && !fuse) return MUMMU_ERR_UNSUPPORTED;       // caller falls back to the separate launch
    if (counts && !fuse) MUMMU_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int32_t) * c.experts, s));
    RouterArgs a;
    a.fuse = fuse ? 1 : 0;
    a.p_counts = grouped ? grouped->counts : m->counts;
    a.p_offsets = grouped ? grouped->offsets : m->offsets;
    a.p_row_token = grouped ? grouped->row_token : m->row_token;
    a.p_pos = grouped ? grouped->pos : m->pos;
    a.p_active = m->active;
    a.p_n_active = m->n_active;
    a.x = x;
    a.w = m->router_w;
    a.wt = m->router_wt;
    a.bias = m->router_bias;
    a.logits = m->logits;
    a.tile_done = m->tile_done;
    a.ids = ids;
    a.wts = wts;
    a.counts = fuse ? nullptr : counts;
    a.hits = m->hits;
    a.status = m->status;
    a.T = (int)tokens;
    a.H = c.hidden;
    a.E = c.experts;
    a.k = top_k;
    a.norm = norm;
    switch (c.act_dtype) {
        case MUMMU_F32: return launch_router_t<float>(m, a, s);
        case MUMMU_F16: return launch_router_t<__half>(m, a, s);
        case MUMMU_BF16: return launch_router_t<__nv_bfloat16>(m, a, s);
    }
    set_error("router: bad activation dtype %d", c.act_dtype);
    return MUMMU_ERR_CONTRACT;
}

// ---------------------------------------------------------------------------------------------
// checked mode (switch CHECKED): the routing plan drives every hand-computed address of the
// layer.  These kernels verify it and make it safe in place: a bad index is replaced by one that
// stays inside its buffer, and the status word is raised (MUMMU_ERR_CONTRACT at the next sync).
// The reference arms its backend's bounds validation for tests the same way (burn.toml:17).
// ---------------------------------------------------------------------------------------------
// whole plan: pair i = (token, slot): ids[i] an expert, pos[i] inside that expert's segment,
// row_token[pos[i]] the pair's token; per expert: segments tile [0, pairs)
__global__ void check_plan_kernel(int32_t* ids, int32_t* pos, int32_t* row_token, const int32_t* counts,
                                  const int32_t* offsets, int64_t pairs, int top_k, int E, int32_t* status) {
    bool bad = false;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
        int e = ids[i];
        if (e < 0 || e >= E) {
            bad = true;
            ids[i] = e = 0;
        }
        int p = pos[i];
        if (p < 0 || p >= pairs) {
            bad = true;
            pos[i] = p = 0;
        }
        if (p < offsets[e] || p >= offsets[e] + counts[e]) bad = true;
        const int t = row_token[i];                      // entry i of the sorted order
        if (t < 0 || (int64_t)t * top_k >= pairs) {
            bad = true;
            row_token[i] = 0;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int64_t run = 0;
        for (int e = 0; e < E; ++e) {
            if (offsets[e] != run || counts[e] < 0) bad = true;
            run += counts[e];
        }
        if (run != pairs) bad = true;
    }
    if (bad) atomicOr(status, STATUS_BOUNDS);
}

// caller-given (ids, pos) of a combine: copied, with every index made safe
__global__ void check_combine_kernel(const int32_t* ids, const int32_t* pos, int32_t* ids_out, int32_t* pos_out,
                                     int64_t pairs, int E, int32_t* status) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
        int e = ids[i], p = pos[i];
        if (e < 0 || e >= E || p < 0 || p >= pairs) {
            atomicOr(status, STATUS_BOUNDS);
            e = min(max(e, 0), E - 1);
            p = 0;
        }
        ids_out[i] = e;
        pos_out[i] = p;
    }
}

// caller-given per-expert row counts: copied, clipped so that the segments stay inside `rows`
__global__ void check_counts_kernel(const int32_t* counts, int32_t* counts_out, int n, int64_t rows, int32_t* status) {
    if (blockIdx.x || threadIdx.x) return;
    int64_t run = 0;
    bool bad = false;
    for (int e = 0; e < n; ++e) {
        int64_t c = counts[e];
        if (c < 0 || run + c > rows) {
            bad = true;
            c = c < 0 ? 0 : rows - run;
        }
        counts_out[e] = (int32_t)c;
        run += c;
    }
    if (bad) atomicOr(status, STATUS_BOUNDS);
}

int launch_check_plan(MummuMoe* m, int32_t* ids, int32_t* pos, int32_t* row_token, const int32_t* counts,
                      const int32_t* offsets, int64_t tokens, int top_k, cudaStream_t s) {
    const int64_t pairs = tokens * top_k;
    if (pairs == 0) return MUMMU_OK;
    LaunchScope scope(m, s, "check_plan");
    check_plan_kernel<<<(unsigned)std::min<int64_t>((pairs + 255) / 256, 1024), 256, 0, s>>>(
        ids, pos, row_token, counts, offsets, pairs, top_k, m->cfg.experts, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int launch_check_combine(MummuMoe* m, const int32_t* ids, const int32_t* pos, int32_t* ids_out, int32_t* pos_out,
                         int64_t pairs, cudaStream_t s) {
    if (pairs == 0) return MUMMU_OK;
    LaunchScope scope(m, s, "check_combine");
    check_combine_kernel<<<(unsigned)std::min<int64_t>((pairs + 255) / 256, 1024), 256, 0, s>>>(ids, pos, ids_out, pos_out,
                                                                                             pairs, m->cfg.experts, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int launch_check_counts(MummuMoe* m, const int32_t* counts, int32_t* counts_out, int n, int64_t rows, cudaStream_t s) {
    LaunchScope scope(m, s, "check_counts");
    check_counts_kernel<<<1, 32, 0, s>>>(counts, counts_out, n, rows, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// ---------------------------------------------------------------------------------------------
// histogram / offsets / permute
// ---------------------------------------------------------------------------------------------
__global__ void count_kernel(const int32_t* ids, int64_t n, int E, int32_t* counts, int32_t* status) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(counts + e, 1);
    }
}

int launch_count(MummuMoe* m, const int32_t* ids, int64_t n, int32_t* counts, cudaStream_t s) {
    MUMMU_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int32_t) * m->cfg.experts, s));
    if (n == 0) return MUMMU_OK;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 1184) blocks = 1184;
    LaunchScope scope(m, s, "count");
    count_kernel<<<blocks, 256, 0, s>>>(ids, n, m->cfg.experts, counts, m->status);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

__global__ void offsets_kernel(const int32_t* counts, int n, int32_t* offsets, int32_t* active,
                               int32_t* n_active) {
    // one warp: 32 counts at a time, prefix by shuffles
    const int lane = threadIdx.x;
    int acc = 0, nz = 0;
    for (int e0 = 0; e0 < n; e0 += 32) {
        const int e = e0 + lane;
        const int c = e < n ? counts[e] : 0;
        int incl = c, zincl = c > 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, incl, off);
            const int zup = __shfl_up_sync(0xFFFFFFFFu, zincl, off);
            if (lane >= off) { incl += up; zincl += zup; }
        }
        if (e < n) {
            offsets[e] = acc + incl - c;
            if (c > 0 && active) active[nz + zincl - 1] = e;
        }
        acc += __shfl_sync(0xFFFFFFFFu, incl, 31);
        nz += __shfl_sync(0xFFFFFFFFu, zincl, 31);
    }
    if (lane == 0) {
        offsets[n] = acc;
        if (n_active) *n_active = nz;
    }
}

int launch_offsets_from_counts(MummuMoe* m, const int32_t* counts, int n, int32_t* offsets,
                               cudaStream_t s) {
    LaunchScope scope(m, s, "offsets");
    offsets_kernel<<<1, 32, 0, s>>>(counts, n, offsets, m->active, m->n_active);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// One block per expert: stable compaction of the (token, slot) pairs routed to it, so rows of one
// expert come out in ascending token order (the order nn/moe.rs:276-285 builds its lists in).
constexpr int P_THREADS = 1024;
__global__ void __launch_bounds__(P_THREADS) permute_kernel(const int32_t* ids, int64_t n, int top_k,
                                                            int E, const int32_t* counts,
                                                            int32_t* offsets, int32_t* row_token,
                                                            int32_t* pos, int32_t* active,
                                                            int32_t* n_active) {
    __shared__ int warp_sums[P_THREADS / 32];
    __shared__ int warp_nz[P_THREADS / 32];
    __shared__ int base_s;
    const int e = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // exclusive prefix of counts up to e
    // part: rows of experts before e (exclusive prefix).  nz: experts that come before e in the
    // work order "most rows first, then lower id" - longest jobs are scheduled first so that the
    // CTAs of the expert kernels finish together.
    const int mine_c = counts[e];
    int part = 0, nz = 0;
    for (int i = tid; i < E; i += P_THREADS) {
        int c = counts[i];
        if (i < e) part += c;
        nz += (c > mine_c || (c == mine_c && i < e)) && c > 0;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        part += __shfl_xor_sync(0xFFFFFFFFu, part, off);
        nz += __shfl_xor_sync(0xFFFFFFFFu, nz, off);
    }
    if (lane == 0) {
        warp_sums[warp] = part;
        warp_nz[warp] = nz;
    }
    __syncthreads();
    if (tid == 0) {
        int b = 0, z = 0;
        for (int w = 0; w < P_THREADS / 32; ++w) {
            b += warp_sums[w];
            z += warp_nz[w];
        }
        base_s = b;
        const int mine = counts[e];
        if (offsets) {
            offsets[e] = b;
            if (e == E - 1) offsets[E] = b + mine;
        }
        if (active && mine > 0) active[z] = e;
        if (n_active && mine > 0) atomicMax(n_active, z + 1);   // the last in the order sets the count
    }
    __syncthreads();
    int running = base_s;
    if (counts[e] == 0) return;
    // four consecutive entries per thread per step (in order, so the compaction stays stable)
    for (int64_t start = 0; start < n; start += 4 * P_THREADS) {
        const int64_t i0 = start + 4 * (int64_t)tid;
        int v[4];
        if (i0 + 3 < n && (reinterpret_cast<uintptr_t>(ids) & 15) == 0) {
            const int4 q = *reinterpret_cast<const int4*>(ids + i0);
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = i0 + u < n ? ids[i0 + u] : -1;
        }
        const int mine = (v[0] == e) + (v[1] == e) + (v[2] == e) + (v[3] == e);
        int incl = mine;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, incl, off);
            if (lane >= off) incl += up;
        }
        __syncthreads();  // warp_sums reuse
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int wbase = 0, total = 0;
        for (int w = 0; w < P_THREADS / 32; ++w) {
            const int c = warp_sums[w];
            if (w < warp) wbase += c;
            total += c;
        }
        int p = running + wbase + incl - mine;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (v[u] == e) {
                if (row_token) row_token[p] = (int32_t)((i0 + u) / top_k);
                if (pos) pos[i0 + u] = p;
                ++p;
            }
        }
        running += total;
    }
}

// Large calls: a counting sort in three launches instead of one block per expert scanning every
// pair.  A warp owns 256 consecutive pairs (8 steps of 32, in index order, so the order inside an
// expert stays ascending by token):
//   count   : per-warp histogram by expert (warp match)            -> whist[warp][expert]
//   scan    : per expert, exclusive prefix over the warps + the expert's first row
//             (also offsets and the heaviest-first list of active experts) -> whist in place
//   scatter : the same walk again; pos = whist[warp][expert] + earlier pairs of the expert in the warp
constexpr int PS_PAIRS_PER_WARP = 256, PS_WARPS = 8, PS_PAIRS_PER_BLOCK = PS_PAIRS_PER_WARP * PS_WARPS;

__global__ void __launch_bounds__(PS_WARPS * 32) permute_count_kernel(const int32_t* __restrict__ ids, int64_t n, int E,
                                                                      int32_t* __restrict__ whist) {
    extern __shared__ int32_t s_tbl[];                           // [PS_WARPS][E]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t* tbl = s_tbl + warp * E;
    for (int e = lane; e < E; e += 32) tbl[e] = 0;
    __syncwarp();
    const int64_t first = ((int64_t)blockIdx.x * PS_WARPS + warp) * PS_PAIRS_PER_WARP;
    for (int st = 0; st < PS_PAIRS_PER_WARP / 32; ++st) {
        const int64_t i = first + st * 32 + lane;
        const int e = i < n ? ids[i] : -1;
        const int key = (e >= 0 && e < E) ? e : -1 - lane;       // pairs without a valid expert match nobody
        const unsigned mask = __match_any_sync(0xFFFFFFFFu, key);
        if (key >= 0 && lane == __ffs(mask) - 1) tbl[key] += __popc(mask);
        __syncwarp();
    }
    int32_t* out = whist + ((int64_t)blockIdx.x * PS_WARPS + warp) * E;
    for (int e = lane; e < E; e += 32) out[e] = tbl[e];
}

// one warp per expert
__global__ void __launch_bounds__(32) permute_scan_kernel(const int32_t* __restrict__ counts, int E, int64_t n_warps,
                                                          int32_t* __restrict__ whist, int32_t* offsets, int32_t* active,
                                                          int32_t* n_active) {
    const int e = blockIdx.x, lane = threadIdx.x;
    const int mine = counts[e];
    int before = 0, nz = 0;
    for (int i = lane; i < E; i += 32) {
        const int c = counts[i];
        if (i < e) before += c;
        nz += (c > mine || (c == mine && i < e)) && c > 0;       // work order: most rows first, then lower id
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        before += __shfl_xor_sync(0xFFFFFFFFu, before, off);
        nz += __shfl_xor_sync(0xFFFFFFFFu, nz, off);
    }
    if (lane == 0) {
        if (offsets) {
            offsets[e] = before;
            if (e == E - 1) offsets[E] = before + mine;
        }
        if (active && mine > 0) active[nz] = e;
        if (n_active && mine > 0) atomicMax(n_active, nz + 1);
    }
    int run = before;
    for (int64_t k0 = 0; k0 < n_warps; k0 += 32) {
        const int64_t k = k0 + lane;
        const int c = k < n_warps ? whist[k * E + e] : 0;
        int incl = c;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, incl, off);
            if (lane >= off) incl += up;
        }
        if (k < n_warps) whist[k * E + e] = run + incl - c;
        run += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
}

__global__ void __launch_bounds__(PS_WARPS * 32) permute_scatter_kernel(const int32_t* __restrict__ ids, int64_t n, int top_k,
                                                                        int E, const int32_t* __restrict__ whist,
                                                                        int32_t* __restrict__ row_token,
                                                                        int32_t* __restrict__ pos) {
    extern __shared__ int32_t s_tbl[];                           // [PS_WARPS][E]: next row of the expert for this warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t* nxt = s_tbl + warp * E;
    const int32_t* base = whist + ((int64_t)blockIdx.x * PS_WARPS + warp) * E;
    for (int e = lane; e < E; e += 32) nxt[e] = base[e];
    __syncwarp();
    const int64_t first = ((int64_t)blockIdx.x * PS_WARPS + warp) * PS_PAIRS_PER_WARP;
    for (int st = 0; st < PS_PAIRS_PER_WARP / 32; ++st) {
        const int64_t i = first + st * 32 + lane;
        const int e = i < n ? ids[i] : -1;
        const int key = (e >= 0 && e < E) ? e : -1 - lane;
        const unsigned mask = __match_any_sync(0xFFFFFFFFu, key);
        if (key >= 0) {
            const int p = nxt[key] + __popc(mask & ((1u << lane) - 1u));
            if (pos) pos[i] = p;
            if (row_token) row_token[p] = (int32_t)(i / top_k);
        }
        __syncwarp();
        if (key >= 0 && lane == __ffs(mask) - 1) nxt[key] += __popc(mask);
        __syncwarp();
    }
}

int launch_permute(MummuMoe* m, const int32_t* ids, int64_t tokens, int top_k,
                   const int32_t* counts, int32_t* offsets, int32_t* row_token, int32_t* pos,
                   cudaStream_t s) {
    MUMMU_CUDA_TRY(cudaMemsetAsync(m->n_active, 0, sizeof(int32_t), s));
    const int64_t n = tokens * top_k;
    const int E = m->cfg.experts;
    const int64_t blocks = (n + PS_PAIRS_PER_BLOCK - 1) / PS_PAIRS_PER_BLOCK;
    const size_t tbl_bytes = (size_t)PS_WARPS * E * sizeof(int32_t);
    // three launches cost about 15 us of launch latency: they pay from about 64 K pairs on
    if (n >= 65536 && m->whist && blocks * PS_WARPS * E <= m->whist_elems && tbl_bytes <= 48 * 1024) {
        LaunchScope scope(m, s, "permute");
        permute_count_kernel<<<(unsigned)blocks, PS_WARPS * 32, tbl_bytes, s>>>(ids, n, E, m->whist);
        permute_scan_kernel<<<E, 32, 0, s>>>(counts, E, blocks * PS_WARPS, m->whist, offsets, m->active, m->n_active);
        permute_scatter_kernel<<<(unsigned)blocks, PS_WARPS * 32, tbl_bytes, s>>>(ids, n, top_k, E, m->whist, row_token, pos);
        MUMMU_CUDA_TRY(cudaGetLastError());
        return MUMMU_OK;
    }
    LaunchScope scope(m, s, "permute");
    permute_kernel<<<m->cfg.experts, P_THREADS, 0, s>>>(ids, tokens * top_k, top_k, m->cfg.experts,
                                                        counts, offsets, row_token, pos, m->active,
                                                        m->n_active);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// ---------------------------------------------------------------------------------------------
// combine: per token, ascending expert id, scaled = w * y; out += scaled (two roundings)
// ---------------------------------------------------------------------------------------------
template <typename TY, typename TO>
__global__ void __launch_bounds__(256) combine_kernel(const TY* ys, const int32_t* ids, const float* w,
                                                      const int32_t* pos, int top_k, int H, TO* out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int32_t* s_pos = reinterpret_cast<int32_t*>(smem_raw);
    float* s_w = reinterpret_cast<float*>(s_pos + top_k);
    const int64_t t = blockIdx.x;
    for (int r = threadIdx.x; r < top_k; r += blockDim.x) {
        int id = ids[t * top_k + r];
        int rank = 0;
        for (int q = 0; q < top_k; ++q) {
            int other = ids[t * top_k + q];
            rank += (other < id || (other == id && q < r)) ? 1 : 0;
        }
        s_pos[rank] = pos[t * top_k + r];
        s_w[rank] = w[t * top_k + r];
    }
    __syncthreads();
    for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < H; h += gridDim.y * blockDim.x) {
        float acc = 0.0f;
        for (int r0 = 0; r0 < top_k; r0 += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)      // independent loads first, then the ordered sum
                v[u] = r0 + u < top_k ? to_f32(ys[(size_t)s_pos[r0 + u] * H + h]) : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (r0 + u < top_k) acc = __fadd_rn(acc, __fmul_rn(s_w[r0 + u], v[u]));
        }
        out[t * H + h] = from_f32<TO>(acc);
    }
}

// 8 outputs per thread: the k source rows are read with 16-byte loads before the ordered sum
template <typename T> struct Vec8 { uint4 raw[sizeof(T) * 8 / 16]; };
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
    Vec8<T> r = *reinterpret_cast<const Vec8<T>*>(p);
    const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32(e[i]);
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
    Vec8<T> r;
    T* e = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(v[i]);
    *reinterpret_cast<Vec8<T>*>(p) = r;
}

// BATCH expert rows in flight per thread: 8 for decode-sized calls (latency), 4 for large T (occupancy)
template <typename TY, typename TO, int BATCH>
__global__ void __launch_bounds__(256) combine_vec8_kernel(const TY* ys, const int32_t* ids, const float* w,
                                                           const int32_t* pos, int top_k, int H, TO* out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int32_t* s_pos = reinterpret_cast<int32_t*>(smem_raw);
    float* s_w = reinterpret_cast<float*>(s_pos + top_k);
    const int64_t t = blockIdx.x;
    for (int r = threadIdx.x; r < top_k; r += blockDim.x) {
        int id = ids[t * top_k + r];
        int rank = 0;
        for (int q = 0; q < top_k; ++q) {
            int other = ids[t * top_k + q];
            rank += (other < id || (other == id && q < r)) ? 1 : 0;
        }
        s_pos[rank] = pos[t * top_k + r];
        s_w[rank] = w[t * top_k + r];
    }
    __syncthreads();
    for (int h = (blockIdx.y * blockDim.x + threadIdx.x) * 8; h < H; h += gridDim.y * blockDim.x * 8) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r0 = 0; r0 < top_k; r0 += BATCH) {
            // the rows stay as loaded (16-bit rows: 4 registers each) until they are summed: the
            // kernel lives on loads in flight, and registers decide how many blocks an SM holds
            Vec8<TY> raw[BATCH];
#pragma unroll
            for (int u = 0; u < BATCH; ++u)
                if (r0 + u < top_k) raw[u] = *reinterpret_cast<const Vec8<TY>*>(ys + (size_t)s_pos[r0 + u] * H + h);
#pragma unroll
            for (int u = 0; u < BATCH; ++u)
                if (r0 + u < top_k) {
                    const float wv = s_w[r0 + u];
                    const TY* e = reinterpret_cast<const TY*>(&raw[u]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(wv, to_f32(e[i])));
                }
        }
        store8(out + t * H + h, acc);
    }
}

template <typename TY>
static int launch_combine_y(MummuMoe* m, const void* ys, const int32_t* ids, const float* w,
                            const int32_t* pos, int64_t tokens, int top_k, void* out,
                            cudaStream_t s) {
    size_t smem = (size_t)top_k * 8;
    const int H = m->cfg.hidden;
    const bool vec = (H & 7) == 0 && (reinterpret_cast<uintptr_t>(ys) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    // few tokens: 64-thread blocks so that a decode batch still spreads over the SMs
    const unsigned vthreads = tokens < 128 ? 64u : 256u;
    const dim3 grid((unsigned)tokens, vec ? (tokens < 512 ? (unsigned)((H / 8 + vthreads - 1) / vthreads) : 1u)
                                          : (tokens < 512 ? (unsigned)((H + 255) / 256) : 1u));
    LaunchScope scope(m, s, "combine");
    if (vec) {
        switch (m->cfg.act_dtype) {
            case MUMMU_F32:
                if (tokens < 128) combine_vec8_kernel<TY, float, 8><<<grid, vthreads, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (float*)out);
                else combine_vec8_kernel<TY, float, 4><<<grid, vthreads, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (float*)out);
                break;
            case MUMMU_F16:
                if (tokens < 128) combine_vec8_kernel<TY, __half, 8><<<grid, vthreads, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (__half*)out);
                else combine_vec8_kernel<TY, __half, 4><<<grid, vthreads, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (__half*)out);
                break;
            case MUMMU_BF16:
                if (tokens < 128) combine_vec8_kernel<TY, __nv_bfloat16, 8><<<grid, vthreads, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (__nv_bfloat16*)out);
                else combine_vec8_kernel<TY, __nv_bfloat16, 4><<<grid, vthreads, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (__nv_bfloat16*)out);
                break;
        }
        MUMMU_CUDA_TRY(cudaGetLastError());
        return MUMMU_OK;
    }
    switch (m->cfg.act_dtype) {
        case MUMMU_F32:
            combine_kernel<TY, float><<<grid, 256, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (float*)out);
            break;
        case MUMMU_F16:
            combine_kernel<TY, __half><<<grid, 256, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (__half*)out);
            break;
        case MUMMU_BF16:
            combine_kernel<TY, __nv_bfloat16><<<grid, 256, smem, s>>>((const TY*)ys, ids, w, pos, top_k, H, (__nv_bfloat16*)out);
            break;
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int launch_combine(MummuMoe* m, const void* ys, int ys_dtype, const int32_t* ids, const float* w,
                   const int32_t* pos, int64_t tokens, int top_k, void* out, cudaStream_t s) {
    if (tokens == 0) return MUMMU_OK;
    switch (ys_dtype) {
        case MUMMU_F32: return launch_combine_y<float>(m, ys, ids, w, pos, tokens, top_k, out, s);
        case MUMMU_F16: return launch_combine_y<__half>(m, ys, ids, w, pos, tokens, top_k, out, s);
        case MUMMU_BF16: return launch_combine_y<__nv_bfloat16>(m, ys, ids, w, pos, tokens, top_k, out, s);
    }
    set_error("combine: bad dtype %d", ys_dtype);
    return MUMMU_ERR_CONTRACT;
}

// ---------------------------------------------------------------------------------------------
// SIMT grouped SwiGLU: every weight format, f32 accumulation.  The correctness path and the
// fallback for shapes the tensor-core kernels do not take.
// ---------------------------------------------------------------------------------------------
template <typename TW> __device__ __forceinline__ float load_w(const uint8_t* row, int k) {
    return to_f32(reinterpret_cast<const TW*>(row)[k]);
}
template <> __device__ __forceinline__ float load_w<q4k_t>(const uint8_t* row, int k) {
    return q4k_decode_elem(row, k);
}
template <> __device__ __forceinline__ float load_w<q80_t>(const uint8_t* row, int k) { return q80_decode_elem(row, k); }
template <> __device__ __forceinline__ float load_w<q5k_t>(const uint8_t* row, int k) { return q5k_decode_elem(row, k); }
template <> __device__ __forceinline__ float load_w<q6k_t>(const uint8_t* row, int k) { return q6k_decode_elem(row, k); }

// rows of a block-quantised matrix -> f32 [rows, cols] (mummu_moe_dequant_bank for the sibling formats)
template <typename TW>
__global__ void block_dequant_kernel(const uint8_t* src, float* dst, int64_t rows, int64_t cols, size_t row_bytes) {
    const int64_t n = rows * cols;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols;
        dst[i] = load_w<TW>(src + (size_t)r * row_bytes, (int)(i - r * cols));
    }
}

// rows of a block-quantised bank -> f16 [rows, cols], eight values per thread, only for experts
// that have rows this call (the image feeds the tensor-core GEMMs; the element decoders keep the
// reference's operation order in f32, the f16 rounding comes last)
template <typename TW>
__global__ void block_expand_f16_kernel(const uint8_t* src, __half* dst, int64_t rows, int64_t cols, size_t row_bytes,
                                        int64_t rows_per_expert, const int32_t* counts) {
    const int64_t n8 = rows * cols / 8;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = (i * 8) / cols;
        if (counts[r / rows_per_expert] == 0) continue;
        const int k0 = (int)(i * 8 - r * cols);
        const uint8_t* row = src + (size_t)r * row_bytes;
        __half out[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) out[u] = __float2half_rn(load_w<TW>(row, k0 + u));
        *reinterpret_cast<uint4*>(dst + i * 8) = *reinterpret_cast<const uint4*>(out);
    }
}

int launch_block_expand_f16(MummuMoe* m, int which, __half* dst, const int32_t* counts, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    const int64_t out_dim = which == MUMMU_BANK_DOWN ? c.hidden : c.inter, cols = which == MUMMU_BANK_DOWN ? c.inter : c.hidden;
    const int64_t rows = out_dim * c.experts_local;
    const size_t row_bytes = bank_row_bytes(c, which);
    const unsigned blocks = (unsigned)std::min<int64_t>((rows * cols / 8 + 255) / 256, 148 * 16);
    const uint8_t* p = (const uint8_t*)m->bank[which];
    switch (c.weight_dtype) {
        case MUMMU_Q8_0: block_expand_f16_kernel<q80_t><<<blocks, 256, 0, s>>>(p, dst, rows, cols, row_bytes, out_dim, counts); break;
        case MUMMU_Q5_K: block_expand_f16_kernel<q5k_t><<<blocks, 256, 0, s>>>(p, dst, rows, cols, row_bytes, out_dim, counts); break;
        case MUMMU_Q6_K: block_expand_f16_kernel<q6k_t><<<blocks, 256, 0, s>>>(p, dst, rows, cols, row_bytes, out_dim, counts); break;
        default:
            set_error("block expand: dtype %d has no generic expander", c.weight_dtype);
            return MUMMU_ERR_CONTRACT;
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int launch_block_dequant(const void* src, int dtype, float* dst, int64_t rows, int64_t cols, size_t row_bytes,
                         cudaStream_t s) {
    const int64_t n = rows * cols;
    const unsigned blocks = (unsigned)std::min<int64_t>((n + 255) / 256, 148 * 16);
    const uint8_t* p = (const uint8_t*)src;
    switch (dtype) {
        case MUMMU_Q4_K: block_dequant_kernel<q4k_t><<<blocks, 256, 0, s>>>(p, dst, rows, cols, row_bytes); break;
        case MUMMU_Q8_0: block_dequant_kernel<q80_t><<<blocks, 256, 0, s>>>(p, dst, rows, cols, row_bytes); break;
        case MUMMU_Q5_K: block_dequant_kernel<q5k_t><<<blocks, 256, 0, s>>>(p, dst, rows, cols, row_bytes); break;
        case MUMMU_Q6_K: block_dequant_kernel<q6k_t><<<blocks, 256, 0, s>>>(p, dst, rows, cols, row_bytes); break;
        default:
            set_error("block dequant: dtype %d is not a block format", dtype);
            return MUMMU_ERR_CONTRACT;
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

struct SimtArgs {
    const void* A;          // activations
    int64_t lda;
    const int32_t* row_index;   // sorted row -> source row, or null (identity)
    const int32_t* counts;      // per local expert, or null (single expert, rows_single rows)
    const int32_t* offsets;     // per local expert exclusive prefix, or null
    int rows_single;
    int expert_single;          // >= 0: only this expert
    const uint8_t* W0;          // gate (or down)
    const uint8_t* W1;          // up (GATEUP only)
    size_t expert_stride;       // bytes between experts
    size_t row_bytes;           // bytes per weight row
    void* out;
    int64_t ldo;
    int N, K;
};

constexpr int S_BM = 64, S_BN = 64, S_BK = 16;

template <typename TA, typename TW, bool GATEUP, typename TO>
__global__ void __launch_bounds__(256) simt_grouped_kernel(SimtArgs a) {
    __shared__ float As[S_BK][S_BM + 4];
    __shared__ float B0[S_BK][S_BN + 4];
    __shared__ float B1[GATEUP ? S_BK : 1][S_BN + 4];
    const int e = a.expert_single >= 0 ? a.expert_single : (int)blockIdx.z;
    const int cnt = a.counts ? a.counts[e] : a.rows_single;
    const int m0 = blockIdx.y * S_BM;
    if (m0 >= cnt) return;
    const int base = a.offsets ? a.offsets[e] : 0;
    const int n0 = blockIdx.x * S_BN;
    const int tid = threadIdx.x;
    const int lr = tid >> 2, lk = (tid & 3) * 4;   // loader: row, first k
    const int ty = tid >> 4, tx = tid & 15;
    const TA* A = reinterpret_cast<const TA*>(a.A);

    int64_t src_row = -1;
    if (m0 + lr < cnt) {
        int p = base + m0 + lr;
        src_row = a.row_index ? a.row_index[p] : p;
    }
    const uint8_t* w0row = nullptr;
    const uint8_t* w1row = nullptr;
    if (n0 + lr < a.N) {
        w0row = a.W0 + (size_t)e * a.expert_stride + (size_t)(n0 + lr) * a.row_bytes;
        if (GATEUP) w1row = a.W1 + (size_t)e * a.expert_stride + (size_t)(n0 + lr) * a.row_bytes;
    }
    float acc0[4][4], acc1[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc0[i][j] = acc1[i][j] = 0.0f;

    for (int k0 = 0; k0 < a.K; k0 += S_BK) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            int k = k0 + lk + u;
            As[lk + u][lr] = (src_row >= 0 && k < a.K) ? to_f32(A[src_row * a.lda + k]) : 0.0f;
            B0[lk + u][lr] = (w0row && k < a.K) ? load_w<TW>(w0row, k) : 0.0f;
            if (GATEUP) B1[lk + u][lr] = (w1row && k < a.K) ? load_w<TW>(w1row, k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < S_BK; ++kk) {
            float av[4], b0[4], b1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b0[j] = B0[kk][tx * 4 + j];
                if (GATEUP) b1[j] = B1[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc0[i][j] = fmaf(av[i], b0[j], acc0[i][j]);
                    if (GATEUP) acc1[i][j] = fmaf(av[i], b1[j], acc1[i][j]);
                }
        }
        __syncthreads();
    }
    TO* out = reinterpret_cast<TO*>(a.out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int r = m0 + ty * 4 + i;
        if (r >= cnt) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            float v = GATEUP ? silu_f(acc0[i][j]) * acc1[i][j] : acc0[i][j];
            out[(size_t)(base + r) * a.ldo + n] = from_f32<TO>(v);
        }
    }
}

template <typename TA, typename TW, bool GATEUP, typename TO>
static int simt_launch(MummuMoe* m, SimtArgs& a, int experts, int64_t max_rows, cudaStream_t s,
                       const char* name) {
    if (max_rows <= 0) return MUMMU_OK;
    dim3 grid((a.N + S_BN - 1) / S_BN, (unsigned)((max_rows + S_BM - 1) / S_BM), experts);
    LaunchScope scope(m, s, name);
    simt_grouped_kernel<TA, TW, GATEUP, TO><<<grid, 256, 0, s>>>(a);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

template <typename TA, typename TW>
static int simt_two_stage(MummuMoe* m, const void* x, const int32_t* row_index,
                          const int32_t* counts, const int32_t* offsets, int64_t max_rows,
                          void* ys, int ys_dtype, int expert_only, int rows_single, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    SimtArgs a{};
    a.A = x;
    a.lda = c.hidden;
    a.row_index = row_index;
    a.counts = counts;
    a.offsets = offsets;
    a.rows_single = rows_single;
    a.expert_single = expert_only;
    a.W0 = (const uint8_t*)m->bank[MUMMU_BANK_GATE];
    a.W1 = (const uint8_t*)m->bank[MUMMU_BANK_UP];
    a.row_bytes = bank_row_bytes(c, MUMMU_BANK_GATE);
    a.expert_stride = a.row_bytes * c.inter;
    a.out = m->hact;
    a.ldo = c.inter;
    a.N = c.inter;
    a.K = c.hidden;
    int experts = expert_only >= 0 ? 1 : c.experts_local;
    int rc = simt_launch<TA, TW, true, float>(m, a, experts, max_rows, s, "simt_gate_up");
    if (rc) return rc;
    SimtArgs d{};
    d.A = m->hact;
    d.lda = c.inter;
    d.row_index = nullptr;
    d.counts = counts;
    d.offsets = offsets;
    d.rows_single = rows_single;
    d.expert_single = expert_only;
    d.W0 = (const uint8_t*)m->bank[MUMMU_BANK_DOWN];
    d.W1 = nullptr;
    d.row_bytes = bank_row_bytes(c, MUMMU_BANK_DOWN);
    d.expert_stride = d.row_bytes * c.hidden;
    d.out = ys;
    d.ldo = c.hidden;
    d.N = c.hidden;
    d.K = c.inter;
    switch (ys_dtype) {
        case MUMMU_F32: return simt_launch<float, TW, false, float>(m, d, experts, max_rows, s, "simt_down");
        case MUMMU_F16: return simt_launch<float, TW, false, __half>(m, d, experts, max_rows, s, "simt_down");
        case MUMMU_BF16: return simt_launch<float, TW, false, __nv_bfloat16>(m, d, experts, max_rows, s, "simt_down");
    }
    set_error("experts: bad output dtype %d", ys_dtype);
    return MUMMU_ERR_CONTRACT;
}

template <typename TA>
static int simt_by_weight(MummuMoe* m, const void* x, const int32_t* row_index,
                          const int32_t* counts, const int32_t* offsets, int64_t max_rows, void* ys,
                          int ys_dtype, int expert_only, int rows_single, cudaStream_t s) {
    switch (m->cfg.weight_dtype) {
        case MUMMU_F32: return simt_two_stage<TA, float>(m, x, row_index, counts, offsets, max_rows, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_F16: return simt_two_stage<TA, __half>(m, x, row_index, counts, offsets, max_rows, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_BF16: return simt_two_stage<TA, __nv_bfloat16>(m, x, row_index, counts, offsets, max_rows, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_Q4_K: return simt_two_stage<TA, q4k_t>(m, x, row_index, counts, offsets, max_rows, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_Q8_0: return simt_two_stage<TA, q80_t>(m, x, row_index, counts, offsets, max_rows, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_Q5_K: return simt_two_stage<TA, q5k_t>(m, x, row_index, counts, offsets, max_rows, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_Q6_K: return simt_two_stage<TA, q6k_t>(m, x, row_index, counts, offsets, max_rows, ys, ys_dtype, expert_only, rows_single, s);
    }
    set_error("experts: bad weight dtype %d", m->cfg.weight_dtype);
    return MUMMU_ERR_CONTRACT;
}

int launch_experts_simt(MummuMoe* m, const void* x, int x_dtype, const int32_t* row_index,
                        const int32_t* counts, const int32_t* offsets, int64_t max_rows_per_expert,
                        int64_t total_rows, void* ys, int ys_dtype, int expert_only,
                        cudaStream_t s) {
    int rows_single = expert_only >= 0 ? (int)total_rows : 0;
    switch (x_dtype) {
        case MUMMU_F32: return simt_by_weight<float>(m, x, row_index, counts, offsets, max_rows_per_expert, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_F16: return simt_by_weight<__half>(m, x, row_index, counts, offsets, max_rows_per_expert, ys, ys_dtype, expert_only, rows_single, s);
        case MUMMU_BF16: return simt_by_weight<__nv_bfloat16>(m, x, row_index, counts, offsets, max_rows_per_expert, ys, ys_dtype, expert_only, rows_single, s);
    }
    set_error("experts: bad activation dtype %d", x_dtype);
    return MUMMU_ERR_CONTRACT;
}

// ---------------------------------------------------------------------------------------------
// Q4_K decode / encode, widening
// ---------------------------------------------------------------------------------------------
__global__ void q4k_dequant_kernel(const uint8_t* src, float* dst, int64_t n_elems) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_elems;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint8_t* blk = src + (i >> 8) * Q4K_BLOCK_BYTES;
        dst[i] = q4k_decode_elem(blk, (int)(i & 255));
    }
}

int launch_q4k_dequant(const void* src, float* dst, int64_t n_blocks, cudaStream_t s) {
    int64_t n = n_blocks * Q4K_BLOCK_ELEMS;
    if (n == 0) return MUMMU_OK;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    q4k_dequant_kernel<<<(unsigned)blocks, 256, 0, s>>>((const uint8_t*)src, dst, n);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// One warp per super-block; lane l owns values 8l..8l+7 (sub-block l/4).  The arithmetic is the
// host encoder's (mummu_b200/q4k.py), operation for operation, so both produce the same bytes.
__global__ void __launch_bounds__(256) q4k_quantize_kernel(const float* src, uint8_t* dst, int64_t n_blocks) {
    const unsigned full = 0xFFFFFFFFu;
    const int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t blk = warp; blk < n_blocks; blk += nwarps) {
        const float* x = src + blk * 256 + lane * 8;
        float v[8];
        float4 lo4 = *reinterpret_cast<const float4*>(x);
        float4 hi4 = *reinterpret_cast<const float4*>(x + 4);
        v[0] = lo4.x; v[1] = lo4.y; v[2] = lo4.z; v[3] = lo4.w;
        v[4] = hi4.x; v[5] = hi4.y; v[6] = hi4.z; v[7] = hi4.w;
        float mn = v[0], mx = v[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) { mn = fminf(mn, v[i]); mx = fmaxf(mx, v[i]); }
        mn = fminf(mn, __shfl_xor_sync(full, mn, 1)); mx = fmaxf(mx, __shfl_xor_sync(full, mx, 1));
        mn = fminf(mn, __shfl_xor_sync(full, mn, 2)); mx = fmaxf(mx, __shfl_xor_sync(full, mx, 2));
        float lo = fminf(mn, 0.0f);
        float hi = fmaxf(mx, lo);
        float scale = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
        float mnv = -lo;
        float ms = scale, mm = mnv;
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            ms = fmaxf(ms, __shfl_xor_sync(full, ms, off));
            mm = fmaxf(mm, __shfl_xor_sync(full, mm, off));
        }
        __half dh = __float2half_rn(__fdiv_rn(ms, 63.0f));
        __half dminh = __float2half_rn(__fdiv_rn(mm, 63.0f));
        float df = __half2float(dh), dminf = __half2float(dminh);
        float sc = df > 0.0f ? fminf(fmaxf(rintf(__fdiv_rn(scale, df)), 0.0f), 63.0f) : 0.0f;
        float mq = dminf > 0.0f ? fminf(fmaxf(rintf(__fdiv_rn(mnv, dminf)), 0.0f), 63.0f) : 0.0f;
        float dsc = __fmul_rn(df, sc);
        float dm = __fmul_rn(dminf, mq);
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float q = dsc > 0.0f ? fminf(fmaxf(rintf(__fdiv_rn(__fadd_rn(v[i], dm), dsc)), 0.0f), 15.0f) : 0.0f;
            packed |= ((uint32_t)q) << (4 * i);
        }
        uint8_t* out = dst + blk * Q4K_BLOCK_BYTES;
        uint32_t sci = (uint32_t)sc, mi = (uint32_t)mq;
        // scale bytes: lane b < 12 builds byte b from sub-block values held by lanes 4*j
        int b = lane < 12 ? lane : 0;
        int j_lo = b < 4 ? b : (b < 8 ? b - 4 : b - 4);      // first source sub-block
        int j_hi = b < 4 ? b + 4 : (b < 8 ? b : b - 4);      // second source sub-block
        uint32_t sc_a = __shfl_sync(full, sci, 4 * j_lo), m_a = __shfl_sync(full, mi, 4 * j_lo);
        uint32_t sc_b = __shfl_sync(full, sci, 4 * j_hi), m_b = __shfl_sync(full, mi, 4 * j_hi);
        uint32_t byte;
        if (b < 4) byte = sc_a | ((sc_b >> 4) << 6);
        else if (b < 8) byte = m_a | ((m_b >> 4) << 6);
        else byte = (sc_b & 0x0Fu) | ((m_b & 0x0Fu) << 4);
        if (lane < 12) out[4 + lane] = (uint8_t)byte;
        if (lane == 0) {
            *reinterpret_cast<unsigned short*>(out) = __half_as_ushort(dh);
            *reinterpret_cast<unsigned short*>(out + 2) = __half_as_ushort(dminh);
        }
        // quants: lane L with L%8 < 4 holds low nibbles of chunk L/8, lane L+4 the high nibbles
        uint32_t partner = __shfl_down_sync(full, packed, 4);
        if ((lane & 7) < 4) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t by = ((packed >> (4 * i)) & 0xFu) | (((partner >> (4 * i)) & 0xFu) << 4);
                w0 |= by << (8 * i);
                uint32_t by2 = ((packed >> (4 * (i + 4))) & 0xFu) | (((partner >> (4 * (i + 4))) & 0xFu) << 4);
                w1 |= by2 << (8 * i);
            }
            uint32_t* q = reinterpret_cast<uint32_t*>(out + 16 + 32 * (lane >> 3) + 8 * (lane & 7));
            q[0] = w0;
            q[1] = w1;
        }
    }
}

int launch_q4k_quantize(const float* src, void* dst, int64_t n_blocks, cudaStream_t s) {
    if (n_blocks == 0) return MUMMU_OK;
    int64_t blocks = (n_blocks + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    q4k_quantize_kernel<<<(unsigned)blocks, 256, 0, s>>>(src, (uint8_t*)dst, n_blocks);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

template <typename T>
__global__ void narrow_kernel(const float* src, T* dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = from_f32<T>(src[i]);
}

int launch_narrow(const float* src, void* dst, int dtype, int64_t n, cudaStream_t s) {
    if (n == 0) return MUMMU_OK;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    switch (dtype) {
        case MUMMU_F32: narrow_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(src, (float*)dst, n); break;
        case MUMMU_F16: narrow_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(src, (__half*)dst, n); break;
        case MUMMU_BF16: narrow_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(src, (__nv_bfloat16*)dst, n); break;
        default: set_error("narrow: bad dtype %d", dtype); return MUMMU_ERR_CONTRACT;
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

template <typename T>
__global__ void widen_kernel(const T* src, float* dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = to_f32(src[i]);
}

int launch_widen(const void* src, int dtype, float* dst, int64_t n, cudaStream_t s) {
    if (n == 0) return MUMMU_OK;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    switch (dtype) {
        case MUMMU_F32: widen_kernel<float><<<(unsigned)blocks, 256, 0, s>>>((const float*)src, dst, n); break;
        case MUMMU_F16: widen_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((const __half*)src, dst, n); break;
        case MUMMU_BF16: widen_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)src, dst, n); break;
        default: set_error("widen: bad dtype %d", dtype); return MUMMU_ERR_CONTRACT;
    }
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// ---------------------------------------------------------------------------------------------
// one expert on its own (ExpertExec::run and friends)
// ---------------------------------------------------------------------------------------------
// counts / offsets / work order for "`rows` rows, all of expert e"
__global__ void single_expert_plan_kernel(int e, int rows, int E, int32_t* counts, int32_t* offsets, int32_t* active,
                                          int32_t* n_active) {
    for (int i = threadIdx.x; i <= E; i += blockDim.x) {
        if (i < E) counts[i] = i == e ? rows : 0;
        offsets[i] = i <= e ? 0 : rows;
    }
    if (threadIdx.x == 0) {
        active[0] = e;
        *n_active = rows > 0 ? 1 : 0;
    }
}

int launch_single_expert_plan(MummuMoe* m, int expert, int rows, cudaStream_t s) {
    LaunchScope scope(m, s, "expert_plan");
    single_expert_plan_kernel<<<1, 256, 0, s>>>(expert, rows, m->cfg.experts_local, m->counts, m->offsets, m->active,
                                                m->n_active);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// energy[row] = sum over the expert's intermediate columns n of silu(x[row,:] . gate[n,:])^2
// (ExpertExec::gate_energy, nn/moe.rs:413-418).  One block per row; the columns are summed in a
// fixed order (a thread's columns ascending, then a tree over the threads), so the result does not
// depend on scheduling.
template <typename TW>
__global__ void __launch_bounds__(256) gate_energy_kernel(const float* x, const uint8_t* gate, size_t row_bytes, int H,
                                                          int I, float* energy) {
    extern __shared__ float s_x[];
    __shared__ float s_part[256];
    const int row = blockIdx.x;
    for (int k = threadIdx.x; k < H; k += blockDim.x) s_x[k] = x[(size_t)row * H + k];
    __syncthreads();
    float acc = 0.0f;
    for (int n = threadIdx.x; n < I; n += blockDim.x) {
        const uint8_t* wrow = gate + (size_t)n * row_bytes;
        float d = 0.0f;
        for (int k = 0; k < H; ++k) d = fmaf(s_x[k], load_w<TW>(wrow, k), d);
        const float a = silu_f(d);
        acc += a * a;
    }
    s_part[threadIdx.x] = acc;
    __syncthreads();
    for (int off = 128; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) s_part[threadIdx.x] += s_part[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) energy[row] = s_part[0];
}

int launch_gate_energy(MummuMoe* m, int expert, const float* x, int rows, float* energy, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    const size_t row_bytes = bank_row_bytes(c, MUMMU_BANK_GATE);
    const uint8_t* gate = (const uint8_t*)m->bank[MUMMU_BANK_GATE] + (size_t)expert * row_bytes * c.inter;
    const size_t smem = (size_t)c.hidden * sizeof(float);
    if (smem > 200 * 1024) {
        set_error("gate_energy: hidden %d too wide", c.hidden);
        return MUMMU_ERR_UNSUPPORTED;
    }
    LaunchScope scope(m, s, "gate_energy");
#define MUMMU_GE(TW)                                                                          \
    do {                                                                                      \
        MUMMU_CUDA_TRY(allow_big_smem(gate_energy_kernel<TW>, c.device));                     \
        gate_energy_kernel<TW><<<rows, 256, smem, s>>>(x, gate, row_bytes, c.hidden, c.inter, energy); \
    } while (0)
    switch (c.weight_dtype) {
        case MUMMU_F32: MUMMU_GE(float); break;
        case MUMMU_F16: MUMMU_GE(__half); break;
        case MUMMU_BF16: MUMMU_GE(__nv_bfloat16); break;
        case MUMMU_Q4_K: MUMMU_GE(q4k_t); break;
        case MUMMU_Q8_0: MUMMU_GE(q80_t); break;
        case MUMMU_Q5_K: MUMMU_GE(q5k_t); break;
        case MUMMU_Q6_K: MUMMU_GE(q6k_t); break;
        default: set_error("gate_energy: bad weight dtype %d", c.weight_dtype); return MUMMU_ERR_CONTRACT;
    }
#undef MUMMU_GE
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

// ---------------------------------------------------------------------------------------------
// Router for callers that must not allocate (mummu_moe_route_noalloc)
// ---------------------------------------------------------------------------------------------
// The router kernel needs scratch beyond its inputs and outputs: the [tokens, experts] logits that
// its expert-slice blocks hand to the block that selects, one arrival counter per token tile, and a
// status word.  Here that scratch is a fixed array in the library's device image, so the call
// allocates nothing.  Every GPU that loads the library holds the array (about 1 MiB) until exit.
constexpr int NOALLOC_MAX_TOKENS = 1024;
constexpr int NOALLOC_MAX_LOGITS = 256 * 1024;                 // tokens * experts
constexpr int NOALLOC_TILES = NOALLOC_MAX_TOKENS / 4 + 8;

struct NoAllocScratch {
    float logits[NOALLOC_MAX_LOGITS];
    int32_t tile_done[NOALLOC_TILES];
    int32_t status;
};

static __device__ __align__(256) unsigned char g_route_scratch[sizeof(NoAllocScratch)];

// In host code `g_route_scratch` is only a stand-in for the symbol, never a device address: the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
static NoAllocScratch* route_scratch_for(int device, cudaError_t* err) {
    static std::mutex mu;
    static NoAllocScratch* ptrs[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    *err = cudaSuccess;
    if (device < 0 || device >= 64) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    if (!ptrs[device]) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_route_scratch);
        if (*err != cudaSuccess) return nullptr;
        ptrs[device] = static_cast<NoAllocScratch*>(p);
    }
    return ptrs[device];
}

template <typename TX>
static int route_noalloc_launch(RouterArgs& a, int device, cudaStream_t s) {
    const size_t smem = router_smem(a.H, a.E, a.k, 4);
    if (smem > 220 * 1024) {
        set_error("mummu_moe_route_noalloc: hidden %d too wide for the shared-memory staged router", a.H);
        return MUMMU_ERR_UNSUPPORTED;
    }
    MUMMU_CUDA_TRY(allow_big_smem(router_kernel<TX, 1, false>, device));
    dim3 grid((a.E + R_ES - 1) / R_ES, (a.T + 3) / 4);
    router_kernel<TX, 1, false><<<grid, R_THREADS, smem, s>>>(a);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

}  // namespace mummu

extern "C" int32_t mummu_moe_route_noalloc(const void* x, int32_t act_dtype, const float* router_w,
                                           const float* bias, int32_t tokens, int32_t hidden,
                                           int32_t experts, int32_t top_k, int32_t norm_topk_prob,
                                           int32_t* ids_out, float* w_out, int32_t device, void* stream) {
    using namespace mummu;
    MUMMU_REQUIRE(tokens >= 0, "mummu_moe_route_noalloc: negative token count %d", tokens);
    MUMMU_REQUIRE(hidden >= 1 && experts >= 2 && experts <= 32 * R_MAXV,
                  "mummu_moe_route_noalloc: hidden %d, experts %d (2..=%d)", hidden, experts, 32 * R_MAXV);
    MUMMU_REQUIRE(top_k >= 1 && top_k <= experts,
                  "MoE forward: top_k (%d) must be in 1..=num_experts (%d)", top_k, experts);
    MUMMU_REQUIRE(tokens <= NOALLOC_MAX_TOKENS && (int64_t)tokens * experts <= NOALLOC_MAX_LOGITS,
                  "mummu_moe_route_noalloc: %d tokens x %d experts exceed the fixed scratch "
                  "(at most %d tokens and %d tokens*experts); use mummu_moe_route",
                  tokens, experts, NOALLOC_MAX_TOKENS, NOALLOC_MAX_LOGITS);
    if (tokens == 0) return MUMMU_OK;
    MUMMU_REQUIRE(x && router_w && ids_out && w_out, "mummu_moe_route_noalloc: null pointer");
    // the kernel reads eight experts of one router row as two 128-bit words: a pointer into the
    // middle of a packed buffer that is only 4-byte aligned would fault on the device
    MUMMU_REQUIRE((reinterpret_cast<uintptr_t>(router_w) & 15) == 0,
                  "mummu_moe_route_noalloc: router_w must be 16-byte aligned (got %p)", (const void*)router_w);
    MUMMU_REQUIRE((reinterpret_cast<uintptr_t>(x) & (act_dtype == MUMMU_F32 ? 3 : 1)) == 0 &&
                      (reinterpret_cast<uintptr_t>(ids_out) & 3) == 0 &&
                      (reinterpret_cast<uintptr_t>(w_out) & 3) == 0 &&
                      (!bias || (reinterpret_cast<uintptr_t>(bias) & 3) == 0),
                  "mummu_moe_route_noalloc: x, bias, ids_out and w_out must be aligned to their element size");
    int prev = -1;
    MUMMU_CUDA_TRY(cudaGetDevice(&prev));
    if (prev != device) MUMMU_CUDA_TRY(cudaSetDevice(device));
    int rc = MUMMU_OK;
    do {
        cudaError_t err;
        NoAllocScratch* sc = route_scratch_for(device, &err);
        if (!sc) {
            set_error("mummu_moe_route_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
            rc = MUMMU_ERR_DEVICE;
            break;
        }
        cudaStream_t s = (cudaStream_t)stream;
        // the array keeps the previous call's contents: counters and status must start at zero
        err = cudaMemsetAsync(sc->tile_done, 0, sizeof(sc->tile_done) + sizeof(sc->status), s);
        if (err != cudaSuccess) {
            set_error("mummu_moe_route_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(err));
            rc = MUMMU_ERR_DEVICE;
            break;
        }
        RouterArgs a;
        a.x = x;
        a.w = router_w;
        a.wt = nullptr;
        a.bias = bias;
        a.logits = sc->logits;
        a.tile_done = sc->tile_done;
        a.ids = ids_out;
        a.wts = w_out;
        a.counts = nullptr;
        a.hits = nullptr;
        a.fuse = 0;
        a.p_counts = a.p_offsets = a.p_row_token = a.p_pos = a.p_active = a.p_n_active = nullptr;
        a.status = &sc->status;
        a.T = tokens;
        a.H = hidden;
        a.E = experts;
        a.k = top_k;
        a.norm = norm_topk_prob;
        switch (act_dtype) {
            case MUMMU_F32: rc = route_noalloc_launch<float>(a, device, s); break;
            case MUMMU_F16: rc = route_noalloc_launch<__half>(a, device, s); break;
            case MUMMU_BF16: rc = route_noalloc_launch<__nv_bfloat16>(a, device, s); break;
            default:
                set_error("mummu_moe_route_noalloc: activation dtype %d is not F32, F16 or BF16", act_dtype);
                rc = MUMMU_ERR_CONTRACT;
        }
    } while (0);
    if (prev != device) cudaSetDevice(prev);
    return rc;
}
