// Decode-step trunk of the OLMoE decoder around the expert bank: everything a token passes
// between two MoE layers, for `slots` independent sequences with one new token each
// (reference: crates/mummu/src/models/olmoe.rs:522-587; nn/attention.rs:182-295 - whole-projection
// q/k RMSNorm :196-200, f32 score island :275-289, additive -1e4 mask :28-48; nn/rope.rs:21-105;
// the fixed-shape step of nn/static_kv.rs:36-72 and capture.rs:48-107: preallocated
// [slots, kv_heads, max_ctx, head_dim] cache written in place, positions read on the device).
//
// HBM-bound like the expert bank: per step the f16 projection weights (4 * hidden^2 per layer), the
// lm_head and the keys and values cached so far are streamed once.  Kernels:
//   add_rms        x (+= y) ; h = rmsnorm(x) * gamma                          one block per slot
//   gemv           out[slot, n] = sum_k W[n, k] h[slot, k]   f16 weights read with 128-bit loads,
//                  16 rows per warp against the slots' activations in shared memory, m16n8k16 MMAs
//                  with f32 accumulation; K may be split over blockIdx.y into f32 partials that the
//                  consumer adds in a fixed order
//   qk_norm_rope   partials -> q, k, v; RMSNorm of q and of k over the WHOLE projection; rotate-half
//                  RoPE at each slot's position; k and v written into the cache at that position
//   attention      per (head, slot, key split): scores in f32 against the cached keys up to the
//                  slot's position (keys beyond it would get -1e4 and vanish in the softmax: they
//                  are skipped), partial softmax and value sum; combine folds the splits
//   residual_rms   x += o-projection partials ; h2 = rmsnorm(x) * gamma_post
//   head           final norm (add_rms), lm_head (gemv), argmax with ties to the lowest id
// Every kernel is shape-static for fixed (slots, key_len), so a step replays from one CUDA graph.
#include <cfloat>
#include <cmath>
#include <cstring>

#include "common.cuh"

struct MummuTrunk {
    MummuTrunkConfig cfg{};
    std::mutex mu;
    cudaStream_t stream = nullptr;
    __half* embed = nullptr;        // [vocab, hidden]
    __half* lm_head = nullptr;      // [vocab, hidden]
    float* final_norm = nullptr;    // [hidden]
    float* norms = nullptr;         // [layers][4][hidden]: in, post, q, k
    __half* wqkv = nullptr;         // [layers][(heads + 2 kv_heads) * head_dim, hidden]
    __half* wo = nullptr;           // [layers][hidden, heads * head_dim]
    __half* kc = nullptr;           // [layers][slots][kv_heads][max_ctx][head_dim]
    __half* vc = nullptr;
    float* rope_cos = nullptr;      // [max_ctx][head_dim / 2]
    float* rope_sin = nullptr;
    // per-step scratch
    __half* h = nullptr;            // [slots, hidden] normalised activations
    float* part = nullptr;          // GEMV partials [ksplit][slots][n_max]
    __half* q = nullptr;            // [slots, heads * head_dim]
    __half* ctx = nullptr;          // [slots, heads * head_dim]
    float* apart = nullptr;         // attention partials [slots][heads][splits][head_dim + 2]
    int64_t launches = 0;
};

namespace mummu {

constexpr int TR_MAX_SPLITS = 32;

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float block_sum(float v, float* s_red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; ++w) t += s_red[w];      // same order in every thread
    return t;
}

// x[slot] (+= y[slot]); h[slot] = x / sqrt(mean(x^2) + eps) * gamma        (models/olmoe.rs:561, 566)
__global__ void __launch_bounds__(512) add_rms_kernel(__half* x, const __half* y, const float* gamma, __half* h, int H,
                                                      float eps) {
    __shared__ float s_red[16];
    extern __shared__ float s_row[];
    const int slot = blockIdx.x;
    float ss = 0.0f;
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
        float v = __half2float(x[(size_t)slot * H + k]);
        if (y) {
            v = __half2float(__float2half_rn(v + __half2float(y[(size_t)slot * H + k])));
            x[(size_t)slot * H + k] = __float2half_rn(v);
        }
        s_row[k] = v;
        ss += v * v;
    }
    const float tot = block_sum(ss, s_red);
    const float r = rsqrtf(tot / (float)H + eps);
    for (int k = threadIdx.x; k < H; k += blockDim.x) h[(size_t)slot * H + k] = __float2half_rn(s_row[k] * r * gamma[k]);
}

// out partials: part[(ks * B + b) * N + n] = sum over this block's K range of W[n, k] * x[b, k]
// grid (N / 128 rounded up, ksplit); 8 warps, 16 rows each.  NTT token tiles of 8.
template <int NTT>
__global__ void __launch_bounds__(256) gemv_f16_kernel(const __half* __restrict__ W, const __half* __restrict__ x,
                                                        float* __restrict__ part, int N, int K, int k_per_block, int B) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int KC = 512;                         // K staged per round
    constexpr int XS = KC + 32;                     // padded row (halves): rows 16 words apart mod 32 banks
    __half* xs = reinterpret_cast<__half*>(smem_raw);     // [8 * NTT][XS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 128 + warp * 16;
    const int k_begin = blockIdx.y * k_per_block, k_end = min(K, k_begin + k_per_block);
    const bool rows_ok = row0 + 16 <= N;
    const __half* wa = W + (size_t)(row0 + g) * K;
    const __half* wb = wa + (size_t)8 * K;
    float acc[NTT][4];
#pragma unroll
    for (int nt = 0; nt < NTT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    for (int k0 = k_begin; k0 < k_end; k0 += KC) {
        const int kc = min(KC, k_end - k0);
        __syncthreads();
        for (int idx = tid; idx < 8 * NTT * (KC / 8); idx += 256) {
            const int b = idx / (KC / 8), q8 = idx - b * (KC / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (b < B && q8 * 8 < kc) v = *reinterpret_cast<const uint4*>(x + (size_t)b * K + k0 + q8 * 8);
            *reinterpret_cast<uint4*>(xs + (size_t)b * XS + q8 * 8) = v;
        }
        __syncthreads();
        if (rows_ok) {
            // a lane reads 16 contiguous bytes (8 values) of its two rows per 32-value step; the MMA's
            // k slots are labelled so that those 8 values are the lane's slots of two MMAs
#pragma unroll 4
            for (int c = 0; c < kc / 32; ++c) {
                const uint4 a_lo = __ldcs(reinterpret_cast<const uint4*>(wa + k0 + c * 32 + t * 8));
                const uint4 a_hi = __ldcs(reinterpret_cast<const uint4*>(wb + k0 + c * 32 + t * 8));
#pragma unroll
                for (int nt = 0; nt < NTT; ++nt) {
                    const uint4 b = *reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + g) * XS + c * 32 + t * 8);
                    mma_f16(acc[nt], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
                    mma_f16(acc[nt], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
                }
            }
        }
    }
    if (!rows_ok) return;
#pragma unroll
    for (int nt = 0; nt < NTT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int b = nt * 8 + 2 * t + (i & 1);
            const int n = row0 + g + ((i >> 1) << 3);
            if (b < B) part[((size_t)blockIdx.y * B + b) * N + n] = acc[nt][i];
        }
}

// per (slot, part): part 0 = q, 1 = k, 2 = v.  The projection's output from its partials; RMSNorm of
// q and of k over the whole projection (nn/attention.rs:196-200); rotate-half RoPE
// (nn/rope.rs:66-105); k and v stored in the cache at the slot's position (nn/static_kv.rs:
// index-driven assignment in place)
__global__ void __launch_bounds__(512) qk_norm_rope_kernel(const float* part, int ksplit, int B, const float* gq,
                                                           const float* gk, const float* cosv, const float* sinv,
                                                           const int32_t* positions, __half* q_out, __half* kc, __half* vc,
                                                           int heads, int kv_heads, int hd, int max_ctx, float eps) {
    extern __shared__ float s_v[];
    __shared__ float s_red[16];
    const int slot = blockIdx.x, which = blockIdx.y;
    const int nq = heads * hd, nkv = kv_heads * hd, N = nq + 2 * nkv;
    const int n0 = which == 0 ? 0 : (which == 1 ? nq : nq + nkv), nn = which == 0 ? nq : nkv;
    float ss = 0.0f;
    for (int n = threadIdx.x; n < nn; n += blockDim.x) {
        float s = 0.0f;
        for (int ks = 0; ks < ksplit; ++ks) s += part[((size_t)ks * B + slot) * N + n0 + n];
        s = __half2float(__float2half_rn(s));       // the projection's output in the trunk's dtype
        s_v[n] = s;
        ss += s * s;
    }
    const int pos = positions[slot];
    if (which == 2) {
        __syncthreads();
        for (int n = threadIdx.x; n < nkv; n += blockDim.x) {
            const int hh = n / hd, d = n - hh * hd;
            vc[(((size_t)slot * kv_heads + hh) * max_ctx + pos) * hd + d] = __float2half_rn(s_v[n]);
        }
        return;
    }
    const float r = rsqrtf(block_sum(ss, s_red) / (float)nn + eps);
    const float* gamma = which == 0 ? gq : gk;
    for (int n = threadIdx.x; n < nn; n += blockDim.x) s_v[n] = __half2float(__float2half_rn(s_v[n] * r * gamma[n]));
    __syncthreads();
    const int half = hd >> 1;
    const float* cr = cosv + (size_t)pos * half;
    const float* sr = sinv + (size_t)pos * half;
    for (int n = threadIdx.x; n < nn; n += blockDim.x) {
        const int hh = n / hd, d = n - hh * hd, i = d < half ? d : d - half;
        const float other = d < half ? -s_v[n + half] : s_v[n - half];
        const __half o = __float2half_rn(s_v[n] * cr[i] + other * sr[i]);
        if (which == 0) q_out[(size_t)slot * nq + n] = o;
        else kc[(((size_t)slot * kv_heads + hh) * max_ctx + pos) * hd + d] = o;
    }
}

constexpr int ATT_UN = 8;                           // 16-byte loads in flight per lane

// a 16-byte load that does not displace the weights in L1: each key and value is read once per step
__device__ __forceinline__ uint4 ld_stream16(const __half* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// grid (heads, slots, splits); 128 threads; one partial (max, sum, value sum) per block.
// A key or value row of `hd` halves is read by hd/8 lanes with one 16-byte load each, so a warp
// covers 256 / hd rows... (hd = 128: two rows) per instruction, fully coalesced.
__global__ void __launch_bounds__(128) decode_attn_kernel(const __half* q, const __half* kc, const __half* vc,
                                                          const int32_t* positions, float* apart, int heads, int kv_heads,
                                                          int hd, int max_ctx, int key_len, int splits, float scale) {
    extern __shared__ float s_attn[];               // scores [chunk] | per-warp value sums [4][hd]
    __shared__ float s_red[4];
    const int head = blockIdx.x, slot = blockIdx.y, sp = blockIdx.z;
    const int pos = min(positions[slot], key_len - 1);
    const int chunk = (key_len + splits - 1) / splits;
    const int lo = sp * chunk, hi = min(pos + 1, lo + chunk);
    float* s_sc = s_attn;
    float* s_acc = s_attn + chunk;
    float* out = apart + (((size_t)slot * heads + head) * splits + sp) * (hd + 2);
    if (lo >= hi) {                                 // nothing for this split (uniform over the block)
        if (threadIdx.x == 0) {
            out[0] = -FLT_MAX;
            out[1] = 0.0f;
        }
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lpr = hd >> 3;                        // lanes per row (16 for head_dim 128)
    const int rpw = 32 / lpr;                       // rows per warp instruction
    const int sub = lane / lpr, li = lane - sub * lpr;
    const int hkv = head / (heads / kv_heads);
    const __half* kbase = kc + ((size_t)slot * kv_heads + hkv) * max_ctx * hd;
    const __half* vbase = vc + ((size_t)slot * kv_heads + hkv) * max_ctx * hd;
    // this lane's 8 values of q
    float qf[8];
    {
        const uint4 qv = *reinterpret_cast<const uint4*>(q + ((size_t)slot * heads + head) * hd + li * 8);
        const __half2* h2 = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float2 f = __half22float2(h2[u]);
            qf[2 * u] = f.x * scale;
            qf[2 * u + 1] = f.y * scale;
        }
    }
    // ATT_UN loads per lane are issued before any is used: the kernel is bound by bytes in flight
    float mx = -FLT_MAX;
    for (int jb = lo + warp * (rpw * ATT_UN); jb < hi; jb += 4 * rpw * ATT_UN) {
        uint4 kv[ATT_UN];
#pragma unroll
        for (int u = 0; u < ATT_UN; ++u) {
            const int j = jb + u * rpw + sub;
            kv[u] = j < hi ? ld_stream16(kbase + (size_t)j * hd + li * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < ATT_UN; ++u) {
            const int j = jb + u * rpw + sub;
            const __half2* h2 = reinterpret_cast<const __half2*>(&kv[u]);
            float s = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h2[e]);
                s = fmaf(f.x, qf[2 * e], s);
                s = fmaf(f.y, qf[2 * e + 1], s);
            }
            for (int off = lpr >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
            if (j < hi) {
                if (li == 0) s_sc[j - lo] = s;
                mx = fmaxf(mx, s);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    float psum = 0.0f;
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        const float p = __expf(s_sc[j - lo] - mx);
        s_sc[j - lo] = p;
        psum += p;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) psum += __shfl_xor_sync(0xFFFFFFFFu, psum, off);
    __syncthreads();                                // everyone has read s_red (the maxima)
    if (lane == 0) s_red[warp] = psum;
    __syncthreads();
    // values: the lane keeps 8 output dimensions, summed over the rows it reads
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int jb = lo + warp * (rpw * ATT_UN); jb < hi; jb += 4 * rpw * ATT_UN) {
        uint4 vv[ATT_UN];
#pragma unroll
        for (int u = 0; u < ATT_UN; ++u) {
            const int j = jb + u * rpw + sub;
            vv[u] = j < hi ? ld_stream16(vbase + (size_t)j * hd + li * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < ATT_UN; ++u) {
            const int j = jb + u * rpw + sub;
            const float p = j < hi ? s_sc[j - lo] : 0.0f;
            const __half2* h2 = reinterpret_cast<const __half2*>(&vv[u]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h2[e]);
                acc[2 * e] = fmaf(p, f.x, acc[2 * e]);
                acc[2 * e + 1] = fmaf(p, f.y, acc[2 * e + 1]);
            }
        }
    }
    // fold the row groups of a warp, then the warps (fixed order)
    for (int off = lpr; off < 32; off <<= 1)
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] += __shfl_xor_sync(0xFFFFFFFFu, acc[u], off);
    if (sub == 0)
#pragma unroll
        for (int u = 0; u < 8; ++u) s_acc[warp * hd + li * 8 + u] = acc[u];
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += blockDim.x)
        out[2 + d] = (s_acc[d] + s_acc[hd + d]) + (s_acc[2 * hd + d] + s_acc[3 * hd + d]);
    if (threadIdx.x == 0) {
        out[0] = mx;
        out[1] = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
    }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const float* apart, __half* ctx, int heads, int hd, int splits) {
    const int head = blockIdx.x, slot = blockIdx.y;
    const float* base = apart + ((size_t)slot * heads + head) * splits * (hd + 2);
    float M = -FLT_MAX;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, base[(size_t)s * (hd + 2)]);
    float L = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float l = base[(size_t)s * (hd + 2) + 1];
        if (l > 0.0f) L += l * __expf(base[(size_t)s * (hd + 2)] - M);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float l = base[(size_t)s * (hd + 2) + 1];
            if (l > 0.0f) acc += base[(size_t)s * (hd + 2) + 2 + d] * __expf(base[(size_t)s * (hd + 2)] - M);
        }
        ctx[((size_t)slot * heads + head) * hd + d] = __float2half_rn(acc / L);
    }
}

// x += sum of the o-projection partials ; h2 = rmsnorm(x) * gamma     (models/olmoe.rs:565-566)
__global__ void __launch_bounds__(512) residual_rms_kernel(__half* x, const float* part, int ksplit, int B,
                                                           const float* gamma, __half* h2, int H, float eps) {
    __shared__ float s_red[16];
    extern __shared__ float s_row[];
    const int slot = blockIdx.x;
    float ss = 0.0f;
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
        float o = 0.0f;
        for (int ks = 0; ks < ksplit; ++ks) o += part[((size_t)ks * B + slot) * H + k];
        const float v = __half2float(__float2half_rn(__half2float(x[(size_t)slot * H + k]) + __half2float(__float2half_rn(o))));
        x[(size_t)slot * H + k] = __float2half_rn(v);
        s_row[k] = v;
        ss += v * v;
    }
    const float tot = block_sum(ss, s_red);
    const float r = rsqrtf(tot / (float)H + eps);
    for (int k = threadIdx.x; k < H; k += blockDim.x) h2[(size_t)slot * H + k] = __float2half_rn(s_row[k] * r * gamma[k]);
}

__global__ void __launch_bounds__(256) embed_kernel(const __half* embed, const int32_t* tokens, __half* x, int H, int vocab) {
    const int slot = blockIdx.x;
    int tok = tokens[slot];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const uint4* src = reinterpret_cast<const uint4*>(embed + (size_t)tok * H);
    uint4* dst = reinterpret_cast<uint4*>(x + (size_t)slot * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// greedy pick: the largest logit, ties to the lowest id (decode.rs:33-48)
__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, int V, int32_t* out) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const int slot = blockIdx.x;
    const float* row = logits + (size_t)slot * V;
    float bv = -FLT_MAX;
    int bi = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > bv) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        s_v[threadIdx.x >> 5] = bv;
        s_i[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = threadIdx.x < (blockDim.x >> 5) ? s_v[threadIdx.x] : -FLT_MAX;
        bi = threadIdx.x < (blockDim.x >> 5) ? s_i[threadIdx.x] : 0x7FFFFFFF;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (threadIdx.x == 0) out[slot] = bi;
    }
}

__global__ void kv_write_kernel(const __half* k, const __half* v, __half* kc, __half* vc, int kv_heads, int hd, int max_ctx,
                                int slot, int first, int count) {
    const size_t n = (size_t)kv_heads * count * hd;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % hd);
        const int p = (int)((i / hd) % count);
        const int hh = (int)(i / ((size_t)hd * count));
        const size_t at = (((size_t)slot * kv_heads + hh) * max_ctx + first + p) * hd + d;
        kc[at] = k[i];
        vc[at] = v[i];
    }
}

struct TrunkLaunch {
    MummuTrunk* t;
    explicit TrunkLaunch(MummuTrunk* t_) : t(t_) { t->launches += 1; }
};

static int gemv(MummuTrunk* t, const __half* W, const __half* x, float* part, int N, int K, int ksplit, int B,
                cudaStream_t s) {
    const int k_per_block = ((K / ksplit + 31) / 32) * 32;
    const dim3 grid((unsigned)((N + 127) / 128), (unsigned)ksplit);
    const int ntt = (B + 7) / 8;
    TrunkLaunch l(t);
#define MUMMU_GEMV(NTT)                                                                                         \
    do {                                                                                                        \
        const size_t smem = (size_t)8 * NTT * (512 + 32) * sizeof(__half);                                      \
        MUMMU_CUDA_TRY(allow_big_smem(gemv_f16_kernel<NTT>, t->cfg.device));                                    \
        gemv_f16_kernel<NTT><<<grid, 256, smem, s>>>(W, x, part, N, K, k_per_block, B);                         \
    } while (0)
    if (ntt <= 1) MUMMU_GEMV(1);
    else if (ntt <= 2) MUMMU_GEMV(2);
    else if (ntt <= 4) MUMMU_GEMV(4);
    else MUMMU_GEMV(8);
#undef MUMMU_GEMV
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

struct TrunkDevice {
    int prev = -1;
    explicit TrunkDevice(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~TrunkDevice() {
        int cur = -1;
        cudaGetDevice(&cur);
        if (prev >= 0 && cur != prev) cudaSetDevice(prev);
    }
};

static size_t trunk_weight_elems(const MummuTrunkConfig& c, int which) {
    const size_t H = c.hidden, nq = (size_t)c.heads * c.head_dim, nkv = (size_t)c.kv_heads * c.head_dim;
    switch (which) {
        case MUMMU_TRUNK_EMBED:
        case MUMMU_TRUNK_LM_HEAD: return (size_t)c.vocab * H;
        case MUMMU_TRUNK_FINAL_NORM:
        case MUMMU_TRUNK_IN_NORM:
        case MUMMU_TRUNK_POST_NORM: return H;
        case MUMMU_TRUNK_Q_NORM: return nq;
        case MUMMU_TRUNK_K_NORM: return nkv;
        case MUMMU_TRUNK_Q: return nq * H;
        case MUMMU_TRUNK_K:
        case MUMMU_TRUNK_V: return nkv * H;
        case MUMMU_TRUNK_O: return H * nq;
    }
    return 0;
}

}  // namespace mummu

using namespace mummu;

extern "C" {

uint64_t mummu_trunk_static_bytes(const MummuTrunkConfig* c) {
    if (!c) return 0;
    return (uint64_t)2 * c->layers * c->slots * c->kv_heads * c->max_ctx * c->head_dim * sizeof(__half);
}

int32_t mummu_trunk_create(const MummuTrunkConfig* cfg, MummuTrunk** out) {
    MUMMU_REQUIRE(cfg && out, "mummu_trunk_create: null argument");
    *out = nullptr;
    const MummuTrunkConfig& c = *cfg;
    MUMMU_REQUIRE(c.hidden >= 8 && c.hidden % 32 == 0 && c.heads >= 1 && c.kv_heads >= 1 && c.heads % c.kv_heads == 0 &&
                      c.head_dim >= 8 && c.head_dim <= 256 && (c.head_dim & (c.head_dim - 1)) == 0 && c.layers >= 1 &&
                      c.vocab >= 1,
                  "trunk: hidden %d (a multiple of 32), %d heads over %d kv heads of %d (a power of two, 8..256), %d layers, "
                  "vocabulary %d",
                  c.hidden, c.heads, c.kv_heads, c.head_dim, c.layers, c.vocab);
    MUMMU_REQUIRE((c.heads * c.head_dim) % 32 == 0 && ((c.heads + 2 * c.kv_heads) * c.head_dim) % 128 == 0 &&
                      c.hidden % 128 == 0 && c.vocab % 128 == 0,
                  "trunk: projection widths must be multiples of 128 rows (q+k+v %d, hidden %d, vocabulary %d)",
                  (c.heads + 2 * c.kv_heads) * c.head_dim, c.hidden, c.vocab);
    MUMMU_REQUIRE(c.slots >= 1 && c.slots <= 64, "trunk: %d slots (1..=64 sequences per step)", c.slots);
    MUMMU_REQUIRE(c.max_ctx >= 1 && c.max_ctx <= 131072, "trunk: max_ctx %d", c.max_ctx);
    int ndev = 0;
    MUMMU_CUDA_TRY(cudaGetDeviceCount(&ndev));
    MUMMU_REQUIRE(c.device >= 0 && c.device < ndev, "trunk: CUDA device %d of %d", c.device, ndev);
    TrunkDevice guard(c.device);
    MummuTrunk* t = new MummuTrunk();
    t->cfg = c;
    const size_t H = c.hidden, nq = (size_t)c.heads * c.head_dim, nkv = (size_t)c.kv_heads * c.head_dim;
    const size_t nqkv = nq + 2 * nkv, L = c.layers;
    const size_t n_max = std::max<size_t>(std::max(nqkv, H), (size_t)c.vocab);
    cudaError_t err = cudaStreamCreateWithFlags(&t->stream, cudaStreamNonBlocking);
    auto alloc = [&](void** p, size_t bytes) {
        if (err == cudaSuccess) err = cudaMalloc(p, bytes ? bytes : 1);
    };
    alloc((void**)&t->embed, (size_t)c.vocab * H * 2);
    alloc((void**)&t->lm_head, (size_t)c.vocab * H * 2);
    alloc((void**)&t->final_norm, H * 4);
    alloc((void**)&t->norms, L * 4 * std::max(H, nq) * 4);
    alloc((void**)&t->wqkv, L * nqkv * H * 2);
    alloc((void**)&t->wo, L * H * nq * 2);
    alloc((void**)&t->kc, mummu_trunk_static_bytes(&c) / 2);
    alloc((void**)&t->vc, mummu_trunk_static_bytes(&c) / 2);
    alloc((void**)&t->rope_cos, (size_t)c.max_ctx * (c.head_dim / 2) * 4);
    alloc((void**)&t->rope_sin, (size_t)c.max_ctx * (c.head_dim / 2) * 4);
    alloc((void**)&t->h, (size_t)c.slots * std::max(H, nq) * 2);
    alloc((void**)&t->part, (size_t)8 * c.slots * n_max * 4);
    alloc((void**)&t->q, (size_t)c.slots * nq * 2);
    alloc((void**)&t->ctx, (size_t)c.slots * nq * 2);
    alloc((void**)&t->apart, (size_t)c.slots * c.heads * TR_MAX_SPLITS * (c.head_dim + 2) * 4);
    if (err == cudaSuccess) err = cudaMemset(t->kc, 0, mummu_trunk_static_bytes(&c) / 2);
    if (err == cudaSuccess) err = cudaMemset(t->vc, 0, mummu_trunk_static_bytes(&c) / 2);
    if (err == cudaSuccess) {
        // RoPE tables as the reference builds them (nn/rope.rs:21-63): f32 arithmetic on the host
        const int half = c.head_dim / 2;
        std::vector<float> cs((size_t)c.max_ctx * half), sn((size_t)c.max_ctx * half);
        for (int i = 0; i < half; ++i) {
            const float inv = 1.0f / powf(c.rope_theta, 2.0f * (float)i / (float)c.head_dim);
            for (int p = 0; p < c.max_ctx; ++p) {
                const float ang = (float)p * inv;
                cs[(size_t)p * half + i] = cosf(ang);
                sn[(size_t)p * half + i] = sinf(ang);
            }
        }
        err = cudaMemcpy(t->rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice);
        if (err == cudaSuccess) err = cudaMemcpy(t->rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice);
    }
    if (err != cudaSuccess) {
        set_error("mummu_trunk_create: %s", cudaGetErrorString(err));
        mummu_trunk_destroy(t);
        return MUMMU_ERR_DEVICE;
    }
    *out = t;
    return MUMMU_OK;
}

int32_t mummu_trunk_destroy(MummuTrunk* t) {
    if (!t) return MUMMU_OK;
    {
        TrunkDevice guard(t->cfg.device);
        if (t->stream) cudaStreamSynchronize(t->stream);
        cudaFree(t->embed); cudaFree(t->lm_head); cudaFree(t->final_norm); cudaFree(t->norms); cudaFree(t->wqkv);
        cudaFree(t->wo); cudaFree(t->kc); cudaFree(t->vc); cudaFree(t->rope_cos); cudaFree(t->rope_sin); cudaFree(t->h);
        cudaFree(t->part); cudaFree(t->q); cudaFree(t->ctx); cudaFree(t->apart);
        if (t->stream) cudaStreamDestroy(t->stream);
    }
    delete t;
    return MUMMU_OK;
}

int32_t mummu_trunk_set_weight(MummuTrunk* t, int32_t which, int32_t layer, const void* data, size_t bytes,
                               int32_t on_device) {
    MUMMU_REQUIRE(t && data, "mummu_trunk_set_weight: null argument");
    MUMMU_REQUIRE(which >= MUMMU_TRUNK_EMBED && which <= MUMMU_TRUNK_K_NORM, "mummu_trunk_set_weight: weight %d", which);
    const MummuTrunkConfig& c = t->cfg;
    const bool per_layer = which >= MUMMU_TRUNK_IN_NORM;
    MUMMU_REQUIRE(!per_layer || (layer >= 0 && layer < c.layers), "mummu_trunk_set_weight: layer %d of %d", layer, c.layers);
    const bool is_norm = which == MUMMU_TRUNK_FINAL_NORM || which == MUMMU_TRUNK_IN_NORM || which == MUMMU_TRUNK_POST_NORM ||
                         which == MUMMU_TRUNK_Q_NORM || which == MUMMU_TRUNK_K_NORM;
    const size_t elems = trunk_weight_elems(c, which);
    const size_t want = elems * (is_norm ? 4 : 2);
    MUMMU_REQUIRE(bytes == want, "mummu_trunk_set_weight: weight %d needs %zu bytes (%s), got %zu", which, want,
                  is_norm ? "f32" : "f16", bytes);
    std::lock_guard<std::mutex> lock(t->mu);
    TrunkDevice guard(c.device);
    const size_t H = c.hidden, nq = (size_t)c.heads * c.head_dim, nkv = (size_t)c.kv_heads * c.head_dim;
    const size_t nqkv = nq + 2 * nkv, nstride = std::max(H, nq);
    void* dst = nullptr;
    switch (which) {
        case MUMMU_TRUNK_EMBED: dst = t->embed; break;
        case MUMMU_TRUNK_LM_HEAD: dst = t->lm_head; break;
        case MUMMU_TRUNK_FINAL_NORM: dst = t->final_norm; break;
        case MUMMU_TRUNK_IN_NORM: dst = t->norms + ((size_t)layer * 4 + 0) * nstride; break;
        case MUMMU_TRUNK_POST_NORM: dst = t->norms + ((size_t)layer * 4 + 1) * nstride; break;
        case MUMMU_TRUNK_Q_NORM: dst = t->norms + ((size_t)layer * 4 + 2) * nstride; break;
        case MUMMU_TRUNK_K_NORM: dst = t->norms + ((size_t)layer * 4 + 3) * nstride; break;
        case MUMMU_TRUNK_Q: dst = t->wqkv + (size_t)layer * nqkv * H; break;
        case MUMMU_TRUNK_K: dst = t->wqkv + (size_t)layer * nqkv * H + nq * H; break;
        case MUMMU_TRUNK_V: dst = t->wqkv + (size_t)layer * nqkv * H + (nq + nkv) * H; break;
        case MUMMU_TRUNK_O: dst = t->wo + (size_t)layer * H * nq; break;
    }
    MUMMU_CUDA_TRY(cudaDeviceSynchronize());
    MUMMU_CUDA_TRY(cudaMemcpy(dst, data, bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    MUMMU_CUDA_TRY(cudaDeviceSynchronize());
    return MUMMU_OK;
}

int32_t mummu_trunk_embed(MummuTrunk* t, const int32_t* tokens, int32_t slots, void* x, void* stream) {
    MUMMU_REQUIRE(t && tokens && x, "mummu_trunk_embed: null argument");
    MUMMU_REQUIRE(slots >= 1 && slots <= t->cfg.slots, "mummu_trunk_embed: %d slots of %d", slots, t->cfg.slots);
    std::lock_guard<std::mutex> lock(t->mu);
    TrunkDevice guard(t->cfg.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : t->stream;
    TrunkLaunch l(t);
    embed_kernel<<<slots, 256, 0, s>>>(t->embed, tokens, (__half*)x, t->cfg.hidden, t->cfg.vocab);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

int32_t mummu_trunk_attention_step(MummuTrunk* t, int32_t layer, void* x, const void* y_prev, const int32_t* positions,
                                   int32_t slots, int32_t key_len, void* h2, void* stream) {
    MUMMU_REQUIRE(t && x && positions && h2, "mummu_trunk_attention_step: null argument");
    const MummuTrunkConfig& c = t->cfg;
    MUMMU_REQUIRE(layer >= 0 && layer < c.layers, "mummu_trunk_attention_step: layer %d of %d", layer, c.layers);
    MUMMU_REQUIRE(slots >= 1 && slots <= c.slots, "mummu_trunk_attention_step: %d slots of %d", slots, c.slots);
    MUMMU_REQUIRE(key_len >= 1 && key_len <= c.max_ctx, "mummu_trunk_attention_step: key_len %d of %d", key_len, c.max_ctx);
    std::lock_guard<std::mutex> lock(t->mu);
    TrunkDevice guard(c.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : t->stream;
    const int H = c.hidden, nq = c.heads * c.head_dim, nkv = c.kv_heads * c.head_dim, nqkv = nq + 2 * nkv;
    const size_t nstride = (size_t)std::max(H, nq);
    const float* g_in = t->norms + ((size_t)layer * 4 + 0) * nstride;
    const float* g_post = t->norms + ((size_t)layer * 4 + 1) * nstride;
    const float* g_q = t->norms + ((size_t)layer * 4 + 2) * nstride;
    const float* g_k = t->norms + ((size_t)layer * 4 + 3) * nstride;
    int rc;
    {   // x += y_prev (the previous layer's expert bank joins the residual stream); h = rmsnorm(x) * gamma_in
        TrunkLaunch l(t);
        MUMMU_CUDA_TRY(allow_big_smem(add_rms_kernel, c.device));
        add_rms_kernel<<<slots, 512, (size_t)H * 4, s>>>((__half*)x, (const __half*)y_prev, g_in, t->h, H, c.rms_eps);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    const int ks_qkv = H >= 2048 ? 4 : (H >= 1024 ? 2 : 1);
    if ((rc = gemv(t, t->wqkv + (size_t)layer * nqkv * H, t->h, t->part, nqkv, H, ks_qkv, slots, s))) return rc;
    const size_t kv_layer = (size_t)c.slots * c.kv_heads * c.max_ctx * c.head_dim;
    __half* kc = t->kc + (size_t)layer * kv_layer;
    __half* vc = t->vc + (size_t)layer * kv_layer;
    {
        TrunkLaunch l(t);
        MUMMU_CUDA_TRY(allow_big_smem(qk_norm_rope_kernel, c.device));
        qk_norm_rope_kernel<<<dim3(slots, 3), 512, (size_t)std::max(nq, nkv) * 4, s>>>(t->part, ks_qkv, slots, g_q, g_k, t->rope_cos, t->rope_sin,
                                                                 positions, t->q, kc, vc, c.heads, c.kv_heads, c.head_dim,
                                                                 c.max_ctx, c.rms_eps);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    // key splits: enough blocks to fill the GPU when few sequences decode, chunks of at most 1024 keys
    int splits = (8 * 148 + slots * c.heads - 1) / (slots * c.heads);
    splits = std::max(splits, (key_len + 1023) / 1024);
    splits = std::min(std::min(splits, TR_MAX_SPLITS), std::max(1, key_len / 32));
    const int chunk = (key_len + splits - 1) / splits;
    MUMMU_REQUIRE(chunk <= 8192, "mummu_trunk_attention_step: %d keys need more than %d splits", key_len, TR_MAX_SPLITS);
    {
        TrunkLaunch l(t);
        MUMMU_CUDA_TRY(allow_big_smem(decode_attn_kernel, c.device));
        decode_attn_kernel<<<dim3(c.heads, slots, splits), 128, (size_t)(4 * c.head_dim + chunk) * 4, s>>>(
            t->q, kc, vc, positions, t->apart, c.heads, c.kv_heads, c.head_dim, c.max_ctx, key_len, splits,
            1.0f / sqrtf((float)c.head_dim));
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    {
        TrunkLaunch l(t);
        attn_combine_kernel<<<dim3(c.heads, slots), 128, 0, s>>>(t->apart, t->ctx, c.heads, c.head_dim, splits);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    const int ks_o = nq >= 2048 ? 8 : (nq >= 1024 ? 4 : 1);
    if ((rc = gemv(t, t->wo + (size_t)layer * H * nq, t->ctx, t->part, H, nq, ks_o, slots, s))) return rc;
    {
        TrunkLaunch l(t);
        MUMMU_CUDA_TRY(allow_big_smem(residual_rms_kernel, c.device));
        residual_rms_kernel<<<slots, 512, (size_t)H * 4, s>>>((__half*)x, t->part, ks_o, slots, g_post, (__half*)h2, H, c.rms_eps);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    return MUMMU_OK;
}

int32_t mummu_trunk_head(MummuTrunk* t, void* x, const void* y_prev, int32_t slots, float* logits, int32_t* argmax,
                         void* stream) {
    MUMMU_REQUIRE(t && x && logits, "mummu_trunk_head: null argument (logits are always written)");
    const MummuTrunkConfig& c = t->cfg;
    MUMMU_REQUIRE(slots >= 1 && slots <= c.slots, "mummu_trunk_head: %d slots of %d", slots, c.slots);
    std::lock_guard<std::mutex> lock(t->mu);
    TrunkDevice guard(c.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : t->stream;
    int rc;
    {
        TrunkLaunch l(t);
        MUMMU_CUDA_TRY(allow_big_smem(add_rms_kernel, c.device));
        add_rms_kernel<<<slots, 512, (size_t)c.hidden * 4, s>>>((__half*)x, (const __half*)y_prev, t->final_norm, t->h, c.hidden,
                                                                c.rms_eps);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    if ((rc = gemv(t, t->lm_head, t->h, logits, c.vocab, c.hidden, 1, slots, s))) return rc;
    if (argmax) {
        TrunkLaunch l(t);
        argmax_kernel<<<slots, 1024, 0, s>>>(logits, c.vocab, argmax);
        MUMMU_CUDA_TRY(cudaGetLastError());
    }
    return MUMMU_OK;
}

int32_t mummu_trunk_kv_write(MummuTrunk* t, int32_t layer, int32_t slot, int32_t first, int32_t count, const void* k,
                             const void* v, void* stream) {
    MUMMU_REQUIRE(t && k && v, "mummu_trunk_kv_write: null argument");
    const MummuTrunkConfig& c = t->cfg;
    MUMMU_REQUIRE(layer >= 0 && layer < c.layers && slot >= 0 && slot < c.slots && first >= 0 && count >= 0 &&
                      first + count <= c.max_ctx,
                  "mummu_trunk_kv_write: layer %d, slot %d, positions [%d, %d) of %d", layer, slot, first, first + count,
                  c.max_ctx);
    if (count == 0) return MUMMU_OK;
    std::lock_guard<std::mutex> lock(t->mu);
    TrunkDevice guard(c.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : t->stream;
    const size_t kv_layer = (size_t)c.slots * c.kv_heads * c.max_ctx * c.head_dim;
    TrunkLaunch l(t);
    kv_write_kernel<<<148, 256, 0, s>>>((const __half*)k, (const __half*)v, t->kc + (size_t)layer * kv_layer,
                                        t->vc + (size_t)layer * kv_layer, c.kv_heads, c.head_dim, c.max_ctx, slot, first, count);
    MUMMU_CUDA_TRY(cudaGetLastError());
    return MUMMU_OK;
}

}  // extern "C"
