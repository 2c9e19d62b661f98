/*
 * mummu_oracle.c — CPU restatement of the reference's sparse-MoE expert bank.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT.  Only the tests, the smoke check and the benchmark's CPU
 * baseline leg may call this file; the CUDA library never does.
 *
 * The reference (physics515/Mummu, Rust on the burn tensor library) cannot be compiled where this
 * is built (no Rust toolchain, burn/gemm/half crates not vendored), so each function restates the
 * reference's algorithm from its source and cites the lines it follows (paths are relative to
 * `crates/mummu/src/` in the reference tree).
 *
 * What is pinned and what is not:
 *  - Q4_K decoding is pinned by the reference's known-answer super-block (gguf.rs:2408-2429) and
 *    cross-checked against the `gguf` Python package where that is installed.
 *  - Router selection and tie order are pinned by the reference's router tests
 *    (models/qwen4exp/experts.rs:1366-1408).
 *  - The layer as a whole is pinned only as far as the reference pins it: its tests recompute the
 *    expected output with a scalar loop (nn/moe.rs:2101-2175) at 1e-5; that loop is restated here
 *    (orc_moe_routed with ORC_SUM_SEQUENTIAL).  PARITY UNPINNED for what lives inside burn 0.22.0-pre.3 /
 *    gemm 0.19.0: the summation order of its matmul, the rounding of its `exp`, and the order
 *    `topk_with_indices` gives exactly equal probabilities.  This file fixes those three choices:
 *    dot products use the reference's own fixed 8-lane order (models/qwen4exp/experts.rs:463-478;
 *    the router's lanes step with a fused multiply-add, as the gemm crate behind burn's Linear does),
 *    the softmax exponential is orc_exp below (same IEEE operation sequence on CPU and GPU, within
 *    1 ulp of the true value), ties go to the lowest expert id (experts.rs:532-535, 564-573).
 *
 * Build: see the Makefile beside this file (-ffp-contract=off is required: the reference rounds
 * products and sums separately wherever it says "two roundings on purpose").
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_OK 0
#define ORC_ERR_ARG 1
#define ORC_ERR_NONFINITE 5

/* ------------------------------------------------------------------------------------------ */
/* half precision                                                                              */
/* ------------------------------------------------------------------------------------------ */

/* IEEE 754 binary16 -> binary32, every bit pattern (gguf.rs:1464-1468 does this through the
 * `half` crate; the conversion is exact so there is only one right answer). */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int shift = 0;
            while ((man & 0x400u) == 0) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

float orc_bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* ------------------------------------------------------------------------------------------ */
/* GGUF Q4_K                                                                                    */
/* ------------------------------------------------------------------------------------------ */

/* The 6-bit (scale, min) pair of sub-block j — gguf.rs:1685-1698 (`scale_min_k4`). */
static void scale_min_k4(const uint8_t* scales, int j, float* sc, float* m) {
    uint8_t s, mn;
    if (j < 4) {
        s = scales[j] & 63;
        mn = scales[j + 4] & 63;
    } else {
        s = (uint8_t)((scales[j + 4] & 0x0F) | ((scales[j - 4] >> 6) << 4));
        mn = (uint8_t)((scales[j + 4] >> 4) | ((scales[j] >> 6) << 4));
    }
    *sc = (float)s;
    *m = (float)mn;
}

/* One 144-byte super-block -> 256 f32 — gguf.rs:1701-1726 (`dequant_q4_k`).
 * x = d*sc*q - dmin*m: `d*sc` first, then `*q`, each rounded to f32; the min product `dmin*m`
 * rounded on its own; then one subtraction.  Chunk c (64 values) reads 32 bytes: the 32 low
 * nibbles with sub-block 2c's pair, then the 32 high nibbles with sub-block 2c+1's. */
void orc_dequant_q4_k(const uint8_t* block, float* out) {
    float d = orc_f16_to_f32((uint16_t)(block[0] | (block[1] << 8)));
    float dmin = orc_f16_to_f32((uint16_t)(block[2] | (block[3] << 8)));
    const uint8_t* scales = block + 4;
    const uint8_t* qs = block + 16;
    for (int chunk = 0; chunk < 4; ++chunk) {
        float sc1, m1, sc2, m2;
        scale_min_k4(scales, chunk * 2, &sc1, &m1);
        scale_min_k4(scales, chunk * 2 + 1, &sc2, &m2);
        const uint8_t* q = qs + chunk * 32;
        float min1 = dmin * m1;
        float min2 = dmin * m2;
        float ds1 = d * sc1;
        float ds2 = d * sc2;
        for (int b = 0; b < 32; ++b) {
            float product = ds1 * (float)(q[b] & 0x0F);
            out[chunk * 64 + b] = product - min1;
        }
        for (int b = 0; b < 32; ++b) {
            float product = ds2 * (float)(q[b] >> 4);
            out[chunk * 64 + 32 + b] = product - min2;
        }
    }
}

/* Whole blocks, in order — gguf.rs:1442-1461 (`dequantize` over `chunks_exact`). */
void orc_dequant_q4_k_blocks(const uint8_t* bytes, int64_t n_blocks, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < n_blocks; ++b) orc_dequant_q4_k(bytes + b * 144, out + b * 256);
}

/* Q8_0 — gguf.rs:1535-1543: 34 bytes = f16 d + 32 i8; x = d * q. */
void orc_dequant_q8_0(const uint8_t* block, float* out) {
    float d = orc_f16_to_f32((uint16_t)(block[0] | (block[1] << 8)));
    for (int i = 0; i < 32; ++i) out[i] = d * (float)(int8_t)block[2 + i];
}

/* Q5_K — gguf.rs:1731-1765: 176 bytes = f16 d, f16 dmin, 12 B packed 6-bit (scale, min) pairs,
 * 32 B of fifth bits, 128 B of nibbles.  Chunk c (64 values) reads 32 nibble bytes (low nibbles
 * first) and bit planes 2c (low nibbles) and 2c+1 (high nibbles) of the shared 32 bytes;
 * x = d*sc*(q + 16*bit) - dmin*m with the products rounded as in Q4_K. */
void orc_dequant_q5_k(const uint8_t* block, float* out) {
    float d = orc_f16_to_f32((uint16_t)(block[0] | (block[1] << 8)));
    float dmin = orc_f16_to_f32((uint16_t)(block[2] | (block[3] << 8)));
    const uint8_t* scales = block + 4;
    const uint8_t* qh = block + 16;
    const uint8_t* qs = block + 48;
    uint8_t u1 = 1, u2 = 2;
    for (int chunk = 0; chunk < 4; ++chunk) {
        float sc1, m1, sc2, m2;
        scale_min_k4(scales, chunk * 2, &sc1, &m1);
        scale_min_k4(scales, chunk * 2 + 1, &sc2, &m2);
        const uint8_t* q = qs + chunk * 32;
        float min1 = dmin * m1;
        float min2 = dmin * m2;
        for (int b = 0; b < 32; ++b) {
            int top = (qh[b] & u1) ? 16 : 0;
            float ds = d * sc1;
            float product = ds * (float)((q[b] & 0x0F) + top);
            out[chunk * 64 + b] = product - min1;
        }
        for (int b = 0; b < 32; ++b) {
            int top = (qh[b] & u2) ? 16 : 0;
            float ds = d * sc2;
            float product = ds * (float)((q[b] >> 4) + top);
            out[chunk * 64 + 32 + b] = product - min2;
        }
        u1 = (uint8_t)(u1 << 2);
        u2 = (uint8_t)(u2 << 2);
    }
}

/* Q6_K — gguf.rs:1769-1797: 210 bytes = 128 B low nibbles, 64 B high bit pairs, 16 i8 sub-scales,
 * f16 d; two halves of 128 values; x = d * s * (q - 32), `d*s` first. */
void orc_dequant_q6_k(const uint8_t* block, float* out) {
    const uint8_t* lows = block;
    const uint8_t* highs = block + 128;
    const uint8_t* scales = block + 192;
    float d = orc_f16_to_f32((uint16_t)(block[208] | (block[209] << 8)));
    for (int h = 0; h < 2; ++h) {
        const uint8_t* ql = lows + h * 64;
        const uint8_t* qh = highs + h * 32;
        const uint8_t* sc = scales + h * 8;
        float* y = out + h * 128;
        for (int l = 0; l < 32; ++l) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 0x0F) | ((qh[l] & 3) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            float s0 = d * (float)(int8_t)sc[is], s2 = d * (float)(int8_t)sc[is + 2];
            float s4 = d * (float)(int8_t)sc[is + 4], s6 = d * (float)(int8_t)sc[is + 6];
            y[l] = s0 * (float)q1;
            y[l + 32] = s2 * (float)q2;
            y[l + 64] = s4 * (float)q3;
            y[l + 96] = s6 * (float)q4;
        }
    }
}

/* kind: 4 = Q8_0, 5 = Q5_K, 6 = Q6_K, 3 = Q4_K (the codes of the C ABI's weight dtypes) */
int orc_dequant_blocks(int kind, const uint8_t* bytes, int64_t n_blocks, float* out) {
    if (kind != 3 && kind != 4 && kind != 5 && kind != 6) return 1;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < n_blocks; ++b) {
        if (kind == 3) orc_dequant_q4_k(bytes + b * 144, out + b * 256);
        else if (kind == 4) orc_dequant_q8_0(bytes + b * 34, out + b * 32);
        else if (kind == 5) orc_dequant_q5_k(bytes + b * 176, out + b * 256);
        else orc_dequant_q6_k(bytes + b * 210, out + b * 256);
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* scalar pieces                                                                               */
/* ------------------------------------------------------------------------------------------ */

/* Inner product in the reference's fixed 8-lane order — models/qwen4exp/experts.rs:463-478:
 * lane l accumulates elements l, l+8, ... (product and sum rounded separately), the lanes fold as
 * ((a0+a4)+(a1+a5))+((a2+a6)+(a3+a7)), the <8 leftover elements are added one by one. */
float orc_dot8(const float* a, const float* b, int64_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t chunks = n / 8;
    for (int64_t c = 0; c < chunks; ++c) {
        for (int l = 0; l < 8; ++l) {
            float p = a[c * 8 + l] * b[c * 8 + l];
            acc[l] = acc[l] + p;
        }
    }
    float s = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
    for (int64_t i = chunks * 8; i < n; ++i) {
        float p = a[i] * b[i];
        s = s + p;
    }
    return s;
}

/* The router's inner product: the same 8 lanes and the same fold as orc_dot8, but each lane step
 * is ONE fused multiply-add.  The reference computes router logits with burn's `Linear`
 * (nn/moe.rs:139, 255), i.e. the `gemm` crate's matmul (0.19.0, not in the tree), whose x86
 * microkernels are built on fused multiply-add; the summation order inside it cannot be read
 * here (parity unpinned), so the lane order of the reference's own `dot`
 * (models/qwen4exp/experts.rs:463-478) is kept and only the rounding per step follows gemm. */
float orc_dot8_fma(const float* a, const float* b, int64_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int64_t chunks = n / 8;
    for (int64_t c = 0; c < chunks; ++c)
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(a[c * 8 + l], b[c * 8 + l], acc[l]);
    float s = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
    for (int64_t i = chunks * 8; i < n; ++i) s = fmaf(a[i], b[i], s);
    return s;
}

/* Plain left-to-right inner product — the reference tests' scalar loop
 * (`(0..HIDDEN).map(|i| x[i]*w[i]).sum()`, nn/moe.rs:2136, 2156-2167). */
static float dot_seq(const float* a, const float* b, int64_t n, int64_t stride_b) {
    float s = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        float p = a[i] * b[i * stride_b];
        s = s + p;
    }
    return s;
}

/* x * sigmoid(x) written as x / (1 + e^-x) — nn/moe.rs:2095-2097, experts.rs:484-487. */
float orc_silu(float x) { return x / (1.0f + expf(-x)); }

/* e^x for the softmax, x <= 0 in use.  The reference calls burn's softmax, whose exponential is
 * not in the tree; this one is a fixed sequence of IEEE-754 single operations (fused multiply-adds
 * spelled out), so the CUDA router evaluates it bit for bit the same way and routing can be
 * compared exactly.  n = round(x*log2 e); r = x - n*ln2 (two-term Cody-Waite); Taylor degree 7 on
 * |r| <= 0.347 (truncation 5e-9 relative); scale by 2^n in two exact-or-once-rounded steps so
 * subnormal results round once.  Within 1 ulp of expf over [-104, 0] (tests check this). */
float orc_exp(float x) {
    if (x != x) return x;
    if (x > 88.7f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    const float LOG2E = 1.4426950216293335f;   /* 0x3FB8AA3B */
    const float LN2_HI = 0.693145751953125f;   /* 0x3F317200: 15 significant bits, n*LN2_HI exact */
    const float LN2_LO = 1.4286068203094172e-06f; /* ln2 - LN2_HI */
    const float MAGIC = 12582912.0f;           /* 1.5 * 2^23: adding it rounds to an integer */
    float t = fmaf(x, LOG2E, MAGIC);
    float n = t - MAGIC;
    float r = fmaf(-n, LN2_HI, x);
    r = fmaf(-n, LN2_LO, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int ni = (int)n;
    /* 2^ni split as 2^a * 2^b with both factors normal floats */
    int a = ni / 2;
    int b = ni - a;
    uint32_t ba = (uint32_t)(a + 127) << 23;
    uint32_t bb = (uint32_t)(b + 127) << 23;
    float fa, fb;
    memcpy(&fa, &ba, 4);
    memcpy(&fb, &bb, 4);
    float y = p * fa; /* exact: p in [0.7, 1.42], fa a power of two >= 2^-76 */
    return y * fb;    /* rounds once, only if the result is subnormal */
}

/* ------------------------------------------------------------------------------------------ */
/* router                                                                                      */
/* ------------------------------------------------------------------------------------------ */

/* logits[t, e] = x[t, :] . W[:, e] (+ bias[e]) — `self.gate.forward(xt)` (nn/moe.rs:139, 255).
 * w is [hidden, experts] row-major (burn Linear [in, out], nn/moe.rs:1642-1646).
 * order: 0 = 8 fused-multiply-add lanes (orc_dot8_fma; what the CUDA router is compared against),
 * 1 = left to right with separate roundings (the reference tests' scalar loop, nn/moe.rs:2136). */
#define ORC_SUM_LANES8 0
#define ORC_SUM_SEQUENTIAL 1

void orc_router_logits(const float* x, const float* w, const float* bias, int64_t tokens,
                       int64_t hidden, int64_t experts, int order, float* logits) {
    /* transpose W once so each expert's column is contiguous */
    float* wt = (float*)malloc(sizeof(float) * (size_t)(hidden * experts));
    for (int64_t i = 0; i < hidden; ++i)
        for (int64_t e = 0; e < experts; ++e) wt[e * hidden + i] = w[i * experts + e];
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tokens; ++t) {
        for (int64_t e = 0; e < experts; ++e) {
            float l = order == ORC_SUM_LANES8 ? orc_dot8_fma(x + t * hidden, wt + e * hidden, hidden)
                                              : dot_seq(x + t * hidden, wt + e * hidden, hidden, 1);
            if (bias) l = l + bias[e];
            logits[t * experts + e] = l;
        }
    }
    free(wt);
}

/* Softmax over ALL experts in f32, then the top_k PROBABILITIES, optional renormalisation —
 * nn/moe.rs:144-150 and 256-262; scalar form nn/moe.rs:2138-2152 (shift by the max, exp, divide by
 * the left-to-right sum; weights = p / (sum of the picked p, in slot order) when renormalising).
 * Selection: descending probability, equal probabilities in ascending expert id, a tie at the
 * boundary keeps the lower id — models/qwen4exp/experts.rs:532-535, 562-574.  Slots come out in
 * descending probability.  Non-finite logits are refused (experts.rs:553-560): returns
 * ORC_ERR_NONFINITE and writes the offending flat index to *bad_index.
 * exp_kind: 0 = orc_exp (what the CUDA router is compared against), 1 = libm expf. */
int orc_route(const float* logits, int64_t tokens, int64_t experts, int64_t top_k,
              int norm_topk_prob, int exp_kind, int32_t* ids, float* weights, int64_t* bad_index) {
    if (experts <= 0 || top_k <= 0 || top_k > experts) return ORC_ERR_ARG;
    for (int64_t i = 0; i < tokens * experts; ++i) {
        if (!isfinite(logits[i])) {
            if (bad_index) *bad_index = i;
            return ORC_ERR_NONFINITE;
        }
    }
    int status = ORC_OK;
#pragma omp parallel
    {
        float* probs = (float*)malloc(sizeof(float) * (size_t)experts);
        float* best_p = (float*)malloc(sizeof(float) * (size_t)(top_k + 1));
        int32_t* best_id = (int32_t*)malloc(sizeof(int32_t) * (size_t)(top_k + 1));
#pragma omp for schedule(static)
        for (int64_t t = 0; t < tokens; ++t) {
            const float* row = logits + t * experts;
            float mx = row[0];
            for (int64_t e = 1; e < experts; ++e) mx = row[e] > mx ? row[e] : mx;
            float total = 0.0f;
            for (int64_t e = 0; e < experts; ++e) {
                float v = exp_kind == 0 ? orc_exp(row[e] - mx) : expf(row[e] - mx);
                probs[e] = v;
                total = total + v;
            }
            for (int64_t e = 0; e < experts; ++e) probs[e] = probs[e] / total;
            /* (prob, id) list, descending prob then ascending id, at most top_k long */
            int64_t len = 0;
            for (int64_t e = 0; e < experts; ++e) {
                float p = probs[e];
                if (len == top_k && p <= best_p[top_k - 1]) continue;
                int64_t pos = 0;
                while (pos < len && best_p[pos] >= p) ++pos; /* partition_point(q >= p) */
                for (int64_t j = len; j > pos; --j) {
                    best_p[j] = best_p[j - 1];
                    best_id[j] = best_id[j - 1];
                }
                best_p[pos] = p;
                best_id[pos] = (int32_t)e;
                if (len < top_k) ++len;
            }
            float denom = 1.0f;
            if (norm_topk_prob) {
                denom = 0.0f;
                for (int64_t s = 0; s < top_k; ++s) denom = denom + best_p[s];
            }
            for (int64_t s = 0; s < top_k; ++s) {
                ids[t * top_k + s] = best_id[s];
                weights[t * top_k + s] = norm_topk_prob ? best_p[s] / denom : best_p[s];
            }
        }
        free(probs);
        free(best_p);
        free(best_id);
    }
    return status;
}

/* ------------------------------------------------------------------------------------------ */
/* experts                                                                                     */
/* ------------------------------------------------------------------------------------------ */

/* out[r, o] = dot(w[o, :], x[r, :]) for `rows` rows; w is [out_dim, in_dim] row-major — the
 * per-row kernel of models/qwen4exp/experts.rs:401-457 (`matvec_rows`: output (t, r) is
 * dot(row r, x_t) whatever the chunking). */
static void matvec_rows(const float* w, int64_t out_dim, int64_t in_dim, const float* x,
                        int64_t rows, int order, float* out) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t o = 0; o < out_dim; ++o)
            out[r * out_dim + o] = order == ORC_SUM_LANES8
                                       ? orc_dot8(w + o * in_dim, x + r * in_dim, in_dim)
                                       : dot_seq(x + r * in_dim, w + o * in_dim, in_dim, 1);
}

/* One expert's SwiGLU on `rows` rows: down(silu(gate x) * (up x)) — nn/moe.rs:314-316, 455-457;
 * models/qwen4exp/experts.rs:781-806 (`ffn`).  gate, up: [inter, hidden]; down: [hidden, inter]
 * (the bank slices of nn/moe.rs:24-29).  y: [rows, hidden]. */
void orc_expert_ffn(const float* gate, const float* up, const float* down, int64_t hidden,
                    int64_t inter, const float* x, int64_t rows, int order, float* y) {
    float* g = (float*)malloc(sizeof(float) * (size_t)(rows * inter));
    float* u = (float*)malloc(sizeof(float) * (size_t)(rows * inter));
    matvec_rows(gate, inter, hidden, x, rows, order, g);
    matvec_rows(up, inter, hidden, x, rows, order, u);
    for (int64_t i = 0; i < rows * inter; ++i) g[i] = orc_silu(g[i]) * u[i];
    matvec_rows(down, hidden, inter, g, rows, order, y);
    free(g);
    free(u);
}

/* Routed bank: group rows per expert (token-major, nn/moe.rs:275-285), run each non-empty expert
 * once in ascending id on its rows (nn/moe.rs:301-316), scatter-add `scaled = w*y; out += scaled`
 * with two roundings in ascending expert id (nn/moe.rs:317-325, 1589-1602;
 * models/qwen4exp/experts.rs:1137-1148).
 * Weights are f32 banks [experts, out, in] (q4k == 0) or Q4_K bytes (q4k != 0, rows of in/256
 * super-blocks of 144 B, dequantised per expert first: experts.rs:430-437).
 * hits (may be NULL): rows served per expert are added (nn/moe.rs:1562-1564). */
int orc_moe_routed(const float* x, const int32_t* ids, const float* weights, int64_t tokens,
                   int64_t top_k, int64_t hidden, int64_t inter, int64_t experts,
                   const void* gate, const void* up, const void* down, int q4k, int order,
                   float* out, uint64_t* hits) {
    if (q4k && (hidden % 256 != 0 || inter % 256 != 0)) return ORC_ERR_ARG;
    for (int64_t i = 0; i < tokens * top_k; ++i)
        if (ids[i] < 0 || ids[i] >= experts) return ORC_ERR_ARG;
    int64_t* count = (int64_t*)calloc((size_t)experts + 1, sizeof(int64_t));
    for (int64_t i = 0; i < tokens * top_k; ++i) count[ids[i] + 1]++;
    for (int64_t e = 0; e < experts; ++e) count[e + 1] += count[e];
    int64_t total = tokens * top_k;
    int64_t* row_tok = (int64_t*)malloc(sizeof(int64_t) * (size_t)(total ? total : 1));
    float* row_w = (float*)malloc(sizeof(float) * (size_t)(total ? total : 1));
    int64_t* fill = (int64_t*)calloc((size_t)experts, sizeof(int64_t));
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t s = 0; s < top_k; ++s) {
            int64_t e = ids[t * top_k + s];
            int64_t p = count[e] + fill[e]++;
            row_tok[p] = t;
            row_w[p] = weights[t * top_k + s];
        }
    float* ys = (float*)malloc(sizeof(float) * (size_t)((total ? total : 1) * hidden));
    size_t bank_elems = (size_t)(inter * hidden);
    size_t bank_bytes_q = (size_t)(inter * hidden / 256 * 144);
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t e = 0; e < experts; ++e) {
        int64_t n = count[e + 1] - count[e];
        if (n == 0) continue;
        float* xe = (float*)malloc(sizeof(float) * (size_t)(n * hidden));
        for (int64_t i = 0; i < n; ++i)
            memcpy(xe + i * hidden, x + row_tok[count[e] + i] * hidden, sizeof(float) * (size_t)hidden);
        const float *g, *u, *d;
        float* tmp = NULL;
        if (q4k) {
            tmp = (float*)malloc(sizeof(float) * bank_elems * 3);
            int64_t nb = inter * hidden / 256;
            for (int64_t b = 0; b < nb; ++b) {
                orc_dequant_q4_k((const uint8_t*)gate + e * bank_bytes_q + b * 144, tmp + b * 256);
                orc_dequant_q4_k((const uint8_t*)up + e * bank_bytes_q + b * 144, tmp + bank_elems + b * 256);
                orc_dequant_q4_k((const uint8_t*)down + e * bank_bytes_q + b * 144, tmp + 2 * bank_elems + b * 256);
            }
            g = tmp;
            u = tmp + bank_elems;
            d = tmp + 2 * bank_elems;
        } else {
            g = (const float*)gate + e * bank_elems;
            u = (const float*)up + e * bank_elems;
            d = (const float*)down + e * bank_elems;
        }
        orc_expert_ffn(g, u, d, hidden, inter, xe, n, order, ys + count[e] * hidden);
        free(xe);
        free(tmp);
    }
    memset(out, 0, sizeof(float) * (size_t)(tokens * hidden));
    for (int64_t e = 0; e < experts; ++e) {
        if (hits) hits[e] += (uint64_t)(count[e + 1] - count[e]);
        for (int64_t p = count[e]; p < count[e + 1]; ++p) {
            float w = row_w[p];
            float* dst = out + row_tok[p] * hidden;
            const float* y = ys + p * hidden;
            for (int64_t i = 0; i < hidden; ++i) {
                float scaled = w * y[i];
                dst[i] = dst[i] + scaled;
            }
        }
    }
    free(count);
    free(row_tok);
    free(row_w);
    free(fill);
    free(ys);
    return ORC_OK;
}

/* Dense-mask bank — nn/moe.rs:151-177: the sparse weight row [tokens, experts] (zero where an
 * expert is not in the token's top_k), EVERY expert computes every token, and the outputs are
 * scaled and summed over experts in index order.  f32 banks only (what `LoadedOlmoe` runs). */
int orc_moe_dense_mask(const float* x, const int32_t* ids, const float* weights, int64_t tokens,
                       int64_t top_k, int64_t hidden, int64_t inter, int64_t experts,
                       const float* gate, const float* up, const float* down, int order,
                       float* out) {
    float* wrow = (float*)calloc((size_t)(tokens * experts), sizeof(float));
    for (int64_t t = 0; t < tokens; ++t)
        for (int64_t s = 0; s < top_k; ++s) {
            int64_t e = ids[t * top_k + s];
            if (e < 0 || e >= experts) { free(wrow); return ORC_ERR_ARG; }
            wrow[t * experts + e] = wrow[t * experts + e] + weights[t * top_k + s];
        }
    float* ys = (float*)malloc(sizeof(float) * (size_t)(experts * tokens * hidden));
    size_t bank_elems = (size_t)(inter * hidden);
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t e = 0; e < experts; ++e)
        orc_expert_ffn(gate + e * bank_elems, up + e * bank_elems, down + e * bank_elems, hidden,
                       inter, x, tokens, order, ys + e * tokens * hidden);
    memset(out, 0, sizeof(float) * (size_t)(tokens * hidden));
    for (int64_t e = 0; e < experts; ++e)
        for (int64_t t = 0; t < tokens; ++t) {
            float w = wrow[t * experts + e];
            const float* y = ys + (e * tokens + t) * hidden;
            float* dst = out + t * hidden;
            for (int64_t i = 0; i < hidden; ++i) {
                float scaled = y[i] * w;
                dst[i] = dst[i] + scaled;
            }
        }
    free(wrow);
    free(ys);
    return ORC_OK;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* The benchmark's reference arm sizes the pool itself: a launcher may have exported
 * OMP_NUM_THREADS=1 for every rank. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
