// extern "C" surface of the library: handle life cycle, weight upload, the layer call and its
// stages.  Declarations and the reference interface each call stands in for: include/mummu_cuda.h.
#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace mummu {

static thread_local std::string g_error;

void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
}

cudaError_t allow_big_smem_impl(const void* kernel, int device) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, bool> done;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_pair(kernel, device);
    if (done.count(key)) return cudaSuccess;
    int optin = 0;
    cudaError_t err = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (err != cudaSuccess) return err;
    cudaFuncAttributes fa;
    err = cudaFuncGetAttributes(&fa, kernel);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               optin - (int)fa.sharedSizeBytes);
    if (err == cudaSuccess) done[key] = true;
    return err;
}

size_t bank_row_bytes(const MummuMoeConfig& c, int which) {
    size_t in_dim = which == MUMMU_BANK_DOWN ? c.inter : c.hidden;
    switch (c.weight_dtype) {
        case MUMMU_Q4_K: return in_dim / Q4K_BLOCK_ELEMS * Q4K_BLOCK_BYTES;
        case MUMMU_Q8_0: return in_dim / Q80_BLOCK_ELEMS * Q80_BLOCK_BYTES;
        case MUMMU_Q5_K: return in_dim / 256 * Q5K_BLOCK_BYTES;
        case MUMMU_Q6_K: return in_dim / 256 * Q6K_BLOCK_BYTES;
        default: break;
    }
    return in_dim * dtype_size(c.weight_dtype);
}

size_t bank_total_bytes(const MummuMoeConfig& c, int which) {
    size_t out_dim = which == MUMMU_BANK_DOWN ? c.hidden : c.inter;
    return bank_row_bytes(c, which) * out_dim * (size_t)c.experts_local;
}

LaunchScope::LaunchScope(MummuMoe* m_, cudaStream_t s_, const char* name_) : m(m_), s(s_), name(name_) {
    m->launches += 1;
    if (!m->prof.enabled) return;
    auto take = [&]() {
        cudaEvent_t e;
        if (!m->prof.pool.empty()) {
            e = m->prof.pool.back();
            m->prof.pool.pop_back();
        } else {
            cudaEventCreate(&e);
        }
        return e;
    };
    a = take();
    b = take();
    cudaEventRecord(a, s);
}

LaunchScope::~LaunchScope() {
    if (!a) return;
    cudaEventRecord(b, s);
    m->prof.pending.push_back({name, a, b});
}

template <typename T>
static int dev_alloc(T** p, size_t n) {
    *p = nullptr;
    if (n == 0) n = 1;
    MUMMU_CUDA_TRY(cudaMalloc((void**)p, n * sizeof(T)));
    return MUMMU_OK;
}

static void free_scratch(MummuMoe* m) {
    if (m->scratch_borrowed) {
        m->logits = nullptr; m->tile_done = nullptr; m->ids = nullptr; m->wts = nullptr;
        m->row_token = nullptr; m->pos = nullptr; m->xs = nullptr; m->hact = nullptr; m->ys = nullptr;
        m->io_x = nullptr; m->io_y = nullptr;
        m->whist = nullptr;
        m->whist_elems = 0;
        m->cap_tokens = 0;
        m->scratch_borrowed = false;
        return;
    }
    cudaFree(m->logits); cudaFree(m->tile_done); cudaFree(m->ids); cudaFree(m->wts); cudaFree(m->whist);
    cudaFree(m->row_token); cudaFree(m->pos); cudaFree(m->xs); cudaFree(m->hact); cudaFree(m->ys);
    cudaFree(m->io_x); cudaFree(m->io_y);
    m->logits = nullptr; m->tile_done = nullptr; m->ids = nullptr; m->wts = nullptr; m->whist = nullptr;
    m->whist_elems = 0;
    m->row_token = nullptr; m->pos = nullptr; m->xs = nullptr; m->hact = nullptr; m->ys = nullptr;
    m->io_x = nullptr; m->io_y = nullptr;
    m->cap_tokens = 0;
}

void clear_host_graphs(MummuMoe* m) {
    for (auto& kv : m->host_graphs)
        if (kv.second) cudaGraphExecDestroy(kv.second);
    m->host_graphs.clear();
    m->host_calls.clear();
}

int ensure_scratch(MummuMoe* m, int64_t tokens) {
    if (tokens <= m->cap_tokens) return MUMMU_OK;
    clear_host_graphs(m);
    if (m->scratch_borrowed) {
        set_error("MoE: %lld tokens exceed the %lld the adopted scratch was sized for", (long long)tokens,
                  (long long)m->cap_tokens);
        return MUMMU_ERR_CONTRACT;
    }
    const MummuMoeConfig& c = m->cfg;
    MUMMU_CUDA_TRY(cudaStreamSynchronize(m->stream));
    MUMMU_CUDA_TRY(cudaDeviceSynchronize());
    free_scratch(m);
    int64_t T = tokens;
    int64_t rows = T * c.top_k;
    size_t act = dtype_size(c.act_dtype);
    int rc;
    if ((rc = dev_alloc(&m->logits, (size_t)T * c.experts))) return rc;
    if ((rc = dev_alloc(&m->tile_done, (size_t)T / 4 + 2))) return rc;
    MUMMU_CUDA_TRY(cudaMemset(m->tile_done, 0, ((size_t)T / 4 + 2) * sizeof(int32_t)));
    if ((rc = dev_alloc(&m->ids, (size_t)rows))) return rc;
    if ((rc = dev_alloc(&m->wts, (size_t)rows))) return rc;
    if ((rc = dev_alloc(&m->row_token, (size_t)rows))) return rc;
    m->whist_elems = ((rows + 2047) / 2048) * 8 * (int64_t)c.experts;
    if ((rc = dev_alloc(&m->whist, (size_t)m->whist_elems))) return rc;
    if ((rc = dev_alloc(&m->pos, (size_t)rows))) return rc;
    if ((rc = dev_alloc((uint8_t**)&m->xs, (size_t)rows * c.hidden * act))) return rc;
    if ((rc = dev_alloc((float**)&m->hact, (size_t)rows * c.inter))) return rc;
    if ((rc = dev_alloc((float**)&m->ys, (size_t)rows * c.hidden))) return rc;
    if ((rc = dev_alloc((uint8_t**)&m->io_x, (size_t)T * c.hidden * act))) return rc;
    if ((rc = dev_alloc((uint8_t**)&m->io_y, (size_t)T * c.hidden * act))) return rc;
    m->cap_tokens = T;
    return MUMMU_OK;
}

static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    if (!v) return dflt;
    return *v ? atoi(v) : 1;         // a variable set to the empty string counts as "on"
}

struct SwitchName {
    const char* name;
    int MummuSwitches::*field;
};
static const SwitchName kSwitches[] = {
    {"NO_TC", &MummuSwitches::no_tc},
    {"NO_HOST_GRAPH", &MummuSwitches::no_host_graph},
    {"ROUTER_PLAIN", &MummuSwitches::router_plain},
    {"DECODE_NO_PDL", &MummuSwitches::decode_no_pdl},
    {"DECODE_NT", &MummuSwitches::decode_nt},
    {"DECODE_STREAM_MIN", &MummuSwitches::decode_stream_min},
    {"DECODE_RB_GATEUP", &MummuSwitches::decode_rb_gateup},
    {"DECODE_RB_DOWN", &MummuSwitches::decode_rb_down},
    {"CHECKED", &MummuSwitches::checked},
};

static void switches_from_env(MummuSwitches& sw) {
    for (const SwitchName& e : kSwitches) {
        const std::string var = std::string("MUMMU_CUDA_") + e.name;
        sw.*(e.field) = env_int(var.c_str(), 0);
    }
    sw.wait_polls = (uint32_t)env_int("MUMMU_CUDA_WAIT_POLLS", 0);
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        int cur = -1;
        cudaGetDevice(&cur);
        if (prev >= 0 && cur != prev) cudaSetDevice(prev);
    }
};

static int check_ready(MummuMoe* m, bool need_router, bool need_banks) {
    if (need_router) MUMMU_REQUIRE(m->router_set, "MoE: router weight was never set (mummu_moe_set_router)");
    if (need_banks)
        MUMMU_REQUIRE(m->bank_set[0] && m->bank_set[1] && m->bank_set[2],
                      "MoE: expert banks were never set (mummu_moe_set_bank gate/up/down)");
    return MUMMU_OK;
}

static int check_top_k(const MummuMoe* m, int top_k) {
    MUMMU_REQUIRE(top_k >= 1 && top_k <= m->cfg.experts,
                  "MoE forward: top_k (%d) must be in 1..=num_experts (%d)", top_k, m->cfg.experts);
    MUMMU_REQUIRE(top_k <= m->cfg.top_k,
                  "MoE forward: top_k (%d) exceeds the num_experts_per_tok (%d) this handle was "
                  "created for", top_k, m->cfg.top_k);
    return MUMMU_OK;
}

static int read_status(MummuMoe* m, cudaStream_t s) {
    int32_t st = 0;
    if (m->status_host) {
        MUMMU_CUDA_TRY(cudaMemcpyAsync(m->status_host, m->status, sizeof(st), cudaMemcpyDeviceToHost, s));
        MUMMU_CUDA_TRY(cudaStreamSynchronize(s));
        st = *m->status_host;
    } else {
        MUMMU_CUDA_TRY(cudaMemcpyAsync(&st, m->status, sizeof(st), cudaMemcpyDeviceToHost, s));
        MUMMU_CUDA_TRY(cudaStreamSynchronize(s));
    }
    if (st == 0) return MUMMU_OK;
    MUMMU_CUDA_TRY(cudaMemsetAsync(m->status, 0, sizeof(int32_t), s));
    if (st & STATUS_TIMEOUT) {
        set_error("a bounded device-side wait ran out");
        return MUMMU_ERR_TIMEOUT;
    }
    if (st & STATUS_BOUNDS) {
        set_error("an index left its buffer on the device (a receive buffer smaller than the rows routed to it, "
                  "or a checked kernel caught a bad index); the access was skipped");
        return MUMMU_ERR_CONTRACT;
    }
    set_error("router logit is not finite (NaN or infinity in the activations or router weight)");
    return MUMMU_ERR_NUMERIC;
}

// router -> permute -> experts -> combine, all on stream s, device pointers
static int forward_device(MummuMoe* m, const void* x, void* y, int64_t tokens, int top_k, int norm,
                          cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    int rc;
    if (decode_q4k_supported(c, tokens) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // decode: router and grouping in one launch when the call is small enough
        rc = launch_router(m, x, tokens, top_k, norm, m->ids, m->wts, m->counts, s, true);
        if (rc == MUMMU_ERR_UNSUPPORTED) {
            if ((rc = launch_router(m, x, tokens, top_k, norm, m->ids, m->wts, m->counts, s))) return rc;
            rc = launch_permute(m, m->ids, tokens, top_k, m->counts, m->offsets, m->row_token, m->pos, s);
        }
        if (rc) return rc;
        if (m->sw.checked && (rc = launch_check_plan(m, m->ids, m->pos, m->row_token, m->counts, m->offsets, tokens, top_k, s)))
            return rc;
        if ((rc = launch_decode_q4k(m, x, tokens, top_k, s))) return rc;
        return launch_combine(m, m->ys, MUMMU_F32, m->ids, m->wts, m->pos, tokens, top_k, y, s);
    }
    if ((rc = launch_router(m, x, tokens, top_k, norm, m->ids, m->wts, m->counts, s))) return rc;
    if (prefill_tc_supported(c, tokens * top_k) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && !m->sw.no_tc) {
        // tensor-core path: sorted copy of the routed rows, two grouped GEMMs, 16-bit expert outputs
        if ((rc = launch_permute(m, m->ids, tokens, top_k, m->counts, m->offsets, m->row_token, m->pos, s))) return rc;
        if (m->sw.checked && (rc = launch_check_plan(m, m->ids, m->pos, m->row_token, m->counts, m->offsets, tokens, top_k, s)))
            return rc;
        if ((rc = launch_gather_rows(m, x, m->row_token, m->xs, tokens * top_k, s))) return rc;
        if ((rc = launch_experts_tc(m, m->xs, m->cap_tokens * c.top_k, m->counts, m->offsets, m->ys, c.act_dtype, s)))
            return rc;
        return launch_combine(m, m->ys, c.act_dtype, m->ids, m->wts, m->pos, tokens, top_k, y, s);
    } else if (q4k_tc_supported(c, tokens * top_k) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && !m->sw.no_tc) {
        // Q4_K with more tokens than the packed-weight kernels take: expand the experts that have
        // rows to f16, then the tensor-core path
        if ((rc = launch_permute(m, m->ids, tokens, top_k, m->counts, m->offsets, m->row_token, m->pos, s))) return rc;
        if (m->sw.checked && (rc = launch_check_plan(m, m->ids, m->pos, m->row_token, m->counts, m->offsets, tokens, top_k, s)))
            return rc;
        if ((rc = launch_gather_rows(m, x, m->row_token, m->xs, tokens * top_k, s))) return rc;
        if ((rc = launch_experts_q4k_tc(m, m->xs, m->cap_tokens * c.top_k, m->counts, m->offsets, m->ys, c.act_dtype, s)))
            return rc;
        return launch_combine(m, m->ys, c.act_dtype, m->ids, m->wts, m->pos, tokens, top_k, y, s);
    } else {
        if ((rc = launch_permute(m, m->ids, tokens, top_k, m->counts, m->offsets, m->row_token, m->pos, s))) return rc;
        if (m->sw.checked && (rc = launch_check_plan(m, m->ids, m->pos, m->row_token, m->counts, m->offsets, tokens, top_k, s)))
            return rc;
        int64_t max_rows = tokens;  // an expert serves a token at most once
        if ((rc = launch_experts_simt(m, x, c.act_dtype, m->row_token, m->counts, m->offsets, max_rows,
                                      tokens * top_k, m->ys, MUMMU_F32, -1, s)))
            return rc;
    }
    return launch_combine(m, m->ys, MUMMU_F32, m->ids, m->wts, m->pos, tokens, top_k, y, s);
}

}  // namespace mummu

using namespace mummu;

extern "C" {

const char* mummu_cuda_last_error(void) { return g_error.c_str(); }
const char* mummu_cuda_version(void) { return "mummu-cuda 0.1 (sm_100a)"; }

int32_t mummu_moe_create(const MummuMoeConfig* cfg, MummuMoe** out) {
    MUMMU_REQUIRE(cfg && out, "mummu_moe_create: null argument");
    *out = nullptr;
    MUMMU_REQUIRE(cfg->experts >= 2,
                  "MoE: num_experts must be >= 2 (got %d); use SwiGluMlp for a dense FFN", cfg->experts);
    MUMMU_REQUIRE(cfg->top_k >= 1 && cfg->top_k <= cfg->experts,
                  "MoE: num_experts_per_tok (%d) must be in 1..=num_experts (%d)", cfg->top_k, cfg->experts);
    MUMMU_REQUIRE(cfg->hidden >= 1 && cfg->inter >= 1,
                  "MoE: hidden_size and expert_intermediate_size must be >= 1");
    MUMMU_REQUIRE(cfg->act_dtype == MUMMU_F32 || cfg->act_dtype == MUMMU_F16 || cfg->act_dtype == MUMMU_BF16,
                  "MoE: activation dtype %d is not F32, F16 or BF16", cfg->act_dtype);
    MUMMU_REQUIRE(cfg->weight_dtype >= MUMMU_F32 && cfg->weight_dtype <= MUMMU_Q6_K,
                  "MoE: weight dtype %d is not F32, F16, BF16, Q4_K, Q8_0, Q5_K or Q6_K", cfg->weight_dtype);
    MUMMU_REQUIRE(cfg->experts_local >= 1 && cfg->expert_first >= 0 &&
                      cfg->expert_first + cfg->experts_local <= cfg->experts,
                  "MoE: local experts [%d, %d) are not inside 0..%d", cfg->expert_first,
                  cfg->expert_first + cfg->experts_local, cfg->experts);
    if (cfg->weight_dtype == MUMMU_Q4_K || cfg->weight_dtype == MUMMU_Q5_K || cfg->weight_dtype == MUMMU_Q6_K)
        MUMMU_REQUIRE(cfg->hidden % Q4K_BLOCK_ELEMS == 0 && cfg->inter % Q4K_BLOCK_ELEMS == 0,
                      "MoE: K-quant rows hold whole 256-value super-blocks (hidden %d, intermediate %d)",
                      cfg->hidden, cfg->inter);
    if (cfg->weight_dtype == MUMMU_Q8_0)
        MUMMU_REQUIRE(cfg->hidden % Q80_BLOCK_ELEMS == 0 && cfg->inter % Q80_BLOCK_ELEMS == 0,
                      "MoE: Q8_0 rows hold whole 32-value blocks (hidden %d, intermediate %d)", cfg->hidden,
                      cfg->inter);
    int ndev = 0;
    MUMMU_CUDA_TRY(cudaGetDeviceCount(&ndev));
    MUMMU_REQUIRE(cfg->device >= 0 && cfg->device < ndev, "MoE: CUDA device %d of %d", cfg->device, ndev);
    DeviceGuard guard(cfg->device);
    MummuMoe* m = new MummuMoe();
    m->cfg = *cfg;
    switches_from_env(m->sw);
    int rc = MUMMU_OK;
    do {
        cudaError_t err = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
        if (err != cudaSuccess) { set_error("cudaStreamCreate: %s", cudaGetErrorString(err)); rc = MUMMU_ERR_DEVICE; break; }
        if ((rc = dev_alloc(&m->router_w, (size_t)cfg->hidden * cfg->experts))) break;
        for (int b = 0; b < 3 && !rc; ++b) {
            m->bank_bytes[b] = bank_total_bytes(*cfg, b);
            rc = dev_alloc((uint8_t**)&m->bank[b], m->bank_bytes[b]);
        }
        if (rc) break;
        if ((rc = dev_alloc(&m->counts, (size_t)cfg->experts))) break;
        if ((rc = dev_alloc(&m->offsets, (size_t)cfg->experts + 1))) break;
        if ((rc = dev_alloc(&m->active, (size_t)cfg->experts))) break;
        if ((rc = dev_alloc(&m->n_active, 1))) break;
        if ((rc = dev_alloc(&m->ret_seg, (size_t)cfg->experts_local * 16 + 1))) break;
        if ((rc = dev_alloc(&m->ret_dst, (size_t)cfg->experts_local * 16))) break;
        if ((rc = dev_alloc(&m->hits, (size_t)cfg->experts))) break;
        if ((rc = dev_alloc(&m->status, 1))) break;
        cudaMemset(m->hits, 0, sizeof(unsigned long long) * cfg->experts);
        cudaMemset(m->ret_seg, 0, sizeof(int32_t) * ((size_t)cfg->experts_local * 16 + 1));
        cudaMemset(m->ret_dst, 0, sizeof(int32_t) * (size_t)cfg->experts_local * 16);
        cudaMemset(m->status, 0, sizeof(int32_t));
        if (cudaHostAlloc((void**)&m->status_host, sizeof(int32_t), cudaHostAllocDefault) != cudaSuccess) {
            m->status_host = nullptr;       // pageable reads still work
            cudaGetLastError();
        }
        if (cfg->max_tokens > 0) rc = ensure_scratch(m, cfg->max_tokens);
    } while (0);
    if (rc) {
        mummu_moe_destroy(m);
        return rc;
    }
    *out = m;
    return MUMMU_OK;
}

int32_t mummu_moe_destroy(MummuMoe* m) {
    if (!m) return MUMMU_OK;
    {
        DeviceGuard guard(m->cfg.device);
        if (m->stream) cudaStreamSynchronize(m->stream);
        clear_host_graphs(m);
        free_scratch(m);
        cudaFree(m->router_w); cudaFree(m->router_wt); cudaFree(m->router_bias); cudaFree(m->ex_io);
        for (int b = 0; b < 3; ++b) cudaFree(m->bank[b]);
        cudaFree(m->counts); cudaFree(m->offsets); cudaFree(m->hits); cudaFree(m->status);
        if (m->status_host) cudaFreeHost(m->status_host);
        cudaFree(m->active); cudaFree(m->n_active); cudaFree(m->ret_seg); cudaFree(m->ret_dst);
        for (int b = 0; b < 3; ++b) cudaFree(m->wexp[b]);
        for (auto& p : m->prof.pending) { cudaEventDestroy(p.a); cudaEventDestroy(p.b); }
        for (auto e : m->prof.pool) cudaEventDestroy(e);
        if (m->stream) cudaStreamDestroy(m->stream);
    }
    delete m;
    return MUMMU_OK;
}

int32_t mummu_moe_set_router(MummuMoe* m, const void* w, int32_t dtype, int32_t layout, const float* bias) {
    MUMMU_REQUIRE(m && w, "mummu_moe_set_router: null argument");
    MUMMU_REQUIRE(dtype == MUMMU_F32 || dtype == MUMMU_F16 || dtype == MUMMU_BF16,
                  "router weight dtype %d is not F32, F16 or BF16", dtype);
    MUMMU_REQUIRE(layout == MUMMU_ROUTER_IN_OUT || layout == MUMMU_ROUTER_OUT_IN, "router layout %d", layout);
    std::lock_guard<std::mutex> lock(m->mu);
    clear_host_graphs(m);
    DeviceGuard guard(m->cfg.device);
    const int H = m->cfg.hidden, E = m->cfg.experts;
    std::vector<float> host((size_t)H * E);
    for (int i = 0; i < H; ++i)
        for (int e = 0; e < E; ++e) {
            size_t src = layout == MUMMU_ROUTER_IN_OUT ? (size_t)i * E + e : (size_t)e * H + i;
            float v;
            if (dtype == MUMMU_F32) v = ((const float*)w)[src];
            else if (dtype == MUMMU_F16) v = __half2float(((const __half*)w)[src]);
            else v = __bfloat162float(((const __nv_bfloat16*)w)[src]);
            host[(size_t)i * E + e] = v;
        }
    // work queued on the handle's stream may still read the old weights; the copies below run on
    // the legacy default stream, which the handle's non-blocking stream is not ordered with
    MUMMU_CUDA_TRY(cudaStreamSynchronize(m->stream));
    MUMMU_CUDA_TRY(cudaMemcpy(m->router_w, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
    if (H % 32 == 0 && E % 8 == 0) {
        // image of the decode router's shared-memory slice, so that a block fetches its 8 experts
        // with one bulk copy instead of 2048 scattered 32-byte reads
        const int S = H / 8 + 4;
        std::vector<float> img((size_t)E * 8 * S, 0.0f);
        for (int e = 0; e < E; ++e)
            for (int i = 0; i < H; ++i)
                img[((size_t)(e / 8) * 64 + (size_t)(i % 8) * 8 + (e % 8)) * S + i / 8] = host[(size_t)i * E + e];
        if (!m->router_wt) {
            int rc = dev_alloc(&m->router_wt, img.size());
            if (rc) return rc;
        }
        MUMMU_CUDA_TRY(cudaMemcpy(m->router_wt, img.data(), img.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    if (bias) {
        if (!m->router_bias) {
            int rc = dev_alloc(&m->router_bias, (size_t)E);
            if (rc) return rc;
        }
        MUMMU_CUDA_TRY(cudaMemcpy(m->router_bias, bias, sizeof(float) * E, cudaMemcpyHostToDevice));
    } else if (m->router_bias) {
        cudaFree(m->router_bias);
        m->router_bias = nullptr;
    }
    m->router_set = true;
    return MUMMU_OK;
}

int32_t mummu_moe_set_bank(MummuMoe* m, int32_t which, const void* data, size_t bytes, int32_t on_device) {
    MUMMU_REQUIRE(m && data, "mummu_moe_set_bank: null argument");
    MUMMU_REQUIRE(which >= 0 && which < 3, "mummu_moe_set_bank: bank %d is not gate(0), up(1) or down(2)", which);
    MUMMU_REQUIRE(bytes == m->bank_bytes[which],
                  "mummu_moe_set_bank: bank %d needs %zu bytes ([experts %d, out, in]), got %zu", which,
                  m->bank_bytes[which], m->cfg.experts_local, bytes);
    std::lock_guard<std::mutex> lock(m->mu);
    clear_host_graphs(m);
    DeviceGuard guard(m->cfg.device);
    // Earlier calls on the handle's own stream may still read the bank; the handle's stream is
    // non-blocking, so the legacy-stream copy below is not ordered with it by itself.  Work the
    // caller queued on its own streams is the caller's to finish first (said in the header).
    MUMMU_CUDA_TRY(cudaStreamSynchronize(m->stream));
    if (on_device) {
        // the source may still be being written on whatever stream the caller used, and a
        // device-to-device cudaMemcpy may return before the copy has run: wait on both sides
        MUMMU_CUDA_TRY(cudaDeviceSynchronize());
        MUMMU_CUDA_TRY(cudaMemcpyAsync(m->bank[which], data, bytes, cudaMemcpyDeviceToDevice, m->stream));
        MUMMU_CUDA_TRY(cudaStreamSynchronize(m->stream));
    } else {
        MUMMU_CUDA_TRY(cudaMemcpy(m->bank[which], data, bytes, cudaMemcpyHostToDevice));
    }
    m->bank_set[which] = true;
    return MUMMU_OK;
}

// io_x -> io_y for a host-pointer call.  Decode-sized Q4_K calls are launch-bound: from the third
// call with the same (tokens, top_k, norm) on, the layer's launches are replayed from a CUDA graph
// captured on the second (the first runs eagerly so that one-time attribute calls are done).
static int forward_host_staged(MummuMoe* m, int64_t tokens, int top_k, int norm, cudaStream_t s) {
    if (m->sw.no_host_graph || m->prof.enabled || !decode_q4k_supported(m->cfg, tokens))
        return forward_device(m, m->io_x, m->io_y, tokens, top_k, norm, s);
    const uint64_t key = ((uint64_t)tokens << 20) | ((uint64_t)top_k << 1) | (uint64_t)(norm != 0);
    auto it = m->host_graphs.find(key);
    if (it != m->host_graphs.end()) {
        if (!it->second) return forward_device(m, m->io_x, m->io_y, tokens, top_k, norm, s);
        MUMMU_CUDA_TRY(cudaGraphLaunch(it->second, s));
        m->launches += m->host_calls[key];
        return MUMMU_OK;
    }
    if (m->host_calls[key]++ == 0) return forward_device(m, m->io_x, m->io_y, tokens, top_k, norm, s);
    // second call: capture
    cudaGraphExec_t exec = nullptr;
    cudaGraph_t graph = nullptr;
    const int64_t before = m->launches;
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        const int rc = forward_device(m, m->io_x, m->io_y, tokens, top_k, norm, s);
        const cudaError_t end = cudaStreamEndCapture(s, &graph);
        if (rc == MUMMU_OK && end == cudaSuccess && graph) {
            if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) exec = nullptr;
        }
        if (graph) cudaGraphDestroy(graph);
    }
    cudaGetLastError();                         // a failed capture leaves a sticky-free error behind
    m->host_graphs[key] = exec;
    m->host_calls[key] = (int)(m->launches - before);   // launches one replay stands for
    if (!exec) {
        m->launches = before;
        return forward_device(m, m->io_x, m->io_y, tokens, top_k, norm, s);
    }
    MUMMU_CUDA_TRY(cudaGraphLaunch(exec, s));
    return MUMMU_OK;
}

int32_t mummu_moe_forward(MummuMoe* m, const void* x, void* y, int32_t tokens, int32_t top_k,
                          int32_t norm, int32_t on_device, void* stream) {
    MUMMU_REQUIRE(m, "mummu_moe_forward: null handle");
    MUMMU_REQUIRE(tokens >= 0, "MoE forward: negative token count %d", tokens);
    int rc;
    if ((rc = check_top_k(m, top_k))) return rc;
    if ((rc = check_ready(m, true, true))) return rc;
    MUMMU_REQUIRE(m->cfg.expert_first == 0 && m->cfg.experts_local == m->cfg.experts,
                  "MoE forward: this handle holds experts [%d, %d) of %d; the whole-layer call needs "
                  "all of them (use the staged calls for expert parallelism)",
                  m->cfg.expert_first, m->cfg.expert_first + m->cfg.experts_local, m->cfg.experts);
    if (tokens == 0) return MUMMU_OK;
    MUMMU_REQUIRE(x && y, "MoE forward: null activation pointer");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    if ((rc = ensure_scratch(m, tokens))) return rc;
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    size_t bytes = (size_t)tokens * m->cfg.hidden * dtype_size(m->cfg.act_dtype);
    if (on_device) return forward_device(m, x, y, tokens, top_k, norm, s);
    MUMMU_CUDA_TRY(cudaMemcpyAsync(m->io_x, x, bytes, cudaMemcpyHostToDevice, s));
    if ((rc = forward_host_staged(m, tokens, top_k, norm, s))) return rc;
    MUMMU_CUDA_TRY(cudaMemcpyAsync(y, m->io_y, bytes, cudaMemcpyDeviceToHost, s));
    return read_status(m, s);
}

int32_t mummu_moe_route(MummuMoe* m, const void* x, int32_t tokens, int32_t top_k, int32_t norm,
                        int32_t* ids_out, float* w_out, int32_t on_device, void* stream) {
    MUMMU_REQUIRE(m, "mummu_moe_route: null handle");
    MUMMU_REQUIRE(tokens >= 0, "MoE route: negative token count %d", tokens);
    int rc;
    if ((rc = check_top_k(m, top_k))) return rc;
    if ((rc = check_ready(m, true, false))) return rc;
    if (tokens == 0) return MUMMU_OK;
    MUMMU_REQUIRE(x && ids_out && w_out, "MoE route: null pointer");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    if ((rc = ensure_scratch(m, tokens))) return rc;
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    if (on_device) return launch_router(m, x, tokens, top_k, norm, ids_out, w_out, m->counts, s);
    size_t bytes = (size_t)tokens * m->cfg.hidden * dtype_size(m->cfg.act_dtype);
    MUMMU_CUDA_TRY(cudaMemcpyAsync(m->io_x, x, bytes, cudaMemcpyHostToDevice, s));
    if ((rc = launch_router(m, m->io_x, tokens, top_k, norm, m->ids, m->wts, m->counts, s))) return rc;
    size_t n = (size_t)tokens * top_k;
    MUMMU_CUDA_TRY(cudaMemcpyAsync(ids_out, m->ids, n * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    MUMMU_CUDA_TRY(cudaMemcpyAsync(w_out, m->wts, n * sizeof(float), cudaMemcpyDeviceToHost, s));
    return read_status(m, s);
}

int32_t mummu_moe_route_grouped(MummuMoe* m, const void* x, int32_t tokens, int32_t top_k, int32_t norm,
                                int32_t* ids, float* w, int32_t* counts, int32_t* offsets, int32_t* row_token,
                                int32_t* pos, void* stream) {
    MUMMU_REQUIRE(m, "mummu_moe_route_grouped: null handle");
    MUMMU_REQUIRE(tokens >= 0, "MoE route: negative token count %d", tokens);
    int rc;
    if ((rc = check_top_k(m, top_k))) return rc;
    if ((rc = check_ready(m, true, false))) return rc;
    if (tokens == 0) return MUMMU_OK;
    MUMMU_REQUIRE(x && ids && w && counts && offsets && row_token && pos, "mummu_moe_route_grouped: null pointer");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    if ((rc = ensure_scratch(m, tokens))) return rc;
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    // decode-sized calls: one launch (the router's last block groups the pairs); else two
    const GroupedOut out{counts, offsets, row_token, pos};
    rc = launch_router(m, x, tokens, top_k, norm, ids, w, counts, s, true, &out);
    if (rc == MUMMU_ERR_UNSUPPORTED) {
        if ((rc = launch_router(m, x, tokens, top_k, norm, ids, w, counts, s))) return rc;
        rc = launch_permute(m, ids, tokens, top_k, counts, offsets, row_token, pos, s);
    }
    if (rc) return rc;
    return m->sw.checked ? launch_check_plan(m, ids, pos, row_token, counts, offsets, tokens, top_k, s) : MUMMU_OK;
}

int32_t mummu_moe_permute(MummuMoe* m, const int32_t* ids, int32_t tokens, int32_t top_k,
                          int32_t* counts, int32_t* offsets, int32_t* row_token, int32_t* pos,
                          void* stream) {
    MUMMU_REQUIRE(m && ids, "mummu_moe_permute: null argument");
    MUMMU_REQUIRE(tokens >= 0 && top_k >= 1, "mummu_moe_permute: tokens %d, top_k %d", tokens, top_k);
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    int32_t* cnt = counts ? counts : m->counts;
    int rc;
    if ((rc = launch_count(m, ids, (int64_t)tokens * top_k, cnt, s))) return rc;
    return launch_permute(m, ids, tokens, top_k, cnt, offsets, row_token, pos, s);
}

static int32_t experts_rows(MummuMoe* m, const void* xs, const int32_t* counts, int32_t rows, void* ys,
                            void* stream, bool planned, const char* who) {
    MUMMU_REQUIRE(m && counts, "%s: null argument", who);
    MUMMU_REQUIRE(rows >= 0, "%s: negative row count %d", who, rows);
    int rc;
    if ((rc = check_ready(m, false, true))) return rc;
    if (rows == 0) return MUMMU_OK;
    MUMMU_REQUIRE(xs && ys, "%s: null activation pointer", who);
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    int64_t tokens_equiv = ((int64_t)rows + m->cfg.top_k - 1) / m->cfg.top_k;
    if ((rc = ensure_scratch(m, tokens_equiv))) return rc;
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    if (m->sw.checked && counts != m->counts) {
        // the caller's counts are copied with the segments clipped to the rows the buffers hold
        if ((rc = launch_check_counts(m, counts, m->counts, m->cfg.experts_local, rows, s))) return rc;
        counts = m->counts;
        planned = false;                     // offsets and work order are rebuilt from the safe copy
    }
    if (!planned && (rc = launch_offsets_from_counts(m, counts, m->cfg.experts_local, m->offsets, s))) return rc;
    if (prefill_tc_supported(m->cfg, rows) && (reinterpret_cast<uintptr_t>(xs) & 15) == 0 && !m->sw.no_tc)
        return launch_experts_tc(m, xs, rows, counts, m->offsets, ys, m->cfg.act_dtype, s);
    // A shard with few experts and many rows each (expert parallelism over many ranks at decode
    // sizes: 8 experts x 64 rows): the packed-weight kernels would expand every expert's weights once
    // per 16-row pass; expanding them once to f16 and running the tensor-core GEMMs is cheaper.
    // `rows` bounds all ranks' rows; this shard expects its share.
    const int shards = m->cfg.experts / m->cfg.experts_local;
    const int64_t rows_per_expert = (int64_t)rows / shards / m->cfg.experts_local;
    const bool few_fat_experts = m->cfg.experts_local <= 8 && rows_per_expert >= 32;
    if (few_fat_experts && q4k_tc_supported(m->cfg, rows) && (reinterpret_cast<uintptr_t>(xs) & 15) == 0 && !m->sw.no_tc)
        return launch_experts_q4k_tc(m, xs, rows, counts, m->offsets, ys, m->cfg.act_dtype, s);
    if (m->cfg.weight_dtype == MUMMU_Q4_K && m->cfg.act_dtype == MUMMU_F16 && (reinterpret_cast<uintptr_t>(xs) & 15) == 0 &&
        rows <= 8192 && m->cfg.hidden <= 8192 && m->cfg.inter <= 8192) {
        // decode regime: packed-weight kernels (f32 out), then narrowed to the activation dtype
        if ((rc = launch_decode_q4k_rows(m, xs, nullptr, counts, m->offsets, rows, (float*)m->ys, s))) return rc;
        return launch_narrow((const float*)m->ys, ys, m->cfg.act_dtype, (int64_t)rows * m->cfg.hidden, s);
    }
    if (q4k_tc_supported(m->cfg, rows) && (reinterpret_cast<uintptr_t>(xs) & 15) == 0 && !m->sw.no_tc)
        return launch_experts_q4k_tc(m, xs, rows, counts, m->offsets, ys, m->cfg.act_dtype, s);
    return launch_experts_simt(m, xs, m->cfg.act_dtype, nullptr, counts, m->offsets, rows, rows, ys,
                               m->cfg.act_dtype, -1, s);
}

int32_t mummu_moe_experts_grouped(MummuMoe* m, const void* xs, const int32_t* counts, int32_t rows,
                                  void* ys, void* stream) {
    return experts_rows(m, xs, counts, rows, ys, stream, false, "mummu_moe_experts_grouped");
}

int32_t mummu_moe_experts_planned(MummuMoe* m, const void* xs, const int32_t* counts, int32_t rows,
                                  void* ys, void* stream) {
    return experts_rows(m, xs, counts, rows, ys, stream, true, "mummu_moe_experts_planned");
}

int32_t mummu_moe_combine(MummuMoe* m, const void* ys, const int32_t* ids, const float* w,
                          const int32_t* pos, int32_t tokens, int32_t top_k, void* out, void* stream) {
    MUMMU_REQUIRE(m && ys && ids && w && pos && out, "mummu_moe_combine: null argument");
    MUMMU_REQUIRE(tokens >= 0 && top_k >= 1, "mummu_moe_combine: tokens %d, top_k %d", tokens, top_k);
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    if (m->sw.checked) {
        // the caller's indices are copied into the layer's scratch with every one made safe
        int rc;
        if ((rc = ensure_scratch(m, tokens))) return rc;
        if ((rc = launch_check_combine(m, ids, pos, m->ids, m->pos, (int64_t)tokens * top_k, s))) return rc;
        ids = m->ids;
        pos = m->pos;
    }
    return launch_combine(m, ys, m->cfg.act_dtype, ids, w, pos, tokens, top_k, out, s);
}

// f32 staging of the one-expert calls: kept in the handle, grown when a larger call arrives
static int ensure_ex_io(MummuMoe* m, size_t elems) {
    if (elems <= m->ex_io_elems) return MUMMU_OK;
    MUMMU_CUDA_TRY(cudaStreamSynchronize(m->stream));
    cudaFree(m->ex_io);
    m->ex_io = nullptr;
    m->ex_io_elems = 0;
    int rc = dev_alloc(&m->ex_io, elems);
    if (rc) return rc;
    m->ex_io_elems = elems;
    return MUMMU_OK;
}

// One expert over `rows` device rows of the activation dtype, through the same kernels a layer
// call uses (tensor-core grouped GEMM, packed decode kernels, generic bank).
static int expert_rows_device(MummuMoe* m, int expert, const void* xs, int rows, void* ys, cudaStream_t s) {
    const MummuMoeConfig& c = m->cfg;
    int rc;
    if ((rc = launch_single_expert_plan(m, expert, rows, s))) return rc;
    if (prefill_tc_supported(c, rows) && (reinterpret_cast<uintptr_t>(xs) & 15) == 0 && !m->sw.no_tc)
        return launch_experts_tc(m, xs, rows, m->counts, m->offsets, ys, c.act_dtype, s);
    if (c.weight_dtype == MUMMU_Q4_K && c.act_dtype == MUMMU_F16 && (reinterpret_cast<uintptr_t>(xs) & 15) == 0 &&
        rows <= 8192 && c.hidden <= 8192 && c.inter <= 8192) {
        if ((rc = launch_decode_q4k_rows(m, xs, nullptr, m->counts, m->offsets, rows, (float*)m->ys, s))) return rc;
        return launch_narrow((const float*)m->ys, ys, c.act_dtype, (int64_t)rows * c.hidden, s);
    }
    return launch_experts_simt(m, xs, c.act_dtype, nullptr, nullptr, nullptr, rows, rows, ys, c.act_dtype, expert, s);
}

static int expert_args(MummuMoe* m, int32_t expert, int32_t rows, const char* who) {
    MUMMU_REQUIRE(m, "%s: null handle", who);
    MUMMU_REQUIRE(expert >= 0 && expert < m->cfg.experts_local, "expert %d out of range (%d)", expert,
                  m->cfg.experts_local);
    MUMMU_REQUIRE(rows >= 0, "%s: negative row count %d", who, rows);
    return check_ready(m, false, true);
}

int32_t mummu_expert_run(MummuMoe* m, int32_t expert, const float* x, int32_t rows, float* y) {
    int rc;
    if ((rc = expert_args(m, expert, rows, "mummu_expert_run"))) return rc;
    if (rows == 0) return MUMMU_OK;
    MUMMU_REQUIRE(x && y, "mummu_expert_run: null pointer");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    const MummuMoeConfig& c = m->cfg;
    int64_t tokens_equiv = ((int64_t)rows + c.top_k - 1) / c.top_k;
    if ((rc = ensure_scratch(m, tokens_equiv))) return rc;
    const size_t n = (size_t)rows * c.hidden;
    if ((rc = ensure_ex_io(m, 3 * n))) return rc;
    cudaStream_t s = m->stream;
    float *dx = m->ex_io, *dy = m->ex_io + n;
    void* y_act = m->ex_io + 2 * n;          // the expert's output rows in the activation dtype
    MUMMU_CUDA_TRY(cudaMemcpyAsync(dx, x, n * sizeof(float), cudaMemcpyHostToDevice, s));
    if (c.act_dtype == MUMMU_F32) {
        // f32 handle: the generic bank takes the f32 rows as they are
        if ((rc = launch_experts_simt(m, dx, MUMMU_F32, nullptr, nullptr, nullptr, rows, rows, dy, MUMMU_F32, expert, s)))
            return rc;
    } else {
        // 16-bit handle: rows narrowed to the activation dtype (as the reference's DeviceExpert casts
        // to its device's float type, nn/moe.rs:448-462), the layer's own kernels, widened back
        if ((rc = launch_narrow(dx, m->xs, c.act_dtype, (int64_t)n, s))) return rc;
        if ((rc = expert_rows_device(m, expert, m->xs, rows, y_act, s))) return rc;
        if ((rc = launch_widen(y_act, c.act_dtype, dy, (int64_t)n, s))) return rc;
    }
    MUMMU_CUDA_TRY(cudaMemcpyAsync(y, dy, n * sizeof(float), cudaMemcpyDeviceToHost, s));
    return read_status(m, s);
}

int32_t mummu_expert_run_device(MummuMoe* m, int32_t expert, const void* x, int32_t rows, void* y, void* stream) {
    int rc;
    if ((rc = expert_args(m, expert, rows, "mummu_expert_run_device"))) return rc;
    if (rows == 0) return MUMMU_OK;
    MUMMU_REQUIRE(x && y, "mummu_expert_run_device: null pointer");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    int64_t tokens_equiv = ((int64_t)rows + m->cfg.top_k - 1) / m->cfg.top_k;
    if ((rc = ensure_scratch(m, tokens_equiv))) return rc;
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    return expert_rows_device(m, expert, x, rows, y, s);
}

int32_t mummu_expert_gate_energy(MummuMoe* m, int32_t expert, const float* x, int32_t rows, float* energy) {
    int rc;
    if ((rc = expert_args(m, expert, rows, "mummu_expert_gate_energy"))) return rc;
    if (rows == 0) return MUMMU_OK;
    MUMMU_REQUIRE(x && energy, "mummu_expert_gate_energy: null pointer");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    const size_t n = (size_t)rows * m->cfg.hidden;
    if ((rc = ensure_ex_io(m, n + (size_t)rows))) return rc;
    cudaStream_t s = m->stream;
    MUMMU_CUDA_TRY(cudaMemcpyAsync(m->ex_io, x, n * sizeof(float), cudaMemcpyHostToDevice, s));
    if ((rc = launch_gate_energy(m, expert, m->ex_io, rows, m->ex_io + n, s))) return rc;
    MUMMU_CUDA_TRY(cudaMemcpyAsync(energy, m->ex_io + n, (size_t)rows * sizeof(float), cudaMemcpyDeviceToHost, s));
    MUMMU_CUDA_TRY(cudaStreamSynchronize(s));
    return MUMMU_OK;
}

uint64_t mummu_expert_resident_bytes(const MummuMoe* m, int32_t expert) {
    if (!m || expert < 0 || expert >= m->cfg.experts_local) return 0;
    uint64_t total = 0;
    for (int b = 0; b < 3; ++b) total += (uint64_t)(bank_total_bytes(m->cfg, b) / (size_t)m->cfg.experts_local);
    return total;
}

int32_t mummu_moe_get_config(const MummuMoe* m, MummuMoeConfig* out) {
    MUMMU_REQUIRE(m && out, "mummu_moe_get_config: null argument");
    *out = m->cfg;
    return MUMMU_OK;
}

int32_t mummu_moe_dequant_bank(MummuMoe* m, int32_t which, int32_t expert, float* out) {
    MUMMU_REQUIRE(m && out, "mummu_moe_dequant_bank: null argument");
    MUMMU_REQUIRE(which >= 0 && which < 3, "bank %d is not gate(0), up(1) or down(2)", which);
    MUMMU_REQUIRE(expert >= 0 && expert < m->cfg.experts_local, "expert %d out of range (%d)", expert,
                  m->cfg.experts_local);
    MUMMU_REQUIRE(m->bank_set[which], "bank %d was never set", which);
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    const MummuMoeConfig& c = m->cfg;
    size_t out_dim = which == MUMMU_BANK_DOWN ? c.hidden : c.inter;
    size_t in_dim = which == MUMMU_BANK_DOWN ? c.inter : c.hidden;
    size_t n = out_dim * in_dim;
    size_t ebytes = bank_row_bytes(c, which) * out_dim;
    const uint8_t* src = (const uint8_t*)m->bank[which] + ebytes * expert;
    float* tmp = nullptr;
    int rc;
    if ((rc = dev_alloc(&tmp, n))) return rc;
    if (c.weight_dtype == MUMMU_Q4_K) rc = launch_q4k_dequant(src, tmp, (int64_t)(n / Q4K_BLOCK_ELEMS), m->stream);
    else if (c.weight_dtype > MUMMU_Q4_K)
        rc = launch_block_dequant(src, c.weight_dtype, tmp, (int64_t)out_dim, (int64_t)in_dim, bank_row_bytes(c, which),
                                  m->stream);
    else rc = launch_widen(src, c.weight_dtype, tmp, (int64_t)n, m->stream);
    cudaError_t err = cudaSuccess;
    if (!rc) err = cudaMemcpyAsync(out, tmp, n * sizeof(float), cudaMemcpyDeviceToHost, m->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(m->stream);
    cudaFree(tmp);
    if (rc) return rc;
    if (err != cudaSuccess) {
        set_error("mummu_moe_dequant_bank: %s", cudaGetErrorString(err));
        return MUMMU_ERR_DEVICE;
    }
    return MUMMU_OK;
}

int32_t mummu_moe_take_hits(MummuMoe* m, uint64_t* per_expert) {
    MUMMU_REQUIRE(m && per_expert, "mummu_moe_take_hits: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    size_t bytes = sizeof(unsigned long long) * m->cfg.experts;
    MUMMU_CUDA_TRY(cudaMemcpyAsync(per_expert, m->hits, bytes, cudaMemcpyDeviceToHost, m->stream));
    MUMMU_CUDA_TRY(cudaMemsetAsync(m->hits, 0, bytes, m->stream));
    MUMMU_CUDA_TRY(cudaStreamSynchronize(m->stream));
    return MUMMU_OK;
}

int32_t mummu_moe_adopt_scratch(MummuMoe* m, MummuMoe* donor) {
    MUMMU_REQUIRE(m && donor && m != donor, "mummu_moe_adopt_scratch: bad handles");
    const MummuMoeConfig &a = m->cfg, &b = donor->cfg;
    MUMMU_REQUIRE(a.device == b.device && a.hidden == b.hidden && a.inter == b.inter && a.experts == b.experts &&
                      a.top_k == b.top_k && a.act_dtype == b.act_dtype && !donor->scratch_borrowed,
                  "mummu_moe_adopt_scratch: the two layers must have the same shape, dtype and device");
    std::lock_guard<std::mutex> lock(m->mu);
    clear_host_graphs(m);
    DeviceGuard guard(a.device);
    MUMMU_CUDA_TRY(cudaDeviceSynchronize());
    free_scratch(m);
    m->logits = donor->logits; m->tile_done = donor->tile_done; m->ids = donor->ids; m->wts = donor->wts;
    m->row_token = donor->row_token; m->pos = donor->pos; m->xs = donor->xs; m->hact = donor->hact;
    m->ys = donor->ys; m->io_x = donor->io_x; m->io_y = donor->io_y;
    m->whist = donor->whist; m->whist_elems = donor->whist_elems;
    m->cap_tokens = donor->cap_tokens;
    m->scratch_borrowed = true;
    m->scratch_donor = donor;
    return MUMMU_OK;
}

int32_t mummu_moe_sync(MummuMoe* m, void* stream) {
    MUMMU_REQUIRE(m, "mummu_moe_sync: null handle");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    cudaStream_t s = stream ? (cudaStream_t)stream : m->stream;
    return read_status(m, s);
}

int32_t mummu_moe_set_profiling(MummuMoe* m, int32_t enabled) {
    MUMMU_REQUIRE(m, "mummu_moe_set_profiling: null handle");
    std::lock_guard<std::mutex> lock(m->mu);
    m->prof.enabled = enabled != 0;
    return MUMMU_OK;
}

int32_t mummu_moe_take_profile(MummuMoe* m, char* names, size_t cap) {
    MUMMU_REQUIRE(m && names && cap > 0, "mummu_moe_take_profile: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    DeviceGuard guard(m->cfg.device);
    MUMMU_CUDA_TRY(cudaDeviceSynchronize());
    for (auto& p : m->prof.pending) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, p.a, p.b) == cudaSuccess) {
            auto& st = m->prof.stats[p.name];
            st.launches += 1;
            st.ms += ms;
        }
        m->prof.pool.push_back(p.a);
        m->prof.pool.push_back(p.b);
    }
    m->prof.pending.clear();
    std::string out;
    for (auto& kv : m->prof.stats) {
        char buf[160];
        snprintf(buf, sizeof(buf), "%s=%lld:%.6f;", kv.first.c_str(), (long long)kv.second.launches,
                 kv.second.launches ? kv.second.ms / (double)kv.second.launches : 0.0);
        out += buf;
    }
    m->prof.stats.clear();
    strncpy(names, out.c_str(), cap - 1);
    names[cap - 1] = 0;
    return MUMMU_OK;
}

int64_t mummu_moe_launch_count(const MummuMoe* m) { return m ? m->launches : 0; }

int32_t mummu_moe_set_switch(MummuMoe* m, const char* name, int32_t value) {
    MUMMU_REQUIRE(m && name, "mummu_moe_set_switch: null argument");
    std::lock_guard<std::mutex> lock(m->mu);
    if (!strcmp(name, "WAIT_POLLS")) {
        MUMMU_REQUIRE(value >= 0, "mummu_moe_set_switch: WAIT_POLLS %d", value);
        m->sw.wait_polls = (uint32_t)value;
        return MUMMU_OK;
    }
    for (const SwitchName& e : kSwitches)
        if (!strcmp(name, e.name)) {
            m->sw.*(e.field) = value;
            clear_host_graphs(m);      // captured replays hold the old variant
            return MUMMU_OK;
        }
    set_error("mummu_moe_set_switch: no switch named %s", name);
    return MUMMU_ERR_CONTRACT;
}

int32_t mummu_q4k_quantize(const float* src, void* dst, int64_t n_superblocks, int32_t device, void* stream) {
    MUMMU_REQUIRE(src && dst && n_superblocks >= 0, "mummu_q4k_quantize: bad argument");
    DeviceGuard guard(device);
    return launch_q4k_quantize(src, dst, n_superblocks, (cudaStream_t)stream);
}

int32_t mummu_q4k_dequantize(const void* src, float* dst, int64_t n_superblocks, int32_t device, void* stream) {
    MUMMU_REQUIRE(src && dst && n_superblocks >= 0, "mummu_q4k_dequantize: bad argument");
    DeviceGuard guard(device);
    return launch_q4k_dequant(src, dst, n_superblocks, (cudaStream_t)stream);
}

}  // extern "C"
