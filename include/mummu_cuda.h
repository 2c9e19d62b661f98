/*
 * mummu_cuda.h — C ABI of the B200 (sm_100a) sparse mixture-of-experts expert bank.
 *
 * This is the boundary a `mummu-cuda` FFI crate binds: plain pointers and sizes, no C++ or
 * framework types.  The reference project (physics515/Mummu) has no FFI for this path; every entry
 * point below names the reference interface it stands in for (file:line inside the reference
 * tree, `crates/mummu/src/...`).
 *
 * Conventions
 *  - Every function returns an int32 status (MUMMU_OK = 0).  Nothing aborts; nothing falls back to
 *    the CPU.  `mummu_cuda_last_error()` returns the calling thread's last message.
 *  - Contract violations (bad top_k, mismatched widths, wrong byte counts) return
 *    MUMMU_ERR_CONTRACT with a message that carries the reference's panic stem ("top_k",
 *    "num_experts_per_tok", ...), so a Rust wrapper can re-raise the panic the reference raises
 *    (nn/moe.rs:62-76, 119-126, 250-253).
 *  - A handle serialises the HOST side of its calls with an internal lock; distinct handles are
 *    independent.  The device side is ordered by the stream a call is given: calls of one handle on
 *    two different streams share the handle's scratch buffers and must not overlap on the GPU
 *    (order them with events, or give each stream its own handle; handles can share weights'
 *    source buffers but not scratch).  mummu_moe_set_router / mummu_moe_set_bank wait for the
 *    handle's own stream; work the caller queued on its own streams must have finished first.
 *  - Device memory is allocated when a handle is created (banks, router, scratch for max_tokens)
 *    and, once, when a call first needs more: a larger token count than max_tokens, and the f16
 *    image of a block-quantised bank (first call of more than 256 tokens on Q4_K, first call on a
 *    Q8_0 / Q5_K / Q6_K bank with f16 activations, first call of a shard of at most 8 experts with
 *    32 or more rows each).  A call that allocates cannot be inside a stream capture: make the
 *    first call of each kind before capturing.
 *  - Matrices are row-major.  Router weight: [hidden, experts] (burn `Linear` stores [in, out],
 *    nn/moe.rs:1642) or [experts, hidden] (GGUF `ffn_gate_inp`, models/olmoe.rs:338-339), chosen by
 *    a flag.  Banks: [experts, out, in], byte-identical to GGUF `ffn_{gate,up,down}_exps`
 *    (nn/moe.rs:19-30).  For MUMMU_Q4_K a bank row is in/256 super-blocks of 144 bytes
 *    (gguf.rs:342, 372).
 */
#ifndef MUMMU_CUDA_H
#define MUMMU_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MUMMU_OK               0
#define MUMMU_ERR_CONTRACT     1   /* caller broke the interface contract (reference: panic)   */
#define MUMMU_ERR_DEVICE       2   /* CUDA runtime / driver error                               */
#define MUMMU_ERR_TIMEOUT      3   /* a bounded device-side wait ran out                        */
#define MUMMU_ERR_UNSUPPORTED  4   /* valid request this build has no kernel for                */
#define MUMMU_ERR_NUMERIC      5   /* non-finite router logit (qwen4exp/experts.rs:553-560)     */

typedef enum {
    MUMMU_F32  = 0,
    MUMMU_F16  = 1,
    MUMMU_BF16 = 2,
    MUMMU_Q4_K = 3,     /* GGUF Q4_K super-blocks; weights only */
    /* sibling GGUF formats (gguf.rs:1535-1543, 1731-1797), weights only: with f16 activations the
     * experts that have rows are expanded to f16 and run the tensor-core GEMMs, otherwise the
     * generic bank decodes every weight element by element (no packed-weight decode kernel) */
    MUMMU_Q8_0 = 4,     /* 34-byte blocks of 32 */
    MUMMU_Q5_K = 5,     /* 176-byte super-blocks of 256 */
    MUMMU_Q6_K = 6      /* 210-byte super-blocks of 256 */
} mummu_dtype;

#define MUMMU_BANK_GATE 0
#define MUMMU_BANK_UP   1
#define MUMMU_BANK_DOWN 2

/* router weight memory order */
#define MUMMU_ROUTER_IN_OUT 0      /* [hidden, experts] — burn Linear (nn/moe.rs:1642)          */
#define MUMMU_ROUTER_OUT_IN 1      /* [experts, hidden] — GGUF ffn_gate_inp (olmoe.rs:338-339)  */

typedef struct MummuMoe MummuMoe;  /* opaque: device weights, scratch, one internal stream     */

/* Stands in for `SparseMoeConfig` (nn/moe.rs:42-50).  `experts` is the router width; this handle
 * stores `experts_local` of them starting at global id `expert_first` (expert parallelism keeps a
 * contiguous block per GPU; single GPU: expert_first = 0, experts_local = experts). */
typedef struct {
    int32_t device;          /* CUDA ordinal                                                   */
    int32_t hidden;          /* hidden_size                                                     */
    int32_t inter;           /* expert_intermediate_size                                        */
    int32_t experts;         /* num_experts (>= 2)                                              */
    int32_t top_k;           /* num_experts_per_tok, 1..=experts: upper bound for later calls   */
    int32_t act_dtype;       /* mummu_dtype of x / y: F32, F16 or BF16                          */
    int32_t weight_dtype;    /* mummu_dtype of the banks: F32, F16, BF16 or Q4_K                */
    int32_t expert_first;    /* first global expert id held by this handle                      */
    int32_t experts_local;   /* number of experts held by this handle                           */
    int32_t max_tokens;      /* scratch is sized for this many tokens (grown on demand if 0)   */
} MummuMoeConfig;

/* -------- life cycle ---------------------------------------------------------------------- */

/* `SparseMoeConfig::init` (nn/moe.rs:61-99): checks experts >= 2, 1 <= top_k <= experts,
 * hidden, inter >= 1 (messages keep the reference's wording), allocates the device banks. Weights
 * start undefined; set them with the two calls below.  Q4_K needs hidden % 256 == 0 and
 * inter % 256 == 0 (whole super-blocks per row, gguf.rs:1442-1460). */
int32_t mummu_moe_create(const MummuMoeConfig* cfg, MummuMoe** out);
int32_t mummu_moe_destroy(MummuMoe* moe);

/* Router `gate: Linear` weight (nn/moe.rs:36-37, 92; olmoe.rs:338-339).  `w` is a HOST pointer to
 * hidden*experts values of `dtype` (F32/F16/BF16) in `layout` order; copied.  `bias` is NULL (the
 * reference builds the router without bias) or `experts` f32 values added to the logits. */
int32_t mummu_moe_set_router(MummuMoe* moe, const void* w, int32_t dtype, int32_t layout,
                             const float* bias);

/* One of `MoeExperts::{gate, up, down}` (nn/moe.rs:22-30): `data` points to experts_local*out*in
 * values of the handle's weight_dtype (for Q4_K: the raw ggml bytes), `bytes` is checked.
 * `on_device` != 0 means `data` is a device pointer on the handle's device.  Copied. */
int32_t mummu_moe_set_bank(MummuMoe* moe, int32_t which, const void* data, size_t bytes,
                           int32_t on_device);

/* Let `moe` use `donor`'s per-call scratch instead of its own (a stack of identical layers that
 * run one after another needs one set, not one per layer).  Same shape, dtype and device; the
 * donor must outlive `moe` and must not run at the same time; size the donor (max_tokens) first.
 * No counterpart in the reference (burn allocates intermediates per op). */
int32_t mummu_moe_adopt_scratch(MummuMoe* moe, MummuMoe* donor);

/* -------- the layer ------------------------------------------------------------------------- */

/* `SparseMoe::forward` / `SparseMoePerExpert::forward` (nn/moe.rs:116-177, 214-219) on the
 * flattened [tokens, hidden] input: router -> softmax over all experts (f32) -> top_k of the
 * probabilities (ties: lowest expert id) -> optional renormalisation -> routed SwiGLU experts ->
 * weighted sum in ascending expert order.  x and y hold tokens*hidden values of act_dtype;
 * `on_device` != 0: both are device pointers and the work is queued on `stream` (a cudaStream_t;
 * NULL = the handle's own non-blocking stream, so pass cudaStreamLegacy / cudaStreamPerThread to
 * name a default stream) without waiting; otherwise both are host pointers and the call
 * returns when y is written.  Requires expert_first == 0 and experts_local == experts. */
int32_t mummu_moe_forward(MummuMoe* moe, const void* x, void* y, int32_t tokens, int32_t top_k,
                          int32_t norm_topk_prob, int32_t on_device, void* stream);

/* Router only — `SparseMoePerExpert::route` (nn/moe.rs:247-290) / `qwen4exp::experts::route`
 * (models/qwen4exp/experts.rs:541-582): ids_out[tokens*top_k] (descending probability, ties to
 * the lowest id) and w_out[tokens*top_k] (f32).  Pointers follow `on_device` as above. */
int32_t mummu_moe_route(MummuMoe* moe, const void* x, int32_t tokens, int32_t top_k,
                        int32_t norm_topk_prob, int32_t* ids_out, float* w_out,
                        int32_t on_device, void* stream);

/* mummu_moe_route followed by mummu_moe_permute, device pointers only; for decode-sized calls (at
 * most 1024 (token, slot) pairs) it is one launch: the router's last block groups the pairs.
 * Same outputs as the two calls (SparseMoePerExpert::route, nn/moe.rs:247-290, then the grouping
 * of Routing.per_expert, nn/moe.rs:275-289). */
int32_t mummu_moe_route_grouped(MummuMoe* moe, const void* x, int32_t tokens, int32_t top_k,
                                int32_t norm_topk_prob, int32_t* ids, float* w, int32_t* counts,
                                int32_t* offsets, int32_t* row_token, int32_t* pos, void* stream);

/* Group the routed (token, slot) pairs by expert — the `Routing.per_expert` lists of
 * nn/moe.rs:275-289 as flat device arrays.  ids: device [tokens*top_k] global expert ids.
 * Outputs (device): counts[experts] rows per expert; offsets[experts+1] exclusive prefix sum;
 * row_token[tokens*top_k] token of each sorted row (ascending token within an expert);
 * pos[tokens*top_k] sorted row of pair (token, slot).  Any output may be NULL. */
int32_t mummu_moe_permute(MummuMoe* moe, const int32_t* ids, int32_t tokens, int32_t top_k,
                          int32_t* counts, int32_t* offsets, int32_t* row_token, int32_t* pos,
                          void* stream);

/* Expert bank over rows already grouped by expert — the loop body of
 * `SparseMoePerExpert::run_local` (nn/moe.rs:301-326) without the scatter: xs device
 * [rows, hidden] act_dtype holding, expert by expert in ascending LOCAL id, counts[e] rows;
 * counts device [experts_local]; ys device [rows, hidden] act_dtype receives
 * down(silu(gate x) * (up x)) per row. */
int32_t mummu_moe_experts_grouped(MummuMoe* moe, const void* xs, const int32_t* counts,
                                  int32_t rows, void* ys, void* stream);
/* The same when the handle already holds the experts' first rows and work order for `counts`
 * (left there by mummu_ep_dispatch, which plans them from the gathered counts): saves the launch
 * that derives them. */
int32_t mummu_moe_experts_planned(MummuMoe* moe, const void* xs, const int32_t* counts,
                                  int32_t rows, void* ys, void* stream);

/* Weighted un-permute — the scatter-add of nn/moe.rs:317-325 / 1589-1602 as a gather: for every
 * token, out = sum over its top_k slots in ASCENDING EXPERT ID of (w * y) with the product and the
 * sum rounded separately (no fused multiply-add).  ys device [tokens*top_k, hidden] act_dtype,
 * indexed through pos; ids, w, pos device [tokens*top_k]; out device [tokens, hidden]. */
int32_t mummu_moe_combine(MummuMoe* moe, const void* ys, const int32_t* ids, const float* w,
                          const int32_t* pos, int32_t tokens, int32_t top_k, void* out,
                          void* stream);

/* `ExpertExec::run(&[f32], rows, hidden) -> Vec<f32>` (nn/moe.rs:353-357) and
 * `RoutedExperts::expert_ffn` (models/qwen4exp/experts.rs:1015-1057): one expert (LOCAL id) on
 * `rows` f32 rows from host memory, f32 rows back to host memory. */
int32_t mummu_expert_run(MummuMoe* moe, int32_t expert, const float* x, int32_t rows, float* y);

/* `ExpertExec::run_tensor` / `run_tensor_resident` (nn/moe.rs:366-412): the same expert on `rows`
 * DEVICE rows of act_dtype, result left on the device, queued on `stream` without waiting (the
 * caller moves or reads it later, batched with every other partial, nn/moe.rs:358-367). */
int32_t mummu_expert_run_device(MummuMoe* moe, int32_t expert, const void* x, int32_t rows, void* y,
                                void* stream);

/* `ExpertExec::gate_energy` (nn/moe.rs:413-418): per row, the sum over the expert's intermediate
 * columns of silu(x . gate_row)^2; x and energy are HOST f32 arrays ([rows, hidden] and [rows]). */
int32_t mummu_expert_gate_energy(MummuMoe* moe, int32_t expert, const float* x, int32_t rows,
                                 float* energy);

/* `ExpertExec::resident_bytes` (nn/moe.rs:351-352): bytes one expert's gate, up and down weights
 * hold on the device (0 for a bad argument). */
uint64_t mummu_expert_resident_bytes(const MummuMoe* moe, int32_t expert);

/* The configuration a handle was created with: device and weight dtype are what
 * `ExpertExec::tier` (nn/moe.rs:349-350) reports as the expert's (device, precision). */
int32_t mummu_moe_get_config(const MummuMoe* moe, MummuMoeConfig* out);

/* -------- expert parallelism over peer memory (no counterpart in the reference: its devices
 * exchange through host memory, backend.rs:128-143, nn/moe.rs:1219-1272) ----------------------- */

/* A device buffer other processes on the node can map: cudaMalloc + cudaIpcGetMemHandle.  handle64
 * receives 64 opaque bytes to hand to the peers (any transport); peers map it with mummu_ep_open
 * and unmap with mummu_ep_close; the owner frees with mummu_ep_free. */
int32_t mummu_ep_alloc(int32_t device, size_t bytes, void** ptr, uint8_t* handle64);
int32_t mummu_ep_open(int32_t device, const uint8_t* handle64, void** ptr);
int32_t mummu_ep_close(void* ptr);
int32_t mummu_ep_free(void* ptr);

/* One expert-parallel layer on one rank is four stages that signal each other ONE WAY through the
 * ranks' sync blocks (every rank allocates mummu_ep_sync_bytes(world, experts) with mummu_ep_alloc,
 * which zeroes it, and maps the peers' blocks; peer_sync[r] is rank r's block as seen from this
 * device): a stage's last block stores its epoch into a flag of every peer, a later stage polls its
 * own flags.  No kernel both signals and waits, no library collective and no host round trip is
 * inside a step, so a step can be replayed from a CUDA graph; and the stages of several rank
 * handles may be issued stage by stage on one stream of ONE device (how the exchange is tested on
 * a single GPU).  Every rank issues the same sequence.  Waits are bounded (switch WAIT_POLLS; the
 * default is a few seconds): on expiry the stage skips its data movement, raises the status word
 * (MUMMU_ERR_TIMEOUT from the next mummu_moe_sync) and returns; the group must then be re-zeroed
 * with mummu_ep_reset on every rank, behind a host barrier, before it is used again.
 *
 *   mummu_ep_post_counts  stage 1: counts[experts] (this rank's rows per global expert, device)
 *                         -> every rank; replaces the host exchange of backend.rs:128-143.
 *   mummu_ep_dispatch     stage 2: waits for every rank's counts; computes dst_base[experts] (first
 *                         row, in the owning rank's buffers, of THIS rank's rows per expert; buffers
 *                         are expert-major with sources in rank order, so every expert's rows are in
 *                         a fixed order) and local_counts[experts_local]; copies x[row_token[p]] for
 *                         every sorted row p (mummu_moe_permute order) into the owner's receive
 *                         buffer peer_recv[owner] ([cap_rows, hidden], 16-bit) with peer stores.  A
 *                         row that would land at or beyond cap_rows is dropped and reported
 *                         (MUMMU_ERR_CONTRACT from the next mummu_moe_sync).
 *   mummu_ep_experts      stage 3: waits for every rank's rows; runs this rank's experts over its
 *                         receive buffer into its private output buffer ys_own ([rows_cap, hidden]),
 *                         then stores every output row into the buffer of the rank the row came
 *                         from, peer_back[source] ([back_rows, hidden]: that rank's (token, slot)
 *                         pairs in its own mummu_moe_permute order) with peer stores.  Both
 *                         directions push: no load crosses NVLink.
 *   mummu_ep_combine      stage 4: waits for every rank's outputs; mummu_moe_combine over the own
 *                         buffer back_own.  order_ids (NULL: ids) gives the expert id of each pair
 *                         where `ids` are bank slots (mummu_ep_place): a token's terms are summed
 *                         in ascending expert id either way. */
size_t mummu_ep_sync_bytes(int32_t world, int32_t experts);
/* Small-batch form (decode): with few tokens per rank the three hops above cost more than the rows
 * they move.  Every rank pushes its tokens to every rank (mummu_ep_gather_tokens: x [tokens,
 * hidden] -> rows [rank * tokens, (rank + 1) * tokens) of every peer_gx[r]; one signal), waits for
 * everybody's (mummu_ep_wait, channel 0), and routes ALL world * tokens tokens itself with
 * mummu_moe_route_grouped: the router is replicated and bit-reproducible, so every rank holds the
 * same plan and no counts are exchanged.  mummu_ep_experts_gathered then runs this rank's experts
 * on the rows that plan gives them, read in place from the gathered tokens, and stores each output
 * row into peer_back[rank of the row's token] at the row's position in the common sorted order
 * ([world * tokens * top_k, hidden] per rank); mummu_ep_combine, given the slice of ids, w and pos
 * of this rank's own tokens, finishes the layer.  Two hops instead of three and no row copy on
 * the way out.  f16 activations on Q4_K experts, at most 8192 (token, slot) pairs over all ranks;
 * otherwise MUMMU_ERR_UNSUPPORTED. */
int32_t mummu_ep_gather_tokens(MummuMoe* moe, const void* x, int32_t tokens, void* const* peer_sync,
                               void* const* peer_gx, int32_t rank, int32_t world, void* stream);
/* Wait (bounded) until every rank has signalled the next epoch of `channel` (0: counts or gathered
 * tokens, 1: rows, 2: outputs) to this rank. */
int32_t mummu_ep_wait(MummuMoe* moe, void* const* peer_sync, int32_t rank, int32_t world,
                      int32_t channel, void* stream);
int32_t mummu_ep_experts_gathered(MummuMoe* moe, void* const* peer_sync, void* const* peer_back,
                                  const void* gx_own, const int32_t* row_token, const int32_t* counts,
                                  const int32_t* offsets, int32_t rank, int32_t world,
                                  int32_t tokens_per_rank, int32_t top_k, int64_t back_rows,
                                  void* stream);
/* Hot-expert placement (nn/moe.rs:1527-1535 hands the hit counters to the planner; tier.rs:353-431
 * plans from them).  A group whose handles are created over `world * slots_per_rank` bank SLOTS
 * instead of experts can hold an expert in several slots, on different ranks, and any expert on
 * any rank.  The router (a handle over the real experts) still emits real expert ids; this call
 * turns them into slot ids for this rank's tokens, ids_out[i] = table[ids[i]] (table: device
 * int32 [experts_real], every entry a slot of `moe`), and the stages above run on slot ids
 * unchanged.  The same expert's weights give the same numbers in whichever slot they sit, so the
 * layer's output does not depend on the placement.  An id or a table entry out of range raises
 * MUMMU_ERR_CONTRACT at the next mummu_moe_sync. */
int32_t mummu_ep_place(MummuMoe* moe, const int32_t* ids, const int32_t* table, int32_t experts_real,
                       int64_t n, int32_t* ids_out, void* stream);
int32_t mummu_ep_reset(int32_t device, void* own_sync, int32_t world, int32_t experts);
int32_t mummu_ep_post_counts(MummuMoe* moe, const int32_t* counts, void* const* peer_sync,
                             int32_t rank, int32_t world, void* stream);
int32_t mummu_ep_dispatch(MummuMoe* moe, const void* x, const int32_t* row_token,
                          const int32_t* offsets, void* const* peer_sync, void* const* peer_recv,
                          int32_t rank, int32_t world, int32_t rows, int64_t cap_rows,
                          int32_t* dst_base, int32_t* local_counts, void* stream);
int32_t mummu_ep_experts(MummuMoe* moe, void* const* peer_sync, void* const* peer_back, int32_t rank,
                         int32_t world, const void* recv_own, const int32_t* local_counts,
                         int64_t rows_cap, void* ys_own, int64_t back_rows, void* stream);
int32_t mummu_ep_combine(MummuMoe* moe, void* const* peer_sync, const void* back_own,
                         const int32_t* ids, const int32_t* order_ids, const float* w,
                         const int32_t* pos, int32_t rank, int32_t world, int32_t tokens,
                         int32_t top_k, void* out, void* stream);

/* -------- parity taps and counters ----------------------------------------------------------- */

/* The dequantised (or widened) f32 weights of one expert of one bank, [out, in], to HOST memory.
 * For Q4_K this is `gguf::dequant_q4_k` (gguf.rs:1701-1726) and must match it bit for bit. */
int32_t mummu_moe_dequant_bank(MummuMoe* moe, int32_t which, int32_t expert, float* out);

/* `ExpertPool::take_hits` (nn/moe.rs:1527-1535): rows served per GLOBAL expert id since the last
 * call (accumulated by forward); per_expert is a HOST array of `experts` counters; resets them. */
int32_t mummu_moe_take_hits(MummuMoe* moe, uint64_t* per_expert);

/* Wait for everything queued on the handle's own stream (or `stream`) and report the sticky
 * device status word: MUMMU_OK, MUMMU_ERR_NUMERIC (non-finite router logit) or
 * MUMMU_ERR_TIMEOUT. */
int32_t mummu_moe_sync(MummuMoe* moe, void* stream);

/* Average device time (milliseconds, CUDA events on the launching stream) and launch count of
 * each internal kernel since the last call — the (bytes, elapsed) ledger of
 * nn/packed_gemv.rs:1260-1296.  Enable with mummu_moe_set_profiling; names is a HOST buffer that
 * receives a ';'-separated "name=launches:ms" list. */
int32_t mummu_moe_set_profiling(MummuMoe* moe, int32_t enabled);
int32_t mummu_moe_take_profile(MummuMoe* moe, char* names, size_t cap);

/* Number of kernels this handle has launched (for accounting in benchmarks). */
int64_t mummu_moe_launch_count(const MummuMoe* moe);

/* Kernel-variant switches of one handle.  They are read once from the environment when the handle
 * is created (MUMMU_CUDA_<NAME>, as the reference reads MUMMU_PACKED_GEMV / MUMMU_GEMV_SPLIT once,
 * nn/packed_gemv.rs:85-92, 686-694); this call changes one afterwards.  Names: NO_TC, NO_HOST_GRAPH,
 * ROUTER_PLAIN, DECODE_NO_PDL, DECODE_NT, DECODE_STREAM_MIN, DECODE_RB_GATEUP, DECODE_RB_DOWN,
 * CHECKED (kernels verify their indices and raise the status word: the reference arms CubeCL's
 * check_mode = "validate" for its test suites, burn.toml:17), WAIT_POLLS (bound of the
 * device-side waits on peers, in polls of about 0.2 us; 0 = the default of a few seconds). */
int32_t mummu_moe_set_switch(MummuMoe* moe, const char* name, int32_t value);

/* -------- Q4_K helpers (no counterpart in the reference: it only dequantises Q4_K) ----------- */

/* Encode n_superblocks*256 f32 values (device) to n_superblocks*144 Q4_K bytes (device). */
int32_t mummu_q4k_quantize(const float* src, void* dst, int64_t n_superblocks, int32_t device,
                           void* stream);
/* Decode device Q4_K bytes to device f32 exactly as gguf.rs:1701-1726 does. */
int32_t mummu_q4k_dequantize(const void* src, float* dst, int64_t n_superblocks, int32_t device,
                             void* stream);

/* -------- for callers that cannot allocate device memory ------------------------------------ */

/* The router of mummu_moe_route as a free function that allocates nothing and needs no handle.
 * It has no counterpart in the reference.  It exists for code that runs where device allocation is
 * off limits: inside a real-time or latency-critical serving loop that has fixed its memory plan,
 * under a framework that owns every byte of device memory and forbids cudaMalloc from plug-ins,
 * or in a process that has already committed the GPU's memory to weights and KV cache.
 *
 * All device pointers are the caller's: x [tokens, hidden] of act_dtype, router_w [hidden,
 * experts] f32 (the order mummu_moe_set_router stores), bias NULL or [experts] f32,
 * ids_out / w_out [tokens, top_k].  Results equal mummu_moe_route's bit for bit.  The work is
 * queued on `stream` (a cudaStream_t; 0 is the default stream) and the call does not wait.
 *
 * The kernel's scratch (the logits it hands from its expert-slice blocks to the block that
 * selects, plus a few counters; about 1 MiB) is a fixed array inside the library's device image,
 * held by every GPU that loads the library until the process exits.  Limits, refused with
 * MUMMU_ERR_CONTRACT and a message: tokens <= 1024, tokens * experts <= 262144, experts <= 256.
 * router_w must be 16-byte aligned (the kernel reads it in 128-bit words; a pointer into the
 * middle of a packed buffer is refused with MUMMU_ERR_CONTRACT rather than left to fault on the
 * device); the other pointers need the alignment of their element type.  hidden is limited by the
 * shared memory the kernel stages one 8-expert weight slice and 4 token rows in (48 * hidden + 2 KB
 * <= 220 KB, so hidden <= about 4600): wider inputs return MUMMU_ERR_UNSUPPORTED.
 * The first call on a device looks the array's address up (cudaGetSymbolAddress); make that first
 * call before any stream capture.  All calls on a device share the one array: two calls whose
 * kernels may overlap on the GPU (different streams, no dependency) race on it and give wrong
 * routing — order them.  A non-finite logit is not reported here (there is no handle to carry
 * the status): that token gets experts 0..top_k-1 with zero weights. */
int32_t mummu_moe_route_noalloc(const void* x, int32_t act_dtype, const float* router_w,
                                const float* bias, int32_t tokens, int32_t hidden,
                                int32_t experts, int32_t top_k, int32_t norm_topk_prob,
                                int32_t* ids_out, float* w_out, int32_t device, void* stream);

/* -------- decode trunk: what a token passes between two expert banks ------------------------ */

/* The fixed-shape decode step of the OLMoE decoder around the expert bank, for `slots` independent
 * sequences with one new token each: the arithmetic of `LoadedOlmoe::forward` (models/olmoe.rs:
 * 522-587) and `Attention` (nn/attention.rs:182-295: RMSNorm of q and k over the whole projection
 * :196-200, f32 scores :275-289, the -1e4 causal mask :28-48; RoPE nn/rope.rs:21-105) laid out as
 * `StaticDecode::forward_static` wants it (capture.rs:48-107, nn/static_kv.rs:36-72): a
 * preallocated cache [slots, kv_heads, max_ctx, head_dim] per layer written in place at each
 * slot's position, positions read on the device, nothing uploaded inside a step - so a step can be
 * captured.  f16 weights and activations, f32 norms, f32 accumulation. */
typedef struct MummuTrunk MummuTrunk;

typedef struct {
    int32_t device;
    int32_t hidden;
    int32_t heads;
    int32_t kv_heads;
    int32_t head_dim;
    int32_t layers;
    int32_t vocab;
    int32_t slots;           /* sequences decoded per step (`StaticKvConfig::slots`), 1..=64 */
    int32_t max_ctx;         /* positions each slot can hold                                  */
    float rope_theta;
    float rms_eps;
} MummuTrunkConfig;

#define MUMMU_TRUNK_EMBED      0   /* [vocab, hidden] f16            */
#define MUMMU_TRUNK_LM_HEAD    1   /* [vocab, hidden] f16            */
#define MUMMU_TRUNK_FINAL_NORM 2   /* [hidden] f32                   */
#define MUMMU_TRUNK_IN_NORM    3   /* per layer from here: [hidden] f32 */
#define MUMMU_TRUNK_POST_NORM  4
#define MUMMU_TRUNK_Q          5   /* [heads*head_dim, hidden] f16   */
#define MUMMU_TRUNK_K          6   /* [kv_heads*head_dim, hidden]    */
#define MUMMU_TRUNK_V          7
#define MUMMU_TRUNK_O          8   /* [hidden, heads*head_dim] f16   */
#define MUMMU_TRUNK_Q_NORM     9   /* [heads*head_dim] f32           */
#define MUMMU_TRUNK_K_NORM     10  /* [kv_heads*head_dim] f32        */

/* `StaticDecode::static_bytes` (capture.rs:77-79): bytes of the cache a state of this shape holds. */
uint64_t mummu_trunk_static_bytes(const MummuTrunkConfig* cfg);
/* Weights, the zeroed cache (`StaticDecode::static_state`, capture.rs:81-83) and RoPE tables. */
int32_t mummu_trunk_create(const MummuTrunkConfig* cfg, MummuTrunk** out);
int32_t mummu_trunk_destroy(MummuTrunk* trunk);
/* One weight (MUMMU_TRUNK_*), row-major as the checkpoint stores `Linear` weights [out, in]
 * (models/olmoe.rs:319-349); `layer` is ignored for the first three.  Copied. */
int32_t mummu_trunk_set_weight(MummuTrunk* trunk, int32_t which, int32_t layer, const void* data,
                               size_t bytes, int32_t on_device);
/* x[slot] = embedding of tokens[slot] (device int32) - models/olmoe.rs:550. */
int32_t mummu_trunk_embed(MummuTrunk* trunk, const int32_t* tokens, int32_t slots, void* x,
                          void* stream);
/* One layer's attention half (models/olmoe.rs:561-566).  First x += y_prev when y_prev is not
 * NULL: the previous layer's expert-bank output joins the residual stream (models/olmoe.rs:567-571)
 * in the same launch that normalises it.  Then h = rmsnorm(x); q, k, v; q/k norm; RoPE at
 * positions[slot] (device int32); k, v stored at that position; attention over the keys up to it
 * inside the bucket of `key_len` keys; x += o-projection; h2 = rmsnorm(x) with the
 * post-attention weight - the input of this layer's expert bank.  x: device f16 [slots, hidden],
 * updated in place; y_prev, h2: device f16 [slots, hidden]. */
int32_t mummu_trunk_attention_step(MummuTrunk* trunk, int32_t layer, void* x, const void* y_prev,
                                   const int32_t* positions, int32_t slots, int32_t key_len, void* h2,
                                   void* stream);
/* x += y_prev (the last layer's expert bank; NULL: nothing to add), final norm, lm_head and the
 * greedy pick (models/olmoe.rs:573-585; decode.rs:33-48: the largest logit, ties to the lowest
 * id).  logits: device f32 [slots, vocab]; argmax: device int32 [slots] or NULL. */
int32_t mummu_trunk_head(MummuTrunk* trunk, void* x, const void* y_prev, int32_t slots, float* logits,
                         int32_t* argmax, void* stream);
/* `StaticDecode::seed_static` (capture.rs:105-106): copy `count` prefilled positions of one slot,
 * k and v as device f16 [kv_heads, count, head_dim], into the cache from position `first`. */
int32_t mummu_trunk_kv_write(MummuTrunk* trunk, int32_t layer, int32_t slot, int32_t first,
                             int32_t count, const void* k, const void* v, void* stream);

const char* mummu_cuda_last_error(void);
const char* mummu_cuda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MUMMU_CUDA_H */
