//! mummu-cuda — the B200 (sm_100a) top-k routed SwiGLU expert bank behind a C ABI.
//!
//! NOT COMPILED IN THIS REPOSITORY'S IMAGE: there is no cargo/rustc there.  The C ABI this file
//! binds (`include/mummu_cuda.h`) is built, loaded and tested through the ctypes table
//! `mummu_b200/_lib.py`; a CPU test keeps the `extern "C"` block below and that header in step.
//!
//! Layers of this file:
//!  * `sys`        — the raw `extern "C"` declarations, one per export of `mummu_cuda.h`;
//!  * `CudaBank`   — one MoE layer on one GPU: what `SparseMoe` / `SparseMoePerExpert`
//!                   (crates/mummu/src/nn/moe.rs:34-39, 201-329) hold when the `cuda-b200` feature is
//!                   on, with `forward`, `route`, `take_hits` under the reference's names;
//!  * `CudaTrunk`  — the decode trunk (attention half of every layer, embedding, head) that
//!                   `impl StaticDecode for Olmoe` (capture.rs:48-107) drives between the banks;
//!  * `CudaExpert` — one expert of a bank with the method set of `ExpertExec`
//!                   (nn/moe.rs:348-419).  The trait itself lives in crates/mummu (which depends on
//!                   this crate, not the other way round); the five-line `impl ExpertExec for
//!                   CudaExpert` that forwards to these methods is shown at the end of this file.
//!
//! Contract violations come back as status 1 with the reference's own message ("MoE forward: top_k
//! (..) must be in 1..=num_experts (..)"): `check` re-raises them as the panic the reference raises,
//! so `#[should_panic(expected = "top_k")]` (nn/moe.rs:2354-2374) still holds.

use std::ffi::{c_char, c_void, CStr, CString};
use std::ptr;

pub mod sys {
    use std::ffi::{c_char, c_void};

    #[repr(C)]
    #[derive(Debug, Clone, Copy, Default)]
    pub struct MummuMoeConfig {
        pub device: i32,
        pub hidden: i32,
        pub inter: i32,
        pub experts: i32,
        pub top_k: i32,
        pub act_dtype: i32,
        pub weight_dtype: i32,
        pub expert_first: i32,
        pub experts_local: i32,
        pub max_tokens: i32,
    }

    #[repr(C)]
    pub struct MummuMoe {
        _private: [u8; 0],
    }

    pub const MUMMU_OK: i32 = 0;
    pub const MUMMU_ERR_CONTRACT: i32 = 1;
    pub const MUMMU_ERR_DEVICE: i32 = 2;
    pub const MUMMU_ERR_TIMEOUT: i32 = 3;
    pub const MUMMU_ERR_UNSUPPORTED: i32 = 4;
    pub const MUMMU_ERR_NUMERIC: i32 = 5;

    pub const MUMMU_F32: i32 = 0;
    pub const MUMMU_F16: i32 = 1;
    pub const MUMMU_BF16: i32 = 2;
    pub const MUMMU_Q4_K: i32 = 3;
    pub const MUMMU_Q8_0: i32 = 4;
    pub const MUMMU_Q5_K: i32 = 5;
    pub const MUMMU_Q6_K: i32 = 6;

    pub const MUMMU_BANK_GATE: i32 = 0;
    pub const MUMMU_BANK_UP: i32 = 1;
    pub const MUMMU_BANK_DOWN: i32 = 2;

    pub const MUMMU_ROUTER_IN_OUT: i32 = 0;
    pub const MUMMU_ROUTER_OUT_IN: i32 = 1;

    extern "C" {
        // life cycle
        pub fn mummu_moe_create(cfg: *const MummuMoeConfig, out: *mut *mut MummuMoe) -> i32;
        pub fn mummu_moe_destroy(moe: *mut MummuMoe) -> i32;
        pub fn mummu_moe_set_router(moe: *mut MummuMoe, w: *const c_void, dtype: i32, layout: i32, bias: *const f32) -> i32;
        pub fn mummu_moe_set_bank(moe: *mut MummuMoe, which: i32, data: *const c_void, bytes: usize, on_device: i32) -> i32;
        pub fn mummu_moe_adopt_scratch(moe: *mut MummuMoe, donor: *mut MummuMoe) -> i32;
        pub fn mummu_moe_get_config(moe: *const MummuMoe, out: *mut MummuMoeConfig) -> i32;
        pub fn mummu_moe_set_switch(moe: *mut MummuMoe, name: *const c_char, value: i32) -> i32;
        // the layer and its stages
        pub fn mummu_moe_forward(moe: *mut MummuMoe, x: *const c_void, y: *mut c_void, tokens: i32, top_k: i32,
                                 norm_topk_prob: i32, on_device: i32, stream: *mut c_void) -> i32;
        pub fn mummu_moe_route(moe: *mut MummuMoe, x: *const c_void, tokens: i32, top_k: i32, norm_topk_prob: i32,
                               ids_out: *mut i32, w_out: *mut f32, on_device: i32, stream: *mut c_void) -> i32;
        pub fn mummu_moe_route_grouped(moe: *mut MummuMoe, x: *const c_void, tokens: i32, top_k: i32, norm_topk_prob: i32,
                                       ids: *mut i32, w: *mut f32, counts: *mut i32, offsets: *mut i32,
                                       row_token: *mut i32, pos: *mut i32, stream: *mut c_void) -> i32;
        pub fn mummu_moe_permute(moe: *mut MummuMoe, ids: *const i32, tokens: i32, top_k: i32, counts: *mut i32,
                                 offsets: *mut i32, row_token: *mut i32, pos: *mut i32, stream: *mut c_void) -> i32;
        pub fn mummu_moe_experts_grouped(moe: *mut MummuMoe, xs: *const c_void, counts: *const i32, rows: i32,
                                         ys: *mut c_void, stream: *mut c_void) -> i32;
        pub fn mummu_moe_experts_planned(moe: *mut MummuMoe, xs: *const c_void, counts: *const i32, rows: i32,
                                         ys: *mut c_void, stream: *mut c_void) -> i32;
        pub fn mummu_moe_combine(moe: *mut MummuMoe, ys: *const c_void, ids: *const i32, w: *const f32, pos: *const i32,
                                 tokens: i32, top_k: i32, out: *mut c_void, stream: *mut c_void) -> i32;
        // one expert (ExpertExec)
        pub fn mummu_expert_run(moe: *mut MummuMoe, expert: i32, x: *const f32, rows: i32, y: *mut f32) -> i32;
        pub fn mummu_expert_run_device(moe: *mut MummuMoe, expert: i32, x: *const c_void, rows: i32, y: *mut c_void,
                                       stream: *mut c_void) -> i32;
        pub fn mummu_expert_gate_energy(moe: *mut MummuMoe, expert: i32, x: *const f32, rows: i32, energy: *mut f32) -> i32;
        pub fn mummu_expert_resident_bytes(moe: *const MummuMoe, expert: i32) -> u64;
        // expert parallelism over peer memory
        pub fn mummu_ep_alloc(device: i32, bytes: usize, ptr: *mut *mut c_void, handle64: *mut u8) -> i32;
        pub fn mummu_ep_open(device: i32, handle64: *const u8, ptr: *mut *mut c_void) -> i32;
        pub fn mummu_ep_close(ptr: *mut c_void) -> i32;
        pub fn mummu_ep_free(ptr: *mut c_void) -> i32;
        pub fn mummu_ep_sync_bytes(world: i32, experts: i32) -> usize;
        pub fn mummu_ep_reset(device: i32, own_sync: *mut c_void, world: i32, experts: i32) -> i32;
        pub fn mummu_ep_gather_tokens(moe: *mut MummuMoe, x: *const c_void, tokens: i32, peer_sync: *const *mut c_void,
                                      peer_gx: *const *mut c_void, rank: i32, world: i32, stream: *mut c_void) -> i32;
        pub fn mummu_ep_wait(moe: *mut MummuMoe, peer_sync: *const *mut c_void, rank: i32, world: i32, channel: i32,
                             stream: *mut c_void) -> i32;
        pub fn mummu_ep_experts_gathered(moe: *mut MummuMoe, peer_sync: *const *mut c_void, peer_back: *const *mut c_void,
                                         gx_own: *const c_void, row_token: *const i32, counts: *const i32,
                                         offsets: *const i32, rank: i32, world: i32, tokens_per_rank: i32, top_k: i32,
                                         back_rows: i64, stream: *mut c_void) -> i32;
        pub fn mummu_ep_place(moe: *mut MummuMoe, ids: *const i32, table: *const i32, experts_real: i32, n: i64,
                              ids_out: *mut i32, stream: *mut c_void) -> i32;
        pub fn mummu_ep_post_counts(moe: *mut MummuMoe, counts: *const i32, peer_sync: *const *mut c_void, rank: i32,
                                    world: i32, stream: *mut c_void) -> i32;
        pub fn mummu_ep_dispatch(moe: *mut MummuMoe, x: *const c_void, row_token: *const i32, offsets: *const i32,
                                 peer_sync: *const *mut c_void, peer_recv: *const *mut c_void, rank: i32, world: i32,
                                 rows: i32, cap_rows: i64, dst_base: *mut i32, local_counts: *mut i32,
                                 stream: *mut c_void) -> i32;
        pub fn mummu_ep_experts(moe: *mut MummuMoe, peer_sync: *const *mut c_void, peer_back: *const *mut c_void,
                                rank: i32, world: i32, recv_own: *const c_void, local_counts: *const i32, rows_cap: i64,
                                ys_own: *mut c_void, back_rows: i64, stream: *mut c_void) -> i32;
        pub fn mummu_ep_combine(moe: *mut MummuMoe, peer_sync: *const *mut c_void, back_own: *const c_void,
                                ids: *const i32, order_ids: *const i32, w: *const f32, pos: *const i32, rank: i32,
                                world: i32, tokens: i32, top_k: i32, out: *mut c_void, stream: *mut c_void) -> i32;
        // parity taps, counters, profiling
        pub fn mummu_moe_dequant_bank(moe: *mut MummuMoe, which: i32, expert: i32, out: *mut f32) -> i32;
        pub fn mummu_moe_take_hits(moe: *mut MummuMoe, per_expert: *mut u64) -> i32;
        pub fn mummu_moe_sync(moe: *mut MummuMoe, stream: *mut c_void) -> i32;
        pub fn mummu_moe_set_profiling(moe: *mut MummuMoe, enabled: i32) -> i32;
        pub fn mummu_moe_take_profile(moe: *mut MummuMoe, names: *mut c_char, cap: usize) -> i32;
        pub fn mummu_moe_launch_count(moe: *const MummuMoe) -> i64;
        // Q4_K helpers and the allocation-free router
        pub fn mummu_q4k_quantize(src: *const f32, dst: *mut c_void, n_superblocks: i64, device: i32, stream: *mut c_void) -> i32;
        pub fn mummu_q4k_dequantize(src: *const c_void, dst: *mut f32, n_superblocks: i64, device: i32, stream: *mut c_void) -> i32;
        pub fn mummu_moe_route_noalloc(x: *const c_void, act_dtype: i32, router_w: *const f32, bias: *const f32,
                                       tokens: i32, hidden: i32, experts: i32, top_k: i32, norm_topk_prob: i32,
                                       ids_out: *mut i32, w_out: *mut f32, device: i32, stream: *mut c_void) -> i32;
        // trunk of the OLMoE decode step (see mummu_cuda.h, "decode trunk")
        pub fn mummu_trunk_create(cfg: *const MummuTrunkConfig, out: *mut *mut MummuTrunk) -> i32;
        pub fn mummu_trunk_destroy(trunk: *mut MummuTrunk) -> i32;
        pub fn mummu_trunk_set_weight(trunk: *mut MummuTrunk, which: i32, layer: i32, data: *const c_void, bytes: usize,
                                      on_device: i32) -> i32;
        pub fn mummu_trunk_attention_step(trunk: *mut MummuTrunk, layer: i32, x: *mut c_void, y_prev: *const c_void,
                                          positions: *const i32, slots: i32, key_len: i32, h2: *mut c_void,
                                          stream: *mut c_void) -> i32;
        pub fn mummu_trunk_embed(trunk: *mut MummuTrunk, tokens: *const i32, slots: i32, x: *mut c_void, stream: *mut c_void) -> i32;
        pub fn mummu_trunk_head(trunk: *mut MummuTrunk, x: *mut c_void, y_prev: *const c_void, slots: i32, logits: *mut f32,
                                argmax: *mut i32, stream: *mut c_void) -> i32;
        pub fn mummu_trunk_kv_write(trunk: *mut MummuTrunk, layer: i32, slot: i32, first: i32, count: i32, k: *const c_void,
                                    v: *const c_void, stream: *mut c_void) -> i32;
        pub fn mummu_trunk_static_bytes(cfg: *const MummuTrunkConfig) -> u64;
        // diagnostics
        pub fn mummu_cuda_last_error() -> *const c_char;
        pub fn mummu_cuda_version() -> *const c_char;
    }

    #[repr(C)]
    #[derive(Debug, Clone, Copy, Default)]
    pub struct MummuTrunkConfig {
        pub device: i32,
        pub hidden: i32,
        pub heads: i32,
        pub kv_heads: i32,
        pub head_dim: i32,
        pub layers: i32,
        pub vocab: i32,
        pub slots: i32,
        pub max_ctx: i32,
        pub rope_theta: f32,
        pub rms_eps: f32,
    }

    #[repr(C)]
    pub struct MummuTrunk {
        _private: [u8; 0],
    }
}

pub use sys::{MUMMU_BF16, MUMMU_F16, MUMMU_F32, MUMMU_Q4_K, MUMMU_Q5_K, MUMMU_Q6_K, MUMMU_Q8_0};

/// The calling thread's last message from the library.
pub fn last_error() -> String {
    unsafe {
        let p = sys::mummu_cuda_last_error();
        if p.is_null() { String::new() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
    }
}

/// What went wrong in a call that does not panic.
#[derive(Debug, Clone, PartialEq, Eq)]
pub enum CudaMoeError {
    /// CUDA runtime / driver error.
    Device(String),
    /// A bounded device-side wait ran out (a peer never signalled).
    Timeout(String),
    /// Valid request this build has no kernel for.
    Unsupported(String),
    /// Non-finite router logit (the reference's host router returns `Err`,
    /// models/qwen4exp/experts.rs:553-560).
    Numeric(String),
}

/// Status -> `Result`; a contract violation is the reference's panic (nn/moe.rs:62-76, 119-126).
fn check(rc: i32) -> Result<(), CudaMoeError> {
    match rc {
        sys::MUMMU_OK => Ok(()),
        sys::MUMMU_ERR_CONTRACT => panic!("{}", last_error()),
        sys::MUMMU_ERR_TIMEOUT => Err(CudaMoeError::Timeout(last_error())),
        sys::MUMMU_ERR_UNSUPPORTED => Err(CudaMoeError::Unsupported(last_error())),
        sys::MUMMU_ERR_NUMERIC => Err(CudaMoeError::Numeric(last_error())),
        _ => Err(CudaMoeError::Device(last_error())),
    }
}

/// Stored precision of a bank, as `tier::Precision` names them plus the GGUF block formats.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum BankDtype {
    F32,
    F16,
    Bf16,
    Q4K,
    Q8_0,
    Q5K,
    Q6K,
}

impl BankDtype {
    pub fn code(self) -> i32 {
        match self {
            BankDtype::F32 => sys::MUMMU_F32,
            BankDtype::F16 => sys::MUMMU_F16,
            BankDtype::Bf16 => sys::MUMMU_BF16,
            BankDtype::Q4K => sys::MUMMU_Q4_K,
            BankDtype::Q8_0 => sys::MUMMU_Q8_0,
            BankDtype::Q5K => sys::MUMMU_Q5_K,
            BankDtype::Q6K => sys::MUMMU_Q6_K,
        }
    }
    fn from_code(c: i32) -> Self {
        match c {
            sys::MUMMU_F16 => BankDtype::F16,
            sys::MUMMU_BF16 => BankDtype::Bf16,
            sys::MUMMU_Q4_K => BankDtype::Q4K,
            sys::MUMMU_Q8_0 => BankDtype::Q8_0,
            sys::MUMMU_Q5_K => BankDtype::Q5K,
            sys::MUMMU_Q6_K => BankDtype::Q6K,
            _ => BankDtype::F32,
        }
    }
}

/// `SparseMoeConfig` (nn/moe.rs:42-50) plus where and how the bank is stored.
#[derive(Debug, Clone, Copy)]
pub struct CudaBankConfig {
    pub hidden_size: usize,
    pub expert_intermediate_size: usize,
    pub num_experts: usize,
    pub num_experts_per_tok: usize,
    pub device: usize,
    /// dtype of `x` / `y` on the device: F32, F16 or Bf16 (Q4_K banks run with F16 activations).
    pub act_dtype: BankDtype,
    pub weight_dtype: BankDtype,
    /// Expert parallelism: this handle stores `experts_local` experts from `expert_first`.
    pub expert_first: usize,
    pub experts_local: usize,
    /// Scratch is sized for this many tokens (0: grown on demand).
    pub max_tokens: usize,
}

/// One MoE layer on one B200: router weight, the three expert banks, scratch, one stream.
pub struct CudaBank {
    h: *mut sys::MummuMoe,
    cfg: CudaBankConfig,
}

// The handle serialises the host side of its calls with an internal lock (mummu_cuda.h).
unsafe impl Send for CudaBank {}
unsafe impl Sync for CudaBank {}

impl CudaBank {
    /// `SparseMoeConfig::init` (nn/moe.rs:61-99): the same asserts, with the same messages, come
    /// back from the library and are re-raised as panics.
    pub fn new(cfg: CudaBankConfig) -> Result<Self, CudaMoeError> {
        let c = sys::MummuMoeConfig {
            device: cfg.device as i32,
            hidden: cfg.hidden_size as i32,
            inter: cfg.expert_intermediate_size as i32,
            experts: cfg.num_experts as i32,
            top_k: cfg.num_experts_per_tok as i32,
            act_dtype: cfg.act_dtype.code(),
            weight_dtype: cfg.weight_dtype.code(),
            expert_first: cfg.expert_first as i32,
            experts_local: cfg.experts_local as i32,
            max_tokens: cfg.max_tokens as i32,
        };
        let mut h = ptr::null_mut();
        check(unsafe { sys::mummu_moe_create(&c, &mut h) })?;
        Ok(Self { h, cfg })
    }

    pub fn config(&self) -> &CudaBankConfig {
        &self.cfg
    }

    /// Raw handle for callers that drive the stage calls themselves (device pointers, own stream).
    pub fn raw(&self) -> *mut sys::MummuMoe {
        self.h
    }

    /// Router `gate: Linear` weight as burn stores it, `[hidden, experts]` f32 (nn/moe.rs:1642).
    pub fn set_router_in_out(&self, w: &[f32], bias: Option<&[f32]>) -> Result<(), CudaMoeError> {
        assert_eq!(w.len(), self.cfg.hidden_size * self.cfg.num_experts, "router weight size");
        let b = bias.map_or(ptr::null(), |b| b.as_ptr());
        check(unsafe { sys::mummu_moe_set_router(self.h, w.as_ptr().cast(), sys::MUMMU_F32, sys::MUMMU_ROUTER_IN_OUT, b) })
    }

    /// Router weight as GGUF `ffn_gate_inp` stores it, `[experts, hidden]` (models/olmoe.rs:338-339).
    pub fn set_router_out_in(&self, w: &[f32]) -> Result<(), CudaMoeError> {
        assert_eq!(w.len(), self.cfg.hidden_size * self.cfg.num_experts, "router weight size");
        check(unsafe {
            sys::mummu_moe_set_router(self.h, w.as_ptr().cast(), sys::MUMMU_F32, sys::MUMMU_ROUTER_OUT_IN, ptr::null())
        })
    }

    /// One of `MoeExperts::{gate, up, down}` (nn/moe.rs:22-30) as host bytes of the bank's dtype,
    /// `[experts_local, out, in]`; for Q4_K the raw `ffn_*_exps` tensor bytes of the GGUF file.
    pub fn set_bank(&self, which: i32, bytes: &[u8]) -> Result<(), CudaMoeError> {
        check(unsafe { sys::mummu_moe_set_bank(self.h, which, bytes.as_ptr().cast(), bytes.len(), 0) })
    }

    /// `SparseMoe::forward` / `SparseMoePerExpert::forward` (nn/moe.rs:116-177, 214-219) on host
    /// rows of the activation dtype (`x` and `y` hold `tokens * hidden` values as raw bytes).
    pub fn forward_host(&self, x: &[u8], y: &mut [u8], tokens: usize, top_k: usize, norm_topk_prob: bool) -> Result<(), CudaMoeError> {
        check(unsafe {
            sys::mummu_moe_forward(self.h, x.as_ptr().cast(), y.as_mut_ptr().cast(), tokens as i32, top_k as i32,
                                   norm_topk_prob as i32, 0, ptr::null_mut())
        })
    }

    /// The same on device pointers, queued on `stream` without waiting.
    ///
    /// # Safety
    /// `x` and `y` must be device allocations of `tokens * hidden` activation values on this
    /// bank's device, valid until the stream has passed the call.
    pub unsafe fn forward_device(&self, x: *const c_void, y: *mut c_void, tokens: usize, top_k: usize, norm_topk_prob: bool,
                                 stream: *mut c_void) -> Result<(), CudaMoeError> {
        check(sys::mummu_moe_forward(self.h, x, y, tokens as i32, top_k as i32, norm_topk_prob as i32, 1, stream))
    }

    /// `SparseMoePerExpert::route` (nn/moe.rs:247-290) as flat arrays: ids and weights
    /// `[tokens, top_k]`, descending probability, ties to the lowest expert id.
    pub fn route_host(&self, x: &[u8], tokens: usize, top_k: usize, norm_topk_prob: bool) -> Result<(Vec<i32>, Vec<f32>), CudaMoeError> {
        let mut ids = vec![0i32; tokens * top_k];
        let mut w = vec![0f32; tokens * top_k];
        check(unsafe {
            sys::mummu_moe_route(self.h, x.as_ptr().cast(), tokens as i32, top_k as i32, norm_topk_prob as i32,
                                 ids.as_mut_ptr(), w.as_mut_ptr(), 0, ptr::null_mut())
        })?;
        Ok((ids, w))
    }

    /// `ExpertPool::take_hits` (nn/moe.rs:1527-1535) for this layer.
    pub fn take_hits(&self) -> Result<Vec<u64>, CudaMoeError> {
        let mut hits = vec![0u64; self.cfg.num_experts];
        check(unsafe { sys::mummu_moe_take_hits(self.h, hits.as_mut_ptr()) })?;
        Ok(hits)
    }

    /// Wait for the handle's stream and report the sticky device status word.
    pub fn sync(&self) -> Result<(), CudaMoeError> {
        check(unsafe { sys::mummu_moe_sync(self.h, ptr::null_mut()) })
    }

    /// One kernel-variant switch (`MUMMU_CUDA_<NAME>` read at creation; see mummu_cuda.h).
    pub fn set_switch(&self, name: &str, value: i32) -> Result<(), CudaMoeError> {
        let n = CString::new(name).expect("switch name");
        check(unsafe { sys::mummu_moe_set_switch(self.h, n.as_ptr(), value) })
    }

    /// One expert of this bank as an executor.
    pub fn expert(&self, expert: usize) -> CudaExpert<'_> {
        CudaExpert { bank: self, expert }
    }
}

impl Drop for CudaBank {
    fn drop(&mut self) {
        unsafe {
            sys::mummu_moe_destroy(self.h);
        }
    }
}

/// One expert of a `CudaBank`, with the method set of `ExpertExec` (nn/moe.rs:348-419).
pub struct CudaExpert<'a> {
    bank: &'a CudaBank,
    expert: usize,
}

impl CudaExpert<'_> {
    /// `(device, stored precision)` — the two fields of `tier::Tier` (tier.rs:68-71).
    pub fn tier(&self) -> (usize, BankDtype) {
        let mut c = sys::MummuMoeConfig::default();
        let _ = unsafe { sys::mummu_moe_get_config(self.bank.h, &mut c) };
        (c.device as usize, BankDtype::from_code(c.weight_dtype))
    }

    pub fn resident_bytes(&self) -> u64 {
        unsafe { sys::mummu_expert_resident_bytes(self.bank.h, self.expert as i32) }
    }

    /// `run(&[f32], rows, hidden) -> Vec<f32>` (nn/moe.rs:353-357).
    pub fn run(&self, x: &[f32], rows: usize, hidden: usize) -> Vec<f32> {
        assert_eq!(hidden, self.bank.cfg.hidden_size, "expert input hidden");
        assert_eq!(x.len(), rows * hidden, "expert input size");
        let mut y = vec![0f32; rows * hidden];
        check(unsafe { sys::mummu_expert_run(self.bank.h, self.expert as i32, x.as_ptr(), rows as i32, y.as_mut_ptr()) })
            .expect("a dead worker is a dead generation, never a silently smaller sum (nn/moe.rs:1160-1163)");
        y
    }

    /// `run_tensor` / `run_tensor_resident` on device rows of the activation dtype.
    ///
    /// # Safety
    /// `x` and `y` must be device allocations of `rows * hidden` activation values on the bank's device.
    pub unsafe fn run_device(&self, x: *const c_void, rows: usize, y: *mut c_void, stream: *mut c_void) -> Result<(), CudaMoeError> {
        check(sys::mummu_expert_run_device(self.bank.h, self.expert as i32, x, rows as i32, y, stream))
    }

    /// `gate_energy` (nn/moe.rs:413-418).
    pub fn gate_energy(&self, x: &[f32], rows: usize, hidden: usize) -> Vec<f32> {
        assert_eq!(x.len(), rows * hidden, "gate_energy input size");
        let mut e = vec![0f32; rows];
        check(unsafe { sys::mummu_expert_gate_energy(self.bank.h, self.expert as i32, x.as_ptr(), rows as i32, e.as_mut_ptr()) })
            .expect("gate_energy");
        e
    }

    // pinned to its device: the trait's defaults
    pub fn disable_native(&self) {}
    pub fn stage(&self) {}
    pub fn evict(&self) {}
    pub fn is_staged(&self) -> bool {
        true
    }
}


/// The decode trunk of an OLMoE-shaped model on one B200 (`mummu_cuda.h`, section "decode trunk"):
/// what `impl StaticDecode for Olmoe` (capture.rs:48-107) holds as its `State`.  Every call takes
/// device pointers and one stream, allocates nothing and reads nothing back, so a step can be
/// captured once per bucket of keys.
pub struct CudaTrunk {
    h: *mut sys::MummuTrunk,
    cfg: sys::MummuTrunkConfig,
}

unsafe impl Send for CudaTrunk {}

impl CudaTrunk {
    /// `StaticDecode::static_bytes` (capture.rs:63-66): device bytes of the weights, the KV cache
    /// for `slots` sequences of `max_ctx` positions and the scratch.
    pub fn static_bytes(cfg: &sys::MummuTrunkConfig) -> u64 {
        unsafe { sys::mummu_trunk_static_bytes(cfg) }
    }

    /// `StaticDecode::static_state` (capture.rs:68-75).  A shape the kernels do not take is the
    /// reference's `static_supported() == false`: it comes back as `Unsupported`.
    pub fn new(cfg: sys::MummuTrunkConfig) -> Result<Self, CudaMoeError> {
        let mut h = ptr::null_mut();
        check(unsafe { sys::mummu_trunk_create(&cfg, &mut h) })?;
        Ok(Self { h, cfg })
    }

    pub fn config(&self) -> &sys::MummuTrunkConfig {
        &self.cfg
    }

    /// One weight tensor (`which` = MUMMU_TRUNK_EMBED .. K_NORM; `layer` ignored for the embedding,
    /// the final norm and lm_head) as host bytes: f16 matrices `[out, in]`, f32 norm weights.
    pub fn set_weight(&self, which: i32, layer: usize, bytes: &[u8]) -> Result<(), CudaMoeError> {
        check(unsafe { sys::mummu_trunk_set_weight(self.h, which, layer as i32, bytes.as_ptr().cast(), bytes.len(), 0) })
    }

    /// `StaticDecode::seed_static` (capture.rs:105-106) for one layer: `count` positions of keys
    /// and values from `first` on, device f16 `[kv_heads, count, head_dim]` each.
    ///
    /// # Safety
    /// `k` and `v` are device pointers of that size, valid until `stream` has passed the call.
    pub unsafe fn kv_write(&self, layer: usize, slot: usize, first: usize, count: usize, k: *const c_void,
                           v: *const c_void, stream: *mut c_void) -> Result<(), CudaMoeError> {
        check(sys::mummu_trunk_kv_write(self.h, layer as i32, slot as i32, first as i32, count as i32, k, v, stream))
    }

    /// One `forward_static` step (capture.rs:77-103; models/olmoe.rs:553-587) over `banks`, one
    /// `CudaBank` per layer with f16 activations: embedding, then per layer the attention half
    /// (which first joins the previous layer's expert output to the residual stream) and the
    /// layer's expert bank, then the head.  `tokens`, `positions`: device int32 `[slots]`;
    /// `x`, `h2`, `y`: device f16 `[slots, hidden]` scratch; `logits`: device f32 `[slots, vocab]`;
    /// `argmax`: device int32 `[slots]` or null.  `length`: the bucket of keys attended to.
    ///
    /// # Safety
    /// All pointers are device pointers of the stated sizes, valid until `stream` has passed the
    /// calls; nothing else uses the banks or this trunk on another stream meanwhile.
    #[allow(clippy::too_many_arguments)]
    pub unsafe fn forward_static(&self, banks: &[CudaBank], top_k: usize, norm_topk_prob: bool, tokens: *const i32,
                                 positions: *const i32, slots: usize, length: usize, x: *mut c_void, h2: *mut c_void,
                                 y: *mut c_void, logits: *mut f32, argmax: *mut i32, stream: *mut c_void)
                                 -> Result<(), CudaMoeError> {
        assert_eq!(banks.len(), self.cfg.layers as usize, "one expert bank per layer");
        check(sys::mummu_trunk_embed(self.h, tokens, slots as i32, x, stream))?;
        let mut y_prev: *const c_void = ptr::null();
        for (layer, bank) in banks.iter().enumerate() {
            check(sys::mummu_trunk_attention_step(self.h, layer as i32, x, y_prev, positions, slots as i32, length as i32,
                                                  h2, stream))?;
            check(sys::mummu_moe_forward(bank.raw(), h2, y, slots as i32, top_k as i32, norm_topk_prob as i32, 1, stream))?;
            y_prev = y;
        }
        check(sys::mummu_trunk_head(self.h, x, y_prev, slots as i32, logits, argmax, stream))
    }
}

impl Drop for CudaTrunk {
    fn drop(&mut self) {
        unsafe {
            sys::mummu_trunk_destroy(self.h);
        }
    }
}

// -------------------------------------------------------------------------------------------------
// Glue that lives in crates/mummu/src/nn/moe.rs under `#[cfg(feature = "cuda-b200")]` (shown here
// because this crate cannot name `ExpertExec`, `Tensor` or `Tier`):
//
//     pub struct OwnedCudaExpert { bank: Arc<mummu_cuda::CudaBank>, expert: usize }
//
//     impl ExpertExec for OwnedCudaExpert {
//         fn tier(&self) -> crate::tier::Tier {
//             let (device, dt) = self.bank.expert(self.expert).tier();
//             crate::tier::Tier { device, precision: precision_of(dt) }
//         }
//         fn resident_bytes(&self) -> u64 { self.bank.expert(self.expert).resident_bytes() }
//         fn run(&self, x: &[f32], rows: usize, hidden: usize) -> Vec<f32> {
//             self.bank.expert(self.expert).run(x, rows, hidden)
//         }
//         fn run_tensor(&self, x: Tensor<2>) -> Tensor<2> { /* cubecl CUDA buffer -> run_device */ }
//         fn run_tensor_resident(&self, x: Tensor<2>) -> Tensor<2> { self.run_tensor(x) }
//         fn gate_energy(&self, x: &[f32], rows: usize, hidden: usize) -> Vec<f32> {
//             self.bank.expert(self.expert).gate_energy(x, rows, hidden)
//         }
//         // disable_native, stage, evict, is_staged: the trait's defaults (a pinned executor)
//     }
//
// and in `SparseMoe::forward` (nn/moe.rs:116), unchanged signature:
//
//     #[cfg(feature = "cuda-b200")]
//     if let Some(bank) = &self.cuda {
//         let [b, t, h] = x.dims();
//         let host: Vec<f32> = x.into_data().convert::<f32>().to_vec().unwrap();
//         let mut out = vec![0f32; b * t * h];
//         bank.forward_host(bytemuck::cast_slice(&host), bytemuck::cast_slice_mut(&mut out), b * t, top_k,
//                           norm_topk_prob).expect("cuda expert bank");
//         return Tensor::from_data(TensorData::new(out, [b, t, h]), &self.device);
//     }
// -------------------------------------------------------------------------------------------------
