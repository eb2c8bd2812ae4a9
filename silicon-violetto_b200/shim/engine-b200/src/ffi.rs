//! The C ABI of include/violetto.h, declaration for declaration. Plain data and opaque handles only.
#![allow(non_camel_case_types, dead_code)]
use std::ffi::{c_char, c_int, c_void};

#[repr(C)]
pub struct VltEngine {
    _p: [u8; 0],
}
#[repr(C)]
pub struct VltGenerator {
    _p: [u8; 0],
}
#[repr(C)]
pub struct VltRouter {
    _p: [u8; 0],
}

pub const VLT_FEED_ROW: u32 = 0xffff_0000;
pub const VLT_FEED_W: u32 = 16;
pub const VLT_NO_TOK: u32 = 0xffff_ffff;
pub const VLT_VERIFY_T: u32 = 8;
pub const VLT_MAX_STOP: u32 = 8;
pub const VLT_FLAG_HOST_ONLY: u32 = 1;

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct VltEngineConfig {
    pub max_seqs: u32,
    pub max_step_tokens: u32,
    pub max_chunk: u32,
    pub global_kv_tokens: u32,
    pub max_seq_len: u32,
    pub max_head_rows: u32,
    pub device_ordinal: i32,
    pub flags: u32,
}
#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct VltTuning {
    pub spec_tokens: u32,
    pub spec_tokens_short: u32,
    pub spec_kv: u32,
    pub spec_rows_long: u32,
    pub spec_policy_off: u32,
    pub sm_count: u32,
    pub attn_keys_per_cta: u32,
    pub gemm_min_rows: u32,
    pub plain_attention: u32,
    pub gemm_unpaired: u32,
}
#[repr(C)]
#[derive(Clone, Copy)]
pub struct VltSampling {
    pub temperature: f32,
    pub top_p: f32,
    pub seed: u64,
}
#[repr(C)]
pub struct VltRun {
    pub seq: u32,
    pub tokens: *const u32,
    pub n_tokens: u32,
}
#[repr(C)]
pub struct VltStepOptions {
    pub head: u32,
    pub hidden: u32,
    pub read_logits: u32,
    pub read_taps: u32,
}
#[repr(C)]
pub struct VltStepOutput {
    pub ids: *mut u32,
    pub ids_cap: u32,
    pub n_ids: u32,
    pub logits: *mut f32,
    pub logits_cap: u64,
    pub hidden: *mut f32,
    pub hidden_cap: u64,
    pub n_hidden: u32,
    pub taps: *mut u16,
    pub taps_cap: u64,
    pub gpu_seconds: f64,
    pub n_taps: u32,
}
#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct VltModelDesc {
    pub n_layers: u32,
    pub d_model: u32,
    pub n_heads: u32,
    pub n_kv_heads: u32,
    pub head_dim: u32,
    pub ffn: u32,
    pub vocab: u32,
    pub vocab_real: u32,
    pub page_size: u32,
    pub rms_eps: f32,
    pub attn_scale: f32,
    pub int8: u32,
}
#[repr(C)]
pub struct VltLayerCapture {
    pub layer: u32,
    pub n: u32,
    pub d_model: u32,
    pub qkv_width: u32,
    pub attn_width: u32,
    pub resid_in: *const f32,
    pub attn_in: *const f32,
    pub qkv: *const f32,
    pub sdpa_out: *const f32,
    pub attn_out: *const f32,
    pub mlp_in: *const f32,
    pub mlp_out: *const f32,
    pub resid_base: *const f32,
}
pub type VltCaptureFn = extern "C" fn(layer: *const VltLayerCapture, user: *mut c_void);
#[repr(C)]
pub struct VltRequest {
    pub prompt_kind: u32,
    pub prompt_tokens: *const u32,
    pub n_prompt: u32,
    pub resume_seq: u32,
    pub resume_token: u32,
    pub max_tokens: u32,
    pub stop: *const u32,
    pub n_stop: u32,
    pub sampling: VltSampling,
    pub draft_kind: u32,
    pub draft_rows: u32,
    pub trace: *const u32,
    pub n_trace: u32,
}
#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct VltEvent {
    pub kind: u32,
    pub req: u32,
    pub value: u32,
}
#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct VltStepStats {
    pub tokens: u32,
    pub decode: u32,
    pub emitted: u32,
    pub gpu_seconds: f64,
    pub encode_seconds: f64,
}
#[repr(C)]
pub struct VltReplicaOps {
    pub ctx: *mut c_void,
    pub submit: Option<extern "C" fn(*mut c_void, *const VltRequest, *mut u32) -> c_int>,
    pub step: Option<extern "C" fn(*mut c_void, *mut VltEvent, u32, *mut u32) -> c_int>,
    pub cancel: Option<extern "C" fn(*mut c_void, u32)>,
    pub is_idle: Option<extern "C" fn(*mut c_void) -> c_int>,
    pub counts: Option<extern "C" fn(*mut c_void, *mut u32, *mut u32)>,
}

extern "C" {
    pub fn vlt_last_error() -> *const c_char;
    pub fn vlt_engine_new(path: *const c_char, cfg: *const VltEngineConfig, tuning: *const VltTuning, out: *mut *mut VltEngine) -> c_int;
    pub fn vlt_engine_free(e: *mut VltEngine);
    pub fn vlt_device_name(e: *mut VltEngine, buf: *mut c_char, cap: usize) -> c_int;
    pub fn vlt_model_desc(e: *mut VltEngine, out: *mut VltModelDesc) -> c_int;
    pub fn vlt_seq_new(e: *mut VltEngine, seq: *mut u32) -> c_int;
    pub fn vlt_seq_free(e: *mut VltEngine, seq: u32);
    pub fn vlt_seq_len(e: *mut VltEngine, seq: u32) -> u32;
    pub fn vlt_seq_set_sampling(e: *mut VltEngine, seq: u32, s: *const VltSampling) -> c_int;
    pub fn vlt_step(e: *mut VltEngine, runs: *const VltRun, n_runs: u32, opts: *const VltStepOptions, out: *mut VltStepOutput) -> c_int;
    pub fn vlt_step_capture(e: *mut VltEngine, runs: *const VltRun, n_runs: u32, opts: *const VltStepOptions, f: VltCaptureFn, user: *mut c_void, out: *mut VltStepOutput) -> c_int;
    pub fn vlt_set_taps(e: *mut VltEngine, layers: *const u32, n_layers: u32) -> c_int;
    pub fn vlt_load_drafter(e: *mut VltEngine, path: *const c_char) -> c_int;
    pub fn vlt_has_drafter(e: *mut VltEngine) -> c_int;
    pub fn vlt_set_acceptance(e: *mut VltEngine, rule: u32) -> c_int;
    pub fn vlt_bench_fill(e: *mut VltEngine, seq: u32, len: u32, seed: u32) -> c_int;
    pub fn vlt_sample_logits(e: *mut VltEngine, logits: *const f32, rows: *const VltSampling, pos: *const u32, n: u32, out: *mut u32) -> c_int;
    pub fn vlt_set_profile_skip(e: *mut VltEngine, mask: u32);
    pub fn vlt_bench_matmul(e: *mut VltEngine, kind: *const c_char, n: u32, variant: u32, reps: u32, seconds: *mut f64, bytes: *mut u64) -> c_int;
    pub fn vlt_generator_new(e: *mut VltEngine, out: *mut *mut VltGenerator) -> c_int;
    pub fn vlt_generator_free(g: *mut VltGenerator);
    pub fn vlt_generator_submit(g: *mut VltGenerator, req: *const VltRequest, req_id: *mut u32) -> c_int;
    pub fn vlt_generator_cancel(g: *mut VltGenerator, req_id: u32);
    pub fn vlt_generator_step(g: *mut VltGenerator, events: *mut VltEvent, cap: u32, n_events: *mut u32) -> c_int;
    pub fn vlt_generator_is_idle(g: *mut VltGenerator) -> c_int;
    pub fn vlt_generator_counts(g: *mut VltGenerator, queued: *mut u32, running: *mut u32);
    pub fn vlt_generator_stats(g: *mut VltGenerator, out: *mut VltStepStats, cap: u32, n: *mut u32) -> c_int;
    pub fn vlt_generator_set_hold(g: *mut VltGenerator, hold: u32);
    pub fn vlt_generator_set_replay_mistakes(g: *mut VltGenerator, rate: f32, seed: u32);
    pub fn vlt_replica_of_generator(g: *mut VltGenerator, out: *mut VltReplicaOps);
    pub fn vlt_router_new(replicas: *const VltReplicaOps, n: u32, out: *mut *mut VltRouter) -> c_int;
    pub fn vlt_router_free(r: *mut VltRouter);
    pub fn vlt_router_submit(r: *mut VltRouter, req: *const VltRequest, req_id: *mut u32) -> c_int;
    pub fn vlt_router_cancel(r: *mut VltRouter, req_id: u32);
    pub fn vlt_router_step(r: *mut VltRouter, events: *mut VltEvent, cap: u32, n_events: *mut u32) -> c_int;
    pub fn vlt_router_is_idle(r: *mut VltRouter) -> c_int;
    pub fn vlt_router_alive(r: *mut VltRouter) -> u32;
}
