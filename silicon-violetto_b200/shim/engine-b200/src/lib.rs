//! The reference crate's public API (engine/src/lib.rs:6-10: `Engine`, `EngineConfig`, `Tuning`, `Sampling`, `SeqId`,
//! `Rows`, `Run`, `StepOptions`, `StepOutput`, `LayerCapture`, `Generator`, `Request`, `Prompt`, `Draft`, `ReqId`,
//! `Event`, `Finish`, `StepStats`, `skip`) over libvioletto_b200.so, so that `cli/` builds against this crate unchanged.
//! Each item cites the reference item it stands for. NOT COMPILED where this repository is built (no Rust toolchain
//! there): the Python mirror `silicon-violetto_b200/engine.py` exercises the same C calls in the tests.
//!
//! What differs from the reference's crate, on purpose: the model's shape comes from the weight file (`Engine::desc`)
//! instead of the constants of engine/src/model.rs:6-20; `EngineConfig` has a `device` ordinal (one engine per GPU is a
//! replica); `Tuning` carries B200 knobs in place of the Apple-GPU ones; `Matmul` and `DrafterDebug` (Apple-specific
//! kernel variants, the reference drafter's debug dump) have no counterpart.
mod ffi;

use std::ffi::{c_void, CStr, CString};
use std::marker::PhantomData;
use std::path::Path;

fn check(rc: i32) -> Result<(), String> {
    if rc == 0 {
        return Ok(());
    }
    Err(unsafe { CStr::from_ptr(ffi::vlt_last_error()) }.to_string_lossy().into_owned())
}

/// engine/src/engine.rs:31-57.
#[derive(Clone, Debug)]
pub struct EngineConfig {
    pub max_seqs: usize,
    pub max_step_tokens: usize,
    pub max_chunk: usize,
    pub global_kv_tokens: usize,
    pub max_seq_len: usize,
    pub max_head_rows: usize,
    /// New: the CUDA device this engine runs on.
    pub device: i32,
}
impl Default for EngineConfig {
    fn default() -> Self {
        EngineConfig { max_seqs: 8, max_step_tokens: 512, max_chunk: 512, global_kv_tokens: 65536, max_seq_len: 131072, max_head_rows: 64, device: 0 }
    }
}

/// engine/src/engine.rs:59-95: the rows policy is the reference's; the Apple-GPU knobs are replaced (0 = default).
#[derive(Clone, Debug)]
pub struct Tuning {
    pub spec_tokens: usize,
    pub spec_tokens_short: usize,
    pub spec_kv: usize,
    pub spec_rows_long: usize,
    pub sm_count: usize,
    pub attn_keys_per_cta: usize,
    pub gemm_min_rows: usize,
}
impl Default for Tuning {
    fn default() -> Self {
        Tuning { spec_tokens: 32, spec_tokens_short: 8, spec_kv: 24576, spec_rows_long: 4, sm_count: 0, attn_keys_per_cta: 0, gemm_min_rows: 0 }
    }
}

/// engine/src/engine.rs:98.
#[derive(Clone, Copy, Debug, PartialEq, Eq, Hash)]
pub struct SeqId(pub u32);

/// engine/src/engine.rs:100-138.
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct Sampling {
    pub temperature: f32,
    pub top_p: f32,
    pub seed: u64,
}
impl Sampling {
    pub const GREEDY: Sampling = Sampling { temperature: 0.0, top_p: 1.0, seed: 0 };
    fn c(&self) -> ffi::VltSampling {
        ffi::VltSampling { temperature: self.temperature, top_p: self.top_p, seed: self.seed }
    }
}

/// engine/src/engine.rs:140-147.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum Rows {
    None,
    Last,
    All,
}
/// engine/src/engine.rs:149-152.
pub struct Run<'a> {
    pub seq: SeqId,
    pub tokens: &'a [u32],
}
/// engine/src/engine.rs:154-161.
pub struct StepOptions {
    pub head: Rows,
    pub hidden: Rows,
    pub read_logits: bool,
    pub read_taps: bool,
}
/// engine/src/engine.rs:163-173.
#[derive(Default)]
pub struct StepOutput {
    pub ids: Vec<u32>,
    pub logits: Vec<f32>,
    pub hidden: Vec<f32>,
    pub taps: Vec<u16>,
    pub gpu_seconds: f64,
}
/// engine/src/engine.rs:175-188.
pub struct LayerCapture<'a> {
    pub layer: usize,
    pub n: usize,
    pub resid_in: &'a [f32],
    pub attn_in: &'a [f32],
    pub qkv: &'a [f32],
    pub sdpa_out: &'a [f32],
    pub attn_out: &'a [f32],
    pub mlp_in: &'a [f32],
    pub mlp_out: &'a [f32],
    pub resid_base: Option<&'a [f32]>,
}

/// engine/src/engine/hooks.rs:9-19.
pub mod skip {
    pub const QKV: u32 = 1;
    pub const POST: u32 = 2;
    pub const ATTN: u32 = 4;
    pub const REDUCE: u32 = 8;
    pub const O: u32 = 16;
    pub const GATE_UP: u32 = 32;
    pub const DOWN: u32 = 64;
    pub const HEAD: u32 = 256;
}

/// engine/src/engine.rs:197 `Engine`. Thread-affine, like the reference's (cli/src/serve.rs:100): not Send, not Sync.
pub struct Engine {
    h: *mut ffi::VltEngine,
    cfg: EngineConfig,
    desc: ffi::VltModelDesc,
    taps: usize,
    _not_send: PhantomData<*mut ()>,
}

impl Engine {
    /// engine/src/engine.rs:221.
    pub fn new(weights: &Path, cfg: EngineConfig, tuning: Tuning) -> Result<Self, String> {
        let path = CString::new(weights.to_string_lossy().as_bytes()).map_err(|e| e.to_string())?;
        let c = ffi::VltEngineConfig {
            max_seqs: cfg.max_seqs as u32,
            max_step_tokens: cfg.max_step_tokens as u32,
            max_chunk: cfg.max_chunk as u32,
            global_kv_tokens: cfg.global_kv_tokens as u32,
            max_seq_len: cfg.max_seq_len as u32,
            max_head_rows: cfg.max_head_rows as u32,
            device_ordinal: cfg.device,
            flags: 0,
        };
        let t = ffi::VltTuning {
            spec_tokens: tuning.spec_tokens as u32,
            spec_tokens_short: tuning.spec_tokens_short as u32,
            spec_kv: tuning.spec_kv as u32,
            spec_rows_long: tuning.spec_rows_long as u32,
            spec_policy_off: (tuning.spec_tokens == 0) as u32,
            sm_count: tuning.sm_count as u32,
            attn_keys_per_cta: tuning.attn_keys_per_cta as u32,
            gemm_min_rows: tuning.gemm_min_rows as u32,
            plain_attention: 0,
            gemm_unpaired: 0,
        };
        let mut h = std::ptr::null_mut();
        check(unsafe { ffi::vlt_engine_new(path.as_ptr(), &c, &t, &mut h) })?;
        let mut desc = ffi::VltModelDesc::default();
        check(unsafe { ffi::vlt_model_desc(h, &mut desc) })?;
        Ok(Engine { h, cfg, desc, taps: 0, _not_send: PhantomData })
    }
    /// New: the model's shape (the reference exports constants, engine/src/model.rs:6-20).
    pub fn desc(&self) -> (usize, usize, usize) {
        (self.desc.n_layers as usize, self.desc.d_model as usize, self.desc.vocab as usize)
    }
    /// engine/src/engine.rs:252.
    pub fn device_name(&self) -> String {
        let mut buf = vec![0 as std::ffi::c_char; 256];
        match check(unsafe { ffi::vlt_device_name(self.h, buf.as_mut_ptr(), buf.len()) }) {
            Ok(()) => unsafe { CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned(),
            Err(e) => e,
        }
    }
    /// engine/src/engine.rs:267.
    pub fn new_seq(&mut self) -> Result<SeqId, String> {
        let mut s = 0;
        check(unsafe { ffi::vlt_seq_new(self.h, &mut s) })?;
        Ok(SeqId(s))
    }
    /// engine/src/engine.rs:288.
    pub fn set_sampling(&mut self, id: SeqId, sampling: Sampling) -> Result<(), String> {
        check(unsafe { ffi::vlt_seq_set_sampling(self.h, id.0, &sampling.c()) })
    }
    /// engine/src/engine.rs:299.
    pub fn free_seq(&mut self, id: SeqId) {
        unsafe { ffi::vlt_seq_free(self.h, id.0) }
    }
    /// engine/src/engine.rs:305.
    pub fn seq_len(&self, id: SeqId) -> usize {
        unsafe { ffi::vlt_seq_len(self.h, id.0) as usize }
    }

    fn runs_of(runs: &[Run]) -> Vec<ffi::VltRun> {
        runs.iter().map(|r| ffi::VltRun { seq: r.seq.0, tokens: r.tokens.as_ptr(), n_tokens: r.tokens.len() as u32 }).collect()
    }
    fn opts_of(o: &StepOptions) -> ffi::VltStepOptions {
        let rows = |r: Rows| match r {
            Rows::None => 0,
            Rows::Last => 1,
            Rows::All => 2,
        };
        ffi::VltStepOptions { head: rows(o.head), hidden: rows(o.hidden), read_logits: o.read_logits as u32, read_taps: o.read_taps as u32 }
    }
    fn step_with(&mut self, runs: &[Run], opts: &StepOptions, capture: Option<(ffi::VltCaptureFn, *mut c_void)>) -> Result<StepOutput, String> {
        let n: usize = runs.iter().map(|r| r.tokens.len()).sum();
        let (d, v) = (self.desc.d_model as usize, self.desc.vocab as usize);
        let rows = self.cfg.max_head_rows;
        let mut out = StepOutput { ids: vec![0; rows], ..Default::default() };
        if opts.read_logits {
            out.logits = vec![0.0; rows * v];
        }
        if opts.hidden != Rows::None {
            out.hidden = vec![0.0; n * d];
        }
        if opts.read_taps {
            out.taps = vec![0; (self.taps + 1) * n * d];
        }
        let mut c = ffi::VltStepOutput {
            ids: out.ids.as_mut_ptr(),
            ids_cap: rows as u32,
            n_ids: 0,
            logits: out.logits.as_mut_ptr(),
            logits_cap: out.logits.len() as u64,
            hidden: out.hidden.as_mut_ptr(),
            hidden_cap: out.hidden.len() as u64,
            n_hidden: 0,
            taps: out.taps.as_mut_ptr(),
            taps_cap: out.taps.len() as u64,
            gpu_seconds: 0.0,
            n_taps: 0,
        };
        let (cr, co) = (Self::runs_of(runs), Self::opts_of(opts));
        check(match capture {
            None => unsafe { ffi::vlt_step(self.h, cr.as_ptr(), cr.len() as u32, &co, &mut c) },
            Some((f, user)) => unsafe { ffi::vlt_step_capture(self.h, cr.as_ptr(), cr.len() as u32, &co, f, user, &mut c) },
        })?;
        out.ids.truncate(c.n_ids as usize);
        out.logits.truncate(c.n_ids as usize * v);
        out.hidden.truncate(c.n_hidden as usize * d);
        out.taps.truncate(c.n_taps as usize * n * d);
        out.gpu_seconds = c.gpu_seconds;
        Ok(out)
    }
    /// engine/src/engine.rs:310.
    pub fn step(&mut self, runs: &[Run], opts: &StepOptions) -> Result<StepOutput, String> {
        self.step_with(runs, opts, None)
    }
    /// engine/src/engine.rs:318.
    pub fn step_capture(&mut self, runs: &[Run], opts: &StepOptions, f: &mut dyn FnMut(&LayerCapture)) -> Result<StepOutput, String> {
        extern "C" fn tramp(c: *const ffi::VltLayerCapture, user: *mut c_void) {
            let (c, f) = unsafe { (&*c, &mut *(user as *mut &mut dyn FnMut(&LayerCapture))) };
            let s = |p: *const f32, w: u32| unsafe { std::slice::from_raw_parts(p, (c.n * w) as usize) };
            f(&LayerCapture {
                layer: c.layer as usize,
                n: c.n as usize,
                resid_in: s(c.resid_in, c.d_model),
                attn_in: s(c.attn_in, c.d_model),
                qkv: s(c.qkv, c.qkv_width),
                sdpa_out: s(c.sdpa_out, c.attn_width),
                attn_out: s(c.attn_out, c.d_model),
                mlp_in: s(c.mlp_in, c.d_model),
                mlp_out: s(c.mlp_out, c.d_model),
                resid_base: if c.resid_base.is_null() { None } else { Some(s(c.resid_base, c.d_model)) },
            });
        }
        let mut f = f;
        self.step_with(runs, opts, Some((tramp, &mut f as *mut &mut dyn FnMut(&LayerCapture) as *mut c_void)))
    }
    /// engine/src/engine.rs:382.
    pub fn set_taps(&mut self, layers: &[usize]) -> Result<(), String> {
        let l: Vec<u32> = layers.iter().map(|&x| x as u32).collect();
        check(unsafe { ffi::vlt_set_taps(self.h, l.as_ptr(), l.len() as u32) })?;
        self.taps = layers.len();
        Ok(())
    }
    /// engine/src/engine/drafter.rs:250.
    pub fn load_drafter(&mut self, path: &Path) -> Result<(), String> {
        let p = CString::new(path.to_string_lossy().as_bytes()).map_err(|e| e.to_string())?;
        check(unsafe { ffi::vlt_load_drafter(self.h, p.as_ptr()) })
    }
    /// engine/src/engine/drafter.rs:257.
    pub fn has_drafter(&self) -> bool {
        unsafe { ffi::vlt_has_drafter(self.h) != 0 }
    }
    /// New: 0 the reference's sample-then-match acceptance, 1 rejection sampling against the drafter's distribution.
    pub fn set_acceptance(&mut self, rule: u32) -> Result<(), String> {
        check(unsafe { ffi::vlt_set_acceptance(self.h, rule) })
    }
    /// engine/src/engine/hooks.rs:24.
    pub fn set_profile_skip(&mut self, mask: u32) {
        unsafe { ffi::vlt_set_profile_skip(self.h, mask) }
    }
    /// engine/src/engine/hooks.rs:31.
    pub fn bench_fill(&mut self, id: SeqId, len: usize) -> Result<(), String> {
        check(unsafe { ffi::vlt_bench_fill(self.h, id.0, len as u32, 0) })
    }
    /// engine/src/engine/hooks.rs:41.
    pub fn sample_logits(&mut self, logits: Option<&[f32]>, rows: &[(Sampling, usize)]) -> Result<Vec<u32>, String> {
        let s: Vec<ffi::VltSampling> = rows.iter().map(|(s, _)| s.c()).collect();
        let p: Vec<u32> = rows.iter().map(|&(_, p)| p as u32).collect();
        let mut out = vec![0u32; rows.len()];
        let lp = logits.map_or(std::ptr::null(), |l| l.as_ptr());
        check(unsafe { ffi::vlt_sample_logits(self.h, lp, s.as_ptr(), p.as_ptr(), rows.len() as u32, out.as_mut_ptr()) })?;
        Ok(out)
    }
    /// engine/src/engine/generate.rs:170.
    pub fn generator(&mut self) -> Result<Generator<'_>, String> {
        let mut g = std::ptr::null_mut();
        check(unsafe { ffi::vlt_generator_new(self.h, &mut g) })?;
        Ok(Generator { h: g, stats: Vec::new(), _engine: PhantomData })
    }
}
impl Drop for Engine {
    fn drop(&mut self) {
        unsafe { ffi::vlt_engine_free(self.h) }
    }
}

/// engine/src/engine/generate.rs:12-21.
pub struct Request {
    pub prompt: Prompt,
    pub max_tokens: usize,
    pub stop: Vec<u32>,
    pub sampling: Sampling,
    pub draft: Draft,
}
/// engine/src/engine/generate.rs:24-33.
#[derive(Clone, Debug, PartialEq)]
pub enum Draft {
    None,
    Replay { rows: usize, trace: Vec<u32> },
    Model { rows: usize },
}
/// engine/src/engine/generate.rs:55-61.
pub enum Prompt {
    Tokens(Vec<u32>),
    Resume(SeqId, u32),
}
/// engine/src/engine/generate.rs:65.
#[derive(Clone, Copy, Debug, PartialEq, Eq, Hash)]
pub struct ReqId(pub usize);
/// engine/src/engine/generate.rs:68-73.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum Finish {
    Stop,
    Length,
}
/// engine/src/engine/generate.rs:76-79.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum Event {
    Token(ReqId, u32),
    Done(ReqId, Finish),
}
/// engine/src/engine/generate.rs:81-91.
#[derive(Clone, Copy, Debug)]
pub struct StepStats {
    pub tokens: usize,
    pub decode: bool,
    pub emitted: usize,
    pub gpu_seconds: f64,
    pub encode_seconds: f64,
}

/// engine/src/engine/generate.rs:95 `Generator`: borrows its engine for its lifetime, frees its sequences on drop.
pub struct Generator<'e> {
    h: *mut ffi::VltGenerator,
    /// One entry per collected step (the reference's public `stats` field); refreshed by `step`.
    pub stats: Vec<StepStats>,
    _engine: PhantomData<&'e mut Engine>,
}
impl Generator<'_> {
    /// engine/src/engine/generate.rs:196.
    pub fn set_replay_mistakes(&mut self, rate: f32, seed: u32) {
        unsafe { ffi::vlt_generator_set_replay_mistakes(self.h, rate, seed) }
    }
    /// engine/src/engine/generate.rs:201.
    pub fn submit(&mut self, req: Request) -> Result<ReqId, String> {
        let (kind, prompt, seq, tok): (u32, &[u32], u32, u32) = match &req.prompt {
            Prompt::Tokens(t) => (0, t, 0, 0),
            Prompt::Resume(s, t) => (1, &[], s.0, *t),
        };
        let (dk, rows, trace): (u32, usize, &[u32]) = match &req.draft {
            Draft::None => (0, 1, &[]),
            Draft::Replay { rows, trace } => (1, *rows, trace),
            Draft::Model { rows } => (2, *rows, &[]),
        };
        let c = ffi::VltRequest {
            prompt_kind: kind,
            prompt_tokens: prompt.as_ptr(),
            n_prompt: prompt.len() as u32,
            resume_seq: seq,
            resume_token: tok,
            max_tokens: req.max_tokens as u32,
            stop: req.stop.as_ptr(),
            n_stop: req.stop.len() as u32,
            sampling: req.sampling.c(),
            draft_kind: dk,
            draft_rows: rows as u32,
            trace: trace.as_ptr(),
            n_trace: trace.len() as u32,
        };
        let mut id = 0;
        check(unsafe { ffi::vlt_generator_submit(self.h, &c, &mut id) })?;
        Ok(ReqId(id as usize))
    }
    /// engine/src/engine/generate.rs:248.
    pub fn is_idle(&self) -> bool {
        unsafe { ffi::vlt_generator_is_idle(self.h) != 0 }
    }
    /// engine/src/engine/generate.rs:253.
    pub fn counts(&self) -> (usize, usize) {
        let (mut q, mut r) = (0, 0);
        unsafe { ffi::vlt_generator_counts(self.h, &mut q, &mut r) };
        (q as usize, r as usize)
    }
    /// engine/src/engine/generate.rs:259.
    pub fn cancel(&mut self, id: ReqId) {
        unsafe { ffi::vlt_generator_cancel(self.h, id.0 as u32) }
    }
    /// engine/src/engine/generate.rs:271: commits the next step, returns the previous step's events.
    pub fn step(&mut self) -> Result<Vec<Event>, String> {
        let mut buf = vec![ffi::VltEvent::default(); 4096];
        let mut n = 0;
        check(unsafe { ffi::vlt_generator_step(self.h, buf.as_mut_ptr(), buf.len() as u32, &mut n) })?;
        let mut st = vec![ffi::VltStepStats::default(); 64];
        let mut ns = 0;
        check(unsafe { ffi::vlt_generator_stats(self.h, st.as_mut_ptr(), st.len() as u32, &mut ns) })?;
        self.stats.extend(st[..ns as usize].iter().map(|s| StepStats {
            tokens: s.tokens as usize,
            decode: s.decode != 0,
            emitted: s.emitted as usize,
            gpu_seconds: s.gpu_seconds,
            encode_seconds: s.encode_seconds,
        }));
        Ok(buf[..n as usize]
            .iter()
            .map(|e| match e.kind {
                0 => Event::Token(ReqId(e.req as usize), e.value),
                _ => Event::Done(ReqId(e.req as usize), if e.value == 0 { Finish::Stop } else { Finish::Length }),
            })
            .collect())
    }
    /// The reference's `hold` field (generate.rs:112): decode runs wait while set.
    pub fn set_hold(&mut self, hold: bool) {
        unsafe { ffi::vlt_generator_set_hold(self.h, hold as u32) }
    }
}
impl Drop for Generator<'_> {
    /// engine/src/engine/generate.rs:503-518.
    fn drop(&mut self) {
        unsafe { ffi::vlt_generator_free(self.h) }
    }
}
