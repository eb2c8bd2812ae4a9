/* C ABI of the B200 back end for Silicon Violetto's speculative-decoding decode step.
 *
 * The reference is a Rust crate whose public API is `violetto::{Engine, Generator, ...}`
 * (engine/src/lib.rs:6-10) over Metal. This library offers the same calls over CUDA, one
 * `extern "C"` function per method, so that a thin Rust shim can re-export the crate's API
 * unchanged. Each declaration cites the reference item it replaces (paths are relative to
 * the reference repository).
 *
 * Conventions. Every fallible call returns 0 on success and non-zero on failure;
 * `vlt_last_error()` then gives the message (the reference returns `Result<_, String>`).
 * Handles are opaque and, like the reference's `Engine`, thread-affine: use an engine and its
 * generator from the thread that created them (cli/src/serve.rs:100). Output buffers are
 * owned by the caller and passed with their capacities. All arithmetic runs on the GPU
 * selected by `device_ordinal`; there is no CPU path, and creating an engine without a
 * usable CUDA device fails unless `VLT_FLAG_HOST_ONLY` is set, in which case the engine plans
 * steps (page tables, step layout) but refuses to run them.
 */
#ifndef VIOLETTO_B200_H
#define VIOLETTO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct VltEngine VltEngine;
typedef struct VltGenerator VltGenerator;

/* engine/src/engine/kernels.rs:14-29 */
#define VLT_FEED_ROW 0xffff0000u /* input token VLT_FEED_ROW + i: the slot's GPU-fed token i */
#define VLT_FEED_W 16u
#define VLT_NO_TOK 0xffffffffu
#define VLT_VERIFY_T 8u /* rows per run that one attention tile takes */
#define VLT_MAX_STOP 8u

/* engine/src/engine.rs:31-57 `EngineConfig`; device_ordinal and flags are new. */
typedef struct {
    uint32_t max_seqs;         /* sequence slots */
    uint32_t max_step_tokens;  /* tokens per step, all sequences together */
    uint32_t max_chunk;        /* tokens one sequence may add in one step */
    uint32_t global_kv_tokens; /* capacity of the paged KV pool, in tokens */
    uint32_t max_seq_len;
    uint32_t max_head_rows;    /* rows that can go through the head in one step */
    int32_t device_ordinal;    /* CUDA device; one engine per GPU makes a replica */
    uint32_t flags;            /* VLT_FLAG_* */
} VltEngineConfig;
#define VLT_FLAG_HOST_ONLY 1u /* plan only: no device memory, steps cannot run */

/* engine/src/engine.rs:59-95 `Tuning`. The reference's Apple-GPU knobs (gpu_cores,
 * splitk_target, decode_split, verify_ki) are replaced by B200 ones; the rows policy is kept. 0 = default. */
typedef struct {
    uint32_t spec_tokens;       /* default 32 */
    uint32_t spec_tokens_short; /* default 8 */
    uint32_t spec_kv;           /* default 24576 */
    uint32_t spec_rows_long;    /* default 4 */
    uint32_t spec_policy_off;   /* 1: rows as requested (the reference's spec_tokens = 0) */
    uint32_t sm_count;          /* SMs to size grids for; 0: the device's */
    uint32_t attn_keys_per_cta; /* keys one attention CTA takes; 0: sized to fill the SMs */
    uint32_t gemm_min_rows;     /* steps with at least this many tokens use the tensor-core GEMM; 0: default (9) */
    uint32_t plain_attention;   /* 1: the scalar attention kernel (cross-check only) */
    uint32_t gemm_unpaired;     /* 1: the head GEMM as one block per SM, like the others (cross-check only; results are the same bit for bit) */
} VltTuning;

/* engine/src/engine.rs:100-138 `Sampling`. */
typedef struct {
    float temperature; /* 0: argmax */
    float top_p;       /* (0, 1] */
    uint64_t seed;
} VltSampling;

/* engine/src/engine.rs:140-172 `Rows`, `Run`, `StepOptions`, `StepOutput`. */
enum { VLT_ROWS_NONE = 0, VLT_ROWS_LAST = 1, VLT_ROWS_ALL = 2 };
typedef struct {
    uint32_t seq;
    const uint32_t* tokens;
    uint32_t n_tokens;
} VltRun;
typedef struct {
    uint32_t head;   /* VLT_ROWS_* */
    uint32_t hidden; /* VLT_ROWS_* */
    uint32_t read_logits;
    uint32_t read_taps;
} VltStepOptions;
typedef struct {
    uint32_t* ids; /* the token each head row got */
    uint32_t ids_cap, n_ids;
    float* logits; /* [n_ids][vocab] if read_logits */
    uint64_t logits_cap;
    float* hidden; /* [n_hidden][d_model]: final normed hidden state per hidden row */
    uint64_t hidden_cap;
    uint32_t n_hidden;
    uint16_t* taps; /* [tap][n_tokens][d_model] bf16(rms_norm(a tapped layer's output)) if read_taps (see vlt_set_taps) */
    uint64_t taps_cap;
    double gpu_seconds;
    uint32_t n_taps; /* tapped layers read back */
} VltStepOutput;

/* New: what the weight file's `meta` tensor describes (the reference hard-codes its model,
 * engine/src/model.rs:6-20). */
typedef struct {
    uint32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn, vocab, vocab_real, page_size;
    float rms_eps, attn_scale;
    uint32_t int8; /* 1 if the layer matrices are int8 */
} VltModelDesc;

const char* vlt_last_error(void);

/* Engine::new, engine/src/engine.rs:221-250. `tuning` may be NULL. The weight file is a plain decoder's (its `meta` tensor
 * describes it: the benchmark's models) or one of the reference's own architecture as tools/convert.py:64-114 writes it (no
 * `meta`; engine/src/model.rs:6-20, with the shapes read off the file). */
int vlt_engine_new(const char* weights_path, const VltEngineConfig* cfg, const VltTuning* tuning, VltEngine** out);
/* Drop for Engine. */
void vlt_engine_free(VltEngine* e);
/* Engine::device_name, engine.rs:252-254. */
int vlt_device_name(VltEngine* e, char* buf, size_t cap);
int vlt_model_desc(VltEngine* e, VltModelDesc* out);
/* Engine::new_seq / free_seq / seq_len / set_sampling, engine.rs:259-307. */
int vlt_seq_new(VltEngine* e, uint32_t* seq);
void vlt_seq_free(VltEngine* e, uint32_t seq);
uint32_t vlt_seq_len(VltEngine* e, uint32_t seq);
int vlt_seq_set_sampling(VltEngine* e, uint32_t seq, const VltSampling* s);
/* Engine::step, engine.rs:310-314: one synchronous step of CPU-fed runs. */
int vlt_step(VltEngine* e, const VltRun* runs, uint32_t n_runs, const VltStepOptions* opts, VltStepOutput* out);
/* Engine::step_capture, engine.rs:318-355, with LayerCapture, engine.rs:175-188: a synchronous step that stops after
 * every layer and hands that layer's intermediates (host memory, valid during the call) to `fn`: n rows each of
 * resid_in [d_model] (the residual stream entering the layer), attn_in [d_model] (its RMS-normed rows), qkv [qkv_width]
 * (q | k | v after the folded norm and RoPE, fp32: before the rounding to bf16 and q's softmax scale), sdpa_out
 * [attn_width] (the attention's output), attn_out [d_model] (the o projection's output before the residual add), mlp_in
 * [d_model] (the RMS-normed stream after attention), mlp_out [d_model] (the down projection's output before the residual
 * add); resid_base is the reference's MUDD base (NULL for a plain decoder). */
typedef struct {
    uint32_t layer, n, d_model, qkv_width, attn_width;
    const float *resid_in, *attn_in, *qkv, *sdpa_out, *attn_out, *mlp_in, *mlp_out, *resid_base;
} VltLayerCapture;
typedef void (*VltCaptureFn)(const VltLayerCapture* layer, void* user);
int vlt_step_capture(VltEngine* e, const VltRun* runs, uint32_t n_runs, const VltStepOptions* opts, VltCaptureFn fn, void* user, VltStepOutput* out);
/* Engine::set_taps, engine.rs:381-389: taps these layers' outputs -- bf16(rms_norm(output)), kernels.metal:133-148 -- from the
 * next step on, for VltStepOptions.read_taps ([tap][token][d_model], in the order given; with a drafter loaded the last layer
 * stays tapped and comes last if it was not named). Engine::load_drafter / has_drafter, engine.rs:381-389, engine/drafter.rs:250-262.
 * Two kinds of file load: the reference's block drafter as tools/spec/export.py writes it (recognised by its `kv_all`
 * tensor; engine/drafter.rs:131-240; it taps the layers its `meta` names, needs a target of 64-wide heads whose hidden width
 * is the drafter's, and drafts a tree per step), and the benchmark's one-layer chain drafter (`meta` = [1, 1, 1, draft ids
 * [, attention window]]). */
int vlt_set_taps(VltEngine* e, const uint32_t* layers, uint32_t n_layers);
int vlt_load_drafter(VltEngine* e, const char* path);
int vlt_has_drafter(VltEngine* e);
/* Which rule accepts drafts. VLT_ACCEPT_MATCH is the reference's `accept` (kernels.metal:1578-1657): every verify row
 * draws the target's token, a draft is accepted if it equals the token drawn on its parent row. VLT_ACCEPT_REJECTION has
 * no counterpart in the reference: a verify run whose drafts the chain drafter drew from its own distribution q at the
 * sequence's temperature (top_p = 1, temperature > 0) is decided by speculative sampling -- draft i accepted with
 * probability min(1, P(x) / Q(x)), the first rejected one replaced by a draw from the normalised max(0, P - Q), a bonus
 * token from the last row if all pass -- inside the step, and committed through the same `accept` state (lens, feed,
 * path, on_path, gen, emitted): rejected rows are rolled back by the sequence advancing only by what was accepted.
 * Runs the rule does not fit (greedy or top-p sequences, replay drafts, draft trees) keep the reference's rule. */
enum { VLT_ACCEPT_MATCH = 0, VLT_ACCEPT_REJECTION = 1 };
int vlt_set_acceptance(VltEngine* e, uint32_t rule);

/* Hooks, engine/src/engine/hooks.rs. */
/* bench_fill, hooks.rs:28-36: advance a sequence without computing it. `seed` != 0 also fills
 * the new positions' K/V with small pseudo-random values, so that later steps read finite numbers. */
int vlt_bench_fill(VltEngine* e, uint32_t seq, uint32_t len, uint32_t seed);
/* sample_logits, hooks.rs:41-54: rows of logits [n][vocab] (NULL: the previous call's) through
 * the sampler, each row with its own settings and drawn-token position. */
int vlt_sample_logits(VltEngine* e, const float* logits, const VltSampling* rows, const uint32_t* pos, uint32_t n, uint32_t* out);
/* Rejection-sampling acceptance on caller-supplied logits: p [streams][k+1][vocab] target rows and
 * q [streams][k][vocab] draft rows (bf16), the k draft tokens per stream, one seed and the position
 * of the first draft per stream. Draft i is accepted with probability min(1, P(x)/Q(x)); the first
 * rejected one is replaced by a draw from the normalised max(0, P - Q); with all accepted a bonus
 * token is drawn from the last target row. No counterpart in the reference, whose acceptance is
 * sample-then-match (`accept`, kernels.metal:1578-1657); it reuses the reference sampler's
 * uniforms and summation order (kernels.metal:1462-1576). gpu_seconds (may be NULL): the kernels'
 * time, best of reps. */
int vlt_spec_accept(VltEngine* e, const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, float temperature,
                    const uint64_t* seeds, const uint32_t* pos0, uint32_t reps, uint32_t* accepted, uint32_t* token, uint32_t* rollback, double* gpu_seconds);
/* The reference drafter's candidate kernels on caller-supplied draft logits [n_rows][nv] (host memory): `draft_top`
 * (kernels.metal:1846-1889: the ncand <= 4 best entries of each row, mapped through vocab_ids if not NULL, with their
 * probabilities at temperature 1 / inv_t -> cand, cand_q [n_rows][4]; rows whose tin[2r + 1] is 0 -- a block's first row, the
 * bonus token's own -- are skipped, tin NULL: none are) and `draft_tree` (kernels.metal:1896-1934: per block
 * b of blocks[2b + 1] <= 8 rows starting at row blocks[2b], the draft tree of slot slots[b] grown by path probability).
 * feed and tree receive the engine's whole [max_seqs][16] arrays afterwards. The reference runs them inside its drafter
 * (drafter.rs:420-447). */
int vlt_draft_trees(VltEngine* e, const float* logits, uint32_t n_rows, uint32_t nv, const uint32_t* vocab_ids, const uint32_t* tin, const uint32_t* blocks, const uint32_t* slots,
                    uint32_t n_blocks, float inv_t, uint32_t ncand, uint32_t* cand, float* cand_q, uint32_t* feed, uint32_t* tree);
/* The same acceptance step for a caller that cannot allocate device memory at that point (all of it
 * is in the caller's own pools, or an allocation's device-wide synchronisation is not acceptable
 * inside the decode loop). No counterpart in the reference. It allocates nothing, on the device or
 * (when it succeeds) on the host: its scratch is a pair of static device arrays of fixed size, so
 * streams * (2 k + 1) may be at most vlt_spec_accept_static_max_rows() (2048); beyond that it fails
 * with a message and vlt_spec_accept is the call to use. Every pointer is device memory of the
 * current device; the kernels are queued on cuda_stream (a cudaStream_t; NULL: the default stream)
 * and the call does not wait for them. A draft id >= vocab is read as 0. The first call made with a
 * given device current looks up the arrays' addresses: that call is set-up and should come before
 * the caller begins any stream capture. All calls on one device share the arrays; nothing in them
 * needs clearing between calls, but two calls whose kernels overlap in time (two streams, two
 * threads) race on them. */
int vlt_spec_accept_static(const uint16_t* p_dev, const uint16_t* q_dev, const uint32_t* drafts_dev, uint32_t streams, uint32_t k, uint32_t vocab,
                           float temperature, const uint64_t* seeds_dev, const uint32_t* pos0_dev, uint32_t* accepted_dev, uint32_t* token_dev,
                           uint32_t* rollback_dev, void* cuda_stream);
uint32_t vlt_spec_accept_static_max_rows(void);
/* set_profile_skip, hooks.rs:9-26: leave kernel groups out (results are then wrong). */
enum { VLT_SKIP_QKV = 1, VLT_SKIP_POST = 2, VLT_SKIP_ATTN = 4, VLT_SKIP_REDUCE = 8, VLT_SKIP_O = 16, VLT_SKIP_GATE_UP = 32, VLT_SKIP_DOWN = 64, VLT_SKIP_HEAD = 256 };
void vlt_set_profile_skip(VltEngine* e, uint32_t mask);
/* bench_matmul, hooks.rs:56-111: GPU seconds (best of reps) of one matmul kind ("qkv", "o",
 * "gate_up", "down", "head") over all layers for n tokens, and the weight bytes one pass reads.
 * variant 0: the engine's choice, 1: GEMV, 2: tensor-core GEMM. */
int vlt_bench_matmul(VltEngine* e, const char* kind, uint32_t n, uint32_t variant, uint32_t reps, double* seconds, uint64_t* bytes);

/* Generator, engine/src/engine/generate.rs:12-518. */
enum { VLT_DRAFT_NONE = 0, VLT_DRAFT_REPLAY = 1, VLT_DRAFT_MODEL = 2 };
enum { VLT_PROMPT_TOKENS = 0, VLT_PROMPT_RESUME = 1 };
typedef struct {
    uint32_t prompt_kind;          /* VLT_PROMPT_* */
    const uint32_t* prompt_tokens; /* TOKENS: the prompt */
    uint32_t n_prompt;
    uint32_t resume_seq, resume_token; /* RESUME: a sequence of the engine, continued by this token */
    uint32_t max_tokens;
    const uint32_t* stop; /* at most VLT_MAX_STOP */
    uint32_t n_stop;
    VltSampling sampling;
    uint32_t draft_kind; /* VLT_DRAFT_* */
    uint32_t draft_rows; /* rows verified per step (1 + drafts) */
    const uint32_t* trace; /* REPLAY: the recorded sequence, prompt and continuation */
    uint32_t n_trace;
} VltRequest;
enum { VLT_EVENT_TOKEN = 0, VLT_EVENT_DONE = 1 };
enum { VLT_FINISH_STOP = 0, VLT_FINISH_LENGTH = 1, VLT_FINISH_FAILED = 2 /* router only: no replica could take the request */ };
typedef struct {
    uint32_t kind; /* VLT_EVENT_* */
    uint32_t req;
    uint32_t value; /* TOKEN: the token; DONE: VLT_FINISH_* */
} VltEvent;
/* generate.rs:81-91 `StepStats`. */
typedef struct {
    uint32_t tokens, decode, emitted;
    double gpu_seconds, encode_seconds;
} VltStepStats;

/* Engine::generator, generate.rs:153-176. The generator borrows the engine until freed. */
int vlt_generator_new(VltEngine* e, VltGenerator** out);
/* Drop for Generator, generate.rs:503-518. */
void vlt_generator_free(VltGenerator* g);
int vlt_generator_submit(VltGenerator* g, const VltRequest* req, uint32_t* req_id);
void vlt_generator_cancel(VltGenerator* g, uint32_t req_id);
/* Generator::step, generate.rs:271-280: commits the next step, returns the previous step's events. */
int vlt_generator_step(VltGenerator* g, VltEvent* events, uint32_t cap, uint32_t* n_events);
int vlt_generator_is_idle(VltGenerator* g);
void vlt_generator_counts(VltGenerator* g, uint32_t* queued, uint32_t* running);
/* Takes the step statistics gathered so far (the reference's `stats` field). */
int vlt_generator_stats(VltGenerator* g, VltStepStats* out, uint32_t cap, uint32_t* n);
void vlt_generator_set_hold(VltGenerator* g, uint32_t hold);
void vlt_generator_set_replay_mistakes(VltGenerator* g, float rate, uint32_t seed);

/* Replicas. The model fits one GPU, so a machine's GPUs are used as independent replicas -- one engine and generator per
 * device, no exchange between them -- and a router on the host shards the streams: a request goes to the live replica
 * with the fewest requests, and when a replica's step fails, its unfinished requests are submitted again on the others,
 * continued from the tokens they had emitted (a sequence's draws are keyed by seed and position, engine.rs:100-102, so
 * the continuation is the one the failed replica would have produced). The reference has one engine on one device and
 * exits when it fails (cli/src/serve.rs:147-150): this has no counterpart there. A replica is a table of the generator's
 * calls (generate.rs:185-280), so that it can be a VltGenerator (vlt_replica_of_generator) or anything else that
 * behaves like one; each must be called from the thread that owns it, i.e. the router's. */
typedef struct {
    void* ctx;
    int (*submit)(void* ctx, const VltRequest* req, uint32_t* req_id);
    int (*step)(void* ctx, VltEvent* events, uint32_t cap, uint32_t* n_events); /* non-zero: the replica has failed */
    void (*cancel)(void* ctx, uint32_t req_id);                                 /* may be NULL */
    int (*is_idle)(void* ctx);
    void (*counts)(void* ctx, uint32_t* queued, uint32_t* running);
} VltReplicaOps;
typedef struct VltRouter VltRouter;
void vlt_replica_of_generator(VltGenerator* g, VltReplicaOps* out);
int vlt_router_new(const VltReplicaOps* replicas, uint32_t n_replicas, VltRouter** out);
void vlt_router_free(VltRouter* r);
/* Token prompts only (a resumed sequence lives on one replica's engine). */
int vlt_router_submit(VltRouter* r, const VltRequest* req, uint32_t* req_id);
void vlt_router_cancel(VltRouter* r, uint32_t req_id);
/* One step of every live replica; events carry the router's request ids. A request that no replica can take after a
 * failure ends with VLT_EVENT_DONE / VLT_FINISH_FAILED; with no replica left and requests pending the call fails. */
int vlt_router_step(VltRouter* r, VltEvent* events, uint32_t cap, uint32_t* n_events);
int vlt_router_is_idle(VltRouter* r);
uint32_t vlt_router_alive(VltRouter* r);
/* The replica a pending request is on (VLT_NO_TOK: finished or unknown). */
uint32_t vlt_router_replica_of(VltRouter* r, uint32_t req_id);

/* Inspection, for parity tests against the CPU oracle: copies a named engine array into `out`
 * (u32 words: "lens", "feed", "tree", "gen", "path", "path_len", "on_path", "page_table",
 * "free_pages", "tokens", "tin", "vis", "head_rows", "sample_rows", "runs", "out_ids",
 * "emitted", "meta", "tiles"; "attn_split": the last plan's keys per attention split and its split count;
 * "k_cache", "v_cache": the whole pools as bf16 pairs).
 * Returns the word count through n. */
int vlt_debug_read(VltEngine* e, const char* name, uint32_t* out, uint64_t cap, uint64_t* n);
/* Plans a step without running it (Engine::plan, engine/src/engine/plan.rs:47-150); works on a host-only engine. */
int vlt_debug_plan(VltEngine* e, const VltRun* runs, const uint32_t* verify, const uint32_t* heads, uint32_t n_runs, uint32_t hidden);
/* Corrects a sequence's length as `collect` does (engine.rs:281-285 `settle`). */
void vlt_debug_settle(VltEngine* e, uint32_t seq, uint32_t unused);
/* Overwrites words of "lens", "feed", "tree" or "gen" (the per-slot state the GPU keeps), from word `index`. */
int vlt_debug_write(VltEngine* e, const char* name, uint64_t index, const uint32_t* data, uint64_t n);
/* One synchronous step of runs with their own head rows and verify flags, which may name GPU-fed
 * tokens (what Generator::encode_next plans, generate.rs:380-392); optionally followed by the
 * replay drafter (encode_replay, encode.rs:439-451). */
int vlt_debug_step(VltEngine* e, const VltRun* runs, const uint32_t* verify, const uint32_t* heads, uint32_t n_runs, const VltStepOptions* opts,
                   uint32_t replay, float replay_rate, uint32_t replay_seed, VltStepOutput* out);
/* A slot's generation state as `admit` writes it (generate.rs:307-309), and its replay trace. */
int vlt_debug_set_gen(VltEngine* e, uint32_t slot, uint32_t remaining, const uint32_t* stop, uint32_t n_stop);
int vlt_debug_set_trace(VltEngine* e, uint32_t slot, const uint32_t* trace, uint32_t n);

/* Measurement. Two marks on the engine's stream and the GPU time between them; the number of
 * kernels this library has launched so far; per-group GPU time of the steps queued while
 * profiling is on (groups: the target layers' 0 matmuls, 1 attention, 2 K/V write and split merge; 3 the tail:
 * head, sampling, acceptance; 4 the drafter, everything it launches; the reference times its step with GPUEndTime - GPUStartTime,
 * engine/src/gpu.rs:147-154, and kernel groups by leaving them out, cli/src/profile.rs:44-104);
 * the bytes one step uploads and downloads. */
/* vlt_debug_step then runs the loaded drafter for this many rows after the step (0: not). */
void vlt_debug_set_draft_rows(VltEngine* e, uint32_t rows);
/* Queues, on the engine's stream, a small kernel whose wait on a barrier runs out by design (nobody arrives; it gives up
 * after 1024 polls, sets the device error word and returns -- nothing faults or hangs). Every kernel of a step bounds its
 * waits the same way; this makes the report testable: the next step collected fails with "a kernel's bounded wait ran
 * out", and the engine works on afterwards. */
int vlt_debug_stalled_wait(VltEngine* e);
/* The next vlt_debug_step replaces the logits its head computed ([head rows][vocab]) and the logits of its drafter's
 * passes ([pass][run][draft vocabulary]) by these (either may be NULL / 0) before the sampler, the acceptance and the
 * drafter's pick read them: the integer tail of a step on inputs identical to the oracle's. One step only. */
int vlt_debug_force_logits(VltEngine* e, const float* logits, uint64_t n_logits, const float* draft_logits, uint64_t n_draft);
int vlt_debug_mark(VltEngine* e, uint32_t which);
int vlt_debug_mark_elapsed_ms(VltEngine* e, double* ms);
uint64_t vlt_debug_launches(void);
int vlt_debug_profile(VltEngine* e, uint32_t on);
int vlt_debug_profile_read(VltEngine* e, double* ms5, uint32_t* launches5);
int vlt_debug_step_bytes(VltEngine* e, uint64_t* h2d, uint64_t* d2h);

#ifdef __cplusplus
}
#endif
#endif
