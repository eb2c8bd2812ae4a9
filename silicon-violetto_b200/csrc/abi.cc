// The C ABI (include/violetto.h): one function per method of the reference's public API.
#include <cstring>
#include <memory>
#include <string>

#include "../../include/violetto.h"
#include "engine.h"
#include "generator.h"
#include "router.h"

using namespace vlt;

struct VltEngine {
    std::unique_ptr<Engine> e;
    VltGenerator* generator = nullptr;  // at most one borrows the engine at a time
};
struct VltGenerator {
    std::unique_ptr<Generator> g;
    VltEngine* owner = nullptr;
};

struct VltRouter {
    std::unique_ptr<Router> r;
};

static thread_local std::string g_error;

template <typename F>
static int guard(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& ex) {
        g_error = ex.what();
        return 1;
    } catch (...) {
        g_error = "unknown error";
        return 1;
    }
}
// Every entry that may touch the GPU makes the engine's device current first: one thread may hold engines on
// several devices (one engine per GPU makes a replica), and a launch goes to whichever device is current.
static Engine& eng(VltEngine* e) {
    if (!e || !e->e) throw Error("null engine");
    e->e->make_current();
    return *e->e;
}
static Generator& gen(VltGenerator* g) {
    if (!g || !g->g) throw Error("null generator");
    g->g->eng.make_current();
    return *g->g;
}
// The synchronous step entries use step set 0 and the engine's one stream of state: not while a generator has a step queued.
static void no_step_in_flight(VltEngine* e) {
    if (e->generator && e->generator->g && e->generator->g->has_step_in_flight())
        throw Error("the engine's generator has a step in flight: collect it (vlt_generator_step until idle, or free the generator) before stepping the engine directly");
}
static Sampling sampling_of(const VltSampling& s) { return Sampling{s.temperature, s.top_p, s.seed}; }

extern "C" {

const char* vlt_last_error(void) { return g_error.c_str(); }

int vlt_engine_new(const char* weights_path, const VltEngineConfig* cfg, const VltTuning* tuning, VltEngine** out) {
    return guard([&] {
        if (!weights_path || !cfg || !out) throw Error("vlt_engine_new: null argument");
        EngineConfig c;
        c.max_seqs = cfg->max_seqs;
        c.max_step_tokens = cfg->max_step_tokens;
        c.max_chunk = cfg->max_chunk;
        c.global_kv_tokens = cfg->global_kv_tokens;
        c.max_seq_len = cfg->max_seq_len;
        c.max_head_rows = cfg->max_head_rows;
        c.device = cfg->device_ordinal;
        c.host_only = (cfg->flags & VLT_FLAG_HOST_ONLY) != 0;
        Tuning t;
        if (tuning) {
            if (tuning->spec_tokens) t.spec_tokens = tuning->spec_tokens;
            if (tuning->spec_tokens_short) t.spec_tokens_short = tuning->spec_tokens_short;
            if (tuning->spec_kv) t.spec_kv = tuning->spec_kv;
            if (tuning->spec_rows_long) t.spec_rows_long = tuning->spec_rows_long;
            if (tuning->spec_policy_off) t.spec_tokens = 0;
            t.sm_count = tuning->sm_count;
            t.attn_keys_per_cta = tuning->attn_keys_per_cta;
            t.gemm_min_rows = tuning->gemm_min_rows;
            t.plain_attention = tuning->plain_attention != 0;
            t.gemm_unpaired = tuning->gemm_unpaired != 0;
        }
        auto h = std::make_unique<VltEngine>();
        h->e = std::make_unique<Engine>(weights_path, c, t);
        *out = h.release();
    });
}

#ifdef VLT_STEP_PROBE
extern "C" void vlt_sp_dump_all();
#endif
void vlt_engine_free(VltEngine* e) {
    if (!e) return;
#ifdef VLT_STEP_PROBE
    vlt_sp_dump_all();
#endif
    if (e->e) e->e->make_current();
    if (e->generator) e->generator->g.reset();  // a generator must not outlive its engine
    delete e;
}

int vlt_device_name(VltEngine* e, char* buf, size_t cap) {
    return guard([&] {
        const std::string n = eng(e).device_name();
        if (!buf || cap == 0) throw Error("vlt_device_name: no buffer");
        std::strncpy(buf, n.c_str(), cap - 1);
        buf[cap - 1] = 0;
    });
}

int vlt_model_desc(VltEngine* e, VltModelDesc* out) {
    return guard([&] {
        const Engine& en = eng(e);
        const ModelDesc& m = en.model.md;
        *out = VltModelDesc{m.n_layers, m.d, m.n_heads, m.n_kv, m.hd, m.ffn, m.vocab, m.vocab_real, m.page, m.eps, m.attn_scale, en.model.layers[0].qkv.int8 ? 1u : 0u};
    });
}

int vlt_seq_new(VltEngine* e, uint32_t* seq) { return guard([&] { *seq = eng(e).new_seq(); }); }
void vlt_seq_free(VltEngine* e, uint32_t seq) { if (e && e->e) { e->e->make_current(); e->e->free_seq(seq); } }
uint32_t vlt_seq_len(VltEngine* e, uint32_t seq) { return e && e->e ? e->e->seq_len(seq) : 0; }
int vlt_seq_set_sampling(VltEngine* e, uint32_t seq, const VltSampling* s) { return guard([&] { eng(e).set_sampling(seq, sampling_of(*s)); }); }

static void fill_output(Engine& en, const StepOutput& r, VltStepOutput* out) {
    if (!out) return;
    out->n_ids = uint32_t(r.ids.size());
    if (r.ids.size() > out->ids_cap) throw Error("ids buffer too small");
    if (out->ids) std::memcpy(out->ids, r.ids.data(), r.ids.size() * 4);
    if (!r.logits.empty()) {
        if (!out->logits || r.logits.size() > out->logits_cap) throw Error("logits buffer too small");
        std::memcpy(out->logits, r.logits.data(), r.logits.size() * 4);
    }
    out->n_hidden = uint32_t(r.hidden.size() / en.model.md.d);
    if (!r.hidden.empty()) {
        if (!out->hidden || r.hidden.size() > out->hidden_cap) throw Error("hidden buffer too small");
        std::memcpy(out->hidden, r.hidden.data(), r.hidden.size() * 4);
    }
    out->n_taps = 0;
    if (!r.taps.empty()) {
        if (!out->taps || r.taps.size() > out->taps_cap) throw Error("taps buffer too small");
        std::memcpy(out->taps, r.taps.data(), r.taps.size() * 2);
        out->n_taps = uint32_t(en.tap_layers.size());
    }
    out->gpu_seconds = r.gpu_seconds;
}

int vlt_step(VltEngine* e, const VltRun* runs, uint32_t n_runs, const VltStepOptions* opts, VltStepOutput* out) {
    return guard([&] {
        Engine& en = eng(e);
        no_step_in_flight(e);
        std::vector<PlanRun> rs;
        for (uint32_t i = 0; i < n_runs; i++) {
            for (uint32_t j = 0; j < runs[i].n_tokens; j++)
                if (runs[i].tokens[j] >= en.model.md.vocab) throw Error("token id out of range");  // engine.rs:346-348
            rs.push_back(PlanRun{runs[i].seq, runs[i].tokens, runs[i].n_tokens, Rows(opts->head), false});
        }
        StepOptions o{Rows(opts->head), Rows(opts->hidden), opts->read_logits != 0, opts->read_taps != 0};
        fill_output(en, en.step(rs, o), out);
    });
}

int vlt_set_taps(VltEngine* e, const uint32_t* layers, uint32_t n_layers) {
    return guard([&] { eng(e).set_taps(std::vector<uint32_t>(layers, layers + (layers ? n_layers : 0))); });
}

int vlt_step_capture(VltEngine* e, const VltRun* runs, uint32_t n_runs, const VltStepOptions* opts, VltCaptureFn fn, void* user, VltStepOutput* out) {
    return guard([&] {
        Engine& en = eng(e);
        no_step_in_flight(e);
        if (!fn) throw Error("vlt_step_capture: no callback");
        std::vector<PlanRun> rs;
        for (uint32_t i = 0; i < n_runs; i++) {
            for (uint32_t j = 0; j < runs[i].n_tokens; j++)
                if (runs[i].tokens[j] >= en.model.md.vocab) throw Error("token id out of range");  // engine.rs:346-348
            rs.push_back(PlanRun{runs[i].seq, runs[i].tokens, runs[i].n_tokens, Rows(opts->head), false});
        }
        StepOptions o{Rows(opts->head), Rows(opts->hidden), opts->read_logits != 0, opts->read_taps != 0};
        const ModelDesc& md = en.model.md;
        fill_output(en, en.step_capture(rs, o, [&](const LayerCapture& c) {
            const VltLayerCapture v{c.layer, c.n, md.d, md.qkv_w(), md.n_heads * md.hd, c.resid_in, c.attn_in, c.qkv, c.sdpa_out, c.attn_out, c.mlp_in, c.mlp_out, nullptr};
            fn(&v, user);
        }), out);
    });
}
int vlt_set_acceptance(VltEngine* e, uint32_t rule) { return guard([&] { eng(e).set_acceptance(rule); }); }
int vlt_load_drafter(VltEngine* e, const char* path) { return guard([&] { eng(e).load_drafter(path); }); }
int vlt_has_drafter(VltEngine* e) { return e && e->e && e->e->has_drafter() ? 1 : 0; }

int vlt_bench_fill(VltEngine* e, uint32_t seq, uint32_t len, uint32_t seed) { return guard([&] { eng(e).bench_fill(seq, len, seed); }); }

int vlt_sample_logits(VltEngine* e, const float* logits, const VltSampling* rows, const uint32_t* pos, uint32_t n, uint32_t* out) {
    return guard([&] {
        std::vector<std::pair<Sampling, uint32_t>> r;
        for (uint32_t i = 0; i < n; i++) r.emplace_back(sampling_of(rows[i]), pos[i]);
        const std::vector<uint32_t> ids = eng(e).sample_logits(logits, r);
        std::memcpy(out, ids.data(), ids.size() * 4);
    });
}

int vlt_spec_accept(VltEngine* e, const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, float temperature,
                    const uint64_t* seeds, const uint32_t* pos0, uint32_t reps, uint32_t* accepted, uint32_t* token, uint32_t* rollback, double* gpu_seconds) {
    return guard([&] {
        std::vector<uint32_t> out(size_t(3) * streams);
        const double t = eng(e).spec_accept(p, q, drafts, streams, k, temperature, seeds, pos0, reps, out.data());
        std::memcpy(accepted, out.data(), size_t(streams) * 4);
        std::memcpy(token, out.data() + streams, size_t(streams) * 4);
        std::memcpy(rollback, out.data() + 2 * streams, size_t(streams) * 4);
        if (gpu_seconds) *gpu_seconds = t;
    });
}

int vlt_draft_trees(VltEngine* e, const float* logits, uint32_t n_rows, uint32_t nv, const uint32_t* vocab_ids, const uint32_t* tin, const uint32_t* blocks, const uint32_t* slots,
                    uint32_t n_blocks, float inv_t, uint32_t ncand, uint32_t* cand, float* cand_q, uint32_t* feed, uint32_t* tree) {
    return guard([&] { eng(e).draft_trees(logits, n_rows, nv, vocab_ids, tin, blocks, slots, n_blocks, inv_t, ncand, cand, cand_q, feed, tree); });
}

int vlt_spec_accept_static(const uint16_t* p_dev, const uint16_t* q_dev, const uint32_t* drafts_dev, uint32_t streams, uint32_t k, uint32_t vocab,
                           float temperature, const uint64_t* seeds_dev, const uint32_t* pos0_dev, uint32_t* accepted_dev, uint32_t* token_dev,
                           uint32_t* rollback_dev, void* cuda_stream) {
    // No guard(): nothing on this path throws, and the success path allocates nothing on host or device.
    const char* err = launch_spec_accept_static(p_dev, q_dev, drafts_dev, streams, k, vocab, temperature, seeds_dev, pos0_dev, accepted_dev, token_dev,
                                                rollback_dev, static_cast<cudaStream_t>(cuda_stream));
    if (!err) return 0;
    g_error = err;
    return 1;
}
uint32_t vlt_spec_accept_static_max_rows(void) { return spec_accept_static_max_rows(); }

void vlt_set_profile_skip(VltEngine* e, uint32_t mask) { if (e && e->e) e->e->skip = mask; }

int vlt_bench_matmul(VltEngine* e, const char* kind, uint32_t n, uint32_t variant, uint32_t reps, double* seconds, uint64_t* bytes) {
    return guard([&] { eng(e).bench_matmul(kind, n, variant, reps, seconds, bytes); });
}

// ---- generator
int vlt_generator_new(VltEngine* e, VltGenerator** out) {
    return guard([&] {
        Engine& en = eng(e);
        if (e->generator) throw Error("the engine already has a generator");
        auto g = std::make_unique<VltGenerator>();
        g->g = std::make_unique<Generator>(en);
        g->owner = e;
        e->generator = g.get();
        *out = g.release();
    });
}

void vlt_generator_free(VltGenerator* g) {
    if (!g) return;
    if (g->g) g->g->eng.make_current();
    if (g->owner && g->owner->generator == g) g->owner->generator = nullptr;
    delete g;
}

int vlt_generator_submit(VltGenerator* g, const VltRequest* r, uint32_t* req_id) {
    return guard([&] {
        Request q;
        q.resume = r->prompt_kind == VLT_PROMPT_RESUME;
        if (!q.resume && r->n_prompt) q.prompt.assign(r->prompt_tokens, r->prompt_tokens + r->n_prompt);
        q.resume_seq = r->resume_seq;
        q.resume_token = r->resume_token;
        q.max_tokens = r->max_tokens;
        if (r->n_stop) q.stop.assign(r->stop, r->stop + r->n_stop);
        q.sampling = sampling_of(r->sampling);
        if (r->draft_kind > VLT_DRAFT_MODEL) throw Error("unknown draft kind");
        q.draft = DraftKind(r->draft_kind);
        q.rows = r->draft_rows;
        if (r->n_trace) q.trace.assign(r->trace, r->trace + r->n_trace);
        *req_id = gen(g).submit(q);
    });
}

void vlt_generator_cancel(VltGenerator* g, uint32_t req_id) { if (g && g->g) { g->g->eng.make_current(); g->g->cancel(req_id); } }

int vlt_generator_step(VltGenerator* g, VltEvent* events, uint32_t cap, uint32_t* n_events) {
    return guard([&] {
        const std::vector<Event> ev = gen(g).step();
        if (ev.size() > cap) throw Error("event buffer too small: " + std::to_string(ev.size()) + " events");
        for (size_t i = 0; i < ev.size(); i++) events[i] = VltEvent{uint32_t(ev[i].kind), ev[i].req, ev[i].value};
        *n_events = uint32_t(ev.size());
    });
}

int vlt_generator_is_idle(VltGenerator* g) { return g && g->g && g->g->is_idle() ? 1 : 0; }
void vlt_generator_counts(VltGenerator* g, uint32_t* queued, uint32_t* running) { if (g && g->g) g->g->counts(queued, running); }

int vlt_generator_stats(VltGenerator* g, VltStepStats* out, uint32_t cap, uint32_t* n) {
    return guard([&] {
        Generator& gg = gen(g);
        const size_t k = std::min<size_t>(cap, gg.stats.size());
        for (size_t i = 0; i < k; i++) {
            const StepStats& s = gg.stats[i];
            out[i] = VltStepStats{s.tokens, s.decode ? 1u : 0u, s.emitted, s.gpu_seconds, s.encode_seconds};
        }
        gg.stats.erase(gg.stats.begin(), gg.stats.begin() + k);
        *n = uint32_t(k);
    });
}

void vlt_generator_set_hold(VltGenerator* g, uint32_t hold) { if (g && g->g) g->g->hold = hold != 0; }
void vlt_generator_set_replay_mistakes(VltGenerator* g, float rate, uint32_t seed) { if (g && g->g) g->g->set_replay_mistakes(rate, seed); }

// ---- replicas
static int rep_submit(void* ctx, const VltRequest* req, uint32_t* id) { return vlt_generator_submit(static_cast<VltGenerator*>(ctx), req, id); }
static int rep_step(void* ctx, VltEvent* ev, uint32_t cap, uint32_t* n) { return vlt_generator_step(static_cast<VltGenerator*>(ctx), ev, cap, n); }
static void rep_cancel(void* ctx, uint32_t id) { vlt_generator_cancel(static_cast<VltGenerator*>(ctx), id); }
static int rep_idle(void* ctx) { return vlt_generator_is_idle(static_cast<VltGenerator*>(ctx)); }
static void rep_counts(void* ctx, uint32_t* q, uint32_t* r) { *q = *r = 0; vlt_generator_counts(static_cast<VltGenerator*>(ctx), q, r); }

void vlt_replica_of_generator(VltGenerator* g, VltReplicaOps* out) {
    if (out) *out = VltReplicaOps{g, rep_submit, rep_step, rep_cancel, rep_idle, rep_counts};
}

int vlt_router_new(const VltReplicaOps* replicas, uint32_t n_replicas, VltRouter** out) {
    return guard([&] {
        if (!replicas || !out) throw Error("vlt_router_new: null argument");
        auto h = std::make_unique<VltRouter>();
        h->r = std::make_unique<Router>(std::vector<VltReplicaOps>(replicas, replicas + n_replicas));
        *out = h.release();
    });
}
void vlt_router_free(VltRouter* r) { delete r; }
static Router& router(VltRouter* r) {
    if (!r || !r->r) throw Error("null router");
    return *r->r;
}
int vlt_router_submit(VltRouter* r, const VltRequest* req, uint32_t* req_id) { return guard([&] { *req_id = router(r).submit(*req); }); }
void vlt_router_cancel(VltRouter* r, uint32_t req_id) { if (r && r->r) r->r->cancel(req_id); }
int vlt_router_step(VltRouter* r, VltEvent* events, uint32_t cap, uint32_t* n_events) {
    return guard([&] {
        const std::vector<VltEvent> ev = router(r).step();
        if (ev.size() > cap) throw Error("event buffer too small: " + std::to_string(ev.size()) + " events");
        for (size_t i = 0; i < ev.size(); i++) events[i] = ev[i];
        *n_events = uint32_t(ev.size());
    });
}
int vlt_router_is_idle(VltRouter* r) { return r && r->r && r->r->is_idle() ? 1 : 0; }
uint32_t vlt_router_alive(VltRouter* r) { return r && r->r ? r->r->alive() : 0; }
uint32_t vlt_router_replica_of(VltRouter* r, uint32_t req_id) { return r && r->r ? r->r->replica_of(req_id) : NO_TOK; }

// ---- inspection
int vlt_debug_read(VltEngine* e, const char* name, uint32_t* out, uint64_t cap, uint64_t* n) {
    return guard([&] {
        const std::vector<uint32_t> v = eng(e).debug_read(name);
        *n = v.size();
        if (v.size() > cap) throw Error(std::string(name) + ": " + std::to_string(v.size()) + " words, buffer too small");
        std::memcpy(out, v.data(), v.size() * 4);
    });
}

int vlt_debug_write(VltEngine* e, const char* name, uint64_t index, const uint32_t* data, uint64_t n) {
    return guard([&] { eng(e).debug_write(name, index, data, n); });
}

int vlt_debug_plan(VltEngine* e, const VltRun* runs, const uint32_t* verify, const uint32_t* heads, uint32_t n_runs, uint32_t hidden) {
    return guard([&] {
        eng(e);
        no_step_in_flight(e);
        std::vector<PlanRun> rs;
        for (uint32_t i = 0; i < n_runs; i++) rs.push_back(PlanRun{runs[i].seq, runs[i].tokens, runs[i].n_tokens, Rows(heads[i]), verify[i] != 0});
        eng(e).plan(0, rs, Rows(hidden));
        eng(e).upload_set(0);
    });
}

int vlt_debug_step(VltEngine* e, const VltRun* runs, const uint32_t* verify, const uint32_t* heads, uint32_t n_runs, const VltStepOptions* opts,
                   uint32_t replay, float replay_rate, uint32_t replay_seed, VltStepOutput* out) {
    return guard([&] {
        Engine& en = eng(e);
        no_step_in_flight(e);
        std::vector<PlanRun> rs;
        for (uint32_t i = 0; i < n_runs; i++) rs.push_back(PlanRun{runs[i].seq, runs[i].tokens, runs[i].n_tokens, Rows(heads[i]), verify[i] != 0});
        StepOptions o{Rows::None, Rows(opts->hidden), opts->read_logits != 0, opts->read_taps != 0};
        ReplayArgs ra{en.cfg.max_seq_len, replay_seed, replay_rate, en.model.md.vocab_real};
        fill_output(en, en.step_runs(rs, o, replay ? &ra : nullptr), out);
    });
}

void vlt_debug_set_draft_rows(VltEngine* e, uint32_t rows) { if (e && e->e) e->e->debug_draft_rows = rows; }

int vlt_debug_stalled_wait(VltEngine* e) { return guard([&] { eng(e).debug_stalled_wait(); }); }

int vlt_debug_force_logits(VltEngine* e, const float* logits, uint64_t n_logits, const float* draft_logits, uint64_t n_draft) {
    return guard([&] {
        Engine& en = eng(e);
        en.forced_logits.assign(logits, logits + (logits ? n_logits : 0));
        en.forced_draft_logits.assign(draft_logits, draft_logits + (draft_logits ? n_draft : 0));
    });
}

int vlt_debug_mark(VltEngine* e, uint32_t which) { return guard([&] { eng(e).mark(int(which)); }); }
int vlt_debug_mark_elapsed_ms(VltEngine* e, double* ms) { return guard([&] { *ms = eng(e).mark_elapsed_ms(); }); }
uint64_t vlt_debug_launches(void) { return launch_counter(); }
int vlt_debug_profile(VltEngine* e, uint32_t on) { return guard([&] { eng(e).profile = on != 0; }); }
int vlt_debug_profile_read(VltEngine* e, double* ms5, uint32_t* launches5) { return guard([&] { eng(e).profile_read(ms5, launches5); }); }
int vlt_debug_step_bytes(VltEngine* e, uint64_t* h2d, uint64_t* d2h) {
    return guard([&] { *h2d = eng(e).sets[0].in_bytes; *d2h = eng(e).sets[0].out_bytes; });
}

void vlt_debug_settle(VltEngine* e, uint32_t seq, uint32_t unused) { if (e && e->e) e->e->settle(seq, unused); }

int vlt_debug_set_gen(VltEngine* e, uint32_t slot, uint32_t remaining, const uint32_t* stop, uint32_t n_stop) {
    return guard([&] {
        if (n_stop > MAX_STOP) throw Error(std::to_string(n_stop) + " stop tokens (max " + std::to_string(MAX_STOP) + ")");
        if (slot >= eng(e).cfg.max_seqs) throw Error("slot out of range");
        GenState g = gen_open();
        g.remaining = remaining;
        g.nstop = n_stop;
        for (uint32_t i = 0; i < n_stop && i < MAX_STOP; i++) g.stop[i] = stop[i];
        eng(e).set_gen(slot, g);
    });
}

int vlt_debug_set_trace(VltEngine* e, uint32_t slot, const uint32_t* trace, uint32_t n) { return guard([&] { eng(e).set_trace(slot, trace, n); }); }

}  // extern "C"
