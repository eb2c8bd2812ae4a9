// CPU oracle (test infrastructure only, parity unpinned: see bits.hpp): C entry points for
// the tests' ctypes binding and for the benchmark's CPU-baseline leg.
#include <cstdio>
#include <omp.h>

#include <cstring>
#include <string>

#include "block_drafter.hpp"
#include "model.hpp"

using namespace orc;

static thread_local std::string g_err;
static int fail(const std::exception& e) { g_err = e.what(); return 1; }

extern "C" {

const char* orc_last_error() { return g_err.c_str(); }

void orc_philox(const uint32_t* c, const uint32_t* k, uint32_t* out) {
    U4 r = philox(U4{c[0], c[1], c[2], c[3]}, k[0], k[1]);
    out[0] = r.x; out[1] = r.y; out[2] = r.z; out[3] = r.w;
}
float orc_uniform01(uint32_t lo, uint32_t hi, uint32_t pos, uint32_t round) { return uniform01(lo, hi, pos, round); }
void orc_exp2(const float* x, float* y, uint64_t n) { for (uint64_t i = 0; i < n; i++) y[i] = soft_exp2(x[i]); }
void orc_to_bf16(const float* x, uint16_t* y, uint64_t n) { for (uint64_t i = 0; i < n; i++) y[i] = f32_to_bf16(x[i]); }
uint32_t orc_chain_node(uint32_t row) { return chain_node(row); }
uint32_t orc_dead_node(uint32_t row) { return dead_node(row); }
void orc_quantize(const float* w, uint32_t m, uint32_t k, uint32_t group, int8_t* q, uint16_t* s) { quantize(w, m, k, group, q, s); }

// x, y [rows][hd]; pos [rows]; freq [hd/2]; cs_out [rows][hd/2][2] (may be null).
void orc_rope(const float* x, uint32_t rows, uint32_t hd, const uint32_t* pos, const float* freq, float* y, float* cs_out) {
    std::vector<float> cs(hd);
    for (uint32_t r = 0; r < rows; r++) {
        for (uint32_t i = 0; i < hd / 2; i++) rope_cs(pos[r], freq[i], cs[2 * i], cs[2 * i + 1]);
        std::copy_n(x + size_t(r) * hd, hd, y + size_t(r) * hd);
        rope_pairs(y + size_t(r) * hd, hd, cs.data());
        if (cs_out) std::copy_n(cs.data(), hd, cs_out + size_t(r) * hd);
    }
}

// ---- weight files
void* orc_vlt_load(const char* path) {
    try { return new VltFile(VltFile::load(path)); } catch (const std::exception& e) { fail(e); return nullptr; }
}
void orc_vlt_free(void* h) { delete static_cast<VltFile*>(h); }
uint32_t orc_vlt_count(void* h) { return uint32_t(static_cast<VltFile*>(h)->tensors.size()); }
const void* orc_vlt_tensor(void* h, uint32_t i, char* name64, uint32_t* dtype, uint32_t* ndim, uint32_t* shape4, uint64_t* offset, uint64_t* nbytes) {
    VltFile* f = static_cast<VltFile*>(h);
    const Tensor& t = f->tensors[i];
    std::memset(name64, 0, 64);
    std::memcpy(name64, t.name.data(), std::min<size_t>(63, t.name.size()));
    *dtype = t.dtype;
    *ndim = uint32_t(t.shape.size());
    for (size_t j = 0; j < 4; j++) shape4[j] = j < t.shape.size() ? t.shape[j] : 0;
    *offset = t.offset;
    *nbytes = t.nbytes;
    return f->ptr(t);
}
int orc_vlt_write(const char* path, uint32_t n, const char* const* names, const uint32_t* dtypes, const uint32_t* ndims,
                  const uint32_t* shapes4, const void* const* ptrs, const uint64_t* nbytes) {
    try {
        VltWriter w;
        for (uint32_t i = 0; i < n; i++)
            w.add(names[i], DType(dtypes[i]), std::vector<uint32_t>(shapes4 + 4 * i, shapes4 + 4 * i + ndims[i]), ptrs[i], nbytes[i]);
        w.write(path);
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

// ---- kernels, one call per dispatch
void orc_sample(const float* logits, uint32_t vocab, const SampleRow* rows, uint32_t nrows, const uint32_t* meta, uint32_t* out) {
#pragma omp parallel for schedule(dynamic)
    for (int64_t r = 0; r < int64_t(nrows); r++) {
        const SampleRow& sr = rows[r];
        const uint32_t pos = sr.tok == NO_TOK ? sr.pos : meta[2 * sr.tok + 1] + 1;
        out[r] = sample_row(logits + uint64_t(r) * vocab, vocab, sr, pos);
    }
}
void orc_accept(const RunIn* runs, uint32_t nruns, const uint32_t* tokens, uint32_t* out, uint32_t* lens, uint32_t* feed, GenState* gen,
                uint32_t* emitted, const uint32_t* tree, uint32_t* path, uint32_t* path_len, uint32_t* on_path) {
    for (uint32_t r = 0; r < nruns; r++) accept_run(r, runs, tokens, out, lens, feed, gen, emitted, tree, path, path_len, on_path);
}
void orc_replay_draft(const RunIn* runs, uint32_t nruns, const uint32_t* lens, uint32_t* feed, const uint32_t* trace, const uint32_t* trace_len,
                      uint32_t stride, uint32_t seed, float rate, uint32_t vocab, uint32_t* tree) {
    ReplayArgs ra{stride, seed, rate, vocab};
    for (uint32_t r = 0; r < nruns; r++) replay_draft_run(r, runs, lens, feed, trace, trace_len, ra, tree);
}
void orc_draft_top(const float* logits, uint32_t nrows, uint32_t nv, const uint32_t* vocab_ids, const uint32_t* tin, float inv_t, uint32_t ncand,
                   uint32_t* cand, float* cand_q) {
    for (uint32_t r = 0; r < nrows; r++) {
        if (tin[2 * r + 1] == 0) continue;  // kernels.metal:1862: row 0 is the bonus token's own
        draft_top_row(logits + uint64_t(r) * nv, nv, vocab_ids, inv_t, ncand, cand + r * CANDS, cand_q + r * CANDS);
    }
}
void orc_draft_tree(const uint32_t* blocks, uint32_t nblocks, const uint32_t* tin, const uint32_t* cand, const float* cand_q, uint32_t ncand,
                    uint32_t* feed, uint32_t* tree) {
    for (uint32_t b = 0; b < nblocks; b++) draft_tree_block(blocks[2 * b], blocks[2 * b + 1], tin[2 * blocks[2 * b]], cand, cand_q, ncand, feed, tree);
}
void orc_spec_accept(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, uint32_t vocab, float temperature,
                     const uint64_t* seeds, const uint32_t* pos0, uint32_t* accepted, uint32_t* token, uint32_t* rollback) {
#pragma omp parallel for schedule(dynamic)
    for (int64_t s = 0; s < int64_t(streams); s++) {
        SpecOut o = spec_accept_stream(p + uint64_t(s) * (k + 1) * vocab, q + uint64_t(s) * k * vocab, drafts + s * k, k, vocab, temperature,
                                       uint32_t(seeds[s]), uint32_t(seeds[s] >> 32), pos0[s]);
        accepted[s] = o.accepted; token[s] = o.token; rollback[s] = o.rollback;
    }
}
void orc_draw_drafts(const uint16_t* q, uint32_t streams, uint32_t k, uint32_t vocab, float temperature, const uint64_t* seeds, const uint32_t* pos0,
                     uint32_t* drafts) {
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int64_t s = 0; s < int64_t(streams); s++)
        for (int64_t i = 0; i < int64_t(k); i++)
            drafts[s * k + i] = draw_draft(q + (uint64_t(s) * k + i) * vocab, vocab, temperature, uint32_t(seeds[s]), uint32_t(seeds[s] >> 32), pos0[s] + uint32_t(i));
}

// OpenMP threads of the calls below (a launcher may have set OMP_NUM_THREADS=1 for its workers).
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int orc_max_threads() { return omp_get_max_threads(); }

// ---- the engine
struct OrcConfig { uint32_t max_seqs, max_step_tokens, max_chunk, kv_tokens, max_seq_len, max_head_rows; };

void* orc_engine_new(const char* path, const OrcConfig* c) {
    try {
        EngineConfig cfg{c->max_seqs, c->max_step_tokens, c->max_chunk, c->kv_tokens, c->max_seq_len, c->max_head_rows};
        return new Engine(path, cfg);
    } catch (const std::exception& e) { fail(e); return nullptr; }
}
void orc_engine_free(void* h) { delete static_cast<Engine*>(h); }
int orc_seq_new(void* h, uint32_t* id) { try { *id = static_cast<Engine*>(h)->new_seq(); return 0; } catch (const std::exception& e) { return fail(e); } }
void orc_seq_free(void* h, uint32_t id) { static_cast<Engine*>(h)->free_seq(id); }
uint32_t orc_seq_len(void* h, uint32_t id) { Engine* e = static_cast<Engine*>(h); return id < e->seqs.size() && e->seqs[id] ? e->seqs[id]->len : 0; }
int orc_seq_set_sampling(void* h, uint32_t id, float temperature, float top_p, uint64_t seed) {
    try { static_cast<Engine*>(h)->seq(id).sampling = Sampling{temperature, top_p, seed}; return 0; } catch (const std::exception& e) { return fail(e); }
}
// engine.rs:281-285 `settle`.
void orc_seq_settle(void* h, uint32_t id, uint32_t unused) { Engine* e = static_cast<Engine*>(h); if (id < e->seqs.size() && e->seqs[id]) e->seqs[id]->len -= unused; }
int orc_bench_fill(void* h, uint32_t id, uint32_t len, uint32_t seed) { try { static_cast<Engine*>(h)->bench_fill(id, len, seed); return 0; } catch (const std::exception& e) { return fail(e); } }
void orc_set_gen(void* h, uint32_t slot, uint32_t remaining, const uint32_t* stop, uint32_t nstop) {
    GenState g{remaining, 0, nstop, 0, {0}};
    for (uint32_t i = 0; i < nstop && i < MAX_STOP; i++) g.stop[i] = stop[i];
    static_cast<Engine*>(h)->gen[slot] = g;
}
void orc_set_trace(void* h, uint32_t slot, const uint32_t* trace, uint32_t n) {
    Engine* e = static_cast<Engine*>(h);
    std::copy_n(trace, n, e->trace.begin() + size_t(slot) * e->cfg.max_seq_len);
    e->trace_len[slot] = n;
}
int orc_load_drafter(void* h, const char* path) { try { static_cast<Engine*>(h)->load_drafter(path); return 0; } catch (const std::exception& e) { return fail(e); } }
// 0: the reference's acceptance (sample, then match); 1: rejection sampling for runs whose drafts came with their q rows.
void orc_set_acceptance(void* h, uint32_t rule) { static_cast<Engine*>(h)->accept_rule = rule; }
void orc_set_capture(void* h, uint32_t on) { static_cast<Engine*>(h)->capture = on != 0; }
void orc_set_taps(void* h, const uint32_t* layers, uint32_t n) { static_cast<Engine*>(h)->tap_layers.assign(layers, layers + n); }
void orc_set_replay(void* h, float rate, uint32_t seed) {
    Engine* e = static_cast<Engine*>(h);
    e->replay = ReplayArgs{e->cfg.max_seq_len, seed, rate, e->md.vocab_real};
}

// One step. Runs are (seq, count, verify) with their tokens concatenated in `tokens`;
// `head` and `hidden` are Rows values; mode bit 0: plan only (no forward), bit 1: run the
// replay drafter after the step; bits 8..11: run the chain drafter for that many rows.
int orc_step(void* h, uint32_t n_runs, const uint32_t* seq, const uint32_t* count, const uint32_t* verify, const uint32_t* heads, const uint32_t* tokens,
             uint32_t hidden, uint32_t mode) {
    try {
        Engine* e = static_cast<Engine*>(h);
        std::vector<PlanRun> runs;
        const uint32_t* t = tokens;
        for (uint32_t r = 0; r < n_runs; r++) {
            runs.push_back(PlanRun{seq[r], std::vector<uint32_t>(t, t + count[r]), Rows(heads[r]), verify[r] != 0});
            t += count[r];
        }
        Plan p = e->plan(runs, Rows(hidden));
        if (mode & 1) return 0;
        e->forward(p);
        if ((mode >> 8) & 15) e->draft(p, (mode >> 8) & 15);
        if (mode & 2) e->run_replay(p);
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

// Named views of the engine's arrays, for bit-exact comparison: returns the element count.
uint64_t orc_array(void* h, const char* name, const void** ptr) {
    Engine* e = static_cast<Engine*>(h);
    const std::string n = name;
#define ARR(x) if (n == #x) { *ptr = e->x.data(); return e->x.size(); }
    ARR(lens) ARR(feed) ARR(tree) ARR(path) ARR(path_len) ARR(on_path) ARR(trace_len) ARR(page_table) ARR(free_pages)
    ARR(tokens) ARR(tin) ARR(vis) ARR(head_rows) ARR(hidden_rows) ARR(out_ids) ARR(tiles) ARR(emitted) ARR(meta)
    ARR(logits) ARR(hidden_out) ARR(taps) ARR(k_cache) ARR(v_cache) ARR(draft_logits) ARR(taps_all)
    ARR(cap_resid_in) ARR(cap_attn_in) ARR(cap_qkv) ARR(cap_sdpa_out) ARR(cap_attn_out) ARR(cap_mlp_in) ARR(cap_mlp_out)
#undef ARR
    if (n == "draft_k_cache" && e->drafter) { *ptr = e->drafter->k_cache.data(); return e->drafter->k_cache.size(); }
    if (n == "draft_v_cache" && e->drafter) { *ptr = e->drafter->v_cache.data(); return e->drafter->v_cache.size(); }
    if (n == "carry" && e->drafter) { *ptr = e->drafter->carry.data(); return e->drafter->carry.size(); }
    if (n == "q_rows" && e->drafter) { *ptr = e->drafter->q_rows.data(); return e->drafter->q_rows.size(); }
    if (n == "q_keep" && e->drafter) { *ptr = e->drafter->q_keep.data(); return e->drafter->q_keep.size(); }
    if (e->lim) {
        if (n == "limite_k_local") { *ptr = e->lim->k_local.data(); return e->lim->k_local.size(); }
        if (n == "limite_v_local") { *ptr = e->lim->v_local.data(); return e->lim->v_local.size(); }
    }
    if (e->block_drafter) {
        BlockDrafter& b = *e->block_drafter;
        if (n == "block_logits") { *ptr = b.logits.data(); return b.logits.size(); }
        if (n == "block_hfin") { *ptr = b.hfin.data(); return b.hfin.size(); }
        if (n == "block_ctx_ring") { *ptr = b.ctx_ring.data(); return b.ctx_ring.size(); }
        if (n == "block_k_ring") { *ptr = b.k_ring.data(); return b.k_ring.size(); }
        if (n == "block_v_ring") { *ptr = b.v_ring.data(); return b.v_ring.size(); }
    }
    if (n == "gen") { *ptr = e->gen.data(); return e->gen.size() * sizeof(GenState) / 4; }
    if (n == "runs") { *ptr = e->runs.data(); return e->runs.size() * 6; }
    if (n == "sample_rows") { *ptr = e->sample_rows.data(); return e->sample_rows.size() * 6; }
    *ptr = nullptr;
    return 0;
}
// Overwrites words of lens, feed or tree from word `index`.
int orc_array_write(void* h, const char* name, uint64_t index, const uint32_t* data, uint64_t n) {
    Engine* e = static_cast<Engine*>(h);
    const std::string nm = name;
    if ((nm == "draft_k_cache" || nm == "draft_v_cache") && e->drafter) {  // one cache element (bf16 bits) per word
        std::vector<uint16_t>& c = nm == "draft_k_cache" ? e->drafter->k_cache : e->drafter->v_cache;
        if (index + n > c.size()) { g_err = "orc_array_write: " + nm; return 1; }
        for (uint64_t i = 0; i < n; i++) c[index + i] = uint16_t(data[i]);
        return 0;
    }
    std::vector<uint32_t>* v = nm == "lens" ? &e->lens : nm == "feed" ? &e->feed : nm == "tree" ? &e->tree : nullptr;
    if (!v || index + n > v->size()) { g_err = "orc_array_write: " + nm; return 1; }
    std::copy_n(data, n, v->begin() + index);
    return 0;
}
void orc_model_desc(void* h, uint32_t* out12) {
    const ModelDesc& m = static_cast<Engine*>(h)->md;
    const uint32_t v[12] = {m.n_layers, m.d, m.n_heads, m.n_kv, m.hd, m.ffn, m.vocab, m.vocab_real, m.page, f2u(m.eps), f2u(m.attn_scale),
                            static_cast<Engine*>(h)->n_pages};
    std::memcpy(out12, v, sizeof v);
}

// ---- the reference's block drafter, stand-alone (block_drafter.hpp)
void* orc_block_new(const char* path, float eps, float scale, const float* freq32, uint32_t max_seqs, uint32_t max_chunk) {
    try {
        auto b = std::make_unique<BlockDrafter>(path, eps, scale, std::vector<float>(freq32, freq32 + 32));
        b->init_state(max_seqs, max_chunk);
        return b.release();
    } catch (const std::exception& e) { fail(e); return nullptr; }
}
void orc_block_free(void* h) { delete static_cast<BlockDrafter*>(h); }
void orc_block_desc(void* h, uint32_t* out8) {
    const BlockDrafter* b = static_cast<BlockDrafter*>(h);
    const uint32_t v[8] = {b->n_layers, b->n_taps, b->block, b->window, b->v, b->H, b->FFN, b->ring};
    std::memcpy(out8, v, sizeof v);
}
// taps [n_taps][n][H] fp32 (bf16 values); meta [n][2] (slot, position); on_path [n] or NULL.
int orc_block_context(void* h, uint32_t n, const float* taps, const uint32_t* meta, const uint32_t* on_path) {
    try {
        BlockDrafter* b = static_cast<BlockDrafter*>(h);
        std::vector<const float*> rows;
        for (uint32_t k = 0; k < b->n_taps; k++) rows.push_back(taps + size_t(k) * n * b->H);
        b->context(n, rows, meta, on_path);
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}
// Per block: slot, rows, the bonus token's position, its embedding row ([n_blocks][H] bf16).
int orc_block_run(void* h, uint32_t n_blocks, const uint32_t* slots, const uint32_t* rows, const uint32_t* p0, const uint16_t* bonus_rows) {
    try {
        BlockDrafter* b = static_cast<BlockDrafter*>(h);
        std::vector<BlockDrafter::Block> bl;
        for (uint32_t i = 0; i < n_blocks; i++) bl.push_back(BlockDrafter::Block{slots[i], rows[i], p0[i], bonus_rows + size_t(i) * b->H});
        b->blocks(bl);
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}
uint64_t orc_block_array(void* h, const char* name, const void** ptr) {
    BlockDrafter* b = static_cast<BlockDrafter*>(h);
    const std::string n = name;
    if (n == "hfin") { *ptr = b->hfin.data(); return b->hfin.size(); }
    if (n == "logits") { *ptr = b->logits.data(); return b->logits.size(); }
    if (n == "ctx_ring") { *ptr = b->ctx_ring.data(); return b->ctx_ring.size(); }
    if (n == "k_ring") { *ptr = b->k_ring.data(); return b->k_ring.size(); }
    if (n == "v_ring") { *ptr = b->v_ring.data(); return b->v_ring.size(); }
    if (n == "vocab") { *ptr = b->vocab.data(); return b->vocab.size(); }
    *ptr = nullptr;
    return 0;
}

}  // extern "C"
