// CPU oracle (test infrastructure only, parity unpinned: see bits.hpp): the engine's step --
// plan, forward pass, sampling, acceptance, KV compaction, test drafter -- on host memory,
// for a Llama-style decoder described by the weight file's `meta` tensor.
//
// The reference hard-codes one architecture (engine/src/model.rs:6-20). Here its numeric
// conventions are applied to a plain pre-norm decoder (RMSNorm, RoPE, grouped-query
// attention, SwiGLU), every layer paged ("global", engine/src/engine/kv.rs). What is kept
// from the reference, with the place it comes from:
//   - the residual stream is fp32 and a layer's RMSNorm is folded into the next matmul:
//     y = (W . x) * rsqrt(mean(x^2) + eps)                       kernels.metal:184-199,286
//   - weights are bf16, or int8 with bf16 scales per group of consecutive k   :150-181
//   - gate_up rows are interleaved (gate_0, up_0, gate_1, ...), act = silu(g) * u   :204-209
//   - RoPE rotates interleaved pairs with a (cos, sin) table rounded to bf16   :725-736,
//     engine.rs:392-409
//   - K and V are rounded to bf16 before caching and that rounded value is what attention
//     multiplies, for the step's own rows too                    kernels.metal:925-931
//   - a row's K/V go to cache position p0 + row, its RoPE angle is that of lens + depth  :74-77
//   - softmax in base 2 with scale * log2(e) folded into q       :1036, encode.rs:246
// What differs, because the target device multiplies on bf16 tensor cores: a matmul's input
// activations and the scaled, rotated q are rounded to bf16 first (the reference keeps them
// fp32), and the softmax subtracts the row maximum (the reference's q/k norms bound its
// scores, kernels.metal:803-806; a plain decoder's are unbounded). Sums inside matmuls and
// attention have no pinned order in the reference (Metal's matrix units), so those results are
// compared with a tolerance; everything integer is compared bit for bit.
#pragma once
#include <algorithm>
#include <cmath>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "bits.hpp"
#include "block_drafter.hpp"
#include "limite.hpp"
#include "linear.hpp"
#include "sampling.hpp"
#include "vlt.hpp"

namespace orc {

struct EngineConfig {
    uint32_t max_seqs = 8, max_step_tokens = 512, max_chunk = 512, kv_tokens = 65536, max_seq_len = 131072,
             max_head_rows = 64;
};
struct Sampling { float temperature = 0.0f, top_p = 1.0f; uint64_t seed = 0; };
enum Rows : uint32_t { ROWS_NONE = 0, ROWS_LAST = 1, ROWS_ALL = 2 };
constexpr uint32_t VERIFY_T = 8;

struct PlanRun { uint32_t seq; std::vector<uint32_t> tokens; Rows head; bool verify; };
struct Plan { uint32_t n = 0, n_head = 0, n_hidden = 0, n_runs = 0, n_tiles = 0; bool branches = false; };

struct Seq { uint32_t len = 0; std::vector<uint32_t> pages; Sampling sampling; };

struct Layer { Matrix qkv, o, gate_up, down; };

// The drafter of the benchmark configurations: one decoder layer over
// fc([tapped target hidden of position p-1 ; embedding of token p]) per position p, with its
// own KV cache that shares the target's page table, proposing a chain of drafts one at a time.
// Not in the reference (its drafter is a block drafter with a draft tree,
// engine/src/engine/drafter.rs:278-447); it writes the same feed/tree interface
// (kernels.metal:51-60) and reads the same tapped hidden states (kernels.metal:133-148).
struct Drafter {
    VltFile file;
    Matrix fc;  // [d][2 d]
    Layer layer;
    Matrix head;  // [v][d]
    std::vector<uint32_t> vocab;
    // The draft passes' attention window (meta[4]; 0 or absent: the whole context): a row sees the last `window` keys of
    // its context, extended down to the start of the page that holds the first of them. The reference's drafter layers
    // are sliding-window layers too (tools/spec/drafter.py:17, 1024 positions).
    uint32_t window = 0;
    std::vector<uint16_t> k_cache, v_cache;  // [n_pages][n_kv][page][hd]
    std::vector<float> carry;                // [max_seqs][d]: the tap of each slot's last position
    // For the rejection-sampling rule: the draft rows a slot's drafts were drawn from ([max_seqs][VERIFY_T - 1][v]),
    // how many of them are current (0 once a step has used them), and the draft vocabulary's inverse map.
    std::vector<float> q_keep;
    std::vector<uint32_t> q_rows, index_of;
};

struct Engine;
void limite_forward(Engine& e, const Plan& p);  // limite_forward.hpp

struct Engine {
    VltFile file;
    ModelDesc md{};
    EngineConfig cfg;
    const uint16_t* embed = nullptr;
    Matrix head;
    std::vector<Layer> layers;
    std::vector<float> rope;  // [pos][hd / 2][cos, sin]
    // KV pool: [layer][page][n_kv][page_tok][hd] (kernels.metal:692-711), and the page table.
    std::vector<uint16_t> k_cache, v_cache;
    std::vector<uint32_t> page_table, free_pages;
    uint32_t n_pages = 0, max_pages = 0;
    std::vector<std::optional<Seq>> seqs;
    // Per-slot state that lives on the GPU in the reference (engine/buffers.rs:42-55).
    std::vector<uint32_t> lens, feed, tree, path, path_len, on_path, trace, trace_len;
    std::vector<GenState> gen;
    // One step's inputs and outputs (engine/buffers.rs:120-156).
    std::vector<uint32_t> tokens, tin, vis, head_rows, hidden_rows, out_ids, tiles, emitted, meta;
    std::vector<SampleRow> sample_rows;
    std::vector<RunIn> runs;
    std::vector<float> logits, hidden_out, taps;  // taps: bf16(rms_norm(last layer's output)) as fp32, [n][d]
    ReplayArgs replay{0, 0, 0.0f, 0};
    std::unique_ptr<Drafter> drafter;
    std::unique_ptr<Limite> lim;  // the reference's own architecture (limite.hpp), if the weight file is one of its converter's
    uint32_t kv_layers = 0;       // layers of the paged pool: all of a plain decoder's, the global ones of a Limite model
    std::unique_ptr<BlockDrafter> block_drafter;  // the reference's block drafter (block_drafter.hpp), if that is what was loaded
    std::vector<float> rope_freq;
    std::vector<float> draft_logits;  // the drafter's passes, [rows - 1][runs][v]; rows of runs that did not draft stay 0
    std::vector<uint32_t> write_mask;  // per step token: does its K/V go to the cache (empty: all do)
    // engine.rs:175-188 `LayerCapture`: with `capture` set, `forward` keeps every target layer's intermediates, [layer][n][width].
    bool capture = false;
    std::vector<float> cap_resid_in, cap_attn_in, cap_qkv, cap_sdpa_out, cap_attn_out, cap_mlp_in, cap_mlp_out;
    // engine.rs:381-389 `set_taps`: bf16(rms_norm(output)) of these layers, [tap][n][d] (`taps` is the last layer's, always kept).
    std::vector<uint32_t> tap_layers;
    std::vector<float> taps_all;
    uint32_t attn_window = 0;  // set around the drafter's passes: see Drafter::window
    uint32_t accept_rule = 0;  // 0: the reference's sample-then-match; 1: rejection sampling where a run's drafts came with their q rows

    Engine(const std::string& file_path, const EngineConfig& c) : file(VltFile::load(file_path)), cfg(c) {
        if (Limite::is_limite(file)) {
            // engine/src/model.rs:6-20, read off the file instead of fixed: hidden width and vocabulary from `embed`, kv
            // heads from the qkv projection's rows, FFN from `down`, layers by counting; an optional `limite_vocab_real`
            // (f32[1]) names the first padding id, else the reference's 151 667 of 151 680.
            lim = std::make_unique<Limite>();
            const Tensor& et = file.tensor("embed");
            md.vocab = et.shape.at(0); md.d = et.shape.at(1); md.hd = Limite::D;
            if (md.d % Limite::D) throw std::runtime_error(file_path + ": hidden width is not a multiple of 128");
            md.n_heads = md.d / Limite::D;
            md.n_kv = (file.tensor("L00.qkv").shape.at(0) / Limite::D - md.n_heads) / 2;
            md.ffn = file.tensor("L00.down").shape.at(1);
            md.n_layers = 0;
            while (file.has("L" + std::string(md.n_layers < 10 ? "0" : "") + std::to_string(md.n_layers) + ".qkv")) md.n_layers++;
            md.vocab_real = file.has("limite_vocab_real") ? uint32_t(file.f32s("limite_vocab_real").at(0)) : md.vocab == 151680 ? 151667u : md.vocab;
            md.eps = 0x1p-23f; md.page = Limite::PAGE; md.attn_scale = 0.1f;  // kernels.metal:13, kv.rs:6, model.rs:19
            if (md.n_kv == 0 || md.n_heads % md.n_kv) throw std::runtime_error(file_path + ": the qkv projection's rows do not fit the heads");
        } else {
        std::vector<float> m = file.f32s("meta");
        if (m.size() < 14 || m[0] != 1.0f || m[1] != 0.0f) throw std::runtime_error(file_path + ": meta is not a version-1 llama descriptor");
        md.n_layers = uint32_t(m[2]); md.d = uint32_t(m[3]); md.n_heads = uint32_t(m[4]); md.n_kv = uint32_t(m[5]);
        md.hd = uint32_t(m[6]); md.ffn = uint32_t(m[7]); md.vocab = uint32_t(m[8]); md.vocab_real = uint32_t(m[9]);
        md.eps = m[10]; md.page = uint32_t(m[11]); md.attn_scale = m[13];
        }
        embed = reinterpret_cast<const uint16_t*>(file.ptr(file.get("embed", BF16, {md.vocab, md.d})));
        // engine/src/model.rs:139-140: the head is the embedding unless the file has one.
        if (file.has("head")) head = load_matrix(file, "head", md.vocab, md.d);
        else { head.w = reinterpret_cast<const uint8_t*>(embed); head.m = md.vocab; head.k = md.d; }
        for (uint32_t i = 0; i < md.n_layers; i++) {
            char nm[32];
            auto name = [&](const char* k) { std::snprintf(nm, sizeof nm, "L%02u.%s", i, k); return std::string(nm); };
            Layer l;
            l.qkv = load_matrix(file, name("qkv"), md.qkv_w(), md.d);
            l.o = load_matrix(file, name("o"), md.d, md.n_heads * md.hd);
            l.gate_up = load_matrix(file, name("gate_up"), 2 * md.ffn, md.d);
            l.down = load_matrix(file, name("down"), md.d, md.ffn);
            layers.push_back(l);
            if (!lim) continue;
            LimiteLayer x;  // model.rs:108-135
            auto f32 = [&](const char* k, std::vector<uint32_t> shape) { return reinterpret_cast<const float*>(file.ptr(file.get(name(k), F32, shape))); };
            x.global = i % 4 == 3;
            x.kv_index = x.global ? lim->n_global++ : lim->n_local++;
            x.attn_gate = f32("attn_gate", {md.n_heads, Limite::D});
            if (i % 3 == 1) x.ve_gate = f32("ve_gate", {md.n_kv, 12});
            x.xsa = f32("xsa", {md.n_heads});
            const float* sc = f32("scalars", {8});
            x.qkv_scale = sc[0]; x.o_scale = sc[1]; x.resid_attn = sc[2]; x.post_attn = sc[3]; x.resid_mlp = sc[4]; x.post_mlp = sc[5];
            lim->layers.push_back(x);
        }
        if (lim) {
            lim->value_embed = reinterpret_cast<const uint16_t*>(file.ptr(file.get("value_embed", BF16, {md.vocab, md.n_kv * Limite::D})));
            lim->mudd_dense1 = reinterpret_cast<const float*>(file.ptr(file.get("mudd.dense1", F32, {32, md.d})));
            lim->mudd_mix = reinterpret_cast<const float*>(file.ptr(file.get("mudd.mix", F32, {2, 2, 3, 33})));
            if (lim->n_global == 0 || lim->n_local == 0) throw std::runtime_error(file_path + ": a Limite model has local and global layers (at least 4 layers)");
            lim->init_state(cfg.max_seqs, cfg.max_chunk, md.n_kv);
        }
        // engine.rs:392-421 `rope_table`: theta = float32(pos) * freq, cos and sin rounded to bf16.
        std::vector<float> freq = file.f32s("rope_freq");
        rope_freq = freq;
        // (a Limite head of 128 turns its first 64 dims: 32 pairs, looked up as they are needed)
        if (freq.size() != (lim ? 32 : md.hd / 2)) throw std::runtime_error("rope_freq: expected head_dim / 2 entries (32 for the reference's own model)");
        const uint32_t npos = lim ? 0 : cfg.max_seq_len + FEED_W;
        rope.resize(size_t(npos) * md.hd);
        for (uint32_t p = 0; p < npos; p++)
            for (uint32_t i = 0; i < md.hd / 2; i++)
                rope_cs(p, freq[i], rope[(size_t(p) * (md.hd / 2) + i) * 2], rope[(size_t(p) * (md.hd / 2) + i) * 2 + 1]);
        // kv.rs:23-48 `KvCache::new`.
        n_pages = (cfg.kv_tokens + md.page - 1) / md.page;
        max_pages = (cfg.max_seq_len + md.page - 1) / md.page;
        kv_layers = lim ? lim->n_global : md.n_layers;
        const size_t kv = size_t(kv_layers) * n_pages * md.n_kv * md.page * md.hd;
        k_cache.assign(kv, 0);
        v_cache.assign(kv, 0);
        page_table.assign(size_t(cfg.max_seqs) * max_pages, 0);
        for (uint32_t i = n_pages; i-- > 0;) free_pages.push_back(i);
        seqs.resize(cfg.max_seqs);
        lens.assign(cfg.max_seqs, 0);
        feed.assign(cfg.max_seqs * FEED_W, 0);
        tree.resize(cfg.max_seqs * FEED_W);
        for (uint32_t i = 0; i < tree.size(); i++) tree[i] = chain_node(i % FEED_W);  // buffers.rs:112-113
        gen.assign(cfg.max_seqs, GenState{0xffffffffu, 0, 0, 0, {0}});
        path.assign(cfg.max_seqs * FEED_W, 0);
        path_len.assign(cfg.max_seqs, 0);
        trace.assign(size_t(cfg.max_seqs) * cfg.max_seq_len, 0);
        trace_len.assign(cfg.max_seqs, 0);
    }

    // ---- engine.rs:259-303
    uint32_t new_seq() {
        for (uint32_t s = 0; s < seqs.size(); s++)
            if (!seqs[s]) {
                seqs[s] = Seq{};
                lens[s] = 0;
                trace_len[s] = 0;
                gen[s] = GenState{0xffffffffu, 0, 0, 0, {0}};
                if (drafter) drafter->q_rows[s] = 0;
                return s;
            }
        throw std::runtime_error("no free sequence slot");
    }
    void free_seq(uint32_t s) {
        if (s < seqs.size() && seqs[s]) {
            for (size_t i = seqs[s]->pages.size(); i-- > 0;) free_pages.push_back(seqs[s]->pages[i]);  // kv.rs:60-62
            seqs[s].reset();
        }
    }
    Seq& seq(uint32_t s) {
        if (s >= seqs.size() || !seqs[s]) throw std::runtime_error("unknown sequence");
        return *seqs[s];
    }
    // kv.rs:51-58 `reserve`.
    void reserve(uint32_t slot, std::vector<uint32_t>& pages, uint32_t len) {
        while (pages.size() * md.page < len) {
            if (free_pages.empty()) throw std::runtime_error("global KV pool exhausted");
            uint32_t page = free_pages.back();
            free_pages.pop_back();
            page_table[size_t(slot) * max_pages + pages.size()] = page;
            pages.push_back(page);
        }
    }
    // hooks.rs:28-36 `bench_fill`: the sequence advances without being computed. The reference leaves the new
    // positions' K/V as allocated; with a seed they are filled with the same hashed values the CUDA engine's fill
    // writes (Philox of (position, layer * 64 + kv head, pair of dims, slot) under the key (seed, 0x6b76): four
    // words -> k pair, v pair, each (u >> 8) * 2^-24 mapped to [-1, 1) and rounded to bf16), so that a step over a
    // filled context can be compared value for value.
    void bench_fill(uint32_t s, uint32_t len, uint32_t seed = 0) {
        Seq& q = seq(s);
        const uint32_t from = q.len;
        q.len += len;
        lens[s] = q.len;
        reserve(s, q.pages, q.len);
        if (!seed) return;
        if (lim) throw std::runtime_error("bench_fill with values is for the paged pool of a plain decoder");
        auto val = [](uint32_t u) { return (float(u >> 8) * 0x1p-24f - 0.5f) * 2.0f; };
#pragma omp parallel for schedule(static) collapse(2)
        for (int64_t l = 0; l < int64_t(md.n_layers); l++)
            for (int64_t pos = from; pos < int64_t(q.len); pos++)
                for (uint32_t g = 0; g < md.n_kv; g++) {
                    const size_t at = kv_row(uint32_t(l), s, g, uint32_t(pos));
                    for (uint32_t d = 0; d < md.hd / 2; d++) {
                        const U4 h = philox(U4{uint32_t(pos), uint32_t(l) * 64 + g, d, s}, seed, 0x6b76u);
                        k_cache[at + 2 * d] = f32_to_bf16(val(h.x));
                        k_cache[at + 2 * d + 1] = f32_to_bf16(val(h.y));
                        v_cache[at + 2 * d] = f32_to_bf16(val(h.z));
                        v_cache[at + 2 * d + 1] = f32_to_bf16(val(h.w));
                    }
                }
    }

    // ---- plan.rs:47-150 `plan` (the attention split heuristics are device-specific and left out).
    Plan plan(const std::vector<PlanRun>& in, Rows hidden) {
        uint32_t n = 0;
        for (auto& r : in) n += uint32_t(r.tokens.size());
        if (n == 0 || n > cfg.max_step_tokens) throw std::runtime_error("step has " + std::to_string(n) + " tokens (max " + std::to_string(cfg.max_step_tokens) + ")");
        tokens.clear(); tin.clear(); vis.clear(); head_rows.clear(); hidden_rows.clear(); sample_rows.clear(); tiles.clear(); runs.clear();
        Plan p;
        for (size_t ri = 0; ri < in.size(); ri++) {
            const PlanRun& run = in[ri];
            const uint32_t id = run.seq, count = uint32_t(run.tokens.size());
            if (count == 0 || count > cfg.max_chunk) throw std::runtime_error(std::to_string(count) + " tokens for one sequence in a step (max_chunk " + std::to_string(cfg.max_chunk) + ")");
            for (uint32_t t : run.tokens)
                if (t >= FEED_ROW && t - FEED_ROW >= FEED_W) throw std::runtime_error("only 16 GPU-fed tokens per slot");
            for (size_t j = 0; j < ri; j++)
                if (in[j].seq == id) throw std::runtime_error("a sequence appears twice in one step");
            Seq& s = seq(id);
            const uint32_t new_len = s.len + count;
            if (new_len > cfg.max_seq_len) throw std::runtime_error("sequence would reach " + std::to_string(new_len) + " tokens (max " + std::to_string(cfg.max_seq_len) + ")");
            // With a drafter loaded the draft passes write their own K/V up to VERIFY_T positions past the step.
            reserve(id, s.pages, drafter ? std::min(new_len + VERIFY_T, cfg.max_seq_len) : new_len);
            const uint32_t first_row = uint32_t(tokens.size());
            tokens.insert(tokens.end(), run.tokens.begin(), run.tokens.end());
            for (uint32_t row = 0; row < count; row++) {
                tin.push_back(id);
                tin.push_back(row);
                vis.push_back(0xffffffffu >> (31 - row % 8));
            }
            auto rows = [&](Rows r, std::vector<uint32_t>& v) {
                if (r == ROWS_LAST) v.push_back(first_row + count - 1);
                if (r == ROWS_ALL) for (uint32_t x = first_row; x < first_row + count; x++) v.push_back(x);
            };
            const uint32_t first_head = uint32_t(head_rows.size());
            rows(run.verify ? ROWS_ALL : run.head, head_rows);
            rows(hidden, hidden_rows);
            for (uint32_t h = first_head; h < head_rows.size(); h++)  // engine.rs:123-138 `row_of`
                sample_rows.push_back(SampleRow{uint32_t(s.sampling.seed), uint32_t(s.sampling.seed >> 32), 0, s.sampling.temperature, s.sampling.top_p, head_rows[h]});
            runs.push_back(RunIn{id, first_row, count, first_head, uint32_t(head_rows.size()) - first_head, run.verify ? 1u : 0u});
            for (uint32_t i = 0; i < count; i += 8) {
                tiles.push_back(first_row + i);
                tiles.push_back(std::min(count - i, 8u));
            }
            p.branches = p.branches || (run.verify && count > 2);
            s.len = new_len;
        }
        if (head_rows.size() > cfg.max_head_rows) throw std::runtime_error(std::to_string(head_rows.size()) + " head rows (max " + std::to_string(cfg.max_head_rows) + ")");
        p.n = n;
        p.n_head = uint32_t(head_rows.size());
        p.n_hidden = uint32_t(hidden_rows.size());
        p.n_runs = uint32_t(in.size());
        p.n_tiles = uint32_t(tiles.size() / 2);
        return p;
    }

    // Where kv head g's row for cache position pos starts (kernels.metal:704-711, global layers).
    size_t limite_ring_row(uint32_t layer, uint32_t slot, uint32_t g, uint32_t pos) const {  // kernels.metal:710 `kv_row_of`, local
        return ((size_t(layer) * lim->max_seqs + slot) * md.n_kv + g) * lim->ring * md.hd + size_t(pos % lim->ring) * md.hd;
    }
    size_t kv_row(uint32_t layer, uint32_t slot, uint32_t g, uint32_t pos) const {
        const uint32_t page = page_table[size_t(slot) * max_pages + pos / md.page];
        return ((size_t(layer) * n_pages + page) * md.n_kv + g) * md.page * md.hd + size_t(pos % md.page) * md.hd;
    }

    void rope_head(float* v, uint32_t pos) const { rope_pairs(v, md.hd, rope.data() + size_t(pos) * md.hd); }

    // One decoder layer's attention over the step, K/V written first (kernels.metal:749-801
    // `qkv_post`), then every query tile against the cache (kernels.metal:891-1167).
    void attention(uint32_t layer, uint16_t* kc, uint16_t* vc, const float* qkv, uint32_t n, uint32_t n_tiles, float* out) {
        const uint32_t hd = md.hd, G = md.n_heads / md.n_kv, QW = md.qkv_w();
        const uint32_t koff = md.n_heads * hd, voff = koff + md.n_kv * hd;
        for (uint32_t t = 0; t < n; t++) {
            const uint32_t slot = meta[2 * t], pos = meta[2 * t + 1], row = tin[2 * t + 1];
            const uint32_t cpos = meta[2 * (t - row) + 1] + row;  // kernels.metal:74-77 `cache_pos`
            if (!write_mask.empty() && !write_mask[t]) continue;  // the drafter's passes write the rows that count only
            for (uint32_t g = 0; g < md.n_kv; g++) {
                std::vector<float> k(qkv + size_t(t) * QW + koff + g * hd, qkv + size_t(t) * QW + koff + (g + 1) * hd);
                rope_head(k.data(), pos);
                const size_t at = kv_row(layer, slot, g, cpos);
                for (uint32_t d = 0; d < hd; d++) {
                    kc[at + d] = f32_to_bf16(k[d]);
                    vc[at + d] = f32_to_bf16(qkv[size_t(t) * QW + voff + g * hd + d]);
                }
            }
        }
        const float sl2 = md.attn_scale * LOG2E;
#pragma omp parallel for schedule(dynamic) collapse(2)
        for (int64_t ti = 0; ti < int64_t(n_tiles); ti++) {
            for (int64_t h = 0; h < int64_t(md.n_heads); h++) {
                const uint32_t t0 = tiles[2 * ti], T = tiles[2 * ti + 1], g = uint32_t(h) / G;
                const uint32_t slot = meta[2 * t0], p0 = meta[2 * t0 + 1];
                const uint32_t lo = attn_window && p0 + T > attn_window ? (p0 + T - attn_window) / md.page * md.page : 0;
                std::vector<float> sc(p0 + T), q(hd), o(hd);
                for (uint32_t i = 0; i < T; i++) {
                    const uint32_t t = t0 + i;
                    for (uint32_t d = 0; d < hd; d++) q[d] = qkv[size_t(t) * QW + h * hd + d];
                    rope_head(q.data(), meta[2 * t + 1]);
                    for (uint32_t d = 0; d < hd; d++) q[d] = round_bf16(q[d] * sl2);
                    float mx = -INFINITY;
                    for (uint32_t kp = lo; kp < p0 + T; kp++) {
                        const bool seen = kp < p0 || ((vis[t] >> (kp - p0)) & 1u);
                        if (!seen) { sc[kp] = -INFINITY; continue; }
                        const uint16_t* kr = kc + kv_row(layer, slot, g, kp);
                        float a = 0.0f;
#pragma omp simd reduction(+ : a)
                        for (uint32_t d = 0; d < hd; d++) a += q[d] * bf16_to_f32(kr[d]);
                        sc[kp] = a;
                        mx = std::max(mx, a);
                    }
                    float l = 0.0f;
                    std::fill(o.begin(), o.end(), 0.0f);
                    for (uint32_t kp = lo; kp < p0 + T; kp++) {
                        if (sc[kp] == -INFINITY) continue;
                        const float pz = std::exp2(sc[kp] - mx);
                        l += pz;
                        const uint16_t* vr = vc + kv_row(layer, slot, g, kp);
                        for (uint32_t d = 0; d < hd; d++) o[d] += pz * bf16_to_f32(vr[d]);
                    }
                    for (uint32_t d = 0; d < hd; d++) out[size_t(t) * md.n_heads * hd + h * hd + d] = o[d] / l;
                }
            }
        }
    }

    // One decoder layer on x [n][d] in place: encode.rs:142-192 with the plain decoder's
    // parameters (scales and lambdas 1, no MUDD, gates, XSA or value embeddings).
    void layer_forward(const Layer& L, uint32_t li, uint16_t* kc, uint16_t* vc, float* x, uint32_t n, uint32_t n_tiles, bool keep = false) {
        const uint32_t d = md.d, QW = md.qkv_w();
        std::vector<float> inv(n), qkv(size_t(n) * QW), attn(size_t(n) * md.n_heads * md.hd), acc(size_t(n) * std::max(2 * md.ffn, QW)), act(size_t(n) * md.ffn);
        auto put = [&](std::vector<float>& dst, const float* src, size_t width) { if (keep) dst.insert(dst.end(), src, src + size_t(n) * width); };
        auto put_normed = [&](std::vector<float>& dst) {
            if (!keep) return;
            for (uint32_t t = 0; t < n; t++)
                for (uint32_t j = 0; j < d; j++) dst.push_back(x[size_t(t) * d + j] * inv[t]);
        };
        put(cap_resid_in, x, d);
        inv_rms(x, n, d, md.eps, inv.data());
        put_normed(cap_attn_in);
        matmul_raw(L.qkv, x, n, qkv.data());
        for (uint32_t t = 0; t < n; t++)
            for (uint32_t j = 0; j < QW; j++) qkv[size_t(t) * QW + j] *= inv[t];  // EPI_NORM
        if (keep) {  // q | k | v with RoPE on the q and k heads, before the rounding and q's scale
            std::vector<float> r = qkv;
            for (uint32_t t = 0; t < n; t++)
                for (uint32_t hh = 0; hh < md.n_heads + md.n_kv; hh++) rope_head(r.data() + size_t(t) * QW + hh * md.hd, meta[2 * t + 1]);
            put(cap_qkv, r.data(), QW);
        }
        attention(li, kc, vc, qkv.data(), n, n_tiles, attn.data());
        put(cap_sdpa_out, attn.data(), md.n_heads * md.hd);
        matmul_raw(L.o, attn.data(), n, acc.data());
        put(cap_attn_out, acc.data(), d);
        for (size_t i = 0; i < size_t(n) * d; i++) x[i] += acc[i];  // EPI_RESID: mixed
        inv_rms(x, n, d, md.eps, inv.data());
        put_normed(cap_mlp_in);
        matmul_raw(L.gate_up, x, n, acc.data());
        for (uint32_t t = 0; t < n; t++)
            for (uint32_t j = 0; j < md.ffn; j++) {  // EPI_SWIGLU, kernels.metal:204-209
                const float g = acc[size_t(t) * 2 * md.ffn + 2 * j] * inv[t], u = acc[size_t(t) * 2 * md.ffn + 2 * j + 1] * inv[t];
                act[size_t(t) * md.ffn + j] = g * (1.0f / (1.0f + std::exp(-g))) * u;
            }
        matmul_raw(L.down, act.data(), n, acc.data());
        put(cap_mlp_out, acc.data(), d);
        for (size_t i = 0; i < size_t(n) * d; i++) x[i] += acc[i];
    }

    // encode.rs:99-105 `encode_forward` + :383-412 `encode_tail`.
    void forward(const Plan& p) {
        if (lim) { limite_forward(*this, p); return; }
        const uint32_t n = p.n, d = md.d;
        meta.assign(2 * n, 0);
        std::vector<float> x(size_t(n) * d);
        for (uint32_t t = 0; t < n; t++) {  // kernels.metal:82-114 `embed` (a plain decoder: no norm)
            const uint32_t slot = tin[2 * t];
            uint32_t tok = tokens[t], depth = tin[2 * t + 1];
            if (tok >= FEED_ROW) {
                const uint32_t i = tok - FEED_ROW, node = tree[slot * FEED_W + i];
                tok = feed[slot * FEED_W + i];
                depth = node_depth(node);
                vis[t] = node_sees(node);
            }
            tokens[t] = tok;
            meta[2 * t] = slot;
            meta[2 * t + 1] = lens[slot] + depth;
            for (uint32_t i = 0; i < d; i++) x[size_t(t) * d + i] = bf16_to_f32(embed[size_t(tok) * d + i]);
        }
        for (std::vector<float>* c : {&cap_resid_in, &cap_attn_in, &cap_qkv, &cap_sdpa_out, &cap_attn_out, &cap_mlp_in, &cap_mlp_out}) c->clear();
        taps_all.assign(tap_layers.size() * size_t(n) * d, 0.0f);
        for (uint32_t li = 0; li < md.n_layers; li++) {
            layer_forward(layers[li], li, k_cache.data(), v_cache.data(), x.data(), n, p.n_tiles, capture);
            for (size_t ti = 0; ti < tap_layers.size(); ti++) {
                if (tap_layers[ti] != li) continue;
                std::vector<float> tinv(n);
                inv_rms(x.data(), n, d, md.eps, tinv.data());
                for (uint32_t t = 0; t < n; t++)
                    for (uint32_t i = 0; i < d; i++) taps_all[(ti * n + t) * d + i] = round_bf16(x[size_t(t) * d + i] * tinv[t]);
            }
        }
        std::vector<float> inv(n);
        inv_rms(x.data(), n, d, md.eps, inv.data());
        taps.resize(size_t(n) * d);  // kernels.metal:133-148 `tap_rows`
        for (uint32_t t = 0; t < n; t++)
            for (uint32_t i = 0; i < d; i++) taps[size_t(t) * d + i] = round_bf16(x[size_t(t) * d + i] * inv[t]);
        hidden_out.resize(size_t(p.n_hidden) * d);
        for (uint32_t r = 0; r < p.n_hidden; r++)
            for (uint32_t i = 0; i < d; i++) hidden_out[size_t(r) * d + i] = x[size_t(hidden_rows[r]) * d + i] * inv[hidden_rows[r]];
        out_ids.assign(p.n_head, 0);
        if (p.n_head) {
            std::vector<float> hx(size_t(p.n_head) * d);
            for (uint32_t r = 0; r < p.n_head; r++) std::copy_n(x.data() + size_t(head_rows[r]) * d, d, hx.data() + size_t(r) * d);
            logits.resize(size_t(p.n_head) * md.vocab);
            matmul_raw(head, hx.data(), p.n_head, logits.data());
            for (uint32_t r = 0; r < p.n_head; r++)
                for (uint32_t j = 0; j < md.vocab; j++) {
                    float& l = logits[size_t(r) * md.vocab + j];
                    l = j < md.vocab_real ? l * inv[head_rows[r]] : -INFINITY;
                }
        }
        finish_step(p);
    }

    // encode.rs:395-412, from the logits on: each head row's token, `accept`, and the accepted paths' K/V into place.
    void finish_step(const Plan& p) {
        const uint32_t n = p.n;
        if (p.n_head) {
#pragma omp parallel for schedule(dynamic)
            for (int64_t r = 0; r < int64_t(p.n_head); r++) {
                const SampleRow& sr = sample_rows[r];
                const uint32_t pos = sr.tok == NO_TOK ? sr.pos : meta[2 * sr.tok + 1] + 1;
                out_ids[r] = sample_row(logits.data() + size_t(r) * md.vocab, md.vocab, sr, pos);
            }
        }
        emitted.assign(p.n_runs, 0);
        on_path.assign(n, 0);
        std::vector<uint32_t> decided(p.n_runs, 0);
        if (accept_rule == 1 && drafter) {
            for (uint32_t r = 0; r < p.n_runs; r++) {
                if (spec_applies(r)) decided[r] = spec_decide(r);
                drafter->q_rows[runs[r].slot] = 0;  // a slot's kept rows serve one step
            }
        }
        for (uint32_t r = 0; r < p.n_runs; r++)
            accept_run(r, runs.data(), tokens.data(), out_ids.data(), lens.data(), feed.data(), gen.data(), emitted.data(), tree.data(), path.data(), path_len.data(), on_path.data(), decided[r]);
        if (p.branches) kv_compact(p, k_cache.data(), v_cache.data(), kv_layers);
    }

    // Whether run r is decided by the rejection rule: a verify run of a sequence that samples (temperature > 0, no
    // top-p cut), whose rows are a plain chain and whose drafts all came with a kept q row from the step before.
    bool spec_applies(uint32_t r) const {
        const RunIn& ru = runs[r];
        if (!ru.verify || ru.count < 2 || ru.nhead != ru.count) return false;
        const SampleRow& sr = sample_rows[ru.head0];
        if (!(sr.temperature > 0.0f) || sr.top_p < 1.0f) return false;
        if (drafter->q_rows[ru.slot] + 1 < ru.count) return false;
        for (uint32_t c2 = 1; c2 < ru.count; c2++)
            if (tree[ru.slot * FEED_W + c2] != chain_node(c2)) return false;
        return true;
    }
    uint32_t spec_decide(uint32_t r) {
        const RunIn& ru = runs[r];
        const SampleRow& sr = sample_rows[ru.head0];
        const uint32_t v = drafter->head.m;
        uint32_t pos[FEED_W];
        for (uint32_t i = 0; i < ru.count; i++) pos[i] = meta[2 * (ru.first + i) + 1];
        return spec_step_run(logits.data() + size_t(ru.head0) * md.vocab, md.vocab, drafter->q_keep.data() + size_t(ru.slot) * (VERIFY_T - 1) * v, v,
                             drafter->index_of.data(), tokens.data() + ru.first, pos, ru.count, sr.temperature, sr.seed_lo, sr.seed_hi, out_ids.data() + ru.head0);
    }

    // kernels.metal:1663-1693 `kv_compact` over `nl` layers of a cache with the pool's layout.
    void kv_compact(const Plan& p, uint16_t* kc, uint16_t* vc, uint32_t nl) {
        for (uint32_t r = 0; r < p.n_runs; r++) {
            const uint32_t k = path_len[r], slot = runs[r].slot, p0 = lens[slot] - k;
            if (lim && kc == k_cache.data())  // the local layers' rings as well (kernels.metal:1663-1693 takes both kinds)
                for (uint32_t l = 0; l < lim->n_local; l++)
                    for (uint32_t g = 0; g < md.n_kv; g++)
                        for (uint32_t j = 1; j < k; j++) {
                            const uint32_t from = path[r * FEED_W + j];
                            if (from == j) continue;
                            const size_t src = limite_ring_row(l, slot, g, p0 + from), dst = limite_ring_row(l, slot, g, p0 + j);
                            std::copy_n(lim->k_local.data() + src, md.hd, lim->k_local.data() + dst);
                            std::copy_n(lim->v_local.data() + src, md.hd, lim->v_local.data() + dst);
                        }
            for (uint32_t l = 0; l < nl; l++)
                for (uint32_t g = 0; g < md.n_kv; g++)
                    for (uint32_t j = 1; j < k; j++) {
                        const uint32_t from = path[r * FEED_W + j];
                        if (from == j) continue;
                        const size_t src = kv_row(l, slot, g, p0 + from), dst = kv_row(l, slot, g, p0 + j);
                        std::copy_n(kc + src, md.hd, kc + dst);
                        std::copy_n(vc + src, md.hd, vc + dst);
                    }
        }
    }

    // ---- the chain drafter (a benchmark extension, see `Drafter`)
    void load_drafter(const std::string& path) {
        auto dr = std::make_unique<Drafter>();
        dr->file = VltFile::load(path);
        if (BlockDrafter::is_block_drafter(dr->file)) {  // engine/src/engine.rs:381-389 with a file of tools/spec/export.py
            if (rope_freq.size() != 32 || md.d % BlockDrafter::D) throw std::runtime_error(path + ": the block drafter needs a target whose hidden width is a multiple of 128 and whose RoPE table has 32 pairs");
            block_drafter = std::make_unique<BlockDrafter>(path, md.eps, md.attn_scale, rope_freq);
            if (block_drafter->H != md.d) throw std::runtime_error(path + ": hidden width " + std::to_string(block_drafter->H) + ", the target's is " + std::to_string(md.d));
            block_drafter->init_state(cfg.max_seqs, cfg.max_chunk);
            tap_layers = block_drafter->taps;
            return;
        }
        const std::vector<float> m = dr->file.f32s("meta");
        if (m.size() < 4 || m[0] != 1.0f || m[1] != 1.0f || m[2] != 1.0f) throw std::runtime_error(path + ": meta is not a version-1 one-layer chain drafter");
        const uint32_t v = uint32_t(m[3]), d = md.d;
        dr->window = m.size() > 4 ? uint32_t(m[4]) : 0;
        if (md.ffn < 2 * d) throw std::runtime_error(path + ": the chain drafter needs ffn >= 2 d_model");
        dr->fc = load_matrix(dr->file, "fc", d, 2 * d);
        dr->layer.qkv = load_matrix(dr->file, "D00.qkv", md.qkv_w(), d);
        dr->layer.o = load_matrix(dr->file, "D00.o", d, md.n_heads * md.hd);
        dr->layer.gate_up = load_matrix(dr->file, "D00.gate_up", 2 * md.ffn, d);
        dr->layer.down = load_matrix(dr->file, "D00.down", d, md.ffn);
        dr->head = load_matrix(dr->file, "head", v, d);
        for (float id : dr->file.f32s("vocab")) dr->vocab.push_back(uint32_t(id));
        if (dr->vocab.size() != v) throw std::runtime_error(path + ": vocab has " + std::to_string(dr->vocab.size()) + " ids for a head of " + std::to_string(v));
        for (uint32_t id : dr->vocab)
            if (id >= md.vocab) throw std::runtime_error(path + ": draft vocabulary id out of the target's range");
        const size_t pool = size_t(n_pages) * md.n_kv * md.page * md.hd;
        dr->k_cache.assign(pool, 0);
        dr->v_cache.assign(pool, 0);
        dr->carry.assign(size_t(cfg.max_seqs) * d, 0.0f);
        dr->q_keep.assign(size_t(cfg.max_seqs) * (VERIFY_T - 1) * v, 0.0f);
        dr->q_rows.assign(cfg.max_seqs, 0);
        dr->index_of.assign(md.vocab, NO_TOK);
        for (uint32_t j = 0; j < v; j++) dr->index_of[dr->vocab[j]] = j;
        drafter = std::move(dr);
    }

    // The drafter's part of a step, after `forward`: (1) a catch-up pass over the step's own tokens -- input
    // fc([feature of the position before ; embedding]), the feature being the target's tap of the row before
    // (the slot's carried tap for a run's first row, zero at position 0) -- that writes the drafter's K/V for
    // the rows on the accepted path only; (2) rows - 1 draft passes of one row per run: pass i stands at
    // position lens[slot] + i - 1 on token feed[slot][i - 1], its feature the tap of the path's last row
    // (i = 1) or the drafter's own normed output of the pass before, and writes feed[slot][i] = the draft
    // vocabulary's argmax (ties to the lowest index) and tree[slot][i] = chain_node(i).
    // engine/src/engine/drafter.rs:278-447 `encode_drafter`: the context of the step's tokens (those on the accepted path
    // reach the rings), a block of `rows` rows for every run with head rows, candidates and a draft tree per block.
    void block_draft(const Plan& p, uint32_t rows) {
        BlockDrafter& b = *block_drafter;
        std::vector<const float*> tap_rows;
        for (size_t k = 0; k < tap_layers.size(); k++) tap_rows.push_back(taps_all.data() + k * size_t(p.n) * md.d);
        b.context(p.n, tap_rows, meta.data(), on_path.data());
        std::vector<BlockDrafter::Block> bl;
        std::vector<uint32_t> btin, first;
        for (uint32_t r = 0; r < p.n_runs && rows > 1; r++) {
            if (runs[r].nhead == 0) continue;
            const uint32_t slot = runs[r].slot;
            uint32_t tok = feed[slot * FEED_W];
            if (tok >= md.vocab) tok = 0;
            first.push_back(uint32_t(btin.size() / 2));
            for (uint32_t i = 0; i < rows; i++) { btin.push_back(slot); btin.push_back(i); }
            bl.push_back(BlockDrafter::Block{slot, rows, lens[slot], embed + size_t(tok) * md.d});
        }
        if (bl.empty()) { b.hfin.clear(); b.logits.clear(); return; }
        b.blocks(bl);
        const uint32_t R = uint32_t(btin.size() / 2), ncand = std::min(BlockDrafter::CANDS, rows - 1);
        b.cand.assign(size_t(R) * CANDS, 0);
        b.cand_q.assign(size_t(R) * CANDS, 0.0f);
        for (uint32_t r = 0; r < R; r++)
            if (btin[2 * r + 1]) draft_top_row(b.logits.data() + size_t(r) * b.v, b.v, b.vocab.data(), 1.0f / 0.6f, ncand, b.cand.data() + r * CANDS, b.cand_q.data() + r * CANDS);
        for (size_t i = 0; i < bl.size(); i++) draft_tree_block(first[i], rows, bl[i].slot, b.cand.data(), b.cand_q.data(), ncand, feed.data(), tree.data());
    }

    void draft(const Plan& p, uint32_t rows) {
        if (block_drafter) { block_draft(p, rows); return; }
        if (!drafter) throw std::runtime_error("no drafter loaded");
        if (rows < 1 || rows > VERIFY_T) throw std::runtime_error("the chain drafter proposes for 1.." + std::to_string(VERIFY_T) + " rows");
        Drafter& dr = *drafter;
        const uint32_t d = md.d, n = p.n, nr = p.n_runs, v = dr.head.m;
        auto feature_in = [&](float* x, const float* feat, uint32_t tok) {
            for (uint32_t i = 0; i < d; i++) x[i] = feat ? feat[i] : 0.0f;
            for (uint32_t i = 0; i < d; i++) x[d + i] = bf16_to_f32(embed[size_t(tok) * d + i]);
        };
        // (1) catch-up on the step's layout (meta, tin, vis and tiles are still the step's).
        {
            std::vector<float> x(size_t(n) * 2 * d), h(size_t(n) * d);
            for (uint32_t t = 0; t < n; t++) {
                const uint32_t slot = tin[2 * t], row = tin[2 * t + 1], pos = meta[2 * t + 1];
                const float* feat = row ? taps.data() + size_t(t - 1) * d : pos ? dr.carry.data() + size_t(slot) * d : nullptr;
                feature_in(x.data() + size_t(t) * 2 * d, feat, tokens[t]);
            }
            matmul_raw(dr.fc, x.data(), n, h.data());
            write_mask.assign(on_path.begin(), on_path.end());
            layer_forward(dr.layer, 0, dr.k_cache.data(), dr.v_cache.data(), h.data(), n, p.n_tiles);
            write_mask.clear();
        }
        // The runs that draft: those that emitted this step. Every run with rows on the path carries its last tap over.
        std::vector<uint32_t> last(nr, NO_TOK);
        for (uint32_t r = 0; r < nr; r++) {
            const RunIn& ru = runs[r];
            if (ru.verify) { if (path_len[r]) last[r] = ru.first + path[r * FEED_W + path_len[r] - 1]; }
            else if (on_path[ru.first]) last[r] = ru.first + ru.count - 1;
        }
        // (2) draft passes on a layout of their own: one row per run.
        const std::vector<uint32_t> s_meta = meta, s_tin = tin, s_vis = vis, s_tiles = tiles;
        draft_logits.assign(size_t(rows - 1) * nr * v, 0.0f);
        std::vector<float> feat(size_t(nr) * d, 0.0f), x(size_t(nr) * 2 * d), h(size_t(nr) * d), inv(nr), lg(size_t(nr) * v);
        std::vector<uint8_t> live(nr, 0);
        for (uint32_t i = 1; i < rows; i++) {
            meta.assign(2 * nr, 0); tin.assign(2 * nr, 0); vis.assign(nr, 1); tiles.clear(); write_mask.assign(nr, 0);
            for (uint32_t r = 0; r < nr; r++) {
                const uint32_t slot = runs[r].slot, pos = lens[slot] + i - 1;
                live[r] = last[r] != NO_TOK && emitted[r] > 0 && pos < cfg.max_seq_len;
                meta[2 * r] = slot; meta[2 * r + 1] = live[r] ? pos : 0;
                tin[2 * r] = slot;
                tiles.push_back(r); tiles.push_back(1);
                write_mask[r] = live[r];
                const float* f = i == 1 ? (last[r] != NO_TOK ? taps.data() + size_t(last[r]) * d : nullptr) : feat.data() + size_t(r) * d;
                feature_in(x.data() + size_t(r) * 2 * d, f, live[r] ? feed[slot * FEED_W + i - 1] : 0);
            }
            matmul_raw(dr.fc, x.data(), nr, h.data());
            attn_window = dr.window;
            layer_forward(dr.layer, 0, dr.k_cache.data(), dr.v_cache.data(), h.data(), nr, nr);
            attn_window = 0;
            inv_rms(h.data(), nr, d, md.eps, inv.data());
            matmul_raw(dr.head, h.data(), nr, lg.data());
            for (uint32_t r = 0; r < nr; r++) {
                float* row = lg.data() + size_t(r) * v;
                for (uint32_t j = 0; j < v; j++) row[j] *= inv[r];  // EPI_HEAD
                for (uint32_t j = 0; j < d; j++) feat[size_t(r) * d + j] = round_bf16(h[size_t(r) * d + j] * inv[r]);
                if (!live[r]) continue;
                uint32_t best = 0;
                for (uint32_t j = 1; j < v; j++)
                    if (row[j] > row[best]) best = j;
                const uint32_t slot = runs[r].slot;
                // Under the rejection rule a sampling sequence's draft is drawn from softmax(q / T) and its row is kept
                // for the next step's test; otherwise the argmax, and nothing kept.
                const SampleRow& sr = sample_rows[runs[r].head0];
                if (accept_rule == 1 && sr.temperature > 0.0f && sr.top_p >= 1.0f) {
                    best = draw_draft_index(row, v, sr.temperature, sr.seed_lo, sr.seed_hi, lens[slot] + i);
                    std::copy_n(row, v, dr.q_keep.data() + (size_t(slot) * (VERIFY_T - 1) + i - 1) * v);
                    dr.q_rows[slot] = i;
                } else if (i == 1) {
                    dr.q_rows[slot] = 0;
                }
                feed[slot * FEED_W + i] = dr.vocab[best];
                tree[slot * FEED_W + i] = chain_node(i);
                std::copy_n(row, v, draft_logits.data() + (size_t(i - 1) * nr + r) * v);
            }
        }
        write_mask.clear();
        meta = s_meta; tin = s_tin; vis = s_vis; tiles = s_tiles;
        for (uint32_t r = 0; r < nr; r++)
            if (last[r] != NO_TOK) std::copy_n(taps.data() + size_t(last[r]) * d, d, dr.carry.data() + size_t(runs[r].slot) * d);
    }

    // encode.rs:439-451 `encode_replay`.
    void run_replay(const Plan& p) {
        for (uint32_t r = 0; r < p.n_runs; r++)
            replay_draft_run(r, runs.data(), lens.data(), feed.data(), trace.data(), trace_len.data(), replay, tree.data());
    }
};

}  // namespace orc

#include "limite_forward.hpp"
