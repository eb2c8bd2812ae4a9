#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace vlt {

// engine/src/engine.rs:110-117 `Sampling::check`.
void Sampling::check() const {
    const bool t_ok = temperature == 0.0f || (std::isnormal(temperature) && temperature > 0.0f);
    if (!(t_ok && top_p > 0.0f && top_p <= 1.0f))
        throw Error("sampling {temperature " + std::to_string(temperature) + ", top_p " + std::to_string(top_p) +
                    "}: needs a temperature of 0 or a normal positive one, and 0 < top_p <= 1");
}

// ------------------------------------------------------------------ KV cache
void KvCache::init(const EngineConfig& cfg, const ModelDesc& md, uint32_t n_layers, bool with_pool) {
    page = md.page;
    n_pages = (cfg.global_kv_tokens + page - 1) / page;
    max_pages = (cfg.max_seq_len + page - 1) / page;
    const size_t bytes = size_t(n_layers) * n_pages * page * md.n_kv * md.hd * 2;
    if (with_pool) {
        k.alloc(bytes, false);
        v.alloc(bytes, false);
    }
    page_table.alloc(size_t(cfg.max_seqs) * max_pages * 4, !with_pool);
    free_pages.clear();
    for (uint32_t i = n_pages; i-- > 0;) free_pages.push_back(i);  // kv.rs:43: a stack that pops 0, 1, 2, ...
}

// engine/src/engine/kv.rs:51-58.
void KvCache::reserve(uint32_t slot, std::vector<uint32_t>& pages, uint32_t len) {
    const size_t had = pages.size();
    while (size_t(pages.size()) * page < len) {
        if (free_pages.empty()) {
            // Nothing was written yet: give back what this call took, so that a failed reserve changes nothing.
            while (pages.size() > had) { free_pages.push_back(pages.back()); pages.pop_back(); }
            throw Error("global KV pool exhausted");
        }
        pages.push_back(free_pages.back());
        free_pages.pop_back();
    }
    // A sequence's table entries are consecutive: the new ones go up in one copy, ordered on the engine's stream
    // before the kernels of the step that reads them.
    if (pages.size() > had) page_table.write((size_t(slot) * max_pages + had) * 4, pages.data() + had, (pages.size() - had) * 4);
}

// engine/src/engine/kv.rs:60-62.
void KvCache::release(const std::vector<uint32_t>& pages) {
    for (size_t i = pages.size(); i-- > 0;) free_pages.push_back(pages[i]);
}

// ------------------------------------------------------------------ step sets
void StepSet::init(const EngineConfig& cfg) {
    host_only = cfg.host_only;
    const size_t n = cfg.max_step_tokens, hr = cfg.max_head_rows, ms = cfg.max_seqs;
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t o = at; at += (bytes + 255) / 256 * 256; return o; };
    o_tokens = take(n * 4);
    o_tin = take(2 * n * 4);
    o_vis = take(n * 4);
    o_head_rows = take(hr * 4);
    o_hidden_rows = take(n * 4);
    o_sample_rows = take(hr * sizeof(SampleRow));
    o_tiles = take(2 * (n / 8 + ms + 1) * 4);
    o_runs = take(ms * sizeof(RunIn));
    o_ctiles = take(2 * (n / 64 + ms + 1) * 4);
    in_bytes = at;
    at = 0;
    o_out_ids = take(hr * 4);
    o_emitted = take(ms * 4);
    o_err = take(4);
    out_bytes = at;
    dev_in.alloc(in_bytes, host_only);
    dev_out.alloc(out_bytes, host_only);
    if (host_only) {
        host_in = static_cast<uint8_t*>(dev_in.dev);
        host_out = static_cast<uint8_t*>(dev_out.dev);
    } else {
        VLT_CUDA(cudaMallocHost(reinterpret_cast<void**>(&host_in), in_bytes));
        VLT_CUDA(cudaMallocHost(reinterpret_cast<void**>(&host_out), out_bytes));
        std::memset(host_in, 0, in_bytes);
        std::memset(host_out, 0, out_bytes);
        VLT_CUDA(cudaEventCreate(&start));
        VLT_CUDA(cudaEventCreate(&done));
        VLT_CUDA(cudaEventCreateWithFlags(&uploaded, cudaEventDisableTiming));
        VLT_CUDA(cudaEventCreateWithFlags(&computed, cudaEventDisableTiming));
    }
}

void StepSet::release() {
    if (!host_only) {
        if (host_in) cudaFreeHost(host_in);
        if (host_out) cudaFreeHost(host_out);
        if (start) cudaEventDestroy(start);
        if (done) cudaEventDestroy(done);
        if (uploaded) cudaEventDestroy(uploaded);
        if (computed) cudaEventDestroy(computed);
    }
    host_in = host_out = nullptr;
}

// --------------------------------------------------------------------- engine
Engine::Engine(const std::string& weights, const EngineConfig& c, const Tuning& t) : cfg(c), tuning(t) {
    if (!cfg.host_only) {
        int count = 0;
        const cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0)
            throw Error(std::string("no usable CUDA device (") + cudaGetErrorString(e) + "): this engine has no CPU path");
        if (cfg.device < 0 || cfg.device >= count) throw Error("device_ordinal " + std::to_string(cfg.device) + " of " + std::to_string(count) + " devices");
        VLT_CUDA(cudaSetDevice(cfg.device));
        cudaDeviceProp prop;
        VLT_CUDA(cudaGetDeviceProperties(&prop, cfg.device));
        if (prop.major < 10) throw Error(std::string(prop.name) + ": compute capability " + std::to_string(prop.major) + "." + std::to_string(prop.minor) + " (the kernels are built for sm_100a)");
        sm_count = tuning.sm_count ? tuning.sm_count : uint32_t(prop.multiProcessorCount);
        VLT_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        VLT_CUDA(cudaStreamCreateWithFlags(&copy_in, cudaStreamNonBlocking));
        VLT_CUDA(cudaStreamCreateWithFlags(&copy_out, cudaStreamNonBlocking));
    } else if (tuning.sm_count) {
        sm_count = tuning.sm_count;
    }
    if (cfg.max_seqs == 0 || cfg.max_step_tokens == 0 || cfg.max_chunk == 0 || cfg.max_head_rows == 0) throw Error("engine config: zero capacity");
    model.load(weights, cfg.host_only);
    const ModelDesc& md = model.md;
    kv.init(cfg, md, model.limite ? model.n_global : md.n_layers, !cfg.host_only);  // (the reference's architecture pages its global layers only)
    seqs.resize(cfg.max_seqs);
    for (auto& st : sets) st.init(cfg);

    const bool ho = cfg.host_only;
    const size_t n = cfg.max_step_tokens, hr = cfg.max_head_rows, ms = cfg.max_seqs;
    auto f = [&](Buffer& b, size_t floats) { b.alloc(floats * 4, ho); };
    if (!ho) {
        f(s.h, n * md.d);
        f(s.qkv, n * md.qkv_w());
        f(s.attn, n * md.n_heads * md.hd);
        f(s.act, n * md.ffn);
        f(s.part, n * 16 * md.n_heads * ATTN_PART);  // buffers.rs:9: 16 partial slots per token of a full step
        f(s.hfin_head, hr * md.d);
        f(s.hfin_all, n * md.d);
        f(s.logits, hr * md.vocab);
        f(s.inv, n);
        const size_t n16 = (n + 15) / 16 * 16, hr16 = (hr + 15) / 16 * 16;
        s.h_b.alloc(n16 * md.d * 2, false);
        s.attn_b.alloc(n16 * md.n_heads * md.hd * 2, false);
        s.q_b.alloc(n16 * md.n_heads * md.hd * 2, false);
        s.ssq.alloc(size_t(md.d / 128 + 1) * n16 * 4, false);
        s.act_b.alloc(n16 * md.ffn * 2, false);
        s.hfin_b.alloc(hr16 * md.d * 2, false);
        f(s.inv_head, hr);
    }
    f(s.meta, 2 * n);
    f(s.lens, ms);
    f(s.feed, ms * FEED_W);
    f(s.tree, ms * FEED_W);
    s.gen.alloc(ms * sizeof(GenState), ho);
    f(s.path, ms * FEED_W);
    f(s.path_len, ms);
    f(s.on_path, n);
    f(s.trace, ho ? 1 : ms * size_t(cfg.max_seq_len));
    f(s.trace_len, ms);
    f(s.err_flag, 1);
    // Per-slot state and the page table are written while steps are queued (admission, page reservation): those
    // copies go on the engine's stream, ordered between the steps' kernels.
    for (Buffer* b : {&s.lens, &s.feed, &s.tree, &s.gen, &s.path, &s.path_len, &s.on_path, &s.trace, &s.trace_len, &s.err_flag, &s.meta, &kv.page_table}) b->order = stream;
    std::vector<uint32_t> chains(ms * FEED_W);
    for (size_t i = 0; i < chains.size(); i++) chains[i] = chain_node(uint32_t(i % FEED_W));  // buffers.rs:112-113
    s.tree.write_vec(0, chains);
    std::vector<GenState> open(ms, gen_open());
    s.gen.write_vec(0, open);

    if (!ho) {
        // engine.rs:392-421 `rope_table`: theta = float32(pos) * frequency, cos and sin rounded to bf16.
        const uint32_t npos = cfg.max_seq_len + FEED_W, half = uint32_t(model.rope_freq.size());  // hd / 2; 32 pairs for a head of 128 of the reference's architecture
        std::vector<float> tab(size_t(npos) * half * 2);
        auto rb = [](float x) { uint32_t u; std::memcpy(&u, &x, 4); u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u; std::memcpy(&x, &u, 4); return x; };
        for (uint32_t p = 0; p < npos; p++)
            for (uint32_t i = 0; i < half; i++) {
                const float theta = float(p) * model.rope_freq[i];
                tab[(size_t(p) * half + i) * 2] = rb(std::cos(theta));
                tab[(size_t(p) * half + i) * 2 + 1] = rb(std::sin(theta));
            }
        rope_tab.alloc(tab.size() * 4, false);
        rope_tab.write_vec(0, tab);
        if (!model.limite) attn_maps_init(&attn_maps, kv.k.as<uint16_t>(), kv.v.as<uint16_t>(), uint64_t(md.n_layers) * kv.n_pages * md.n_kv * md.page);
        if (model.limite) {
            lim = std::make_unique<LimiteState>();
            lim->ring = LIMITE_WINDOW + cfg.max_chunk;  // kv.rs:26-28: the window plus a whole chunk
            const size_t n = cfg.max_step_tokens, ring_bytes = size_t(model.n_local) * cfg.max_seqs * md.n_kv * lim->ring * 128 * 2;
            lim->k_local.alloc(ring_bytes, false);
            lim->v_local.alloc(ring_bytes, false);
            for (Buffer* b : {&lim->hist0, &lim->hist12, &lim->hist23, &lim->xattn, &lim->base, &lim->mixed}) b->alloc(n * md.d * 4, false);
            lim->vdir.alloc(n * md.n_kv * 128 * 4, false);
            lim->gates.alloc(n * md.n_heads * 4, false);
            lim->part.alloc(n * md.n_heads * size_t(LIMITE_MAX_SPLITS) * LIMITE_PART * 4, false);
        }
        VLT_CUDA(cudaDeviceSynchronize());
    }
}

Engine::~Engine() {
    if (stream) {
        cudaStreamSynchronize(stream);
        cudaStreamSynchronize(copy_out);
        cudaStreamDestroy(stream);
        cudaStreamDestroy(copy_in);
        cudaStreamDestroy(copy_out);
    }
    for (auto& st : sets) st.release();
}

void Engine::make_current() const {
    if (!cfg.host_only) VLT_CUDA(cudaSetDevice(cfg.device));
}

std::string Engine::device_name() const {
    if (cfg.host_only) return "host (planning only)";
    cudaDeviceProp prop;
    VLT_CUDA(cudaGetDeviceProperties(&prop, cfg.device));
    return prop.name;
}

// engine/src/engine.rs:259-267.
uint32_t Engine::new_seq() {
    for (uint32_t slot = 0; slot < seqs.size(); slot++)
        if (!seqs[slot]) {
            seqs[slot] = Seq{};
            const uint32_t zero = 0;
            s.lens.write(slot * 4, &zero, 4);
            s.trace_len.write(slot * 4, &zero, 4);
            if (drafter && !cfg.host_only) drafter->q_rows.write(slot * 4, &zero, 4);
            set_gen(slot, gen_open());
            return slot;
        }
    throw Error("no free sequence slot");
}

void Engine::set_gen(uint32_t slot, const GenState& g) { s.gen.write(slot * sizeof(GenState), &g, sizeof g); }

void Engine::set_trace(uint32_t slot, const uint32_t* trace, uint32_t n) {
    if (n > cfg.max_seq_len) throw Error("replay trace longer than max_seq_len");
    if (!cfg.host_only) s.trace.write(size_t(slot) * cfg.max_seq_len * 4, trace, size_t(n) * 4);
    s.trace_len.write(slot * 4, &n, 4);
}

// engine/src/engine.rs:281-285.
void Engine::settle(uint32_t id, uint32_t unused) {
    if (id < seqs.size() && seqs[id]) seqs[id]->len -= unused;
}

void Engine::set_sampling(uint32_t id, const Sampling& sm) {
    sm.check();
    if (id >= seqs.size() || !seqs[id]) throw Error("unknown sequence");
    seqs[id]->sampling = sm;
}

// engine/src/engine.rs:298-303.
void Engine::free_seq(uint32_t id) {
    if (id < seqs.size() && seqs[id]) {
        kv.release(seqs[id]->pages);
        seqs[id].reset();
    }
}

uint32_t Engine::seq_len(uint32_t id) const { return id < seqs.size() && seqs[id] ? seqs[id]->len : 0; }

void Engine::set_taps(const std::vector<uint32_t>& layers) {
    std::vector<uint32_t> want = layers;
    const uint32_t last = model.md.n_layers - 1;
    // The chain drafter's features are the last layer's tap: it stays tapped while a drafter is loaded.
    if (drafter && std::find(want.begin(), want.end(), last) == want.end()) want.push_back(last);
    for (size_t i = 0; i < want.size(); i++) {
        if (want[i] >= model.md.n_layers) throw Error("taps: layer " + std::to_string(want[i]) + " of " + std::to_string(model.md.n_layers));
        if (std::find(want.begin(), want.begin() + i, want[i]) != want.begin() + i) throw Error("taps: layer " + std::to_string(want[i]) + " named twice");
    }
    if (!cfg.host_only) VLT_CUDA(cudaStreamSynchronize(stream));  // no queued step writes the buffers that go away
    std::vector<Buffer> bufs(want.size());
    for (size_t i = 0; i < want.size(); i++) {
        auto old = std::find(tap_layers.begin(), tap_layers.end(), want[i]);
        if (old != tap_layers.end()) bufs[i] = std::move(tap_bufs[old - tap_layers.begin()]);
        else bufs[i].alloc(size_t(cfg.max_step_tokens) * model.md.d * 4, cfg.host_only);
    }
    tap_layers = std::move(want);
    tap_bufs = std::move(bufs);
}

float* Engine::last_tap() const {
    auto it = std::find(tap_layers.begin(), tap_layers.end(), model.md.n_layers - 1);
    if (it == tap_layers.end()) throw Error("internal: the last layer is not tapped");
    return tap_bufs[it - tap_layers.begin()].as<float>();
}

void Engine::set_acceptance(uint32_t rule) {
    if (rule > 1) throw Error("acceptance rule " + std::to_string(rule) + ": 0 (sample, then match) or 1 (rejection sampling)");
    accept_rule = rule;
}

KvArgs Engine::kv_args() const {
    uint32_t shift = 0;
    while ((1u << shift) < model.md.page) shift++;
    return KvArgs{kv.n_pages, kv.max_pages, model.md.n_kv, shift, model.md.hd};
}

// How the cached keys are split across attention blocks (the reference's decode_splits,
// engine/src/engine/plan.rs:153-163, re-derived for this GPU): blocks of 4 warps, four per SM.
// A block costs its warps' pages plus a fixed part (loading q, merging and writing the partial)
// worth about six pages; the split count with the lowest waves x block cost wins.
void Engine::attention_split(Plan& p, uint32_t max_keys, uint32_t n_tiles) const {
    const uint32_t page = model.md.page, unit = 4 * page;  // a block's four warps take a page each
    const uint32_t cap = std::min<uint32_t>(std::max<uint32_t>(cfg.max_step_tokens * 16 / std::max(p.n, 1u), 1u), 64u);  // plan.rs:127
    const uint32_t slots = 4 * sm_count, base = std::max(n_tiles * model.md.n_kv, 1u);
    uint32_t best = 1;
    if (tuning.attn_keys_per_cta) {
        best = std::max(1u, (max_keys + tuning.attn_keys_per_cta - 1) / tuning.attn_keys_per_cta);
    } else {
        const double fixed = 6.0, pages = double(max_keys + page - 1) / page;
        double best_cost = 1e30;
        for (uint32_t sp = 1; sp <= cap; sp++) {
            if (sp > 1 && max_keys / sp < 8 * page) break;
            const double waves = std::ceil(double(base) * sp / slots);
            const double cost = waves * (std::ceil(pages / (4.0 * sp)) + fixed);
            if (cost < best_cost) { best_cost = cost; best = sp; }
        }
    }
    best = std::min(best, cap);
    uint32_t kps = ((max_keys + best - 1) / best + unit - 1) / unit * unit;
    kps = std::max(kps, unit);
    p.keys_per_split = kps;
    p.max_splits = std::max(1u, (max_keys + kps - 1) / kps);
}

// engine/src/engine/plan.rs:47-150 `plan`.
Plan Engine::plan(uint32_t set, const std::vector<PlanRun>& runs, Rows hidden) {
    uint32_t n = 0;
    for (const PlanRun& r : runs) n += r.count;
    if (n == 0 || n > cfg.max_step_tokens) throw Error("step has " + std::to_string(n) + " tokens (max " + std::to_string(cfg.max_step_tokens) + ")");
    std::vector<uint32_t> tokens, tin, vis, head_rows, hidden_rows, tiles, ctiles;
    std::vector<SampleRow> samples;
    std::vector<RunIn> run_in;
    uint32_t max_keys = 0, max_count = 0;
    Plan p;
    for (size_t ri = 0; ri < runs.size(); ri++) {
        const PlanRun& run = runs[ri];
        const uint32_t id = run.seq, count = run.count;
        if (count == 0 || count > cfg.max_chunk) throw Error(std::to_string(count) + " tokens for one sequence in a step (max_chunk " + std::to_string(cfg.max_chunk) + ")");
        // A verify run is one attention tile and one slot's feed/tree rows (engine/src/engine/kernels.rs:28-29, generate.rs:216-220).
        if (run.verify && count > VERIFY_T) throw Error("a verify run takes at most " + std::to_string(VERIFY_T) + " rows, not " + std::to_string(count));
        for (uint32_t i = 0; i < count; i++) {
            const uint32_t tk = run.tokens[i];
            if (tk >= FEED_ROW && tk - FEED_ROW >= FEED_W) throw Error("only " + std::to_string(FEED_W) + " GPU-fed tokens per slot");
            if (tk < FEED_ROW && tk >= model.md.vocab) throw Error("token id out of range");
        }
        for (size_t j = 0; j < ri; j++)
            if (runs[j].seq == id) throw Error("a sequence appears twice in one step");
        if (id >= seqs.size() || !seqs[id]) throw Error("unknown sequence");
        Seq& sq = *seqs[id];
        const uint32_t new_len = sq.len + count;
        if (new_len > cfg.max_seq_len) throw Error("sequence would reach " + std::to_string(new_len) + " tokens (max " + std::to_string(cfg.max_seq_len) + ")");
        // With a drafter loaded the draft passes write their own K/V up to VERIFY_T positions past the step.
        kv.reserve(id, sq.pages, drafter ? std::min(new_len + VERIFY_T, cfg.max_seq_len) : new_len);
        const uint32_t first_row = uint32_t(tokens.size());
        tokens.insert(tokens.end(), run.tokens, run.tokens + count);
        for (uint32_t row = 0; row < count; row++) {
            tin.push_back(id);
            tin.push_back(row);
            vis.push_back(0xffffffffu >> (31 - row % 8));  // causal within its tile of 8; `embed` overwrites a draft tree's
        }
        auto rows = [&](Rows r, std::vector<uint32_t>& v) {
            if (r == Rows::Last) v.push_back(first_row + count - 1);
            if (r == Rows::All) for (uint32_t x = first_row; x < first_row + count; x++) v.push_back(x);
        };
        const uint32_t first_head = uint32_t(head_rows.size());
        rows(run.verify ? Rows::All : run.head, head_rows);
        rows(hidden, hidden_rows);
        for (uint32_t h = first_head; h < head_rows.size(); h++) samples.push_back(sq.sampling.row_of(head_rows[h]));
        run_in.push_back(RunIn{id, first_row, count, first_head, uint32_t(head_rows.size()) - first_head, run.verify ? 1u : 0u});
        for (uint32_t i = 0; i < count; i += 8) {
            tiles.push_back(first_row + i);
            tiles.push_back(std::min(count - i, 8u));
        }
        for (uint32_t i = 0; i < count; i += 64) {
            ctiles.push_back(first_row + i);
            ctiles.push_back(std::min(count - i, 64u));
        }
        max_keys = std::max(max_keys, new_len);
        max_count = std::max(max_count, count);
        p.branches = p.branches || (run.verify && count > 2);
        sq.len = new_len;
    }
    if (head_rows.size() > cfg.max_head_rows) throw Error(std::to_string(head_rows.size()) + " head rows (max " + std::to_string(cfg.max_head_rows) + ")");
    StepSet& st = sets[set];
    auto put = [&](size_t off, const void* src, size_t bytes) { if (bytes) std::memcpy(st.host_in + off, src, bytes); };
    put(st.o_tokens, tokens.data(), tokens.size() * 4);
    put(st.o_tin, tin.data(), tin.size() * 4);
    put(st.o_vis, vis.data(), vis.size() * 4);
    put(st.o_head_rows, head_rows.data(), head_rows.size() * 4);
    put(st.o_hidden_rows, hidden_rows.data(), hidden_rows.size() * 4);
    put(st.o_sample_rows, samples.data(), samples.size() * sizeof(SampleRow));
    put(st.o_tiles, tiles.data(), tiles.size() * 4);
    put(st.o_runs, run_in.data(), run_in.size() * sizeof(RunIn));
    put(st.o_ctiles, ctiles.data(), ctiles.size() * 4);
    p.ctiles = uint32_t(ctiles.size() / 2);
    p.n = n;
    p.n_head = uint32_t(head_rows.size());
    p.head_all = p.n_head == n;  // (rows are listed in step order, each once)
    p.n_hidden = uint32_t(hidden_rows.size());
    p.n_runs = uint32_t(runs.size());
    p.tiles = uint32_t(tiles.size() / 2);
    p.max_run = max_count;
    p.chunked = max_count > VERIFY_T;
    p.max_keys = max_keys;
    attention_split(p, max_keys, p.tiles);
    last_plan_n = n;
    last_split[0] = p.keys_per_split;
    last_split[1] = p.max_splits;
    return p;
}

// Y = epilogue(W . X) for n tokens: steps of at most 8 tokens stream the weights through the
// tensor cores from registers; larger ones go in token blocks of 8 (the weights of one matrix
// stay in L2 between blocks).
void Engine::matmul(const Matrix& w, uint32_t n, const float* x, float* y, uint32_t epi, const float* base, float* inv_out, uint32_t vocab_real,
                    const QkvEpilogue* q, const uint16_t* xb, uint16_t* yb, float scale, float ra, float rb) {
    MatArgs a{};
    a.scale = scale;
    a.ra = ra;
    a.rb = rb;
    if (q) a.q = *q;
    a.err_flag = s.err_flag.as<uint32_t>();
    a.W = w.w;
    a.scales = w.scales;
    a.k = w.k;
    a.m = w.m;
    a.group = w.group;
    a.int8 = w.int8;
    a.epi = epi;
    a.vocab_real = vocab_real ? vocab_real : model.md.vocab_real;
    a.eps = model.md.eps;
    const uint32_t out_w = epi == EPI_SWIGLU ? w.m / 2 : w.m;
    for (uint32_t t0 = 0; t0 < n; t0 += 8) {
        a.n = std::min(8u, n - t0);
        a.t0 = t0;
        a.X = x + size_t(t0) * w.k;
        a.Xb = xb ? xb + size_t(t0) * w.k : nullptr;
        a.Y = y ? y + size_t(t0) * out_w : nullptr;
        a.Yb = yb ? yb + size_t(t0) * out_w : nullptr;
        a.base = base ? base + size_t(t0) * out_w : nullptr;
        a.inv_out = inv_out ? inv_out + t0 : nullptr;
        launch_matmul_stream(a, sm_count, stream);
    }
}

// Whether the streamed kernel itself (not its scalar stand-in) takes this matrix.
bool Engine::stream_fits(const Matrix& w) const {
    MatArgs a{};
    a.n = 1;
    a.k = w.k;
    a.m = w.m;
    a.group = w.group;
    a.int8 = w.int8;
    return matmul_stream_fits(a);
}

// The matmul variant by step size (the reference's Matmul::for_tokens, encode.rs:33-44): the
// tcgen05 GEMM from gemm_min_rows tokens (default 9), the streamed kernel below.
bool Engine::use_gemm(const Matrix& w, uint32_t n) const {
    const uint32_t min_rows = tuning.gemm_min_rows ? tuning.gemm_min_rows : 9;  // up to 8 tokens the streamed kernel; 9..15 would take it twice over the weights
    const bool grouped = w.int8 && w.group < w.k;
    return !model.limite && n >= min_rows && w.m % 128 == 0 && w.k % 64 == 0 && !grouped;  // (the reference's architecture decides for itself: gemm_fits)
}

// Whether the tensor-core GEMM takes this matrix at n tokens (the plain decoder's rule, for the reference's architecture).
bool Engine::gemm_fits(const Matrix& w, uint32_t n) const {
    const uint32_t min_rows = tuning.gemm_min_rows ? tuning.gemm_min_rows : 9;
    const bool grouped = w.int8 && w.group < w.k;
    return n >= min_rows && w.m % 128 == 0 && w.k % 64 == 0 && (!grouped || (w.group >= 8 && !(w.group & (w.group - 1))));  // (scale groups: powers of two from 8, as the reference's own int8 files have)
}

bool Engine::layer_carries(const Layer& l, uint32_t n) const {
    return use_gemm(l.qkv, n) && use_gemm(l.o, n) && use_gemm(l.gate_up, n) && use_gemm(l.down, n) && model.md.d % 128 == 0;
}

void Engine::matmul_gemm(const Matrix& w, uint32_t n, const uint16_t* xb, float* y, uint16_t* yb, uint32_t epi, const float* base, const float* inv,
                         uint32_t vocab_real, const QkvEpilogue* q, float* ssq_out, const float* ssq_in, float scale, float ra, float rb) {
    MatArgs a{};
    a.scale = scale;
    a.ra = ra;
    a.rb = rb;
    a.W = w.w;
    a.scales = w.scales;
    a.Xb = xb;
    a.Y = y;
    a.Yb = yb;
    a.base = base;
    a.inv_in = inv;
    a.n = n;
    a.k = w.k;
    a.m = w.m;
    a.group = w.group;
    a.int8 = w.int8;
    a.epi = epi;
    a.vocab_real = vocab_real ? vocab_real : model.md.vocab_real;
    a.eps = model.md.eps;
    if (q) a.q = *q;
    a.ssq_out = ssq_out;
    a.ssq_in = ssq_in;
    a.ssq_tiles = ssq_in ? w.k / 128 : 0;
    a.ssq_stride = (cfg.max_step_tokens + 15) / 16 * 16;
    // The kernel's N is at most 256 tokens: a longer step (a prompt chunk) goes in blocks of 256, the weights read once per
    // block (the reference's tiled GEMM loops its token tiles the same way, kernels.metal:319-514). Everything indexed by
    // token moves along with the block.
    const uint32_t out_w = epi == EPI_SWIGLU ? w.m / 2 : w.m;
    for (uint32_t t0 = 0; t0 < n; t0 += 256) {
        MatArgs b = a;
        b.n = std::min(256u, n - t0);
        b.Xb = xb + size_t(t0) * w.k;
        b.Y = y ? y + size_t(t0) * out_w : nullptr;
        b.Yb = yb ? yb + size_t(t0) * out_w : nullptr;
        b.base = base ? base + size_t(t0) * out_w : nullptr;
        b.inv_in = inv ? inv + t0 : nullptr;
        b.ssq_out = ssq_out ? ssq_out + t0 : nullptr;
        b.ssq_in = ssq_in ? ssq_in + t0 : nullptr;
        if (q) {
            b.q.meta = q->meta + 2 * size_t(t0);
            b.q.tin = q->tin + 2 * size_t(t0);
            b.q.cpos = q->cpos ? q->cpos + t0 : nullptr;
            b.q.q_b = q->q_b + size_t(t0) * q->n_heads * model.md.hd;
        }
        if (!gemm_supported(b)) throw Error("internal: GEMM asked for an unsupported shape");
        launch_gemm(b, sm_count, s.err_flag.as<uint32_t>(), stream, !tuning.gemm_unpaired);
    }
}

// engine/src/engine/encode.rs:142-192 `encode_layer`, a plain decoder's.
void Engine::encode_layer(uint32_t set, const Plan& p, uint32_t li, bool capture) {
    StepSet& st = sets[set];
    LayerIO io{};
    io.l = &model.layers[li];
    io.h_ready = li > 0;  // the layer before ended with the down GEMM (if the step is wide enough for the GEMM at all)
    io.n = p.n;
    io.meta = s.meta.as<uint32_t>();
    io.tin = st.in<uint32_t>(st.o_tin);
    io.tiles = st.in<uint32_t>(st.o_tiles);
    io.vis = st.in<uint32_t>(st.o_vis);
    io.n_tiles = p.tiles;
    io.ctiles = st.in<uint32_t>(st.o_ctiles);
    io.n_ctiles = p.chunked ? p.ctiles : 0;
    io.k_cache = kv.k.as<uint16_t>();
    io.v_cache = kv.v.as<uint16_t>();
    io.maps = &attn_maps;
    io.layer = li;
    io.keys_per_split = p.keys_per_split;
    io.max_splits = p.max_splits;
    io.max_rows = std::min(p.max_run, VERIFY_T);
    encode_layer_io(io, capture);
    // kernels.metal:133-148 `tap_rows`: bf16(rms_norm(the layer's output)), kept as fp32.
    auto tap = std::find(tap_layers.begin(), tap_layers.end(), li);
    if (tap != tap_layers.end())
        launch_prep_rows(s.h.as<float>(), nullptr, p.n, model.md.d, model.md.eps, tap_bufs[tap - tap_layers.begin()].as<float>(), nullptr, nullptr, true, true, stream);
}

// The layer on any step layout, weights and cache: the target's layers and the drafter's one.
// With `capture`, the layer also leaves the intermediates step_capture hands out: the normed inputs by row passes, q | k | v
// by a second qkv projection with the plain norm epilogue and a RoPE pass, the o and down projections' own outputs by
// second launches with the raw epilogue (the same kernels on the same inputs: the same sums), all beside the normal work.
void Engine::encode_layer_io(const LayerIO& io, bool capture) {
    const Layer& l = *io.l;
    const ModelDesc& md = model.md;
    const uint32_t n = io.n, li = io.layer;
    float* h = s.h.as<float>();
    // Steps of 16 tokens or more multiply on tcgen05: activations go in as bf16 copies and 1/rms
    // comes from a row pass, since the GEMM does not see whole rows of X.
    const bool big = use_gemm(l.qkv, n) && use_gemm(l.o, n) && use_gemm(l.gate_up, n) && use_gemm(l.down, n);
    const KvArgs kva = kv_args();
    const float scale_log2 = md.attn_scale * 1.44269504088896340736f;
    // The qkv projection's epilogue does what qkv_post does (RoPE, q for the attention, K/V into the cache), in the
    // tensor-core GEMM and in the streamed matmul alike; the scalar attention reads fp32 q, and odd shapes go through
    // the scalar matmul: those keep the separate kernel.
    const bool fused_post = !tuning.plain_attention && (big || stream_fits(l.qkv));
    QkvEpilogue q{};
    q.meta = io.meta;
    q.tin = io.tin;
    q.cpos = io.cpos;
    q.rope = rope_tab.as<float>();
    q.page_table = kv.page_table.as<uint32_t>();
    q.kv = kva;
    q.layer = li;
    q.n_heads = md.n_heads;
    q.scale_log2 = scale_log2;
    q.q_b = s.q_b.as<uint16_t>();
    q.k_cache = io.k_cache;
    q.v_cache = io.v_cache;
    if (capture) {
        VLT_CUDA(cudaMemcpyAsync(cap->resid_in.dev, h, size_t(n) * md.d * 4, cudaMemcpyDeviceToDevice, stream));
        launch_prep_rows(h, nullptr, n, md.d, md.eps, cap->attn_in.as<float>(), nullptr, nullptr, true, false, stream);
    }
    int sp = span_begin(G_MATMUL);
    if (!(skip & 1)) {
        if (big) {
            // 1/rms of the rows: from the sums of squares the GEMM before left (o or down of the layer before), else a row pass.
            const bool carried = io.h_ready && md.d % 128 == 0;
            if (!carried) launch_prep_rows(h, nullptr, n, md.d, md.eps, nullptr, s.h_b.as<uint16_t>(), s.inv.as<float>(), false, false, stream);
            const float* inv_in = carried ? nullptr : s.inv.as<float>();
            const float* ssq_in = carried ? s.ssq.as<float>() : nullptr;
            if (fused_post) matmul_gemm(l.qkv, n, s.h_b.as<uint16_t>(), nullptr, nullptr, EPI_QKV, nullptr, inv_in, 0, &q, nullptr, ssq_in);
            else matmul_gemm(l.qkv, n, s.h_b.as<uint16_t>(), s.qkv.as<float>(), nullptr, EPI_NORM, nullptr, inv_in, 0, nullptr, nullptr, ssq_in);
            if (capture && fused_post) matmul_gemm(l.qkv, n, s.h_b.as<uint16_t>(), s.qkv.as<float>(), nullptr, EPI_NORM, nullptr, inv_in, 0, nullptr, nullptr, ssq_in);
        } else if (fused_post) {
            matmul(l.qkv, n, h, nullptr, EPI_QKV, nullptr, s.inv.as<float>(), 0, &q);
            if (capture) matmul(l.qkv, n, h, s.qkv.as<float>(), EPI_NORM, nullptr, s.inv.as<float>());
        } else {
            matmul(l.qkv, n, h, s.qkv.as<float>(), EPI_NORM, nullptr, s.inv.as<float>());
        }
        if (capture) launch_qkv_capture(s.qkv.as<float>(), io.meta, rope_tab.as<float>(), n, md.n_heads, kva, cap->qkv.as<float>(), stream);
    }
    span_end(sp);
    if (io.kv_only && fused_post && !capture) return;
    sp = span_begin(G_SMALL);
    if (!(skip & 2) && !fused_post)
        launch_qkv_post(s.qkv.as<float>(), io.meta, io.tin, rope_tab.as<float>(), io.k_cache, io.v_cache, kv.page_table.as<uint32_t>(), kva, li, n,
                        md.n_heads, scale_log2, tuning.plain_attention ? nullptr : s.q_b.as<uint16_t>(), io.cpos, stream);
    span_end(sp);
    if (io.kv_only && !capture) return;
    if (io.window && (tuning.plain_attention || io.n_ctiles)) throw Error("only the split attention kernel takes a window");
    if (tuning.plain_attention) {
        if (!(skip & 4))
            launch_attn_plain(s.qkv.as<float>(), io.meta, io.tiles, io.vis, rope_tab.as<float>(), io.k_cache, io.v_cache, kv.page_table.as<uint32_t>(), kva,
                              li, io.n_tiles, md.n_heads, scale_log2, s.attn.as<float>(), stream);
        if (big) launch_prep_rows(s.attn.as<float>(), nullptr, n, md.n_heads * md.hd, md.eps, nullptr, s.attn_b.as<uint16_t>(), nullptr, false, false, stream);
    } else if (io.n_ctiles) {
        // A step with a prompt chunk: rows as the MMA's M side, the keys read once per 64 rows, no key split and no merge.
        ChunkAttnArgs c{};
        c.maps = io.maps;
        c.err_flag = s.err_flag.as<uint32_t>();
        c.q_b = s.q_b.as<uint16_t>();
        c.meta = io.meta;
        c.tin = io.tin;
        c.ctiles = io.ctiles;
        c.vis = io.vis;
        c.page_table = kv.page_table.as<uint32_t>();
        c.kv = kva;
        c.layer = li;
        c.n_ctiles = io.n_ctiles;
        c.n_heads = md.n_heads;
        c.out = s.attn.as<float>();
        c.out_b = s.attn_b.as<uint16_t>();
        sp = span_begin(G_ATTN);
        if (!(skip & 4)) launch_attn_chunk(c, stream);
        span_end(sp);
    } else {
        AttnArgs a{};
        a.maps = io.maps;
        a.err_flag = s.err_flag.as<uint32_t>();
        a.q_b = s.q_b.as<uint16_t>();
        a.meta = io.meta;
        a.tiles = io.tiles;
        a.vis = io.vis;
        a.k_cache = io.k_cache;
        a.v_cache = io.v_cache;
        a.page_table = kv.page_table.as<uint32_t>();
        a.kv = kva;
        a.layer = li;
        a.n_tiles = io.n_tiles;
        a.n_heads = md.n_heads;
        a.scale_log2 = scale_log2;
        a.keys_per_split = io.keys_per_split;
        a.max_splits = io.max_splits;
        a.max_rows = io.max_rows;
        a.window = io.window;
        a.part = s.part.as<float>();
        a.out = s.attn.as<float>();
        a.out_b = s.attn_b.as<uint16_t>();  // the o projection reads the bf16 copy (GEMM and streamed matmul alike)
        a.n = n;
        sp = span_begin(G_ATTN);
        if (!(skip & 4)) launch_attn_mma(a, stream);
        span_end(sp);
        sp = span_begin(G_SMALL);
        if (!(skip & 8)) launch_attn_combine(a, stream);
        span_end(sp);
    }
    sp = span_begin(G_MATMUL);
    if (big) {
        // The residual GEMMs leave bf16(h) and h's sums of squares per 128-row tile for the GEMM after them (gate_up here,
        // the next layer's qkv after down): no row pass in between.
        const bool carry = md.d % 128 == 0;
        float* ssq = carry ? s.ssq.as<float>() : nullptr;
        uint16_t* hb = carry ? s.h_b.as<uint16_t>() : nullptr;
        if (capture) matmul_gemm(l.o, n, s.attn_b.as<uint16_t>(), cap->attn_out.as<float>(), nullptr, EPI_RAW, nullptr, nullptr);
        if (!(skip & 16)) matmul_gemm(l.o, n, s.attn_b.as<uint16_t>(), h, hb, EPI_RESID, h, nullptr, 0, nullptr, ssq);
        if (capture) launch_prep_rows(h, nullptr, n, md.d, md.eps, cap->mlp_in.as<float>(), nullptr, nullptr, true, false, stream);
        if (!(skip & 32)) {
            if (!carry) launch_prep_rows(h, nullptr, n, md.d, md.eps, nullptr, s.h_b.as<uint16_t>(), s.inv.as<float>(), false, false, stream);
            matmul_gemm(l.gate_up, n, s.h_b.as<uint16_t>(), nullptr, s.act_b.as<uint16_t>(), EPI_SWIGLU, nullptr, carry ? nullptr : s.inv.as<float>(), 0, nullptr,
                        nullptr, ssq);  // the down GEMM reads the bf16 copy only
        }
        if (capture) matmul_gemm(l.down, n, s.act_b.as<uint16_t>(), cap->mlp_out.as<float>(), nullptr, EPI_RAW, nullptr, nullptr);
        if (!(skip & 64)) matmul_gemm(l.down, n, s.act_b.as<uint16_t>(), h, hb, EPI_RESID, h, nullptr, 0, nullptr, ssq);
    } else {
        // o and down fold no RMSNorm: they take the bf16 copies their producers leave (a bulk copy instead of a conversion pass).
        const uint16_t* attn_b = tuning.plain_attention ? nullptr : s.attn_b.as<uint16_t>();  // (the scalar attention leaves fp32 only)
        if (capture) matmul(l.o, n, s.attn.as<float>(), cap->attn_out.as<float>(), EPI_RAW, nullptr, nullptr, 0, nullptr, attn_b);
        if (!(skip & 16)) matmul(l.o, n, s.attn.as<float>(), h, EPI_RESID, h, nullptr, 0, nullptr, attn_b);
        if (capture) launch_prep_rows(h, nullptr, n, md.d, md.eps, cap->mlp_in.as<float>(), nullptr, nullptr, true, false, stream);
        if (!(skip & 32)) matmul(l.gate_up, n, h, s.act.as<float>(), EPI_SWIGLU, nullptr, nullptr, 0, nullptr, nullptr, s.act_b.as<uint16_t>());
        if (capture) matmul(l.down, n, s.act.as<float>(), cap->mlp_out.as<float>(), EPI_RAW, nullptr, nullptr, 0, nullptr, s.act_b.as<uint16_t>());
        if (!(skip & 64)) matmul(l.down, n, s.act.as<float>(), h, EPI_RESID, h, nullptr, 0, nullptr, s.act_b.as<uint16_t>());
    }
    span_end(sp);
}

// engine/src/engine/encode.rs:557-573 `encode_sample`.
void Engine::encode_sample(uint32_t set, uint32_t rows) {
    StepSet& st = sets[set];
    launch_sample(s.logits.as<float>(), st.in<SampleRow>(st.o_sample_rows), st.out<uint32_t>(st.o_out_ids), s.meta.as<uint32_t>(), rows, model.md.vocab, stream);
}

// engine/src/engine/encode.rs:383-412 `encode_tail`.
void Engine::encode_tail(uint32_t set, const Plan& p) {
    StepSet& st = sets[set];
    const ModelDesc& md = model.md;
    const float* h = s.h.as<float>();
    bool spec = false;
    SpecStepArgs sa{};
    if (p.n_hidden) launch_prep_rows(h, st.in<uint32_t>(st.o_hidden_rows), p.n_hidden, md.d, md.eps, s.hfin_all.as<float>(), nullptr, nullptr, true, false, stream);
    if (p.n_head && !(skip & 256)) {
        if (use_gemm(model.head, p.n_head) && p.head_all && !(skip & 64) && layer_carries(model.layers.back(), p.n)) {
            // Every row goes through the head (a verify step): the last down projection left bf16(h) and the sums of squares.
            matmul_gemm(model.head, p.n_head, s.h_b.as<uint16_t>(), s.logits.as<float>(), nullptr, EPI_HEAD, nullptr, nullptr, 0, nullptr, nullptr, s.ssq.as<float>());
        } else if (use_gemm(model.head, p.n_head)) {
            launch_prep_rows(h, st.in<uint32_t>(st.o_head_rows), p.n_head, md.d, md.eps, nullptr, s.hfin_b.as<uint16_t>(), s.inv_head.as<float>(), false, false, stream);
            matmul_gemm(model.head, p.n_head, s.hfin_b.as<uint16_t>(), s.logits.as<float>(), nullptr, EPI_HEAD, nullptr, s.inv_head.as<float>());
        } else {
            launch_prep_rows(h, st.in<uint32_t>(st.o_head_rows), p.n_head, md.d, md.eps, s.hfin_head.as<float>(), nullptr, nullptr, false, false, stream);
            matmul(model.head, p.n_head, s.hfin_head.as<float>(), s.logits.as<float>(), EPI_HEAD, nullptr, nullptr);
        }
        // Under the rejection rule the runs whose drafts came with their q rows are decided by k_spec.cu's kernels: row
        // statistics first (they also tell the sampler which rows to leave alone), the sampler for the other rows, then
        // the decisions; accept commits either kind of run.
        if (!forced_logits.empty()) {
            if (forced_logits.size() != size_t(p.n_head) * md.vocab) throw Error("forced logits: " + std::to_string(forced_logits.size()) + " values for " + std::to_string(p.n_head) + " head rows");
            VLT_CUDA(cudaMemcpyAsync(s.logits.dev, forced_logits.data(), forced_logits.size() * 4, cudaMemcpyHostToDevice, stream));
        }
        spec = accept_rule == 1 && drafter;
        if (spec) {
            Drafter& dr = *drafter;
            sa.runs = st.in<RunIn>(st.o_runs);
            sa.n_runs = p.n_runs;
            sa.n_head = p.n_head;
            sa.max_head_rows = cfg.max_head_rows;
            sa.samples = st.in<SampleRow>(st.o_sample_rows);
            sa.tokens = st.in<uint32_t>(st.o_tokens);
            sa.meta = s.meta.as<uint32_t>();
            sa.tree = s.tree.as<uint32_t>();
            sa.logits = s.logits.as<float>();
            sa.vocab = md.vocab;
            sa.q_keep = dr.q_keep.as<float>();
            sa.v = dr.v;
            sa.q_rows = dr.q_rows.as<uint32_t>();
            sa.index_of = dr.index_of.as<uint32_t>();
            sa.stats = dr.spec_stats.as<SpecRowStats>();
            sa.row_skip = dr.row_skip.as<uint32_t>();
            sa.spec_e = dr.spec_e.as<uint32_t>();
            sa.out = st.out<uint32_t>(st.o_out_ids);
            launch_spec_step_stats(sa, stream);
        }
        launch_sample(s.logits.as<float>(), st.in<SampleRow>(st.o_sample_rows), st.out<uint32_t>(st.o_out_ids), s.meta.as<uint32_t>(), p.n_head, md.vocab, stream,
                      spec ? sa.row_skip : nullptr);
        if (spec) launch_spec_step_decide(sa, stream);
    }
    launch_accept(st.in<RunIn>(st.o_runs), st.in<uint32_t>(st.o_tokens), st.out<uint32_t>(st.o_out_ids), s.lens.as<uint32_t>(), s.feed.as<uint32_t>(),
                  s.gen.as<GenState>(), st.out<uint32_t>(st.o_emitted), p.n_runs, s.tree.as<uint32_t>(), s.path.as<uint32_t>(), s.path_len.as<uint32_t>(),
                  s.on_path.as<uint32_t>(), stream, spec ? sa.spec_e : nullptr);
    if (p.branches)
        launch_kv_compact(st.in<RunIn>(st.o_runs), s.path.as<uint32_t>(), s.path_len.as<uint32_t>(), s.lens.as<uint32_t>(), kv.k.as<uint16_t>(),
                          kv.v.as<uint16_t>(), kv.page_table.as<uint32_t>(), kv_args(), p.n_runs, md.n_layers, stream);
}

// The reference's own architecture, encode.rs:99-192 `encode_forward` / `encode_layer` and :383-412 `encode_tail`: the
// layers' extras are k_limite.cu's kernels, the projections the streamed matmul with the matrix scales and residual
// lambdas in its epilogue. The residual stream moves through hist0 (the normed embedding), hist12 / hist23 (the outputs of
// layers 11 and 22, which the MUDD sites at 24 and 47 mix back in) and h.
LimiteKv Engine::limite_kv(const LimiteLayer& x) const {
    uint32_t shift = 0;
    while ((1u << shift) < model.md.page) shift++;
    return LimiteKv{x.global ? 1u : 0u, x.kv_index, model.md.n_kv, lim->ring, cfg.max_seqs, kv.n_pages, kv.max_pages, shift, kv.page_table.as<uint32_t>()};
}

void Engine::encode_forward_limite(uint32_t set, const Plan& p) {
    const ModelDesc& md = model.md;
    StepSet& st = sets[set];
    LimiteState& L = *lim;
    const uint32_t n = p.n, H = md.d;
    if (p.chunked && p.max_run > cfg.max_chunk) throw Error("a run longer than max_chunk");
    begin_step(set, p);  // upload, embedding rows into h
    int sp = span_begin(G_SMALL);
    launch_prep_rows(s.h.as<float>(), nullptr, n, H, md.eps, L.hist0.as<float>(), nullptr, nullptr, true, false, stream);  // kernels.metal:108-113: rms_norm(embedding)
    span_end(sp);
    const float* cur = L.hist0.as<float>();
    const uint32_t* meta = s.meta.as<uint32_t>();
    const uint32_t* tin = st.in<uint32_t>(st.o_tin);
    // From 9 tokens on, and if the projections' shapes and scales fit it (bf16, or int8 with one scale per row or per 64
    // weights of a row, the reference's own int8 files), a layer takes the tensor-core GEMM: activations go in as bf16
    // copies, 1 / rms from a row pass or from the sums of squares the GEMM before left.
    auto big_of = [&](uint32_t li) {
        const Layer& l = model.layers[li];
        return gemm_fits(l.qkv, n) && gemm_fits(l.o, n) && gemm_fits(l.gate_up, n) && gemm_fits(l.down, n) && md.n_heads / md.n_kv <= 8 && md.d % 128 == 0;
    };
    auto mudd_site = [](uint32_t li) { return li == 24 ? 0 : li == 47 ? 1 : -1; };  // model.rs:20 `MUDD_LAYERS`
    for (uint32_t li = 0; li < md.n_layers; li++) {
        const Layer& l = model.layers[li];
        const LimiteLayer& x = model.lim[li];
        const float* xa = cur;
        const float* base = cur;
        const int site = mudd_site(li);
        if (site >= 0) {
            sp = span_begin(G_SMALL);
            launch_limite_mudd(cur, L.hist0.as<float>(), (site == 0 ? L.hist12 : L.hist23).as<float>(), model.mudd_dense1, model.mudd_mix + size_t(site) * 2 * 3 * 33, H, md.eps, n,
                               L.xattn.as<float>(), L.base.as<float>(), stream);
            span_end(sp);
            xa = L.xattn.as<float>();
            base = L.base.as<float>();
        }
        const LimiteKv kva = limite_kv(x);
        uint16_t* kc = x.global ? kv.k.as<uint16_t>() : L.k_local.as<uint16_t>();
        uint16_t* vc = x.global ? kv.v.as<uint16_t>() : L.v_local.as<uint16_t>();
        // The down projection before this layer left the bf16 copy and the sums of squares of this layer's input, unless
        // a MUDD mix stands in between (or this is the first layer): then a row pass makes them.
        const bool big = big_of(li), carried = big && li > 0 && site < 0 && big_of(li - 1);
        const float* inv_in = carried ? nullptr : s.inv.as<float>();
        const float* ssq_in = carried ? s.ssq.as<float>() : nullptr;
        sp = span_begin(G_MATMUL);
        if (big) {
            if (!carried) launch_prep_rows(xa, nullptr, n, H, md.eps, nullptr, s.h_b.as<uint16_t>(), s.inv.as<float>(), false, false, stream);
            matmul_gemm(l.qkv, n, s.h_b.as<uint16_t>(), s.qkv.as<float>(), nullptr, EPI_NORM, nullptr, inv_in, 0, nullptr, nullptr, ssq_in, x.qkv_scale);
        } else {
            matmul(l.qkv, n, xa, s.qkv.as<float>(), EPI_NORM, nullptr, s.inv.as<float>(), 0, nullptr, nullptr, nullptr, x.qkv_scale);
        }
        span_end(sp);
        sp = span_begin(G_SMALL);
        launch_limite_qkv_post(s.qkv.as<float>(), xa, inv_in, meta, tin, st.in<uint32_t>(st.o_tokens), model.value_embed, x.ve_gate, x.attn_gate, rope_tab.as<float>(), kva,
                               H, md.n_heads, md.eps, md.vocab, n, kc, vc, L.vdir.as<float>(), L.gates.as<float>(), ssq_in, H / 128, (cfg.max_step_tokens + 15) / 16 * 16, stream);
        span_end(sp);
        sp = span_begin(G_ATTN);
        launch_limite_attn(s.qkv.as<float>(), meta, tin, st.in<uint32_t>(st.o_vis), st.in<uint32_t>(st.o_tiles), p.tiles, kc, vc, kva, md.n_heads, LIMITE_WINDOW, md.attn_scale, L.vdir.as<float>(), L.gates.as<float>(), x.xsa,
                           n, (x.global ? p.max_keys : std::min(p.max_keys, LIMITE_WINDOW)) + 8, L.part.as<float>(), s.attn.as<float>(), big ? s.attn_b.as<uint16_t>() : nullptr, tuning.attn_keys_per_cta, stream);
        span_end(sp);
        sp = span_begin(G_MATMUL);
        float* out = li == 11 ? L.hist12.as<float>() : li == 22 ? L.hist23.as<float>() : s.h.as<float>();  // encode.rs:116-122 `resid_out`
        if (big) {
            matmul_gemm(l.o, n, s.attn_b.as<uint16_t>(), L.mixed.as<float>(), s.h_b.as<uint16_t>(), EPI_RESID, base, nullptr, 0, nullptr, s.ssq.as<float>(), nullptr, x.o_scale,
                        x.resid_attn, x.post_attn);
            matmul_gemm(l.gate_up, n, s.h_b.as<uint16_t>(), nullptr, s.act_b.as<uint16_t>(), EPI_SWIGLU, nullptr, nullptr, 0, nullptr, nullptr, s.ssq.as<float>());
            const bool carry = li + 1 < md.n_layers && big_of(li + 1) && mudd_site(li + 1) < 0;
            matmul_gemm(l.down, n, s.act_b.as<uint16_t>(), out, carry ? s.h_b.as<uint16_t>() : nullptr, EPI_RESID, L.mixed.as<float>(), nullptr, 0, nullptr,
                        carry ? s.ssq.as<float>() : nullptr, nullptr, 1.0f, x.resid_mlp, x.post_mlp);
        } else {
            matmul(l.o, n, s.attn.as<float>(), L.mixed.as<float>(), EPI_RESID, base, nullptr, 0, nullptr, nullptr, nullptr, x.o_scale, x.resid_attn, x.post_attn);
            matmul(l.gate_up, n, L.mixed.as<float>(), s.act.as<float>(), EPI_SWIGLU, nullptr, nullptr);
            matmul(l.down, n, s.act.as<float>(), out, EPI_RESID, L.mixed.as<float>(), nullptr, 0, nullptr, nullptr, nullptr, 1.0f, x.resid_mlp, x.post_mlp);
        }
        span_end(sp);
        cur = out;
        auto tap = std::find(tap_layers.begin(), tap_layers.end(), li);
        if (tap != tap_layers.end()) launch_prep_rows(out, nullptr, n, H, md.eps, tap_bufs[tap - tap_layers.begin()].as<float>(), nullptr, nullptr, true, true, stream);
    }
    // The tail: final norm of the hidden and head rows, the head with its cap, sampling, accept, compaction.
    sp = span_begin(G_TAIL);
    if (p.n_hidden) launch_prep_rows(cur, st.in<uint32_t>(st.o_hidden_rows), p.n_hidden, H, md.eps, s.hfin_all.as<float>(), nullptr, nullptr, true, false, stream);
    if (p.n_head) {
        const bool big_head = gemm_fits(model.head, p.n_head);
        launch_prep_rows(cur, st.in<uint32_t>(st.o_head_rows), p.n_head, H, md.eps, s.hfin_head.as<float>(), big_head ? s.hfin_b.as<uint16_t>() : nullptr, nullptr, true, false, stream);
        if (big_head) matmul_gemm(model.head, p.n_head, s.hfin_b.as<uint16_t>(), s.logits.as<float>(), nullptr, EPI_HEAD_CAP, nullptr, nullptr);
        else matmul(model.head, p.n_head, s.hfin_head.as<float>(), s.logits.as<float>(), EPI_HEAD_CAP, nullptr, nullptr);
        if (!forced_logits.empty()) {
            if (forced_logits.size() != size_t(p.n_head) * md.vocab) throw Error("forced logits: wrong size");
            VLT_CUDA(cudaMemcpyAsync(s.logits.dev, forced_logits.data(), forced_logits.size() * 4, cudaMemcpyHostToDevice, stream));
        }
        launch_sample(s.logits.as<float>(), st.in<SampleRow>(st.o_sample_rows), st.out<uint32_t>(st.o_out_ids), s.meta.as<uint32_t>(), p.n_head, md.vocab, stream, nullptr);
    }
    launch_accept(st.in<RunIn>(st.o_runs), st.in<uint32_t>(st.o_tokens), st.out<uint32_t>(st.o_out_ids), s.lens.as<uint32_t>(), s.feed.as<uint32_t>(), s.gen.as<GenState>(),
                  st.out<uint32_t>(st.o_emitted), p.n_runs, s.tree.as<uint32_t>(), s.path.as<uint32_t>(), s.path_len.as<uint32_t>(), s.on_path.as<uint32_t>(), stream, nullptr);
    if (p.branches) {
        LimiteLayer any_local, any_global;
        any_global.global = true;
        launch_limite_compact(st.in<RunIn>(st.o_runs), s.path.as<uint32_t>(), s.path_len.as<uint32_t>(), s.lens.as<uint32_t>(), L.k_local.as<uint16_t>(), L.v_local.as<uint16_t>(),
                              kv.k.as<uint16_t>(), kv.v.as<uint16_t>(), limite_kv(any_local), limite_kv(any_global), model.n_local, model.n_global, p.n_runs, stream);
    }
    span_end(sp);
}

// engine/src/engine/encode.rs:99-105 `encode_forward`, after the step set's upload.
void Engine::encode_forward(uint32_t set, const Plan& p) {
    if (model.limite) { encode_forward_limite(set, p); return; }
    begin_step(set, p);
    for (uint32_t li = 0; li < model.md.n_layers; li++) encode_layer(set, p, li);
    const int sp = span_begin(G_TAIL);
    encode_tail(set, p);
    span_end(sp);
}

void Engine::begin_step(uint32_t set, const Plan& p) {
    if (cfg.host_only) throw Error("this engine was created host-only: it plans steps but cannot run them (no CPU path)");
    StepSet& st = sets[set];
    // The set's device copy is free: the step that used it last has been collected (three sets, at most two steps queued).
    VLT_CUDA(cudaMemcpyAsync(st.dev_in.dev, st.host_in, st.in_bytes, cudaMemcpyHostToDevice, copy_in));
    VLT_CUDA(cudaEventRecord(st.uploaded, copy_in));
    VLT_CUDA(cudaEventRecord(st.start, stream));
    VLT_CUDA(cudaStreamWaitEvent(stream, st.uploaded, 0));
    launch_embed(model.embed, st.in<uint32_t>(st.o_tokens), s.h.as<float>(), st.in<uint32_t>(st.o_tin), s.meta.as<uint32_t>(), s.lens.as<uint32_t>(),
                 s.feed.as<uint32_t>(), s.tree.as<uint32_t>(), st.in<uint32_t>(st.o_vis), p.n, model.md.d, model.md.vocab, stream);
}

// engine/src/engine/encode.rs:439-451 `encode_replay`.
void Engine::encode_replay(uint32_t set, const Plan& p, const ReplayArgs& ra) {
    StepSet& st = sets[set];
    launch_replay_draft(st.in<RunIn>(st.o_runs), s.lens.as<uint32_t>(), s.feed.as<uint32_t>(), s.trace.as<uint32_t>(), s.trace_len.as<uint32_t>(), ra,
                        p.n_runs, s.tree.as<uint32_t>(), stream);
}

void Engine::commit(uint32_t set) {
    StepSet& st = sets[set];
    VLT_CUDA(cudaMemcpyAsync(st.out<uint32_t>(st.o_err), s.err_flag.dev, 4, cudaMemcpyDeviceToDevice, stream));
    VLT_CUDA(cudaEventRecord(st.computed, stream));
    VLT_CUDA(cudaStreamWaitEvent(copy_out, st.computed, 0));
    VLT_CUDA(cudaMemcpyAsync(st.host_out, st.dev_out.dev, st.out_bytes, cudaMemcpyDeviceToHost, copy_out));
    VLT_CUDA(cudaEventRecord(st.done, copy_out));
    VLT_CUDA(cudaGetLastError());
}

double Engine::wait(uint32_t set) {
    StepSet& st = sets[set];
    VLT_CUDA(cudaEventSynchronize(st.done));
    float ms = 0.0f;
    VLT_CUDA(cudaEventElapsedTime(&ms, st.start, st.done));
    return double(ms) * 1e-3;
}

void Engine::debug_stalled_wait() {
    if (cfg.host_only) throw Error("this engine was created host-only: it cannot run kernels");
    launch_stalled_wait(s.err_flag.as<uint32_t>(), 1u << 10, 7u, stream);
}

// The device error word of a collected step (it came down with the step's results: no copy of its own).
void Engine::check_device_error(uint32_t set) {
    const StepSet& st = sets[set];
    const uint32_t flag = *st.hout<uint32_t>(st.o_err);
    if (flag) {
        VLT_CUDA(cudaMemsetAsync(s.err_flag.dev, 0, 4, stream));
        *st.hout<uint32_t>(st.o_err) = 0;
        throw Error("a kernel's bounded wait ran out (device error flag " + std::to_string(flag) + "): the step's results are not valid");
    }
}

// engine/src/engine.rs:310-314 `step` + :357-371 `read_output`.
StepOutput Engine::step(const std::vector<PlanRun>& runs, const StepOptions& opts) { return step_runs(runs, opts, nullptr); }

void Engine::upload_set(uint32_t set) {
    if (cfg.host_only) return;
    StepSet& st = sets[set];
    VLT_CUDA(cudaMemcpyAsync(st.dev_in.dev, st.host_in, st.in_bytes, cudaMemcpyHostToDevice, stream));
    VLT_CUDA(cudaStreamSynchronize(stream));
}

// engine/src/engine.rs:381-389 `load_drafter`, for the chain drafter (see Engine::Drafter).
void Engine::load_drafter(const std::string& path) {
    for (const auto& q : seqs)
        if (q) throw Error("load the drafter before the first sequence (it changes how many pages a step reserves)");
    auto dr = std::make_unique<Drafter>();
    const ModelDesc& md = model.md;
    dr->w.load(path, cfg.host_only);
    if (dr->w.has("kv_all")) {  // the reference's block drafter (tools/spec/export.py), not the chain drafter
        dr.reset();
        load_block_drafter(path);
        return;
    }
    if (model.limite) throw Error(path + ": the chain drafter runs a plain decoder's layer; a target of the reference's own architecture takes the block drafter");
    const std::vector<float> m = dr->w.f32s("meta");
    if (m.size() < 4 || m[0] != 1.0f || m[1] != 1.0f || m[2] != 1.0f) throw Error(path + ": `meta` is not a version-1 one-layer chain drafter");
    const uint32_t v = uint32_t(m[3]), d = md.d;
    dr->window = m.size() > 4 ? uint32_t(m[4]) : 0;
    if (md.ffn < 2 * d) throw Error(path + ": the chain drafter needs ffn >= 2 d_model");
    dr->v = v;
    dr->fc = load_matrix(dr->w, "fc", d, 2 * d);
    dr->layer.qkv = load_matrix(dr->w, "D00.qkv", md.qkv_w(), d);
    dr->layer.o = load_matrix(dr->w, "D00.o", d, md.n_heads * md.hd);
    dr->layer.gate_up = load_matrix(dr->w, "D00.gate_up", 2 * md.ffn, d);
    dr->layer.down = load_matrix(dr->w, "D00.down", d, md.ffn);
    dr->head = load_matrix(dr->w, "head", v, d);
    const std::vector<float> idf = dr->w.f32s("vocab");
    if (idf.size() != v) throw Error(path + ": `vocab` has " + std::to_string(idf.size()) + " ids for a head of " + std::to_string(v));
    std::vector<uint32_t> ids(v);
    for (uint32_t i = 0; i < v; i++) {
        ids[i] = uint32_t(idf[i]);
        if (ids[i] >= md.vocab) throw Error(path + ": draft vocabulary id out of the target's range");
    }
    if (cfg.host_only) {  // a planning engine keeps the drafter's effect on page reservation and admission, nothing else
        drafter = std::move(dr);
        return;
    }
    const size_t ms = cfg.max_seqs, ms16 = (ms + 15) / 16 * 16, n = cfg.max_step_tokens;
    dr->vocab_ids.alloc(size_t(v) * 4, false);
    dr->vocab_ids.write(0, ids.data(), size_t(v) * 4);
    const size_t pool = size_t(kv.n_pages) * md.n_kv * kv.page * md.hd * 2;  // one layer
    dr->k.alloc(pool, false);
    dr->v_cache.alloc(pool, false);
    attn_maps_init(&dr->maps, dr->k.as<uint16_t>(), dr->v_cache.as<uint16_t>(), uint64_t(kv.n_pages) * md.n_kv * kv.page);
    dr->carry.alloc(ms * d * 4, false);
    dr->dfeat.alloc(ms * d * 4, false);
    dr->dmeta.alloc(ms * 8, false);
    dr->dtin.alloc(ms * 8, false);
    dr->dvis.alloc(ms * 4, false);
    dr->dcpos.alloc(ms * 4, false);
    dr->live.alloc(ms * 4, false);
    dr->cpos.alloc(n * 4, false);
    dr->logits.alloc(size_t(VERIFY_T - 1) * ms * v * 4, false);
    dr->hfin.alloc(ms * d * 4, false);
    dr->hfin_b.alloc(ms16 * d * 2, false);
    dr->inv.alloc(ms * 4, false);
    dr->q_keep.alloc(ms * (VERIFY_T - 1) * size_t(v) * 4, false);
    dr->q_rows.alloc(ms * 4, false);
    dr->q_rows.order = stream;
    std::vector<uint32_t> inverse(md.vocab, NO_TOK);
    for (uint32_t i = 0; i < v; i++) inverse[ids[i]] = i;
    dr->index_of.alloc(size_t(md.vocab) * 4, false);
    dr->index_of.write(0, inverse.data(), size_t(md.vocab) * 4);
    dr->spec_stats.alloc((size_t(cfg.max_head_rows) + ms * (VERIFY_T - 1)) * sizeof(SpecRowStats), false);
    dr->row_skip.alloc(size_t(cfg.max_head_rows) * 4, false);
    dr->spec_e.alloc(ms * 4, false);
    std::vector<uint32_t> tiles(2 * ms);
    for (uint32_t r = 0; r < ms; r++) { tiles[2 * r] = r; tiles[2 * r + 1] = 1; }
    dr->dtiles.alloc(ms * 8, false);
    dr->dtiles.write(0, tiles.data(), ms * 8);
    drafter = std::move(dr);
    set_taps(tap_layers);  // the drafter reads the last layer's tapped hidden states: it is tapped from now on
}
bool Engine::has_drafter() const { return drafter != nullptr || block_drafter != nullptr; }

// The drafter's part of a step (the reference queues its drafter at the same point,
// engine/src/engine/generate.rs:427-430): a catch-up pass over the step's own tokens that writes the
// drafter's K/V for the rows on the accepted path, then rows - 1 draft passes of one row per run.
void Engine::encode_drafter(uint32_t set, const Plan& p, uint32_t rows) {
    if (block_drafter) { encode_block_drafter(set, p, rows); return; }
    if (!drafter) throw Error("no drafter loaded");
    if (rows < 1 || rows > VERIFY_T) throw Error("the chain drafter proposes for 1.." + std::to_string(VERIFY_T) + " rows");
    Drafter& dr = *drafter;
    StepSet& st = sets[set];
    const ModelDesc& md = model.md;
    const uint32_t d = md.d, n = p.n, nr = p.n_runs;
    const int sp = span_begin(G_DRAFTER);
    float* x = s.act.as<float>();
    uint16_t* xb = s.act_b.as<uint16_t>();
    float* h = s.h.as<float>();
    const RunIn* runs = st.in<RunIn>(st.o_runs);
    // With the layer on the GEMM, fc leaves bf16(h) and h's sums of squares as a residual projection does (no base here):
    // the qkv projection needs no row pass, nor does the head after the layer.
    auto fc = [&](uint32_t rows_in) {
        const bool carries = use_gemm(dr.fc, rows_in) && layer_carries(dr.layer, rows_in);
        if (carries) matmul_gemm(dr.fc, rows_in, xb, h, s.h_b.as<uint16_t>(), EPI_RESID, nullptr, nullptr, 0, nullptr, s.ssq.as<float>());
        else if (use_gemm(dr.fc, rows_in)) matmul_gemm(dr.fc, rows_in, xb, h, nullptr, EPI_RAW, nullptr, nullptr);
        else matmul(dr.fc, rows_in, x, h, EPI_RAW, nullptr, nullptr);
        return carries;
    };
    LayerIO io{};
    io.l = &dr.layer;
    io.layer = 0;
    io.k_cache = dr.k.as<uint16_t>();
    io.v_cache = dr.v_cache.as<uint16_t>();
    io.maps = &dr.maps;
    // (1) catch-up, on the step's own layout. Only its K/V matter (the passes below take their features from the target's
    // taps, not from this pass's output), and a one-layer drafter's K/V depend on fc and the qkv projection alone: the
    // pass stops there, without attention, o projection or MLP.
    launch_draft_catchup_in(st.in<uint32_t>(st.o_tokens), st.in<uint32_t>(st.o_tin), s.meta.as<uint32_t>(), s.on_path.as<uint32_t>(), last_tap(),
                            dr.carry.as<float>(), model.embed, n, d, x, xb, dr.cpos.as<uint32_t>(), stream);
    io.h_ready = fc(n);
    io.n = n;
    io.meta = s.meta.as<uint32_t>();
    io.tin = st.in<uint32_t>(st.o_tin);
    io.tiles = st.in<uint32_t>(st.o_tiles);
    io.vis = st.in<uint32_t>(st.o_vis);
    io.n_tiles = p.tiles;
    io.ctiles = st.in<uint32_t>(st.o_ctiles);
    io.n_ctiles = p.chunked ? p.ctiles : 0;
    io.cpos = dr.cpos.as<uint32_t>();
    io.keys_per_split = p.keys_per_split;
    io.max_splits = p.max_splits;
    io.max_rows = std::min(p.max_run, VERIFY_T);
    io.kv_only = true;
    encode_layer_io(io);
    io.kv_only = false;
    // (2) the draft passes, one row per run.
    Plan dp;
    dp.n = nr;
    const uint32_t reach = std::min(p.max_keys + VERIFY_T, cfg.max_seq_len);
    attention_split(dp, dr.window ? std::min(reach, dr.window + md.page) : reach, nr);
    io.n = nr;
    io.meta = dr.dmeta.as<uint32_t>();
    io.tin = dr.dtin.as<uint32_t>();
    io.tiles = dr.dtiles.as<uint32_t>();
    io.vis = dr.dvis.as<uint32_t>();
    io.n_tiles = nr;
    io.n_ctiles = 0;
    io.cpos = dr.dcpos.as<uint32_t>();
    io.keys_per_split = dp.keys_per_split;
    io.max_splits = dp.max_splits;
    io.max_rows = 1;
    io.window = dr.window;
    for (uint32_t i = 1; i < rows; i++) {
        launch_draft_pass_in(runs, s.lens.as<uint32_t>(), s.feed.as<uint32_t>(), s.path.as<uint32_t>(), s.path_len.as<uint32_t>(), s.on_path.as<uint32_t>(),
                             st.out<uint32_t>(st.o_emitted), last_tap(), dr.dfeat.as<float>(), model.embed, nr, d, md.vocab, i, cfg.max_seq_len, x, xb,
                             dr.dmeta.as<uint32_t>(), dr.dtin.as<uint32_t>(), dr.dvis.as<uint32_t>(), dr.dcpos.as<uint32_t>(), dr.live.as<uint32_t>(), stream);
        io.h_ready = fc(nr);
        encode_layer_io(io);
        // The pass's normed output is the next pass's feature (rounded like a tap); the head reads the raw rows and 1/rms.
        launch_prep_rows(h, nullptr, nr, d, md.eps, dr.dfeat.as<float>(), nullptr, nullptr, true, true, stream);
        float* lg = dr.logits.as<float>() + size_t(i - 1) * cfg.max_seqs * dr.v;
        if (use_gemm(dr.head, nr) && layer_carries(dr.layer, nr)) {
            matmul_gemm(dr.head, nr, s.h_b.as<uint16_t>(), lg, nullptr, EPI_HEAD, nullptr, nullptr, dr.v, nullptr, nullptr, s.ssq.as<float>());
        } else if (use_gemm(dr.head, nr)) {
            launch_prep_rows(h, nullptr, nr, d, md.eps, nullptr, dr.hfin_b.as<uint16_t>(), dr.inv.as<float>(), false, false, stream);
            matmul_gemm(dr.head, nr, dr.hfin_b.as<uint16_t>(), lg, nullptr, EPI_HEAD, nullptr, dr.inv.as<float>(), dr.v);
        } else {
            launch_prep_rows(h, nullptr, nr, d, md.eps, dr.hfin.as<float>(), nullptr, nullptr, false, false, stream);
            matmul(dr.head, nr, dr.hfin.as<float>(), lg, EPI_HEAD, nullptr, nullptr, dr.v);
        }
        if (!forced_draft_logits.empty()) {
            if (forced_draft_logits.size() != size_t(rows - 1) * nr * dr.v) throw Error("forced draft logits: wrong size");
            VLT_CUDA(cudaMemcpyAsync(lg, forced_draft_logits.data() + size_t(i - 1) * nr * dr.v, size_t(nr) * dr.v * 4, cudaMemcpyHostToDevice, stream));
        }
        launch_draft_draw(lg, dr.v, dr.vocab_ids.as<uint32_t>(), runs, st.in<SampleRow>(st.o_sample_rows), dr.live.as<uint32_t>(), s.lens.as<uint32_t>(), nr, i, accept_rule,
                          s.feed.as<uint32_t>(), s.tree.as<uint32_t>(), dr.q_keep.as<float>(), dr.q_rows.as<uint32_t>(), stream);
    }
    launch_draft_carry(runs, s.path.as<uint32_t>(), s.path_len.as<uint32_t>(), s.on_path.as<uint32_t>(), last_tap(), nr, d, dr.carry.as<float>(), stream);
    span_end(sp);
}

// engine/src/engine/drafter.rs:131-240 `Drafter::load`, for a file of tools/spec/export.py's layout. The reference's
// shapes are its target's constants; here the hidden width must be the target's, heads are 128 wide, and the file gives
// the rest. The drafter turns 32 pairs with the engine's RoPE table: the target's heads are 64 wide, or the target is of the
// reference's own architecture.
void Engine::load_block_drafter(const std::string& path) {
    auto d = std::make_unique<BlockDrafter>();
    const ModelDesc& md = model.md;
    d->w.load(path, cfg.host_only);
    const std::vector<float> m = d->w.f32s("meta");
    if (m.size() < 5 || m.size() != 5 + size_t(m[1])) throw Error(path + ": `meta` is not a block drafter's");
    const uint32_t n_layers = uint32_t(m[0]), n_taps = uint32_t(m[1]);
    d->block = uint32_t(m[2]);
    d->v = uint32_t(m[4]);
    for (uint32_t k = 0; k < n_taps; k++) d->taps.push_back(uint32_t(m[5 + k]));
    const uint32_t H = md.d, D = 128;
    if (H % D || model.rope_freq.size() != 32) throw Error(path + ": the block drafter needs a target whose hidden width is a multiple of 128 and whose RoPE table has 32 pairs (heads of 64, or the reference's own architecture)");
    const uint32_t n_q = H / D, kv_rows = d->w.tensor("kv_all").shape.at(0), n_kv = kv_rows / (n_layers * 2 * D);
    if (n_layers == 0 || n_kv == 0 || n_kv * n_layers * 2 * D != kv_rows || n_q % n_kv || n_q + n_kv > 32) throw Error(path + ": kv_all's rows do not fit the layers and heads");
    d->ffn = d->w.tensor("D00.down").shape.at(1);
    if (H / 16 * 2 > BLOCK_CONV_KC) throw Error(path + ": the convolutions' corrections do not fit 192 rows");
    for (uint32_t k = 0; k < n_taps; k++) d->fc.push_back(load_matrix(d->w, "fc." + std::to_string(k), H, H));
    d->kv_all = load_matrix(d->w, "kv_all", kv_rows, H);
    d->inject = load_matrix(d->w, "inject", H, H);
    d->head = load_matrix(d->w, "head", d->v, H);
    const uint8_t* base = d->w.buffer.as<uint8_t>();
    d->mask_emb = reinterpret_cast<const float*>(base + d->w.get("mask_emb", DType::F32, {H}).offset);
    for (uint32_t i = 0; i < n_layers; i++) {
        char nm[48];
        auto name = [&](const std::string& k) { std::snprintf(nm, sizeof nm, "D%02u.%s", i, k.c_str()); return std::string(nm); };
        BlockDrafter::DLayer l;
        l.qkv = load_matrix(d->w, name("qkv"), (n_q + 2 * n_kv) * D, H);
        l.o = load_matrix(d->w, name("o"), H, n_q * D);
        l.gate_up = load_matrix(d->w, name("gate_up"), 2 * d->ffn, H);
        l.down = load_matrix(d->w, name("down"), H, d->ffn);
        for (uint32_t c = 0; c < 4; c++) {
            l.conv_base[c] = reinterpret_cast<const float*>(base + d->w.get(name("conv" + std::to_string(c) + ".base"), DType::F32, {2, H}).offset);
            l.conv_corr[c] = load_matrix(d->w, name("conv" + std::to_string(c) + ".corr"), BLOCK_CONV_KC, H);
        }
        d->layers.push_back(l);
    }
    const std::vector<float> idf = d->w.f32s("vocab");
    if (idf.size() != d->v) throw Error(path + ": `vocab` has " + std::to_string(idf.size()) + " ids for a head of " + std::to_string(d->v));
    std::vector<uint32_t> ids(d->v);
    for (uint32_t i = 0; i < d->v; i++) {
        ids[i] = uint32_t(idf[i]);
        if (ids[i] >= md.vocab) throw Error(path + ": draft vocabulary id out of the target's range");
    }
    for (uint32_t t : d->taps)
        if (t >= md.n_layers) throw Error(path + ": it reads layer " + std::to_string(t) + " of a target with " + std::to_string(md.n_layers));
    BlockDrafterDims& bd = d->dims;
    bd.hidden = H; bd.n_q = n_q; bd.n_kv = n_kv; bd.n_layers = n_layers;
    bd.window = uint32_t(m[3]);
    bd.ring = bd.window + cfg.max_chunk;  // drafter.rs:175: a step's run is at most max_chunk tokens, so its positions do not collide
    bd.ctx_ring_len = cfg.max_chunk;
    bd.max_seqs = cfg.max_seqs;
    bd.eps = md.eps;
    bd.scale = md.attn_scale;
    if (!cfg.host_only) {
        const size_t n = cfg.max_step_tokens, ms = cfg.max_seqs, rows = ms * VERIFY_T, ring_bytes = size_t(n_layers) * ms * n_kv * bd.ring * D * 2;
        auto f = [&](Buffer& b, size_t floats) { b.alloc(floats * 4, false); };
        d->vocab_ids.alloc(size_t(d->v) * 4, false);
        d->vocab_ids.write(0, ids.data(), size_t(d->v) * 4);
        d->k_ring.alloc(ring_bytes, false);
        d->v_ring.alloc(ring_bytes, false);
        f(d->ctx_ring, ms * bd.ctx_ring_len * H);
        f(d->ctx, n * H);
        f(d->ctx_inv, n);
        f(d->kvp, n * kv_rows);
        for (Buffer* b : {&d->x, &d->last, &d->cx, &d->co, &d->mixed, &d->hfin}) f(*b, rows * H);
        f(d->qkv, rows * (n_q + 2 * n_kv) * D);
        f(d->inv, rows);
        f(d->attn, rows * n_q * D);
        f(d->act, rows * d->ffn);
        // The correction matrices also as copies of 256 rows (zero past the file's 192), which the GEMM's 128-row tiles take:
        // bf16 weights, or int8 weights and behind them their scales.
        d->corr_stride = 2 * 128;
        {
            const size_t one = size_t(d->corr_stride) * H * 2 + 256;  // (room for either format, the scales 256-byte aligned)
            d->conv_pad.alloc(one * 4 * n_layers, false);  // (zeroed)
            for (uint32_t i = 0; i < n_layers; i++)
                for (uint32_t c = 0; c < 4; c++) {
                    uint8_t* at = d->conv_pad.as<uint8_t>() + (size_t(i) * 4 + c) * one;
                    const Matrix& src = d->layers[i].conv_corr[c];
                    Matrix& g = d->layers[i].conv_corr_gemm[c];
                    g = src;
                    g.w = at;
                    g.m = d->corr_stride;
                    if (!src.int8) {
                        VLT_CUDA(cudaMemcpy(at, src.w, size_t(BLOCK_CONV_KC) * H * 2, cudaMemcpyDeviceToDevice));
                        continue;
                    }
                    const size_t w_bytes = size_t(d->corr_stride) * H, groups = H / src.group;
                    uint8_t* sc = at + (w_bytes + 255) / 256 * 256;
                    VLT_CUDA(cudaMemcpy(at, src.w, size_t(BLOCK_CONV_KC) * H, cudaMemcpyDeviceToDevice));
                    VLT_CUDA(cudaMemcpy(sc, src.scales, size_t(BLOCK_CONV_KC) * groups * 2, cudaMemcpyDeviceToDevice));
                    g.scales = reinterpret_cast<const uint16_t*>(sc);
                }
            VLT_CUDA(cudaDeviceSynchronize());  // (device-to-device copies on the legacy stream: done before the engine's own streams read them)
        }
        f(d->corr, rows * d->corr_stride);
        f(d->corr_inv, rows);
        d->xb.alloc((std::max(n, rows) + 16) * std::max<size_t>(H, d->ffn) * 2, false);  // (the GEMM's tensor maps cover whole groups of 16 rows)
        d->act_b.alloc((rows + 16) * d->ffn * 2, false);
        d->attn_b.alloc((rows + 16) * size_t(n_q) * D * 2, false);
        // The attention's partials: a row's keys are at most window + 8, in splits of at least 64.
        d->part.alloc(rows * n_q * size_t(std::min<uint32_t>(LIMITE_MAX_SPLITS, (bd.window + 8 + 63) / 64 + 1)) * LIMITE_PART * 4, false);
        f(d->logits, rows * d->v);
        f(d->cand, rows * 4);
        f(d->cand_q, rows * 4);
        f(d->meta, 2 * rows);
        for (Buffer& b : d->layout) {
            f(b, 4 * rows + 3 * ms);
            b.order = stream;
        }
    }
    block_drafter = std::move(d);
    set_taps(block_drafter->taps);
}

void Engine::drafter_matmul(const Matrix& w, uint32_t n, const float* x, float* y, uint32_t epi, const float* base, float* inv_out, const uint16_t* xb, uint16_t* yb) {
    if (!gemm_fits(w, n)) {
        matmul(w, n, x, y, epi, base, inv_out, 0, nullptr, nullptr, yb);
        return;
    }
    BlockDrafter& d = *block_drafter;
    const bool norms = epi == EPI_NORM || epi == EPI_SWIGLU;
    float* inv = norms ? (inv_out ? inv_out : d.inv.as<float>()) : nullptr;
    if (!xb || norms) launch_prep_rows(x, nullptr, n, w.k, model.md.eps, nullptr, xb ? nullptr : d.xb.as<uint16_t>(), inv, false, false, stream);
    matmul_gemm(w, n, xb ? xb : d.xb.as<uint16_t>(), y, yb, epi, base, inv);
}

// engine/src/engine/drafter.rs:278-447 `encode_drafter`: the context of all of the step's tokens (those on the accepted
// path reach the rings), then a block of `rows` rows for every run of the step that has head rows, then the candidates
// and a draft tree per block into feed / tree.
void Engine::encode_block_drafter(uint32_t set, const Plan& p, uint32_t rows) {
    if (cfg.host_only) throw Error("this engine was created host-only: it plans steps but cannot run them (no CPU path)");
    if (rows < 1 || rows > VERIFY_T) throw Error("a block has 1.." + std::to_string(VERIFY_T) + " rows");
    BlockDrafter& d = *block_drafter;
    const BlockDrafterDims& bd = d.dims;
    const ModelDesc& md = model.md;
    StepSet& st = sets[set];
    const int sp = span_begin(G_DRAFTER);
    const uint32_t n = p.n, H = bd.hidden;
    // 1. Context.
    for (uint32_t k = 0; k < d.fc.size(); k++)
        drafter_matmul(d.fc[k], n, tap_bufs[k].as<float>(), d.ctx.as<float>(), k ? EPI_RESID : EPI_RAW, k ? d.ctx.as<float>() : nullptr, nullptr);
    drafter_matmul(d.kv_all, n, d.ctx.as<float>(), d.kvp.as<float>(), EPI_NORM, nullptr, d.ctx_inv.as<float>());
    launch_block_context(d.kvp.as<float>(), d.ctx.as<float>(), d.ctx_inv.as<float>(), s.meta.as<uint32_t>(), s.on_path.as<uint32_t>(), rope_tab.as<float>(), bd, n,
                         d.k_ring.as<uint16_t>(), d.v_ring.as<uint16_t>(), d.ctx_ring.as<float>(), stream);
    // 2. The blocks' layout, from the step's runs (the host's copy of what the step uploaded).
    const RunIn* runs = st.hin<RunIn>(st.o_runs);
    const size_t max_rows = size_t(cfg.max_seqs) * VERIFY_T;
    std::vector<uint32_t> lay(4 * max_rows + 3 * size_t(cfg.max_seqs), 0);
    uint32_t* tin = lay.data();
    uint32_t* rows_of = tin + 2 * max_rows;
    uint32_t* sees = rows_of + max_rows;  // a block row sees every row of its block
    uint32_t* blocks = sees + max_rows;
    uint32_t* slots = blocks + 2 * cfg.max_seqs;
    uint32_t R = 0, nb = 0;
    for (uint32_t r = 0; r < p.n_runs && rows > 1; r++) {
        if (runs[r].nhead == 0 || nb == cfg.max_seqs) continue;
        blocks[2 * nb] = R;
        blocks[2 * nb + 1] = rows;
        slots[nb++] = runs[r].slot;
        for (uint32_t i = 0; i < rows; i++, R++) {
            tin[2 * R] = runs[r].slot;
            tin[2 * R + 1] = i;
            rows_of[R] = rows;
            sees[R] = (1u << rows) - 1;
        }
    }
    d.last_rows = R;
    if (R == 0) { span_end(sp); return; }
    Buffer& lb = d.layout[set];
    lb.write(0, lay.data(), lay.size() * 4);
    const uint32_t* d_tin = lb.as<uint32_t>();
    const uint32_t* d_rows_of = d_tin + 2 * max_rows;
    const uint32_t* d_sees = d_rows_of + max_rows;
    const uint32_t* d_blocks = d_sees + max_rows;
    const uint32_t* d_slots = d_blocks + 2 * cfg.max_seqs;
    float* x = d.x.as<float>();
    launch_block_embed(model.embed, d_tin, s.lens.as<uint32_t>(), s.feed.as<uint32_t>(), d.mask_emb, d.ctx_ring.as<float>(), bd, md.vocab, R, x, d.last.as<float>(),
                       d.meta.as<uint32_t>(), stream);
    drafter_matmul(d.inject, R, d.last.as<float>(), x, EPI_RESID, x, nullptr);
    // out = resid + conv(in) within each block (or conv(in) alone): the corrections through a matmul, then the two taps.
    auto conv = [&](const BlockDrafter::DLayer& l, uint32_t c, const float* in, const float* resid, float* out) {
        const bool padded = l.conv_corr_gemm[c].m && gemm_fits(l.conv_corr_gemm[c], R);
        drafter_matmul(padded ? l.conv_corr_gemm[c] : l.conv_corr[c], R, in, d.corr.as<float>(), EPI_NORM, nullptr, d.corr_inv.as<float>());
        launch_block_conv(in, d.corr.as<float>(), padded ? d.corr_stride : BLOCK_CONV_KC, l.conv_base[c], d_tin, resid, H, R, out, stream);
    };
    for (uint32_t li = 0; li < d.layers.size(); li++) {
        const BlockDrafter::DLayer& l = d.layers[li];
        conv(l, 0, x, nullptr, d.cx.as<float>());
        drafter_matmul(l.qkv, R, d.cx.as<float>(), d.qkv.as<float>(), EPI_NORM, nullptr, d.inv.as<float>());
        launch_block_qkv_post(d.qkv.as<float>(), d.meta.as<uint32_t>(), rope_tab.as<float>(), bd, li, R, d.k_ring.as<uint16_t>(), d.v_ring.as<uint16_t>(), stream);
        // The attention: the reference architecture's tensor-core kernel over the layer's rings (a block's rows lie in the
        // ring like a verified tile's, each seeing all of them; no XSA, no gate), which also leaves the o projection's bf16
        // input; kv heads with more than eight query heads take the block kernel.
        const bool mma_attn = bd.n_q / bd.n_kv <= 8;
        if (mma_attn) {
            LimiteKv ring{};
            ring.layer = li;
            ring.n_kv = bd.n_kv;
            ring.ring = bd.ring;
            ring.max_seqs = bd.max_seqs;
            launch_limite_attn(d.qkv.as<float>(), d.meta.as<uint32_t>(), d_tin, d_sees, d_blocks, nb, d.k_ring.as<uint16_t>(), d.v_ring.as<uint16_t>(), ring, bd.n_q, bd.window, bd.scale, nullptr,
                               nullptr, nullptr, R, std::min(p.max_keys + VERIFY_T, bd.window) + 8, d.part.as<float>(), d.attn.as<float>(), d.attn_b.as<uint16_t>(),
                               tuning.attn_keys_per_cta, stream);
        } else {
            launch_block_attn(d.qkv.as<float>(), d.meta.as<uint32_t>(), d_tin, d_rows_of, d.k_ring.as<uint16_t>(), d.v_ring.as<uint16_t>(), bd, li, R, d.attn.as<float>(), stream);
        }
        drafter_matmul(l.o, R, d.attn.as<float>(), d.co.as<float>(), EPI_RAW, nullptr, nullptr, mma_attn ? d.attn_b.as<uint16_t>() : nullptr);
        conv(l, 1, d.co.as<float>(), x, d.mixed.as<float>());
        conv(l, 2, d.mixed.as<float>(), nullptr, d.cx.as<float>());
        // The SwiGLU's bf16 output feeds the down projection's GEMM directly.
        const bool chain = gemm_fits(l.gate_up, R) && gemm_fits(l.down, R);
        drafter_matmul(l.gate_up, R, d.cx.as<float>(), chain ? nullptr : d.act.as<float>(), EPI_SWIGLU, nullptr, nullptr, nullptr, chain ? d.act_b.as<uint16_t>() : nullptr);
        drafter_matmul(l.down, R, d.act.as<float>(), d.co.as<float>(), EPI_RAW, nullptr, nullptr, chain ? d.act_b.as<uint16_t>() : nullptr);
        conv(l, 3, d.co.as<float>(), d.mixed.as<float>(), x);
    }
    // 3. Raw logits (drafter.rs:418-419: through the target's cap a trained drafter's largest would tie), candidates, trees.
    launch_prep_rows(x, nullptr, R, H, md.eps, d.hfin.as<float>(), nullptr, nullptr, true, false, stream);
    drafter_matmul(d.head, R, d.hfin.as<float>(), d.logits.as<float>(), EPI_RAW, nullptr, nullptr);
    const uint32_t ncand = std::min(4u, rows - 1);
    launch_draft_top(d.logits.as<float>(), R, d.v, d.vocab_ids.as<uint32_t>(), d_tin, 1.0f / 0.6f, ncand, d.cand.as<uint32_t>(), d.cand_q.as<float>(), stream);
    launch_draft_tree(d_blocks, d_slots, nb, d.cand.as<uint32_t>(), d.cand_q.as<float>(), ncand, s.feed.as<uint32_t>(), s.tree.as<uint32_t>(), stream);
    span_end(sp);
}

StepOutput Engine::step_runs(const std::vector<PlanRun>& runs, const StepOptions& opts, const ReplayArgs* replay) {
    Plan p = plan(0, runs, opts.hidden);
    encode_forward(0, p);
    if (debug_draft_rows && has_drafter()) encode_drafter(0, p, debug_draft_rows);
    if (replay) encode_replay(0, p, *replay);
    commit(0);
    const double secs = wait(0);
    forced_logits.clear();
    forced_draft_logits.clear();
    check_device_error(0);
    return read_output(p, opts, secs);
}

// engine/src/engine.rs:357-371 `read_output`.
StepOutput Engine::read_output(const Plan& p, const StepOptions& opts, double gpu_seconds) {
    StepOutput out;
    out.gpu_seconds = gpu_seconds;
    const StepSet& st = sets[0];
    out.ids.assign(st.hout<uint32_t>(st.o_out_ids), st.hout<uint32_t>(st.o_out_ids) + p.n_head);
    if (opts.read_logits) out.logits = s.logits.read_vec<float>(0, size_t(p.n_head) * model.md.vocab);
    out.hidden = s.hfin_all.read_vec<float>(0, size_t(p.n_hidden) * model.md.d);
    if (opts.read_taps) {
        for (const Buffer& b : tap_bufs) {
            const std::vector<float> tf = b.read_vec<float>(0, size_t(p.n) * model.md.d);
            for (float v : tf) { uint32_t u; std::memcpy(&u, &v, 4); out.taps.push_back(uint16_t(u >> 16)); }  // bf16 values held as f32
        }
    }
    return out;
}

// engine/src/engine.rs:318-355 `step_capture`.
StepOutput Engine::step_capture(const std::vector<PlanRun>& runs, const StepOptions& opts, const std::function<void(const LayerCapture&)>& f) {
    if (cfg.host_only) throw Error("this engine was created host-only: it plans steps but cannot run them (no CPU path)");
    if (model.limite) throw Error("step_capture is built for the plain decoder");
    const ModelDesc& md = model.md;
    if (!cap) {
        cap = std::make_unique<CaptureBufs>();
        const size_t n = cfg.max_step_tokens;
        for (Buffer* b : {&cap->resid_in, &cap->attn_in, &cap->attn_out, &cap->mlp_in, &cap->mlp_out}) b->alloc(n * md.d * 4, false);
        cap->qkv.alloc(n * md.qkv_w() * 4, false);
    }
    Plan p = plan(0, runs, opts.hidden);
    begin_step(0, p);
    const size_t n = p.n;
    for (uint32_t li = 0; li < md.n_layers; li++) {
        encode_layer(0, p, li, true);
        VLT_CUDA(cudaStreamSynchronize(stream));
        const std::vector<float> resid_in = cap->resid_in.read_vec<float>(0, n * md.d), attn_in = cap->attn_in.read_vec<float>(0, n * md.d),
                                 qkv = cap->qkv.read_vec<float>(0, n * md.qkv_w()), sdpa = s.attn.read_vec<float>(0, n * md.n_heads * md.hd),
                                 attn_out = cap->attn_out.read_vec<float>(0, n * md.d), mlp_in = cap->mlp_in.read_vec<float>(0, n * md.d),
                                 mlp_out = cap->mlp_out.read_vec<float>(0, n * md.d);
        f(LayerCapture{li, p.n, resid_in.data(), attn_in.data(), qkv.data(), sdpa.data(), attn_out.data(), mlp_in.data(), mlp_out.data()});
    }
    encode_tail(0, p);
    commit(0);
    const double secs = wait(0);
    check_device_error(0);
    return read_output(p, opts, secs);
}

// engine/src/engine/hooks.rs:28-36 `bench_fill`.
void Engine::bench_fill(uint32_t id, uint32_t len, uint32_t seed) {
    if (id >= seqs.size() || !seqs[id]) throw Error("unknown sequence");
    Seq& sq = *seqs[id];
    const uint32_t from = sq.len;
    if (sq.len + len > cfg.max_seq_len) throw Error("sequence would reach " + std::to_string(sq.len + len) + " tokens (max " + std::to_string(cfg.max_seq_len) + ")");
    sq.len += len;
    s.lens.write(id * 4, &sq.len, 4);
    kv.reserve(id, sq.pages, sq.len);
    if (seed && model.limite) throw Error("bench_fill with values fills a plain decoder's paged pool; a model of the reference's own architecture is filled by computing it");
    if (seed && !cfg.host_only) {
        launch_kv_fill(kv.k.as<uint16_t>(), kv.v.as<uint16_t>(), kv.page_table.as<uint32_t>(), kv_args(), model.md.n_layers, id, from, sq.len, seed, stream);
        VLT_CUDA(cudaStreamSynchronize(stream));
    }
}

// engine/src/engine/hooks.rs:41-54 `sample_logits`.
std::vector<uint32_t> Engine::sample_logits(const float* logits, const std::vector<std::pair<Sampling, uint32_t>>& rows) {
    if (cfg.host_only) throw Error("this engine was created host-only: it cannot run kernels");
    const size_t n = rows.size();
    if (n == 0 || n > cfg.max_head_rows) throw Error(std::to_string(n) + " rows of logits (max " + std::to_string(cfg.max_head_rows) + " rows)");
    StepSet& st = sets[0];
    for (size_t i = 0; i < n; i++) {
        rows[i].first.check();
        st.hin<SampleRow>(st.o_sample_rows)[i] = rows[i].first.row_at(rows[i].second);
    }
    if (logits) VLT_CUDA(cudaMemcpyAsync(s.logits.dev, logits, n * model.md.vocab * 4, cudaMemcpyHostToDevice, stream));
    VLT_CUDA(cudaMemcpyAsync(st.dev_in.dev, st.host_in, st.in_bytes, cudaMemcpyHostToDevice, stream));
    encode_sample(0, uint32_t(n));
    VLT_CUDA(cudaMemcpyAsync(st.host_out, st.dev_out.dev, st.out_bytes, cudaMemcpyDeviceToHost, stream));
    VLT_CUDA(cudaStreamSynchronize(stream));
    return std::vector<uint32_t>(st.hout<uint32_t>(st.o_out_ids), st.hout<uint32_t>(st.o_out_ids) + n);
}

double Engine::spec_accept(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, float temperature,
                           const uint64_t* seeds, const uint32_t* pos0, uint32_t reps, uint32_t* out) {
    if (cfg.host_only) throw Error("this engine was created host-only: it cannot run kernels");
    if (streams == 0 || k == 0 || k > 15) throw Error("spec_accept: needs at least one stream and 1..15 drafts");
    if (!(std::isnormal(temperature) && temperature > 0.0f)) throw Error("spec_accept: needs a normal positive temperature");
    const uint32_t vocab = model.md.vocab;
    for (uint32_t i = 0; i < streams * k; i++)
        if (drafts[i] >= vocab) throw Error("spec_accept: draft token id out of range");
    const size_t pb = size_t(streams) * (k + 1) * vocab * 2, qb = size_t(streams) * k * vocab * 2;
    if (spec_p.bytes < pb) spec_p.alloc(pb, false);
    if (spec_q.bytes < qb) spec_q.alloc(qb, false);
    // small: drafts | seeds | pos0 | accepted | token | rollback | row statistics
    const size_t o_seeds = (size_t(streams) * k * 4 + 255) / 256 * 256, o_pos = o_seeds + (size_t(streams) * 8 + 255) / 256 * 256;
    const size_t o_out = o_pos + (size_t(streams) * 4 + 255) / 256 * 256, o_stats = o_out + (size_t(streams) * 12 + 255) / 256 * 256;
    const size_t small = o_stats + size_t(streams) * (2 * k + 1) * 16;
    if (spec_small.bytes < small) spec_small.alloc(small, false);
    uint8_t* sm = spec_small.as<uint8_t>();
    VLT_CUDA(cudaMemcpyAsync(spec_p.dev, p, pb, cudaMemcpyHostToDevice, stream));
    VLT_CUDA(cudaMemcpyAsync(spec_q.dev, q, qb, cudaMemcpyHostToDevice, stream));
    VLT_CUDA(cudaMemcpyAsync(sm, drafts, size_t(streams) * k * 4, cudaMemcpyHostToDevice, stream));
    VLT_CUDA(cudaMemcpyAsync(sm + o_seeds, seeds, size_t(streams) * 8, cudaMemcpyHostToDevice, stream));
    VLT_CUDA(cudaMemcpyAsync(sm + o_pos, pos0, size_t(streams) * 4, cudaMemcpyHostToDevice, stream));
    cudaEvent_t e0, e1;
    VLT_CUDA(cudaEventCreate(&e0));
    VLT_CUDA(cudaEventCreate(&e1));
    double best = 1e30;
    uint32_t* o = reinterpret_cast<uint32_t*>(sm + o_out);
    for (uint32_t r = 0; r < std::max(reps, 1u); r++) {
        VLT_CUDA(cudaEventRecord(e0, stream));
        launch_spec_accept(spec_p.as<uint16_t>(), spec_q.as<uint16_t>(), reinterpret_cast<const uint32_t*>(sm), streams, k, vocab, temperature,
                           reinterpret_cast<const uint64_t*>(sm + o_seeds), reinterpret_cast<const uint32_t*>(sm + o_pos), sm + o_stats, o, o + streams,
                           o + 2 * streams, stream);
        VLT_CUDA(cudaEventRecord(e1, stream));
        VLT_CUDA(cudaEventSynchronize(e1));
        float ms = 0;
        VLT_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        best = std::min(best, double(ms) * 1e-3);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    VLT_CUDA(cudaMemcpy(out, o, size_t(streams) * 12, cudaMemcpyDeviceToHost));
    return best;
}

// drafter.rs:420-447 runs draft_top and draft_tree on its block's logits; here they run on logits the caller supplies.
void Engine::draft_trees(const float* logits, uint32_t n_rows, uint32_t nv, const uint32_t* vocab_ids, const uint32_t* tin, const uint32_t* blocks, const uint32_t* slots,
                         uint32_t n_blocks, float inv_t, uint32_t ncand, uint32_t* cand, float* cand_q, uint32_t* feed, uint32_t* tree) {
    if (cfg.host_only) throw Error("this engine was created host-only: it cannot run kernels");
    if (n_rows == 0 || nv == 0 || ncand == 0 || ncand > 4) throw Error("draft_trees: needs rows, a vocabulary and 1..4 candidates");
    for (uint32_t b = 0; b < n_blocks; b++) {
        if (slots[b] >= cfg.max_seqs) throw Error("draft_trees: slot out of range");
        if (blocks[2 * b + 1] == 0 || blocks[2 * b + 1] > VERIFY_T || blocks[2 * b] + blocks[2 * b + 1] > n_rows) throw Error("draft_trees: block out of the rows given");
    }
    Buffer d_logits, d_ids, d_tin, d_blocks, d_slots, d_cand, d_q;
    if (tin) { d_tin.alloc(size_t(n_rows) * 8, false); d_tin.write(0, tin, size_t(n_rows) * 8); }
    d_logits.alloc(size_t(n_rows) * nv * 4, false);
    d_logits.write(0, logits, size_t(n_rows) * nv * 4);
    if (vocab_ids) { d_ids.alloc(size_t(nv) * 4, false); d_ids.write(0, vocab_ids, size_t(nv) * 4); }
    d_cand.alloc(size_t(n_rows) * 16, false);
    d_q.alloc(size_t(n_rows) * 16, false);
    VLT_CUDA(cudaMemsetAsync(d_cand.dev, 0, size_t(n_rows) * 16, stream));
    VLT_CUDA(cudaMemsetAsync(d_q.dev, 0, size_t(n_rows) * 16, stream));
    launch_draft_top(d_logits.as<float>(), n_rows, nv, vocab_ids ? d_ids.as<uint32_t>() : nullptr, tin ? d_tin.as<uint32_t>() : nullptr, inv_t, ncand,
                     d_cand.as<uint32_t>(), d_q.as<float>(), stream);
    if (n_blocks) {
        d_blocks.alloc(size_t(n_blocks) * 8, false);
        d_blocks.write(0, blocks, size_t(n_blocks) * 8);
        d_slots.alloc(size_t(n_blocks) * 4, false);
        d_slots.write(0, slots, size_t(n_blocks) * 4);
        launch_draft_tree(d_blocks.as<uint32_t>(), d_slots.as<uint32_t>(), n_blocks, d_cand.as<uint32_t>(), d_q.as<float>(), ncand, s.feed.as<uint32_t>(),
                          s.tree.as<uint32_t>(), stream);
    }
    VLT_CUDA(cudaStreamSynchronize(stream));
    d_cand.read(0, cand, size_t(n_rows) * 16);
    d_q.read(0, cand_q, size_t(n_rows) * 16);
    s.feed.read(0, feed, size_t(cfg.max_seqs) * FEED_W * 4);
    s.tree.read(0, tree, size_t(cfg.max_seqs) * FEED_W * 4);
}

// engine/src/engine/hooks.rs:56-111 `bench_matmul`.
void Engine::bench_matmul(const std::string& kind, uint32_t n, uint32_t variant, uint32_t reps, double* seconds, uint64_t* bytes) {
    if (cfg.host_only) throw Error("this engine was created host-only: it cannot run kernels");
    const bool head = kind == "head";
    if (!head && kind != "qkv" && kind != "o" && kind != "gate_up" && kind != "down") throw Error("unknown matmul " + kind);
    if (n == 0 || n > (head ? cfg.max_head_rows : cfg.max_step_tokens)) throw Error(kind + " can't take " + std::to_string(n) + " tokens");
    cudaEvent_t e0, e1;
    VLT_CUDA(cudaEventCreate(&e0));
    VLT_CUDA(cudaEventCreate(&e1));
    double best = 1e30;
    for (uint32_t r = 0; r < std::max(reps, 1u); r++) {
        VLT_CUDA(cudaEventRecord(e0, stream));
        const bool gemm = variant != 1 && use_gemm(head ? model.head : model.layers[0].o, n);
        if (variant == 2 && !gemm) throw Error(kind + ": the tensor-core GEMM can't take " + std::to_string(n) + " tokens");
        if (head) {
            if (gemm) matmul_gemm(model.head, n, s.hfin_b.as<uint16_t>(), s.logits.as<float>(), nullptr, EPI_HEAD, nullptr, s.inv_head.as<float>());
            else matmul(model.head, n, s.hfin_head.as<float>(), s.logits.as<float>(), EPI_HEAD, nullptr, nullptr);
        } else {
            for (const Layer& l : model.layers) {
                if (gemm) {
                    if (kind == "qkv") matmul_gemm(l.qkv, n, s.h_b.as<uint16_t>(), s.qkv.as<float>(), nullptr, EPI_NORM, nullptr, s.inv.as<float>());
                    else if (kind == "o") matmul_gemm(l.o, n, s.attn_b.as<uint16_t>(), s.hfin_all.as<float>(), nullptr, EPI_RESID, s.h.as<float>(), nullptr);
                    else if (kind == "gate_up") matmul_gemm(l.gate_up, n, s.h_b.as<uint16_t>(), nullptr, s.act_b.as<uint16_t>(), EPI_SWIGLU, nullptr, s.inv.as<float>());  // the down GEMM reads the bf16 copy only
                    else matmul_gemm(l.down, n, s.act_b.as<uint16_t>(), s.hfin_all.as<float>(), nullptr, EPI_RESID, s.h.as<float>(), nullptr);
                } else {
                    if (kind == "qkv") matmul(l.qkv, n, s.h.as<float>(), s.qkv.as<float>(), EPI_NORM, nullptr, s.inv.as<float>());
                    else if (kind == "o") matmul(l.o, n, s.attn.as<float>(), s.hfin_all.as<float>(), EPI_RESID, s.h.as<float>(), nullptr);
                    else if (kind == "gate_up") matmul(l.gate_up, n, s.h.as<float>(), s.act.as<float>(), EPI_SWIGLU, nullptr, nullptr);
                    else matmul(l.down, n, s.act.as<float>(), s.hfin_all.as<float>(), EPI_RESID, s.h.as<float>(), nullptr);
                }
            }
        }
        VLT_CUDA(cudaEventRecord(e1, stream));
        VLT_CUDA(cudaEventSynchronize(e1));
        float ms = 0;
        VLT_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        best = std::min(best, double(ms) * 1e-3);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *seconds = best;
    uint64_t b = 0;
    if (head) b = model.head.bytes();
    else
        for (const Layer& l : model.layers) b += kind == "qkv" ? l.qkv.bytes() : kind == "o" ? l.o.bytes() : kind == "gate_up" ? l.gate_up.bytes() : l.down.bytes();
    *bytes = b;
}

cudaEvent_t Engine::pooled_event() {
    if (!event_pool.empty()) {
        cudaEvent_t e = event_pool.back();
        event_pool.pop_back();
        return e;
    }
    cudaEvent_t e;
    VLT_CUDA(cudaEventCreate(&e));
    return e;
}

int Engine::span_begin(int group) {
    if (!profile || span_open_outer) return -1;
    if (group == G_DRAFTER) span_open_outer = true;
    Span sp{pooled_event(), pooled_event(), group, uint32_t(launch_counter())};
    VLT_CUDA(cudaEventRecord(sp.a, stream));
    spans.push_back(sp);
    return int(spans.size()) - 1;
}

void Engine::span_end(int idx) {
    if (idx < 0) return;
    Span& sp = spans[idx];
    if (sp.group == G_DRAFTER) span_open_outer = false;
    VLT_CUDA(cudaEventRecord(sp.b, stream));
    sp.launches = uint32_t(launch_counter()) - sp.launches;
}

void Engine::profile_read(double* ms, uint32_t* launches) {
    VLT_CUDA(cudaStreamSynchronize(stream));
    for (int g = 0; g < G_COUNT; g++) { ms[g] = 0; launches[g] = 0; }
    for (Span& sp : spans) {
        float t = 0;
        VLT_CUDA(cudaEventElapsedTime(&t, sp.a, sp.b));
        ms[sp.group] += t;
        launches[sp.group] += sp.launches;
        event_pool.push_back(sp.a);
        event_pool.push_back(sp.b);
    }
    spans.clear();
    span_open_outer = false;
}

void Engine::mark(int which) {
    if (which < 0 || which > 1) throw Error("mark 0 or 1");
    if (!marks[which]) VLT_CUDA(cudaEventCreate(&marks[which]));
    VLT_CUDA(cudaEventRecord(marks[which], stream));
}

double Engine::mark_elapsed_ms() {
    if (!marks[0] || !marks[1]) throw Error("both marks must be set");
    VLT_CUDA(cudaEventSynchronize(marks[1]));
    float t = 0;
    VLT_CUDA(cudaEventElapsedTime(&t, marks[0], marks[1]));
    return t;
}

// Named views for parity tests.
std::vector<uint32_t> Engine::debug_read(const std::string& name) {
    if (!cfg.host_only) VLT_CUDA(cudaStreamSynchronize(stream));
    const size_t ms = cfg.max_seqs;
    auto whole = [&](const Buffer& b, size_t words) { return b.read_vec<uint32_t>(0, words); };
    if (name == "lens") return whole(s.lens, ms);
    if (name == "feed") return whole(s.feed, ms * FEED_W);
    if (name == "tree") return whole(s.tree, ms * FEED_W);
    if (name == "gen") return whole(s.gen, ms * sizeof(GenState) / 4);
    if (name == "path") return whole(s.path, ms * FEED_W);
    if (name == "path_len") return whole(s.path_len, ms);
    if (name == "on_path") return whole(s.on_path, last_plan_n);
    if (name == "trace_len") return whole(s.trace_len, ms);
    if (name == "meta") return whole(s.meta, 2 * size_t(last_plan_n));
    if (name == "page_table") return whole(kv.page_table, ms * kv.max_pages);
    if (name == "free_pages") return kv.free_pages;
    if (name == "attn_split") return {last_split[0], last_split[1]};
    if (name == "k_cache") return whole(kv.k, kv.k.bytes / 4);  // bf16 pairs; small pools only
    if (name == "v_cache") return whole(kv.v, kv.v.bytes / 4);
    if (drafter) {
        const size_t pool = size_t(kv.n_pages) * model.md.n_kv * kv.page * model.md.hd;
        if (name == "draft_logits") return whole(drafter->logits, size_t(VERIFY_T - 1) * ms * drafter->v);  // [pass][run slot][v] f32
        if (name == "carry") return whole(drafter->carry, ms * model.md.d);
        if (name == "q_rows") return whole(drafter->q_rows, ms);
        if (name == "q_keep") return whole(drafter->q_keep, ms * (VERIFY_T - 1) * size_t(drafter->v));
        if (name == "draft_k_cache") return whole(drafter->k, pool / 2);  // bf16 pairs
        if (name == "draft_v_cache") return whole(drafter->v_cache, pool / 2);
    }
    if (lim) {
        if (name == "limite_k_local") return whole(lim->k_local, lim->k_local.bytes / 4);  // bf16 pairs
        if (name == "limite_v_local") return whole(lim->v_local, lim->v_local.bytes / 4);
    }
    if (block_drafter) {
        const BlockDrafter& b = *block_drafter;
        if (name == "block_logits") return whole(b.logits, size_t(b.last_rows) * b.v);  // [block row][v] f32
        if (name == "block_hfin") return whole(b.hfin, size_t(b.last_rows) * b.dims.hidden);
        if (name == "block_ctx_ring") return whole(b.ctx_ring, b.ctx_ring.bytes / 4);
        if (name == "block_k_ring") return whole(b.k_ring, b.k_ring.bytes / 4);  // bf16 pairs
        if (name == "block_v_ring") return whole(b.v_ring, b.v_ring.bytes / 4);
    }
    const StepSet& st = sets[0];
    auto in = [&](size_t off, size_t words) {
        std::vector<uint32_t> v(words);
        if (cfg.host_only) std::memcpy(v.data(), st.host_in + off, words * 4);
        else st.dev_in.read(off, v.data(), words * 4);
        return v;
    };
    const size_t n = last_plan_n;
    if (name == "tokens") return in(st.o_tokens, n);
    if (name == "tin") return in(st.o_tin, 2 * n);
    if (name == "vis") return in(st.o_vis, n);
    if (name == "head_rows") return in(st.o_head_rows, cfg.max_head_rows);
    if (name == "hidden_rows") return in(st.o_hidden_rows, n);
    if (name == "sample_rows") return in(st.o_sample_rows, cfg.max_head_rows * 6);
    if (name == "tiles") return in(st.o_tiles, 2 * (cfg.max_step_tokens / 8 + ms + 1));
    if (name == "runs") return in(st.o_runs, ms * 6);
    if (name == "out_ids") return st.dev_out.read_vec<uint32_t>(st.o_out_ids / 4, cfg.max_head_rows);
    if (name == "emitted") return st.dev_out.read_vec<uint32_t>(st.o_emitted / 4, ms);
    throw Error("no engine array named " + name);
}

void Engine::debug_write(const std::string& name, size_t index, const uint32_t* data, size_t n) {
    if (!cfg.host_only) VLT_CUDA(cudaStreamSynchronize(stream));
    Buffer* b = name == "lens" ? &s.lens : name == "feed" ? &s.feed : name == "tree" ? &s.tree : name == "gen" ? &s.gen : nullptr;
    if (!b) throw Error("engine array " + name + " is not writable");
    b->write(index * 4, data, n * 4);
}

}  // namespace vlt

#ifdef VLT_STEP_PROBE
extern "C" void vlt_sp_dump_all() { cudaDeviceSynchronize(); for (auto f : vlt::sp_registry()) f(); }
#endif
