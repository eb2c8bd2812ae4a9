#include "generator.h"

#include <algorithm>
#include <chrono>

namespace vlt {

Generator::Generator(Engine& e) : eng(e) {
    // engine/src/engine/generate.rs:155-162.
    const EngineConfig& c = eng.cfg;
    if (c.max_step_tokens < c.max_seqs || c.max_head_rows < c.max_seqs)
        throw Error("generation needs max_step_tokens (" + std::to_string(c.max_step_tokens) + ") and max_head_rows (" + std::to_string(c.max_head_rows) +
                    ") of at least max_seqs (" + std::to_string(c.max_seqs) + ")");
}

// engine/src/engine/generate.rs:503-518 (Drop): waits for the step in flight, frees every sequence it holds.
Generator::~Generator() {
    try {
        if (in_flight) eng.wait(in_flight->set);
    } catch (...) {
    }
    for (Active& a : active) eng.free_seq(a.seq);
    for (Queued& q : queue)
        if (q.req.resume) eng.free_seq(q.req.resume_seq);
}

// engine/src/engine/generate.rs:185-243 `submit`.
uint32_t Generator::submit(const Request& req) {
    const EngineConfig& c = eng.cfg;
    const uint32_t vocab = eng.model.md.vocab;
    req.sampling.check();
    if (req.stop.size() > MAX_STOP) throw Error(std::to_string(req.stop.size()) + " stop tokens (max " + std::to_string(MAX_STOP) + ")");
    const uint32_t rows = req.draft_rows();
    if (rows == 0 || rows > std::min({FEED_W, c.max_chunk, c.max_head_rows}))
        throw Error(std::to_string(rows) + " rows per step (max " + std::to_string(FEED_W) + ", max_chunk and max_head_rows)");
    if (req.draft == DraftKind::Replay) {
        if (req.trace.size() > c.max_seq_len || std::any_of(req.trace.begin(), req.trace.end(), [&](uint32_t t) { return t >= vocab; }))
            throw Error("replay trace longer than max_seq_len, or with ids out of range");
    }
    if (req.draft == DraftKind::Model) {
        if (!eng.has_drafter() || rows > VERIFY_T) throw Error("Draft::Model needs a loaded drafter and at most " + std::to_string(VERIFY_T) + " rows");
    }
    if ((req.draft == DraftKind::Replay || req.draft == DraftKind::Model) && rows > VERIFY_T)
        throw Error(std::to_string(rows) + " rows per step: a verify run takes at most " + std::to_string(VERIFY_T));
    uint32_t len;
    if (!req.resume) {
        if (req.prompt.empty()) throw Error("empty prompt");
        if (std::any_of(req.prompt.begin(), req.prompt.end(), [&](uint32_t t) { return t >= vocab; })) throw Error("token id out of range");
        len = uint32_t(req.prompt.size());
    } else {
        if (req.resume_token >= vocab) throw Error("token id out of range");
        const bool queued = std::any_of(queue.begin(), queue.end(), [&](const Queued& q) { return q.req.resume && q.req.resume_seq == req.resume_seq; });
        if (queued || std::any_of(active.begin(), active.end(), [&](const Active& a) { return a.seq == req.resume_seq; }))
            throw Error("sequence " + std::to_string(req.resume_seq) + " is already generating");
        if (req.resume_seq >= eng.seqs.size() || !eng.seqs[req.resume_seq]) throw Error("unknown sequence");
        len = eng.seqs[req.resume_seq]->len + 1;
    }
    if (req.max_tokens == 0) throw Error("max_tokens is 0");
    const uint64_t kv_len = uint64_t(len) + req.max_tokens - 1;
    const uint32_t page = eng.kv.page;
    // With a drafter loaded a step reserves pages VERIFY_T positions past itself (the draft passes write their own
    // K/V there, Engine::plan), so the pool is budgeted for that reach; the reference reserves to the step's end
    // only (plan.rs:75) and budgets kv_len (generate.rs:237).
    const uint64_t reach = eng.has_drafter() ? std::min<uint64_t>(kv_len + VERIFY_T, c.max_seq_len) : kv_len;
    if (kv_len > c.max_seq_len || (reach + page - 1) / page > eng.kv.n_pages)
        throw Error("a request reaching " + std::to_string(kv_len) + " positions doesn't fit max_seq_len or the KV pool");
    const uint32_t id = submitted++;
    queue.push_back(Queued{id, req, uint32_t(reach)});
    return id;
}

// engine/src/engine/generate.rs:259-267.
void Generator::cancel(uint32_t id) {
    auto q = std::find_if(queue.begin(), queue.end(), [&](const Queued& x) { return x.id == id; });
    if (q != queue.end()) {
        if (q->req.resume) eng.free_seq(q->req.resume_seq);
        queue.erase(q);
        return;
    }
    for (Active& a : active)
        if (a.id == id) a.done = true;
}

// engine/src/engine/generate.rs:271-280.
std::vector<Event> Generator::step() {
    admit();
    std::optional<InFlight> next = encode_next();
    std::vector<Event> events;
    std::optional<InFlight> prev = std::move(in_flight);
    in_flight = std::move(next);
    if (prev) collect(*prev, events);
    release();
    return events;
}

// engine/src/engine/generate.rs:284-337: queued requests start, in order, while a slot is free and
// the KV pool can hold them at their longest beside the running ones.
void Generator::admit() {
    const uint32_t page = eng.kv.page;
    auto pages_of = [&](uint32_t kv_len) { return (kv_len + page - 1) / page; };
    while (!queue.empty()) {
        const Queued& q = queue.front();
        auto held = [&](uint32_t seq) { return seq < eng.seqs.size() && eng.seqs[seq] ? uint32_t(eng.seqs[seq]->pages.size()) : 0u; };
        uint64_t growth = 0;
        for (const Active& a : active) growth += pages_of(a.kv_len) > held(a.seq) ? pages_of(a.kv_len) - held(a.seq) : 0;
        bool slot_free;
        uint32_t need;
        if (!q.req.resume) {
            slot_free = std::any_of(eng.seqs.begin(), eng.seqs.end(), [](const std::optional<Seq>& s) { return !s; });
            need = pages_of(q.kv_len);
        } else {
            slot_free = true;
            const uint32_t h = held(q.req.resume_seq);
            need = pages_of(q.kv_len) > h ? pages_of(q.kv_len) - h : 0;
        }
        if (!slot_free || eng.kv.free_pages.size() < growth + need) {
            if (active.empty() && !in_flight) throw Error("request " + std::to_string(q.id) + " can't start: no free slot or KV pages, and nothing running");
            return;
        }
        Queued item = std::move(queue.front());
        queue.pop_front();
        Active a;
        a.id = item.id;
        if (!item.req.resume) {
            a.seq = eng.new_seq();
            a.feed = item.req.prompt;
        } else {
            a.seq = item.req.resume_seq;
            a.feed = {item.req.resume_token};
        }
        eng.set_sampling(a.seq, item.req.sampling);
        // No step in flight uses the slot (a new one, or a resumed idle sequence).
        GenState gs = gen_open();
        gs.remaining = item.req.max_tokens;
        gs.nstop = uint32_t(item.req.stop.size());
        for (size_t i = 0; i < item.req.stop.size(); i++) gs.stop[i] = item.req.stop[i];
        eng.set_gen(a.seq, gs);
        a.rows = item.req.draft_rows();
        a.model = item.req.draft == DraftKind::Model;
        a.replay = item.req.draft == DraftKind::Replay;
        eng.set_trace(a.seq, item.req.trace.data(), a.replay ? uint32_t(item.req.trace.size()) : 0);
        a.max_tokens = item.req.max_tokens;
        a.stop = item.req.stop;
        a.kv_len = item.kv_len;
        active.push_back(std::move(a));
    }
}

// engine/src/engine/generate.rs:341-444: a run for every decoding request, then prompt chunks in
// the order the requests started; plans, queues and commits the step.
std::optional<Generator::InFlight> Generator::encode_next() {
    const EngineConfig& cfg = eng.cfg;
    const uint64_t step = steps;
    uint32_t budget = cfg.max_step_tokens;
    auto decoding = [&](const Active& a) { return !hold && !a.done && a.fed == a.feed.size() && a.received + a.inflight < a.max_tokens; };
    uint32_t n_dec = 0;
    uint64_t kv = 0;
    for (const Active& a : active)
        if (decoding(a)) { n_dec++; kv += eng.seq_len(a.seq); }
    const uint32_t nd = std::max(n_dec, 1u);
    const uint32_t row_cap = std::max(std::min(cfg.max_step_tokens, cfg.max_head_rows) / nd, 1u);
    const Tuning& t = eng.tuning;
    const uint32_t short_cap = std::max(t.spec_tokens_short / nd, 2u);
    uint32_t spec_cap;
    if (t.spec_tokens == 0) spec_cap = 0xffffffffu;
    else if (kv < t.spec_kv) spec_cap = short_cap;
    else spec_cap = std::max(short_cap, std::min(std::max(t.spec_tokens / nd, 2u), std::max(t.spec_rows_long, 2u)));

    struct Pick { size_t active; bool cpu; uint32_t from, to, rows; bool draws; };
    std::vector<Pick> picks;
    for (size_t i = 0; i < active.size(); i++) {
        Active& a = active[i];
        if (!decoding(a)) continue;
        // Every row may emit a token: stay within max_tokens.
        const uint32_t rows = std::min({a.rows, row_cap, spec_cap, a.max_tokens - a.received - a.inflight});
        picks.push_back(Pick{i, false, 0, 0, rows, true});
        a.inflight += rows;
        a.last_step = step;
        budget -= rows;
    }
    for (size_t i = 0; i < active.size(); i++) {
        Active& a = active[i];
        if (budget > 0 && a.fed < a.feed.size()) {
            const uint32_t k = std::min({uint32_t(a.feed.size()) - a.fed, cfg.max_chunk, budget});
            const bool draws = a.fed + k == a.feed.size();
            picks.push_back(Pick{i, true, a.fed, a.fed + k, k, draws});
            a.fed += k;
            a.inflight += draws ? 1 : 0;
            a.last_step = step;
            budget -= k;
        }
    }
    if (picks.empty()) return std::nullopt;
    static const std::array<uint32_t, FEED_W> feed_rows = [] { std::array<uint32_t, FEED_W> r{}; for (uint32_t i = 0; i < FEED_W; i++) r[i] = FEED_ROW + i; return r; }();
    std::vector<PlanRun> runs;
    for (const Pick& p : picks) {
        const Active& a = active[p.active];
        PlanRun r;
        r.seq = a.seq;
        r.tokens = p.cpu ? a.feed.data() + p.from : feed_rows.data();
        r.count = p.rows;
        r.head = p.draws ? Rows::Last : Rows::None;
        r.verify = !p.cpu && p.rows > 1;
        runs.push_back(r);
    }
    InFlight f;
    uint32_t head0 = 0;
    for (size_t run = 0; run < picks.size(); run++) {
        if (!picks[run].draws) continue;
        const Active& a = active[picks[run].active];
        const uint32_t verify = runs[run].verify ? picks[run].rows : 0;
        f.drawn.push_back(Drawn{a.id, a.seq, uint32_t(run), runs[run].count, head0, verify});
        head0 += std::max(verify, 1u);
    }
    const bool replay = std::any_of(active.begin(), active.end(), [](const Active& a) { return a.rows > 1 && a.replay; });
    const bool modeled = std::any_of(active.begin(), active.end(), [](const Active& a) { return a.model; });
    const uint32_t set = uint32_t(step % 3);
    const Plan plan = eng.plan(set, runs, Rows::None);
    const auto t0 = std::chrono::steady_clock::now();
    eng.encode_forward(set, plan);
    if (modeled) {
        uint32_t drows = 1;
        for (const Active& a : active)
            if (a.model) drows = std::max(drows, std::min(a.rows, VERIFY_T));
        eng.encode_drafter(set, plan, drows);
    }
    if (replay) eng.encode_replay(set, plan, ReplayArgs{cfg.max_seq_len, replay_seed, replay_rate, eng.model.md.vocab_real});
    eng.commit(set);
    f.set = set;
    f.step = step;
    f.stats.tokens = plan.n;
    f.stats.decode = plan.max_run <= VERIFY_T;
    f.stats.encode_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    steps++;
    return f;
}

// engine/src/engine/generate.rs:446-487 `collect`.
void Generator::collect(const InFlight& f, std::vector<Event>& events) {
    const double gpu_seconds = eng.wait(f.set);
    eng.check_device_error(f.set);
    const size_t before = events.size();
    collected = f.step;
    const StepSet& st = eng.sets[f.set];
    const uint32_t* ids = st.hout<uint32_t>(st.o_out_ids);
    const uint32_t* emitted = st.hout<uint32_t>(st.o_emitted);
    for (const Drawn& d : f.drawn) {
        const uint32_t e = emitted[d.run];
        // The plan advanced the sequence by its whole run: a verify run advances by what it
        // emits, and a slot already done on the GPU not at all.
        if (d.verify > 0) eng.settle(d.seq, d.count - e);
        else if (e == 0) eng.settle(d.seq, d.count);
        auto it = std::find_if(active.begin(), active.end(), [&](const Active& a) { return a.id == d.id; });
        if (it == active.end()) throw Error("a drawing request is not active");
        Active& a = *it;
        a.inflight -= std::max(d.verify, 1u);
        if (a.done) continue;
        for (uint32_t j = 0; j < e; j++) {
            const uint32_t tok = ids[d.head0 + j];
            a.received++;
            events.push_back(Event{EventKind::Token, d.id, tok});
            Finish fin;
            if (std::find(a.stop.begin(), a.stop.end(), tok) != a.stop.end()) fin = Finish::Stop;
            else if (a.received == a.max_tokens) fin = Finish::Length;
            else continue;
            a.done = true;
            events.push_back(Event{EventKind::Done, d.id, uint32_t(fin)});
            break;
        }
    }
    StepStats s = f.stats;
    s.gpu_seconds = gpu_seconds;
    s.emitted = 0;
    for (size_t i = before; i < events.size(); i++) s.emitted += events[i].kind == EventKind::Token ? 1 : 0;
    stats.push_back(s);
}

// engine/src/engine/generate.rs:490-500: frees the sequences of finished requests that no step in flight uses.
void Generator::release() {
    auto keep = std::remove_if(active.begin(), active.end(), [&](const Active& a) {
        const bool free_it = a.done && (!a.last_step || (collected && *a.last_step <= *collected));
        if (free_it) eng.free_seq(a.seq);
        return free_it;
    });
    active.erase(keep, active.end());
}

}  // namespace vlt
