#include "router.h"

#include <algorithm>

namespace vlt {

Router::Router(std::vector<VltReplicaOps> replicas) {
    if (replicas.empty()) throw Error("a router needs at least one replica");
    for (const VltReplicaOps& o : replicas) {
        if (!o.submit || !o.step || !o.is_idle || !o.counts) throw Error("a replica needs submit, step, is_idle and counts");
        reps_.push_back(Replica{o, true});
    }
}

uint32_t Router::alive() const {
    return uint32_t(std::count_if(reps_.begin(), reps_.end(), [](const Replica& r) { return r.alive; }));
}

bool Router::is_idle() const { return jobs_.empty(); }

uint32_t Router::replica_of(uint32_t id) const {
    for (const Job& j : jobs_)
        if (j.id == id) return j.replica;
    return NO_TOK;
}

// The live replica with the fewest requests queued or running (the lowest index among equals): with equal requests
// this deals the streams out round-robin, which is how the benchmark shards them.
uint32_t Router::pick() const {
    uint32_t best = NO_TOK, best_load = 0;
    for (uint32_t i = 0; i < reps_.size(); i++) {
        if (!reps_[i].alive) continue;
        uint32_t queued = 0, running = 0;
        reps_[i].ops.counts(reps_[i].ops.ctx, &queued, &running);
        if (best == NO_TOK || queued + running < best_load) {
            best = i;
            best_load = queued + running;
        }
    }
    if (best == NO_TOK) throw Error("no replica is alive" + (last_failure_.empty() ? std::string() : " (last failure: " + last_failure_ + ")"));
    return best;
}

void Router::place(Job& j) {
    // A replica that refuses the request (it does not fit its pool, say) is not a failed replica: the error is the caller's.
    const uint32_t r = pick();
    VltRequest q = j.shape;
    std::vector<uint32_t> prompt = j.prompt;
    prompt.insert(prompt.end(), j.emitted.begin(), j.emitted.end());
    q.prompt_tokens = prompt.data();
    q.n_prompt = uint32_t(prompt.size());
    q.max_tokens = j.shape.max_tokens - uint32_t(j.emitted.size());
    q.stop = j.stop.data();
    q.n_stop = uint32_t(j.stop.size());
    q.trace = j.trace.data();
    q.n_trace = uint32_t(j.trace.size());
    uint32_t local = 0;
    if (reps_[r].ops.submit(reps_[r].ops.ctx, &q, &local) != 0) throw Error(std::string("replica ") + std::to_string(r) + " refused the request: " + vlt_last_error());
    j.replica = r;
    j.local = local;
}

uint32_t Router::submit(const VltRequest& req) {
    Job j;
    j.id = next_id_;
    j.shape = req;
    j.resume = req.prompt_kind == VLT_PROMPT_RESUME;
    if (j.resume) throw Error("a router takes token prompts only: a resumed sequence lives on one replica's engine");
    if (req.n_prompt) j.prompt.assign(req.prompt_tokens, req.prompt_tokens + req.n_prompt);
    if (req.n_stop) j.stop.assign(req.stop, req.stop + req.n_stop);
    if (req.n_trace) j.trace.assign(req.trace, req.trace + req.n_trace);
    place(j);
    jobs_.push_back(std::move(j));
    return next_id_++;
}

void Router::cancel(uint32_t id) {
    for (Job& j : jobs_)
        if (j.id == id && j.replica != NO_TOK && reps_[j.replica].alive && reps_[j.replica].ops.cancel) reps_[j.replica].ops.cancel(reps_[j.replica].ops.ctx, j.local);
}

// Replica r is gone: its unfinished requests go to the others, each continued from what it had emitted. A request
// nothing can take (no replica left, or every one refuses it) ends with VLT_FINISH_FAILED.
void Router::fail(uint32_t r, const std::string& why, std::vector<VltEvent>& out) {
    reps_[r].alive = false;
    last_failure_ = "replica " + std::to_string(r) + ": " + why;
    for (Job& j : jobs_) {
        if (j.replica != r || j.done) continue;
        try {
            if (j.emitted.size() >= j.shape.max_tokens) throw Error("nothing left to generate");
            place(j);
        } catch (const std::exception&) {
            j.done = true;
            out.push_back(VltEvent{VLT_EVENT_DONE, j.id, VLT_FINISH_FAILED});
        }
    }
}

std::vector<VltEvent> Router::step() {
    std::vector<VltEvent> out;
    std::vector<VltEvent> buf(4096);
    for (uint32_t r = 0; r < reps_.size(); r++) {
        if (!reps_[r].alive) continue;
        uint32_t n = 0;
        if (reps_[r].ops.step(reps_[r].ops.ctx, buf.data(), uint32_t(buf.size()), &n) != 0) {
            fail(r, vlt_last_error(), out);
            continue;
        }
        for (uint32_t i = 0; i < n; i++) {
            auto j = std::find_if(jobs_.begin(), jobs_.end(), [&](const Job& x) { return x.replica == r && x.local == buf[i].req && !x.done; });
            if (j == jobs_.end()) continue;  // (a request cancelled or moved away)
            if (buf[i].kind == VLT_EVENT_TOKEN) j->emitted.push_back(buf[i].value);
            else j->done = true;
            out.push_back(VltEvent{buf[i].kind, j->id, buf[i].value});
        }
    }
    jobs_.erase(std::remove_if(jobs_.begin(), jobs_.end(), [](const Job& j) { return j.done; }), jobs_.end());
    if (alive() == 0 && !jobs_.empty()) throw Error("no replica is alive (last failure: " + last_failure_ + ")");
    return out;
}

}  // namespace vlt
