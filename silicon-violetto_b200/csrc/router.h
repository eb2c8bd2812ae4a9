// Streams sharded over independent replicas (one engine + generator per GPU, no exchange between them), with the
// streams of a replica that fails re-queued on the others.
//
// Not in the reference, which runs one engine on one device and exits when it fails (cli/src/serve.rs:147-150); the
// replicas it would be sharded into each keep the reference's Generator interface (engine/src/engine/generate.rs), which
// is all the router uses -- through a table of functions, so that a replica can be a generator of this library or a
// stand-in on the host in tests.
//
// A request that moves continues where it was: its new prompt is the old one plus the tokens it had emitted, its budget
// what is left. Because a sequence's draws are keyed by (seed, position) (engine/src/engine.rs:100-102), the moved
// request goes on with the very tokens it would have produced on the replica that failed.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <vector>

#include "../../include/violetto.h"
#include "common.h"

namespace vlt {

class Router {
  public:
    explicit Router(std::vector<VltReplicaOps> replicas);
    uint32_t submit(const VltRequest& req);
    void cancel(uint32_t id);
    // One step of every live replica; the events of all of them, with the router's request ids.
    std::vector<VltEvent> step();
    bool is_idle() const;
    uint32_t alive() const;
    bool replica_alive(uint32_t i) const { return i < reps_.size() && reps_[i].alive; }
    uint32_t replica_of(uint32_t id) const;  // NO_TOK if the request is finished or unknown
    const std::string& last_failure() const { return last_failure_; }

  private:
    struct Replica {
        VltReplicaOps ops;
        bool alive = true;
    };
    // A request as the router keeps it: everything needed to submit it again elsewhere.
    struct Job {
        uint32_t id = 0;
        std::vector<uint32_t> prompt, stop, trace, emitted;
        VltRequest shape{};  // the scalar fields (pointers are filled in from the vectors at submission)
        uint32_t replica = NO_TOK, local = 0;
        bool resume = false, done = false;
    };
    uint32_t pick() const;
    void place(Job& j);        // submits j to the least-loaded live replica
    void fail(uint32_t r, const std::string& why, std::vector<VltEvent>& out);
    std::vector<Replica> reps_;
    std::deque<Job> jobs_;  // unfinished requests, oldest first
    uint32_t next_id_ = 0;
    std::string last_failure_;
};

}  // namespace vlt
