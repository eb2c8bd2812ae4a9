// Continuous batching over an engine, pipelined: the CPU plans and queues step t+1 while the
// GPU runs step t, and collects each step's results one step behind. Mirrors the reference's
// `Generator` (engine/src/engine/generate.rs).
#pragma once
#include <deque>
#include <optional>
#include <vector>

#include "engine.h"

namespace vlt {

enum class DraftKind : uint32_t { None = 0, Replay = 1, Model = 2 };

// engine/src/engine/generate.rs:12-61.
struct Request {
    bool resume = false;
    std::vector<uint32_t> prompt;  // !resume
    uint32_t resume_seq = 0, resume_token = 0;
    uint32_t max_tokens = 0;
    std::vector<uint32_t> stop;
    Sampling sampling;
    DraftKind draft = DraftKind::None;
    uint32_t rows = 1;
    std::vector<uint32_t> trace;
    uint32_t draft_rows() const { return draft == DraftKind::None ? 1 : rows; }
};

enum class EventKind : uint32_t { Token = 0, Done = 1 };
enum class Finish : uint32_t { Stop = 0, Length = 1 };
struct Event {
    EventKind kind;
    uint32_t req;
    uint32_t value;
};

// engine/src/engine/generate.rs:81-91.
struct StepStats {
    uint32_t tokens = 0;
    bool decode = false;
    uint32_t emitted = 0;
    double gpu_seconds = 0, encode_seconds = 0;
};

class Generator {
  public:
    explicit Generator(Engine& e);
    ~Generator();
    uint32_t submit(const Request& req);
    void cancel(uint32_t id);
    std::vector<Event> step();
    bool is_idle() const { return queue.empty() && active.empty() && !in_flight; }
    bool has_step_in_flight() const { return in_flight.has_value(); }
    void counts(uint32_t* queued, uint32_t* running) const { *queued = uint32_t(queue.size()); *running = uint32_t(active.size()); }
    void set_replay_mistakes(float rate, uint32_t seed) { replay_rate = rate; replay_seed = seed; }
    std::vector<StepStats> stats;
    bool hold = false;
    Engine& eng;

  private:
    struct Queued { uint32_t id; Request req; uint32_t kv_len; };  // kv_len: the furthest position the request's steps reserve pages for
    struct Active {
        uint32_t id, seq;
        std::vector<uint32_t> feed;  // tokens the CPU feeds: the prompt, or the resumed token
        uint32_t fed = 0, max_tokens = 0;
        std::vector<uint32_t> stop;
        uint32_t kv_len = 0, rows = 1;
        bool model = false, replay = false;
        uint32_t received = 0, inflight = 0;
        bool done = false;
        std::optional<uint64_t> last_step;
    };
    struct Drawn { uint32_t id, seq, run, count, head0, verify; };
    struct InFlight { uint32_t set; uint64_t step; std::vector<Drawn> drawn; StepStats stats; };

    void admit();
    std::optional<InFlight> encode_next();
    void collect(const InFlight& f, std::vector<Event>& events);
    void release();

    std::deque<Queued> queue;
    std::vector<Active> active;
    std::optional<InFlight> in_flight;
    uint32_t submitted = 0;
    uint64_t steps = 0;
    std::optional<uint64_t> collected;
    float replay_rate = 0.0f;
    uint32_t replay_seed = 0;
};

}  // namespace vlt
