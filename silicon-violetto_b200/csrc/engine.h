// The engine: sequences, the paged KV cache, the step planner and the step's kernel sequence.
// Mirrors the reference's `Engine` (engine/src/engine.rs) with CUDA underneath.
#pragma once
#include <array>
#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "common.h"
#include "kernels.h"
#include "weights.h"

namespace vlt {

// engine/src/engine.rs:31-57.
struct EngineConfig {
    uint32_t max_seqs = 8, max_step_tokens = 512, max_chunk = 512, global_kv_tokens = 65536, max_seq_len = 131072, max_head_rows = 64;
    int device = 0;
    bool host_only = false;
};

// engine/src/engine.rs:59-95, with B200 knobs in place of the Apple-GPU ones.
struct Tuning {
    uint32_t spec_tokens = 32, spec_tokens_short = 8, spec_kv = 24576, spec_rows_long = 4;
    uint32_t sm_count = 0, attn_keys_per_cta = 0, gemm_min_rows = 0;
    bool plain_attention = false;
    bool gemm_unpaired = false;  // the many-tile head GEMM as one block per SM (default: two smaller blocks per SM)
};

// engine/src/engine.rs:100-138.
struct Sampling {
    float temperature = 0.0f, top_p = 1.0f;
    uint64_t seed = 0;
    void check() const;
    SampleRow row_at(uint32_t pos) const { return SampleRow{uint32_t(seed), uint32_t(seed >> 32), pos, temperature, top_p, NO_TOK}; }
    SampleRow row_of(uint32_t tok) const { SampleRow r = row_at(0); r.tok = tok; return r; }
};

enum class Rows : uint32_t { None = 0, Last = 1, All = 2 };

// engine/src/engine/plan.rs:8-18.
struct PlanRun {
    uint32_t seq;
    const uint32_t* tokens;
    uint32_t count;
    Rows head;
    bool verify;
};

// engine/src/engine/plan.rs:20-37.
struct Plan {
    uint32_t n = 0, n_head = 0, n_hidden = 0, n_runs = 0, tiles = 0, max_run = 0;
    bool branches = false;
    bool head_all = false;  // every row of the step goes through the head, in order
    uint32_t ctiles = 0;   // chunk tiles of at most 64 rows (the prefill attention's blocks)
    bool chunked = false;  // some run is longer than VERIFY_T rows: the step's attention is the chunk kernel (encode.rs:299-355)
    uint32_t keys_per_split = 0, max_splits = 1;  // the attention's key split
    uint32_t max_keys = 0;                        // the longest run's keys
};

struct Seq {
    uint32_t len = 0;  // positions with KV; while a speculative step is in flight, the most it can reach
    std::vector<uint32_t> pages;
    Sampling sampling;
};

// engine/src/engine/kv.rs:9-90, every layer paged.
struct KvCache {
    Buffer k, v, page_table;
    std::vector<uint32_t> free_pages;
    uint32_t n_pages = 0, max_pages = 0, page = 16;
    void init(const EngineConfig& cfg, const ModelDesc& md, uint32_t n_layers, bool with_pool);
    void reserve(uint32_t slot, std::vector<uint32_t>& pages, uint32_t len);
    void release(const std::vector<uint32_t>& pages);
};

// One step's inputs in one block of pinned host memory mirrored on the device (one upload
// per step), and its outputs (one download). engine/src/engine/buffers.rs:120-156.
struct StepSet {
    Buffer dev_in, dev_out;
    uint8_t* host_in = nullptr;   // pinned
    uint8_t* host_out = nullptr;  // pinned
    size_t in_bytes = 0, out_bytes = 0;
    size_t o_tokens = 0, o_tin = 0, o_vis = 0, o_head_rows = 0, o_hidden_rows = 0, o_sample_rows = 0, o_tiles = 0, o_runs = 0, o_ctiles = 0;  // byte offsets in *_in
    size_t o_out_ids = 0, o_emitted = 0, o_err = 0;  // in *_out; o_err: the device error word as it stood when the step ended
    cudaEvent_t start = nullptr, done = nullptr;        // around the step on the engine's stream / after its results reached the host
    cudaEvent_t uploaded = nullptr, computed = nullptr;  // the step's inputs are on the device / its last kernel has run
    bool host_only = false;
    void init(const EngineConfig& cfg);
    void release();
    template <typename T> T* in(size_t off) const { return reinterpret_cast<T*>(static_cast<uint8_t*>(dev_in.dev) + off); }
    template <typename T> T* out(size_t off) const { return reinterpret_cast<T*>(static_cast<uint8_t*>(dev_out.dev) + off); }
    template <typename T> T* hin(size_t off) const { return reinterpret_cast<T*>(host_in + off); }
    template <typename T> T* hout(size_t off) const { return reinterpret_cast<T*>(host_out + off); }
};

struct StepOptions {
    Rows head = Rows::Last, hidden = Rows::None;
    bool read_logits = false, read_taps = false;
};
struct StepOutput {
    std::vector<uint32_t> ids;
    std::vector<float> logits, hidden;
    std::vector<uint16_t> taps;  // [tap][token][d]
    double gpu_seconds = 0;
};

// engine/src/engine.rs:175-188 `LayerCapture`: one layer's intermediates over a step, n rows each (host memory, valid
// during the callback). For the plain decoder: resid_in the residual stream entering the layer; attn_in its RMS-normed
// rows; qkv = q | k | v after the folded norm and RoPE (fp32, before the rounding to bf16 and q's softmax scale);
// sdpa_out the attention's output; attn_out the o projection's output before the residual add; mlp_in the RMS-normed
// residual stream after attention; mlp_out the down projection's output before the residual add.
struct LayerCapture {
    uint32_t layer, n;
    const float *resid_in, *attn_in, *qkv, *sdpa_out, *attn_out, *mlp_in, *mlp_out;
};

class Engine {
  public:
    Engine(const std::string& weights, const EngineConfig& cfg, const Tuning& tuning);
    ~Engine();
    Engine(const Engine&) = delete;

    std::string device_name() const;
    void make_current() const;  // the engine's device becomes the calling thread's current one
    uint32_t new_seq();
    void free_seq(uint32_t id);
    uint32_t seq_len(uint32_t id) const;
    void set_sampling(uint32_t id, const Sampling& s);
    void settle(uint32_t id, uint32_t unused);
    StepOutput step(const std::vector<PlanRun>& runs, const StepOptions& opts);
    // The same with each run's own head rows and verify flag, optionally followed by the replay drafter (tests).
    StepOutput step_runs(const std::vector<PlanRun>& runs, const StepOptions& opts, const ReplayArgs* replay);
    void upload_set(uint32_t set);
    void load_drafter(const std::string& path);
    bool has_drafter() const;
    void encode_drafter(uint32_t set, const Plan& p, uint32_t rows);  // after encode_forward: catch-up, then rows - 1 draft passes
    uint32_t debug_draft_rows = 0;  // step_runs runs the drafter for this many rows (tests)
    // Tests of the integer tail on identical inputs: the next step_runs replaces the head's logits ([head rows][vocab]) and
    // the drafter's per-pass logits ([pass][run][v]) by these before anything reads them. Cleared after that step.
    std::vector<float> forced_logits, forced_draft_logits;
    // engine/src/engine.rs:381-389: taps these layers' outputs (bf16(rms_norm(output)), kernels.metal:133-148) from the next step on.
    void set_taps(const std::vector<uint32_t>& layers);
    // engine/src/engine.rs:318-355: a step that stops after every layer and hands its intermediates to `f`.
    StepOutput step_capture(const std::vector<PlanRun>& runs, const StepOptions& opts, const std::function<void(const LayerCapture&)>& f);
    // 0: the reference's acceptance (every row draws the target's token, a draft is accepted if it equals its parent
    // row's draw); 1: rejection sampling for verify runs whose drafts the chain drafter drew from its own distribution.
    void set_acceptance(uint32_t rule);
    uint32_t accept_rule = 0;
    void bench_fill(uint32_t id, uint32_t len, uint32_t seed);
    std::vector<uint32_t> sample_logits(const float* logits, const std::vector<std::pair<Sampling, uint32_t>>& rows);
    // Rejection-sampling acceptance on caller-supplied logits (host pointers); out: 3 x streams words
    // (accepted, token, rollback). Returns the kernels' GPU seconds (best of reps).
    double spec_accept(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, float temperature, const uint64_t* seeds,
                       const uint32_t* pos0, uint32_t reps, uint32_t* out);
    // The reference drafter's draft_top + draft_tree on caller-supplied draft logits [n_rows][nv] (host pointers; a test hook
    // like sample_logits): candidates [n_rows][4] and their probabilities, and per block (first row, rows, slot) the slot's
    // feed[16] / tree[16] rows, which start as the engine's current ones.
    void draft_trees(const float* logits, uint32_t n_rows, uint32_t nv, const uint32_t* vocab_ids, const uint32_t* tin, const uint32_t* blocks, const uint32_t* slots,
                     uint32_t n_blocks, float inv_t, uint32_t ncand, uint32_t* cand, float* cand_q, uint32_t* feed, uint32_t* tree);
    void bench_matmul(const std::string& kind, uint32_t n, uint32_t variant, uint32_t reps, double* seconds, uint64_t* bytes);

    // The generator's building blocks (engine/src/engine/generate.rs uses the same ones).
    Plan plan(uint32_t set, const std::vector<PlanRun>& runs, Rows hidden);
    void encode_forward(uint32_t set, const Plan& p);   // uploads the set, queues the whole step
    void encode_replay(uint32_t set, const Plan& p, const ReplayArgs& ra);
    void commit(uint32_t set);                          // queues the result download and the step's end event
    double wait(uint32_t set);                          // waits for it; GPU seconds of the step
    void set_gen(uint32_t slot, const GenState& g);
    void set_trace(uint32_t slot, const uint32_t* trace, uint32_t n);
    std::vector<uint32_t> debug_read(const std::string& name);
    void debug_write(const std::string& name, size_t index, const uint32_t* data, size_t n);
    void check_device_error(uint32_t set);
    void debug_stalled_wait();  // queues a kernel whose bounded wait runs out: the next collected step must report it

    // Measurement: two stream marks (GPU time between them), and, while `profile` is on, the GPU
    // time of each kernel group of the queued steps (cuda events around the group's launches). The groups are disjoint:
    // the first three are the target's layers, G_TAIL its head, sampling and acceptance, G_DRAFTER everything the
    // drafter runs (its own projections and attention included).
    enum Group : int { G_MATMUL = 0, G_ATTN = 1, G_SMALL = 2, G_TAIL = 3, G_DRAFTER = 4, G_COUNT = 5 };
    void mark(int which);
    double mark_elapsed_ms();
    bool profile = false;
    bool span_open_outer = false;  // a G_DRAFTER span is open: the spans inside it are not recorded
    void profile_read(double* ms, uint32_t* launches);

    Model model;
    EngineConfig cfg;
    Tuning tuning;
    uint32_t sm_count = 148;
    KvCache kv;
    std::vector<std::optional<Seq>> seqs;
    std::array<StepSet, 3> sets;  // three rotate, so the CPU prepares step t+1 while the GPU runs step t
    uint32_t skip = 0;
    std::vector<uint32_t> tap_layers;
    std::vector<Buffer> tap_bufs;  // [max_step_tokens][d] fp32 holding bf16 values, one per tapped layer
    cudaStream_t stream = nullptr;
    // A step's inputs go up and its results come down on streams of their own, so that neither copy sits between the
    // last kernel of one step and the first of the next (the next step is queued while this one runs).
    cudaStream_t copy_in = nullptr, copy_out = nullptr;

    // Activations (engine/src/engine/buffers.rs:14-118) and per-slot state on the GPU.
    struct Scratch {
        Buffer h, qkv, attn, act, part, hfin_head, hfin_all, logits, inv, meta;
        Buffer h_b, attn_b, act_b, hfin_b, inv_head, q_b, ssq;  // ssq: [d / 128][n] sums of squares of h per 128-row tile (see MatArgs)  // bf16 copies that feed the tensor-core GEMM, rows padded to 16
        Buffer lens, feed, tree, gen, path, path_len, on_path, trace, trace_len, err_flag;
    } s;
    Buffer rope_tab;
    Buffer spec_p, spec_q, spec_small;  // spec_accept's device copies, grown on demand
    AttnMaps attn_maps;
    // The chain drafter (a benchmark extension; the reference's drafter.rs is a block drafter): fc over
    // (feature ; embedding), one decoder layer with a cache of its own on the target's page table, a head
    // over a draft vocabulary.
    struct Drafter {
        Weights w;
        Matrix fc, head;
        Layer layer;
        uint32_t v = 0;
        uint32_t window = 0;  // the draft passes' attention window in keys (0: the whole context)
        Buffer vocab_ids, k, v_cache, carry, dfeat, dmeta, dtin, dvis, dcpos, dtiles, live, cpos, logits, hfin, hfin_b, inv;
        // The rejection-sampling rule's state: the q rows a slot's drafts were drawn from, how many are current, the
        // draft vocabulary's inverse map, and the step's scratch (row statistics, sampler skips, settled candidates).
        Buffer q_keep, q_rows, index_of, spec_stats, row_skip, spec_e;
        AttnMaps maps;
    };
    // The reference's own architecture (model.limite): the local layers' rings and the scratch its layers need beyond a
    // plain decoder's (buffers.rs:14-40: hist0 / hist12 / hist23, the MUDD outputs, XSA directions, attention gates).
    static constexpr uint32_t LIMITE_WINDOW = 1024;  // model.rs:18
    struct LimiteState {
        uint32_t ring = 0;
        Buffer k_local, v_local;  // [local layer][slot][kv head][ring][128] bf16
        Buffer hist0, hist12, hist23, xattn, base, mixed, vdir, gates, part;  // part: the attention's partials per (token, head, key split)
    };
    std::unique_ptr<LimiteState> lim;
    LimiteKv limite_kv(const LimiteLayer& x) const;
    void encode_forward_limite(uint32_t set, const Plan& p);
    std::unique_ptr<Drafter> drafter;
    // The reference's block drafter (engine/src/engine/drafter.rs:52-100): a file of tools/spec/export.py's layout, the
    // context's keys and values in rings per (layer, slot), the normed context in a ring per slot, scratch for a step's
    // context and for its block rows.
    struct BlockDrafter {
        Weights w;
        std::vector<Matrix> fc;
        Matrix kv_all, inject, head;
        const float* mask_emb = nullptr;
        struct DLayer {
            Matrix qkv, o, gate_up, down;
            const float* conv_base[4];
            Matrix conv_corr[4];       // [192][H] as the file holds them
            Matrix conv_corr_gemm[4];  // copies padded with zero rows to the GEMM's 128-row tiles
        };
        std::vector<DLayer> layers;
        std::vector<uint32_t> taps;
        uint32_t v = 0, block = 0, ffn = 0;
        BlockDrafterDims dims{};
        Buffer vocab_ids, k_ring, v_ring, ctx_ring;
        Buffer ctx, ctx_inv, kvp;                                                                 // per step token
        Buffer x, last, cx, co, mixed, qkv, inv, attn, act, corr, corr_inv, hfin, logits, cand, cand_q, meta;  // per block row
        Buffer conv_pad;        // the padded correction matrices
        Buffer xb, act_b, attn_b;  // bf16 inputs of the tensor-core GEMM: a row pass's copy of any input, the SwiGLU's and the attention's output
        Buffer part;               // the attention's partials per (row, head, key split)
        uint32_t corr_stride = BLOCK_CONV_KC;  // floats per row of `corr`
        Buffer layout[3];  // per step set: tin [rows][2] | rows_of [rows] | sees [rows] | blocks [max_seqs][2] | slots [max_seqs]
        uint32_t last_rows = 0;  // the last pass's block rows (debug reads)
    };
    std::unique_ptr<BlockDrafter> block_drafter;
    void load_block_drafter(const std::string& path);
    void encode_block_drafter(uint32_t set, const Plan& p, uint32_t rows);
    // A projection of the block drafter: the tensor-core GEMM where the matrix and the row count fit it (xb: the input's
    // bf16 copy if something left one, else a row pass makes it -- and 1 / rms for the epilogues that norm), else the
    // streamed kernel in blocks of 8 rows.
    void drafter_matmul(const Matrix& w, uint32_t n, const float* x, float* y, uint32_t epi, const float* base, float* inv_out, const uint16_t* xb = nullptr,
                        uint16_t* yb = nullptr);

  private:
    KvArgs kv_args() const;
    void matmul(const Matrix& w, uint32_t n, const float* x, float* y, uint32_t epi, const float* base, float* inv_out, uint32_t vocab_real = 0, const QkvEpilogue* q = nullptr,
                const uint16_t* xb = nullptr, uint16_t* yb = nullptr, float scale = 1.0f, float ra = 1.0f, float rb = 1.0f);
    bool stream_fits(const Matrix& w) const;
    // The tensor-core GEMM: xb is x in bf16, inv the rows' 1/rms (normed epilogues), yb an optional bf16 copy of y.
    void matmul_gemm(const Matrix& w, uint32_t n, const uint16_t* xb, float* y, uint16_t* yb, uint32_t epi, const float* base, const float* inv,
                     uint32_t vocab_real = 0, const QkvEpilogue* q = nullptr, float* ssq_out = nullptr, const float* ssq_in = nullptr, float scale = 1.0f, float ra = 1.0f,
                     float rb = 1.0f);
    bool use_gemm(const Matrix& w, uint32_t n) const;
    bool gemm_fits(const Matrix& w, uint32_t n) const;
    // A layer of n tokens runs on the tensor-core GEMM and its last projection leaves bf16(h) in h_b and h's sums of squares in ssq.
    bool layer_carries(const Layer& l, uint32_t n) const;
    // What a decoder layer runs on: its weights, the step layout (device arrays), the cache it writes and reads.
    struct LayerIO {
        const Layer* l;
        uint32_t n, n_tiles, layer, keys_per_split, max_splits, max_rows;  // max_rows: the longest tile's rows
        uint32_t window;       // 0: every key; else the tiles' last `window` keys, extended down to a page boundary (the split kernel only)
        const uint32_t *meta, *tin, *tiles, *vis;
        const uint32_t* ctiles;  // chunk tiles, if the step's attention is the chunk kernel (n_ctiles > 0)
        uint32_t n_ctiles;
        bool kv_only;          // stop after the qkv projection has written K/V into the cache (the drafter's catch-up pass: a one-layer drafter's K/V depend on nothing after it)
        bool h_ready;          // the GEMM before this layer left bf16(h) in h_b and its sums of squares in ssq: no row pass before qkv
        const uint32_t* cpos;  // optional, per token: the cache position its K/V go to (NO_TOK: nowhere); NULL: its run's first position + its row
        uint16_t *k_cache, *v_cache;
        const AttnMaps* maps;
    };
    // Device buffers a capturing step fills beside its normal work (allocated by the first step_capture).
    struct CaptureBufs { Buffer resid_in, attn_in, qkv, attn_out, mlp_in, mlp_out; };
    std::unique_ptr<CaptureBufs> cap;
    float* last_tap() const;  // the last layer's tap (the chain drafter's features)
    void begin_step(uint32_t set, const Plan& p);  // upload, start event, embedding
    void encode_layer(uint32_t set, const Plan& p, uint32_t li, bool capture = false);
    void encode_layer_io(const LayerIO& io, bool capture = false);
    StepOutput read_output(const Plan& p, const StepOptions& opts, double gpu_seconds);
    void encode_tail(uint32_t set, const Plan& p);
    void encode_sample(uint32_t set, uint32_t rows);
    void attention_split(Plan& p, uint32_t max_keys, uint32_t n_tiles) const;
    const Buffer* named(const std::string& name, uint32_t* set_off, size_t* words) const;
    uint32_t last_plan_n = 0, last_split[2] = {0, 1};  // the last plan's tokens, keys per attention split and split count
    cudaEvent_t marks[2] = {nullptr, nullptr};
    struct Span { cudaEvent_t a, b; int group; uint32_t launches; };
    std::vector<Span> spans;
    std::vector<cudaEvent_t> event_pool;
    cudaEvent_t pooled_event();
    // Opens a profiled span of `group` if profiling is on; the returned index goes to span_end.
    int span_begin(int group);
    void span_end(int idx);
};

}  // namespace vlt
