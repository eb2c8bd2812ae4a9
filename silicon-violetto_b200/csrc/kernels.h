// Launchers of the CUDA kernels (all asynchronous on the given stream).
#pragma once
#include <cuda_runtime.h>

#include "common.h"
#include "device.cuh"
#include "weights.h"

namespace vlt {

// Epilogues of a matmul, engine/src/engine/kernels.rs:3-9 and kernels.metal:154-209.
enum : uint32_t { EPI_NORM = 1, EPI_RESID = 2, EPI_SWIGLU = 3, EPI_HEAD = 4, EPI_RAW = 5, EPI_QKV = 6, EPI_HEAD_CAP = 7 };  // 7: 23 sigmoid((acc + 5) / 7.5), kernels.metal:196-199

// What the tensor-core GEMM's EPI_QKV epilogue needs to finish the qkv projection the way `qkv_post` does
// (kernels.metal:749-801): RoPE on q and k, q scaled and rounded to bf16 for the attention, k and v rounded
// into the paged cache at each token's position.
struct QkvEpilogue {
    const uint32_t* meta;        // (slot, position) per token
    const uint32_t* tin;         // (slot, row in its run) per token
    const uint32_t* cpos;        // optional: cache position per token (NO_TOK: no write); NULL: its run's first position + its row
    const float* rope;           // [position][head_dim / 2] (cos, sin)
    const uint32_t* page_table;
    KvArgs kv;
    uint32_t layer, n_heads;
    float scale_log2;
    uint16_t* q_b;               // [token][head][head_dim] bf16
    uint16_t* k_cache;
    uint16_t* v_cache;
};

// Y[t][row] = epilogue(W[row] . bf16(X[t])). X fp32 [n][k]; Y fp32 (SWIGLU: [n][m/2]).
struct MatArgs {
    const uint8_t* W;
    const uint16_t* scales;  // int8: bf16 [m][k / group]
    const float* X;          // [n][k]
    const uint16_t* Xb;      // bf16 copy of X [n_pad][k]: the tensor-core GEMM's input; the streamed matmul takes it instead of X if given (needs no 1/rms then)
    float* Y;
    const float* base;  // EPI_RESID: y = base + acc (may alias Y)
    float* inv_out;     // EPI_NORM / EPI_SWIGLU / EPI_HEAD: 1 / rms(X[t]) is computed here ...
    const float* inv_in;  // ... or, if not null, read from here (tensor-core GEMM)
    uint16_t* Yb;       // optional bf16 copy of Y (feeds the next tensor-core GEMM)
    uint32_t n, k, m, group;  // group: 0 for bf16 weights
    uint32_t epi, vocab_real;
    float eps;
    // kernels.metal:164-165,188-193: the matrix scale (qkv_scale, o_scale) and EPI_RESID's y = ra base + rb (scale acc). 1 for a
    // plain decoder.
    float scale = 1.0f, ra = 1.0f, rb = 1.0f;
    bool int8;
    QkvEpilogue q;  // EPI_QKV only
    uint32_t t0;    // EPI_QKV in the streamed matmul: the step's token that this launch's token 0 is
    uint32_t* err_flag;  // streamed matmul: device word set if a bounded wait ran out (optional)
    // The residual stream's sum of squares per token, kept by the tensor-core GEMMs themselves so that no row pass is
    // needed between them: an EPI_RESID GEMM with ssq_out writes, per 128-row tile of its output, sum(y^2) over the
    // tile's rows ([tile][ssq_stride]); a GEMM with ssq_in (and no inv_in) takes 1/rms = rsqrt(sum over ssq_tiles / k + eps).
    float* ssq_out;
    const float* ssq_in;
    uint32_t ssq_tiles, ssq_stride;
};

void launch_embed(const uint16_t* table, uint32_t* tokens, float* out, const uint32_t* tin, uint32_t* meta, const uint32_t* lens,
                  const uint32_t* feed, const uint32_t* tree, uint32_t* vis, uint32_t n, uint32_t d, uint32_t vocab, cudaStream_t s);
void launch_qkv_post(const float* qkv, const uint32_t* meta, const uint32_t* tin, const float* rope, uint16_t* k_cache, uint16_t* v_cache,
                     const uint32_t* page_table, KvArgs kv, uint32_t layer, uint32_t n, uint32_t n_heads, float scale_log2, uint16_t* q_b, const uint32_t* cpos, cudaStream_t s);
// q | k | v rows as the attention sees them before rounding (RoPE on q and k, kernels.metal:727-736), for step_capture.
void launch_qkv_capture(const float* qkv, const uint32_t* meta, const float* rope, uint32_t n, uint32_t n_heads, KvArgs kv, float* out, cudaStream_t s);
void launch_attn_plain(const float* qkv, const uint32_t* meta, const uint32_t* tiles, const uint32_t* vis, const float* rope, const uint16_t* k_cache,
                       const uint16_t* v_cache, const uint32_t* page_table, KvArgs kv, uint32_t layer, uint32_t n_tiles, uint32_t n_heads,
                       float scale_log2, float* out, cudaStream_t s);
// Tensor-core decode attention over paged KV, split over keys; then the merge of the splits.
// The TMA descriptors of the K and V pools (opaque 128-byte CUtensorMap objects).
struct alignas(64) AttnMaps {
    alignas(64) uint8_t k[128];
    alignas(64) uint8_t v[128];
};
void attn_maps_init(AttnMaps* m, const uint16_t* k_cache, const uint16_t* v_cache, uint64_t total_rows);
void make_tensor_map_2d(void* out_map, const void* base, uint64_t inner, uint64_t rows, uint32_t box_inner, uint32_t box_rows, uint32_t elem_bytes,
                        bool swizzle128, bool swizzle64 = false);
struct AttnArgs {
    const AttnMaps* maps;  // host pointer
    uint32_t* err_flag;    // device word set if a bounded wait ran out
    const uint16_t* q_b;  // [token][head][64] bf16: q after RoPE, scale * log2(e) folded in (qkv_post writes it)
    const uint32_t* meta;
    const uint32_t* tiles;
    const uint32_t* vis;
    const uint16_t* k_cache;
    const uint16_t* v_cache;
    const uint32_t* page_table;
    KvArgs kv;
    uint32_t layer, n_tiles, n_heads;
    float scale_log2;
    uint32_t keys_per_split, max_splits;
    uint32_t max_rows;  // the longest tile's rows in this launch (0: unknown, VERIFY_T)
    uint32_t window;    // 0: every key; else a tile sees its last `window` keys, extended down to a page boundary
    float* part;  // [token][head][max_splits][PART]
    float* out;   // [n][n_heads * hd]
    uint16_t* out_b;  // optional bf16 copy
    uint32_t n;
};
constexpr uint32_t ATTN_PART = 68;  // floats per partial: m, l, 2 pad, o[64]
void launch_attn_mma(const AttnArgs& a, cudaStream_t s);
void launch_attn_combine(const AttnArgs& a, cudaStream_t s);

// Chunk (prefill) attention, k_prefill.cu: blocks of 64 rows of one run x one query head over all the keys the rows see,
// no key split; writes the normalised rows (fp32 and, optionally, bf16).
struct ChunkAttnArgs {
    const AttnMaps* maps;  // host pointer
    uint32_t* err_flag;
    const uint16_t* q_b;  // [token][head][64] bf16, rotated and scaled
    const uint32_t* meta;
    const uint32_t* tin;
    const uint32_t* ctiles;  // (first token, rows <= 64) per chunk tile, never across runs
    const uint32_t* vis;
    const uint32_t* page_table;
    KvArgs kv;
    uint32_t layer, n_ctiles, n_heads;
    float* out;
    uint16_t* out_b;
};
void launch_attn_chunk(const ChunkAttnArgs& a, cudaStream_t s);

// The chain drafter's own kernels (k_draft.cu): inputs of the catch-up pass and of a draft pass, the
// carried tap, and the argmax pick into feed / tree.
void launch_draft_catchup_in(const uint32_t* tokens, const uint32_t* tin, const uint32_t* meta, const uint32_t* on_path, const float* taps, const float* carry,
                             const uint16_t* embed, uint32_t n, uint32_t d, float* x, uint16_t* xb, uint32_t* cpos, cudaStream_t s);
void launch_draft_pass_in(const RunIn* runs, const uint32_t* lens, const uint32_t* feed, const uint32_t* path, const uint32_t* path_len, const uint32_t* on_path,
                          const uint32_t* emitted, const float* taps, const float* dfeat, const uint16_t* embed, uint32_t n_runs, uint32_t d, uint32_t vocab,
                          uint32_t i, uint32_t max_seq_len, float* x, uint16_t* xb, uint32_t* dmeta, uint32_t* dtin, uint32_t* dvis, uint32_t* dcpos, uint32_t* live,
                          cudaStream_t s);
void launch_draft_carry(const RunIn* runs, const uint32_t* path, const uint32_t* path_len, const uint32_t* on_path, const float* taps, uint32_t n_runs,
                        uint32_t d, float* carry, cudaStream_t s);
void launch_draft_pick(const float* logits, uint32_t v, const uint32_t* vocab_ids, const RunIn* runs, const uint32_t* live, uint32_t n_runs, uint32_t i,
                       uint32_t* feed, uint32_t* tree, cudaStream_t s);

// The reference drafter's candidate kernels (kernels.metal:1846-1934): the best `ncand` (<= 4) entries of each row of draft
// logits with their probabilities, then a draft tree per block of rows grown by path probability.
void launch_draft_top(const float* logits, uint32_t n_rows, uint32_t nv, const uint32_t* vocab_ids, const uint32_t* tin, float inv_t, uint32_t ncand, uint32_t* cand,
                      float* cand_q, cudaStream_t s);  // tin (optional): (slot, row) per row; rows numbered 0 are skipped
void launch_draft_tree(const uint32_t* blocks, const uint32_t* slots, uint32_t n_blocks, const uint32_t* cand, const float* cand_q, uint32_t ncand, uint32_t* feed,
                       uint32_t* tree, cudaStream_t s);

// The reference's block drafter (k_block.cu): its shapes and state sizes, and its own kernels.
struct BlockDrafterDims {
    uint32_t hidden, n_q, n_kv, n_layers;  // heads are 128 wide
    uint32_t ring, max_seqs, window, ctx_ring_len;
    float eps, scale;
};
constexpr uint32_t BLOCK_CONV_KC = 192;  // a convolution's correction rows (2 * hidden / 16, padded; tools/spec/export.py:14)
void launch_block_context(const float* kvp, const float* ctx, const float* ctx_inv, const uint32_t* meta, const uint32_t* on_path, const float* rope,
                          const BlockDrafterDims& b, uint32_t n, uint16_t* k_ring, uint16_t* v_ring, float* ctx_ring, cudaStream_t s);
void launch_block_embed(const uint16_t* table, const uint32_t* tin, const uint32_t* lens, const uint32_t* feed, const float* mask_emb, const float* ctx_ring,
                        const BlockDrafterDims& b, uint32_t vocab, uint32_t rows, float* x, float* last, uint32_t* meta, cudaStream_t s);
void launch_block_conv(const float* x, const float* corr, uint32_t corr_stride, const float* base, const uint32_t* tin, const float* resid, uint32_t hidden,
                       uint32_t rows, float* out, cudaStream_t s);
void launch_block_qkv_post(float* qkv, const uint32_t* meta, const float* rope, const BlockDrafterDims& b, uint32_t layer, uint32_t rows, uint16_t* k_ring,
                           uint16_t* v_ring, cudaStream_t s);
void launch_block_attn(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* rows_of, const uint16_t* k_ring, const uint16_t* v_ring,
                       const BlockDrafterDims& b, uint32_t layer, uint32_t rows, float* out, cudaStream_t s);

// The reference's own architecture (k_limite.cu). A layer's cache: a ring per (local layer, slot) or the paged pool of the
// global layers (kernels.metal:692-715); heads are 128 wide.
struct LimiteKv {
    uint32_t is_global, layer;  // layer: its index among the local or among the global layers
    uint32_t n_kv, ring, max_seqs;
    uint32_t n_pages, max_pages, page_shift;
    const uint32_t* page_table;
};
void launch_limite_mudd(const float* cur, const float* tap0, const float* tap1, const float* dense1, const float* mix, uint32_t hidden, float eps, uint32_t n,
                        float* out_attn, float* out_base, cudaStream_t s);
void launch_limite_qkv_post(float* qkv, const float* x, const float* inv_rms, const uint32_t* meta, const uint32_t* tin, const uint32_t* tokens, const uint16_t* ve_table,
                            const float* ve_gate, const float* attn_gate, const float* rope, const LimiteKv& kv, uint32_t hidden, uint32_t n_q, float eps, uint32_t vocab,
                            uint32_t n, uint16_t* k_cache, uint16_t* v_cache, float* vdir, float* gates, const float* ssq, uint32_t ssq_tiles, uint32_t ssq_stride,
                            cudaStream_t s);
constexpr uint32_t LIMITE_MAX_SPLITS = 128, LIMITE_PART = 132;  // key splits a row's attention may take; floats per partial
void launch_limite_attn_mma(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint16_t* k_cache, const uint16_t* v_cache,
                            const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, uint32_t n, uint32_t keys_per_split, uint32_t splits, float* part,
                            cudaStream_t s);
void launch_limite_attn_cluster(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint16_t* k_cache, const uint16_t* v_cache,
                                const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, const float* vdir, const float* gates, const float* xsa, uint32_t n,
                                uint32_t keys_per_split, uint32_t splits, float* out, uint16_t* out_b, cudaStream_t s);
void launch_limite_attn_rows(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint32_t* tiles, const uint16_t* k_cache,
                             const uint16_t* v_cache, const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, uint32_t n_tiles, uint32_t keys_per_split,
                             uint32_t splits, float* part, cudaStream_t s);
void launch_limite_attn(const float* qkv, const uint32_t* meta, const uint32_t* tin, const uint32_t* vis, const uint32_t* tiles, uint32_t n_tiles, const uint16_t* k_cache, const uint16_t* v_cache,
                        const LimiteKv& kv, uint32_t n_q, uint32_t window, float scale, const float* vdir, const float* gates, const float* xsa, uint32_t n,
                        uint32_t max_keys, float* part, float* out, uint16_t* out_b, uint32_t keys_per_block, cudaStream_t s);  // out_b: optional bf16 copy (heads per kv head 1, 2 or 5)
void launch_limite_compact(const RunIn* runs, const uint32_t* path, const uint32_t* path_len, const uint32_t* lens, uint16_t* k_local, uint16_t* v_local,
                           uint16_t* k_global, uint16_t* v_global, const LimiteKv& local, const LimiteKv& global, uint32_t n_local, uint32_t n_global, uint32_t n_runs,
                           cudaStream_t s);

// The tcgen05 GEMM for 16..256 tokens: needs Xb (bf16 X, rows padded to 16), inv_in for the
// normed epilogues, m a multiple of 128, one int8 scale per row.
bool gemm_supported(const MatArgs& a);
void launch_gemm(const MatArgs& a, uint32_t sm_count, uint32_t* err_flag, cudaStream_t s, bool allow_paired = true);
void launch_matmul_stream(const MatArgs& a, uint32_t sm_count, cudaStream_t s);  // n <= 8, tensor cores fed from registers
bool matmul_stream_fits(const MatArgs& a);                                      // else launch_matmul_stream falls back to the scalar kernel
void launch_matmul_rows(const MatArgs& a, cudaStream_t s);                      // any n, scalar (cross-check, odd scale groups)
// out[r] = in[rows ? rows[r] : r] as fp32 (and bf16); inv[r] = 1 / rms (kernels.metal:117-148).
void launch_prep_rows(const float* in, const uint32_t* rows, uint32_t n, uint32_t k, float eps, float* out_f32, uint16_t* out_bf16, float* inv,
                      bool normalize, bool round_out, cudaStream_t s);

// row_skip (optional): rows marked 1 are left untouched (another rule decides them).
void launch_sample(const float* logits, const SampleRow* rows, uint32_t* out, const uint32_t* meta, uint32_t n_rows, uint32_t vocab, cudaStream_t s,
                   const uint32_t* row_skip = nullptr);
// spec_e (optional): a run with spec_e[run] != 0 has that many candidates already settled in out[head0 ..], its path rows 0 .. spec_e - 1.
void launch_accept(const RunIn* runs, const uint32_t* tokens, uint32_t* out, uint32_t* lens, uint32_t* feed, GenState* gen, uint32_t* emitted,
                   uint32_t n_runs, const uint32_t* tree, uint32_t* path, uint32_t* path_len, uint32_t* on_path, cudaStream_t s, const uint32_t* spec_e = nullptr);
void launch_kv_compact(const RunIn* runs, const uint32_t* path, const uint32_t* path_len, const uint32_t* lens, uint16_t* k_cache, uint16_t* v_cache,
                       const uint32_t* page_table, KvArgs kv, uint32_t n_runs, uint32_t n_layers, cudaStream_t s);
void launch_replay_draft(const RunIn* runs, const uint32_t* lens, uint32_t* feed, const uint32_t* trace, const uint32_t* trace_len, ReplayArgs ra,
                         uint32_t n_runs, uint32_t* tree, cudaStream_t s);
// A row of logits' statistics for the rejection-sampling rule: maximum, argmax (ties to the lowest id), and the sum
// of 2^((x - max) log2(e) / T) in the sampler's order.
struct SpecRowStats {
    float max;
    uint32_t argmax;
    float z;
    uint32_t pad;
};
// The rule inside the engine's step (k_spec.cu), device pointers throughout.
struct SpecStepArgs {
    const RunIn* runs;
    uint32_t n_runs, n_head, max_head_rows;
    const SampleRow* samples;  // per head row
    const uint32_t* tokens;    // the step's tokens, resolved
    const uint32_t* meta;      // (slot, position) per token
    const uint32_t* tree;      // [slot][FEED_W]
    const float* logits;       // [head row][vocab]
    uint32_t vocab;
    const float* q_keep;       // [slot][VERIFY_T - 1][v]: the rows the slot's drafts were drawn from
    uint32_t v;
    uint32_t* q_rows;          // [slot]: how many of them are current
    const uint32_t* index_of;  // [vocab]: a target id's index in the draft vocabulary, or NO_TOK
    SpecRowStats* stats;       // [max_head_rows + max_seqs (VERIFY_T - 1)]
    uint32_t* row_skip;        // [head row]: 1 if the sampler is to leave the row to this rule
    uint32_t* spec_e;          // [run]: the candidates this rule settled (0: the run is not its)
    uint32_t* out;             // out_ids
};
void launch_spec_step_stats(const SpecStepArgs& a, cudaStream_t s);
void launch_spec_step_decide(const SpecStepArgs& a, cudaStream_t s);
// The chain drafter's pick of pass i: argmax, or (rule 1, a sampling sequence) a draw from softmax(q / T) with the row kept.
void launch_draft_draw(const float* logits, uint32_t v, const uint32_t* vocab_ids, const RunIn* runs, const SampleRow* samples, const uint32_t* live,
                       const uint32_t* lens, uint32_t n_runs, uint32_t i, uint32_t rule, uint32_t* feed, uint32_t* tree, float* q_keep, uint32_t* q_rows,
                       cudaStream_t s);
// Rejection-sampling acceptance over bf16 draft and target logits on the device (k_spec.cu).
void launch_spec_accept(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, uint32_t vocab, float temperature,
                        const uint64_t* seeds, const uint32_t* pos0, void* stats, uint32_t* accepted, uint32_t* token, uint32_t* rollback, cudaStream_t s);
// The same with its scratch in static device arrays: allocates nothing; device pointers throughout.
// Returns NULL or an error message (a literal).
uint32_t spec_accept_static_max_rows();
const char* launch_spec_accept_static(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, uint32_t vocab,
                                      float temperature, const uint64_t* seeds, const uint32_t* pos0, uint32_t* accepted, uint32_t* token,
                                      uint32_t* rollback, cudaStream_t s);
// A kernel whose (bounded) wait runs out on purpose and sets the error word to `code`: for testing how that is reported.
void launch_stalled_wait(uint32_t* err_flag, uint32_t polls, uint32_t code, cudaStream_t s);
void launch_kv_fill(uint16_t* k_cache, uint16_t* v_cache, const uint32_t* page_table, KvArgs kv, uint32_t n_layers, uint32_t slot, uint32_t from,
                    uint32_t to, uint32_t seed, cudaStream_t s);

}  // namespace vlt
