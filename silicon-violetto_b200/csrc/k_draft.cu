// The chain drafter's own kernels (its matmuls, attention and K/V writes are the target's).
// Not in the reference, whose drafter is a block drafter with a draft tree
// (engine/src/engine/drafter.rs:278-447); this one keeps that drafter's interface: it reads the
// tapped hidden states of the rows on the accepted path (kernels.metal:133-148), `lens` and
// `feed[slot][0]` after `accept`, and writes its drafts to `feed[slot][1..]` and chain nodes to
// `tree[slot][1..]` (kernels.metal:51-60), all on the device, in the same step.
#include <cfloat>

#include "kernels.h"

namespace vlt {

// One input row of the drafter: [feature (d) ; embedding of `tok` (d)], as fp32 and as bf16 (both exact:
// features and embeddings are bf16 values).
__device__ __forceinline__ void draft_row_in(const float* feat, const uint16_t* emb, uint32_t d, float* x, uint16_t* xb) {
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float f = feat ? feat[i] : 0.0f;
        x[i] = f;
        xb[i] = f32_to_bf16(f);
        x[d + i] = bf16_to_f32(emb[i]);
        xb[d + i] = emb[i];
    }
}

// The catch-up pass's inputs, one block per step token: the feature of the position before is the tap
// of the row before, or for a run's first row the slot's carried tap (zero at position 0). Rows off the
// accepted path keep their K/V out of the drafter's cache (cpos = NO_TOK).
__global__ void draft_catchup_in_kernel(const uint32_t* __restrict__ tokens, const uint32_t* __restrict__ tin, const uint32_t* __restrict__ meta,
                                        const uint32_t* __restrict__ on_path, const float* __restrict__ taps, const float* __restrict__ carry,
                                        const uint16_t* __restrict__ embed, uint32_t d, float* x, uint16_t* xb, uint32_t* cpos) {
    pdl_start();
    const uint32_t t = blockIdx.x, slot = tin[2 * t], row = tin[2 * t + 1], pos = meta[2 * t + 1];
    const float* feat = row ? taps + size_t(t - 1) * d : pos ? carry + size_t(slot) * d : nullptr;
    draft_row_in(feat, embed + size_t(tokens[t]) * d, d, x + size_t(t) * 2 * d, xb + size_t(t) * 2 * d);
    if (threadIdx.x == 0) cpos[t] = on_path[t] ? pos : NO_TOK;
}

// The last row of run r on the accepted path (NO_TOK: none): a verify run's path end, any other run's last row.
__device__ __forceinline__ uint32_t draft_last_row(const RunIn& ru, uint32_t r, const uint32_t* path, const uint32_t* path_len, const uint32_t* on_path) {
    if (ru.verify) return path_len[r] ? ru.first + path[r * FEED_W + path_len[r] - 1] : NO_TOK;
    return on_path[ru.first] ? ru.first + ru.count - 1 : NO_TOK;
}

// Draft pass i (1-based), one block per run: the row stands at position lens[slot] + i - 1 on token
// feed[slot][i - 1]; its feature is the tap of the path's last row (i = 1) or the drafter's own normed
// output of the pass before. Writes the pass's step layout (meta, tin, vis, cpos) and whether the run drafts.
__global__ void draft_pass_in_kernel(const RunIn* __restrict__ runs, const uint32_t* __restrict__ lens, const uint32_t* __restrict__ feed,
                                     const uint32_t* __restrict__ path, const uint32_t* __restrict__ path_len, const uint32_t* __restrict__ on_path,
                                     const uint32_t* __restrict__ emitted, const float* __restrict__ taps, const float* __restrict__ dfeat,
                                     const uint16_t* __restrict__ embed, uint32_t d, uint32_t vocab, uint32_t i, uint32_t max_seq_len, float* x, uint16_t* xb,
                                     uint32_t* dmeta, uint32_t* dtin, uint32_t* dvis, uint32_t* dcpos, uint32_t* live) {
    pdl_start();
    const uint32_t r = blockIdx.x;
    const RunIn ru = runs[r];
    const uint32_t last = draft_last_row(ru, r, path, path_len, on_path);
    const uint32_t pos = lens[ru.slot] + i - 1;
    const bool lv = last != NO_TOK && emitted[r] > 0 && pos < max_seq_len;
    const float* feat = i == 1 ? (last != NO_TOK ? taps + size_t(last) * d : nullptr) : dfeat + size_t(r) * d;
    uint32_t tok = lv ? feed[ru.slot * FEED_W + i - 1] : 0u;
    if (tok >= vocab) tok = 0;  // (only a row of NaN logits can leave such an id in feed)
    draft_row_in(feat, embed + size_t(tok) * d, d, x + size_t(r) * 2 * d, xb + size_t(r) * 2 * d);
    if (threadIdx.x == 0) {
        dmeta[2 * r] = ru.slot;
        dmeta[2 * r + 1] = lv ? pos : 0u;
        dtin[2 * r] = ru.slot;
        dtin[2 * r + 1] = 0;
        dvis[r] = 1;
        dcpos[r] = lv ? pos : NO_TOK;
        live[r] = lv ? 1u : 0u;
    }
}

// The slot's carried tap for the next step's catch-up: the tap of the path's last row.
__global__ void draft_carry_kernel(const RunIn* __restrict__ runs, const uint32_t* __restrict__ path, const uint32_t* __restrict__ path_len,
                                   const uint32_t* __restrict__ on_path, const float* __restrict__ taps, uint32_t d, float* carry) {
    pdl_start();
    const uint32_t r = blockIdx.x;
    const RunIn ru = runs[r];
    const uint32_t last = draft_last_row(ru, r, path, path_len, on_path);
    if (last == NO_TOK) return;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) carry[size_t(ru.slot) * d + i] = taps[size_t(last) * d + i];
}

// The pass's drafts, one block per run: the draft vocabulary's argmax (ties to the lowest index), mapped
// to the target's id, into feed[slot][i]; tree[slot][i] = chain_node(i).
__global__ void __launch_bounds__(256) draft_pick_kernel(const float* __restrict__ logits, uint32_t v, const uint32_t* __restrict__ vocab_ids,
                                                         const RunIn* __restrict__ runs, const uint32_t* __restrict__ live, uint32_t i, uint32_t* feed,
                                                         uint32_t* tree) {
    pdl_start();
    __shared__ float bv[8];
    __shared__ uint32_t bi[8];
    const uint32_t r = blockIdx.x, tid = threadIdx.x;
    if (!live[r]) return;
    const float* row = logits + size_t(r) * v;
    float mx = -FLT_MAX;
    uint32_t am = 0xffffffffu;
    for (uint32_t j = tid; j < v; j += 256) better(mx, am, row[j], j);
    warp_best(mx, am);
    if (tid % 32 == 0) { bv[tid / 32] = mx; bi[tid / 32] = am; }
    __syncthreads();
    if (tid == 0) {
        for (uint32_t w = 1; w < 8; w++) better(mx, am, bv[w], bi[w]);
        const uint32_t slot = runs[r].slot;
        feed[slot * FEED_W + i] = vocab_ids[am < v ? am : 0];
        tree[slot * FEED_W + i] = d_chain_node(i);
    }
}

// ---------------------------------------------------------------- the reference drafter's candidate kernels
// kernels.metal:1846-1889 `draft_top`: one block of 1024 threads per row of draft logits; the `ncand` (<= 4)
// best draft-vocabulary entries (ties to the lowest index), mapped to target ids, and their probabilities
// at temperature 1 / inv_t. The normaliser's sum: thread t adds entries t, t + 1024, ... in turn, lanes are
// added left to right within a warp and the warps left to right (the reference's simd_sum order is not
// pinned); exp is soft_exp2(x log2 e), every operation a single IEEE one, as in the CPU restatement.
constexpr uint32_t DRAFT_CANDS = 4;
__global__ void __launch_bounds__(1024) draft_top_kernel(const float* __restrict__ logits, uint32_t nv, const uint32_t* __restrict__ vocab_ids,
                                                         const uint32_t* __restrict__ tin, float inv_t, uint32_t ncand, uint32_t* cand, float* cand_q) {
    pdl_start();
    if (tin && tin[2 * blockIdx.x + 1] == 0) return;  // kernels.metal:1862: a block's row 0 is the bonus token's own
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    __shared__ float top_v[DRAFT_CANDS];
    __shared__ uint32_t top_i[DRAFT_CANDS];
    __shared__ float zs[1024];
    __shared__ float groups[32];
    __shared__ float z_s;
    const uint32_t r = blockIdx.x, tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
    const float* row = logits + size_t(r) * nv;
    for (uint32_t c = 0; c < ncand; c++) {
        float mx = -FLT_MAX;
        uint32_t am = 0xffffffffu;
        for (uint32_t j = tid; j < nv; j += 1024) {
            bool taken = false;
            for (uint32_t m = 0; m < c; m++) taken = taken || top_i[m] == j;
            if (!taken) better(mx, am, row[j], j);
        }
        warp_best(mx, am);
        if (lane == 0) { bv[warp] = mx; bi[warp] = am; }
        __syncthreads();
        if (tid == 0) {
            for (uint32_t w = 1; w < 32; w++) better(mx, am, bv[w], bi[w]);
            top_v[c] = mx;
            top_i[c] = am;
        }
        __syncthreads();
    }
    const float t0 = top_v[0];
    float zt = 0.0f;
    for (uint32_t j = tid; j < nv; j += 1024) zt = __fadd_rn(zt, soft_exp2(__fmul_rn(__fmul_rn(__fsub_rn(row[j], t0), inv_t), LOG2E)));
    zs[tid] = zt;
    __syncthreads();
    if (lane == 0) {
        float acc = 0.0f;
        for (uint32_t l = 0; l < 32; l++) acc = __fadd_rn(acc, zs[warp * 32 + l]);
        groups[warp] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        float z = 0.0f;
        for (uint32_t w = 0; w < 32; w++) z = __fadd_rn(z, groups[w]);
        z_s = z;
    }
    __syncthreads();
    if (tid < ncand) {
        cand[r * DRAFT_CANDS + tid] = vocab_ids ? vocab_ids[top_i[tid]] : top_i[tid];
        cand_q[r * DRAFT_CANDS + tid] = __fdiv_rn(soft_exp2(__fmul_rn(__fmul_rn(__fsub_rn(top_v[tid], t0), inv_t), LOG2E)), z_s);
    }
}

// kernels.metal:1896-1934 `draft_tree`: one thread per block of `rows` rows starting at step row `first`
// (blocks[2 b], blocks[2 b + 1]) of slot slots[b]: grows the tree greedily by path probability -- the node
// with the best score x next candidate's probability gets a child -- parents before children, then dead
// nodes up to FEED_W.
__global__ void draft_tree_kernel(const uint32_t* __restrict__ blocks, const uint32_t* __restrict__ slots, uint32_t n_blocks, const uint32_t* __restrict__ cand,
                                  const float* __restrict__ cand_q, uint32_t ncand, uint32_t* feed, uint32_t* tree) {
    pdl_start();
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const uint32_t first = blocks[2 * b], rows = min(blocks[2 * b + 1], VERIFY_T), slot = slots[b];
    float score[8] = {1.0f, 0, 0, 0, 0, 0, 0, 0};
    uint32_t depth[8] = {0, 0, 0, 0, 0, 0, 0, 0}, taken[8] = {0, 0, 0, 0, 0, 0, 0, 0}, sees[8] = {1, 0, 0, 0, 0, 0, 0, 0};
    uint32_t n = 1;
    for (; n < rows; n++) {
        float best = -1.0f;
        uint32_t p = 0;
        for (uint32_t i = 0; i < n; i++) {
            if (depth[i] + 1 == rows || taken[i] == ncand) continue;
            const float sc = __fmul_rn(score[i], cand_q[(first + depth[i] + 1) * DRAFT_CANDS + taken[i]]);
            if (sc > best) { best = sc; p = i; }
        }
        if (best < 0.0f) break;
        const uint32_t d = depth[p] + 1;
        feed[slot * FEED_W + n] = cand[(first + d) * DRAFT_CANDS + taken[p]];
        taken[p]++;
        score[n] = best;
        depth[n] = d;
        taken[n] = 0;
        sees[n] = sees[p] | 1u << n;
        tree[slot * FEED_W + n] = d_tree_node(d, p, sees[n]);
    }
    for (; n < FEED_W; n++) tree[slot * FEED_W + n] = d_dead_node(n);
}

void launch_draft_top(const float* logits, uint32_t n_rows, uint32_t nv, const uint32_t* vocab_ids, const uint32_t* tin, float inv_t, uint32_t ncand, uint32_t* cand,
                      float* cand_q, cudaStream_t s) {
    if (n_rows) launch_pdl(draft_top_kernel, n_rows, 1024, 0, s, logits, nv, vocab_ids, tin, inv_t, ncand, cand, cand_q);
}
void launch_draft_tree(const uint32_t* blocks, const uint32_t* slots, uint32_t n_blocks, const uint32_t* cand, const float* cand_q, uint32_t ncand, uint32_t* feed,
                       uint32_t* tree, cudaStream_t s) {
    if (n_blocks) launch_pdl(draft_tree_kernel, (n_blocks + 31) / 32, 32, 0, s, blocks, slots, n_blocks, cand, cand_q, ncand, feed, tree);
}

void launch_draft_catchup_in(const uint32_t* tokens, const uint32_t* tin, const uint32_t* meta, const uint32_t* on_path, const float* taps, const float* carry,
                             const uint16_t* embed, uint32_t n, uint32_t d, float* x, uint16_t* xb, uint32_t* cpos, cudaStream_t s) {
    launch_pdl(draft_catchup_in_kernel, n, 256, 0, s, tokens, tin, meta, on_path, taps, carry, embed, d, x, xb, cpos);
}
void launch_draft_pass_in(const RunIn* runs, const uint32_t* lens, const uint32_t* feed, const uint32_t* path, const uint32_t* path_len, const uint32_t* on_path,
                          const uint32_t* emitted, const float* taps, const float* dfeat, const uint16_t* embed, uint32_t n_runs, uint32_t d, uint32_t vocab,
                          uint32_t i, uint32_t max_seq_len, float* x, uint16_t* xb, uint32_t* dmeta, uint32_t* dtin, uint32_t* dvis, uint32_t* dcpos, uint32_t* live,
                          cudaStream_t s) {
    launch_pdl(draft_pass_in_kernel, n_runs, 256, 0, s, runs, lens, feed, path, path_len, on_path, emitted, taps, dfeat, embed, d, vocab, i, max_seq_len, x, xb, dmeta,
               dtin, dvis, dcpos, live);
}
void launch_draft_carry(const RunIn* runs, const uint32_t* path, const uint32_t* path_len, const uint32_t* on_path, const float* taps, uint32_t n_runs,
                        uint32_t d, float* carry, cudaStream_t s) {
    launch_pdl(draft_carry_kernel, n_runs, 256, 0, s, runs, path, path_len, on_path, taps, d, carry);
}
void launch_draft_pick(const float* logits, uint32_t v, const uint32_t* vocab_ids, const RunIn* runs, const uint32_t* live, uint32_t n_runs, uint32_t i,
                       uint32_t* feed, uint32_t* tree, cudaStream_t s) {
    launch_pdl(draft_pick_kernel, n_runs, 256, 0, s, logits, v, vocab_ids, runs, live, i, feed, tree);
}

}  // namespace vlt
