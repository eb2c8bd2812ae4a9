// CPU oracle (test infrastructure only, parity unpinned: see bits.hpp): the token sampler,
// the acceptance walk, the KV compaction and the test drafters of the reference, restated
// one GPU thread at a time so that every float sum has the reference's order.
#pragma once
#include <algorithm>
#include <cfloat>
#include <cstdint>
#include <vector>

#include "bits.hpp"

namespace orc {

constexpr uint32_t SAMPLE_THREADS = 1024;  // kernels.metal:1415
constexpr uint32_t SAMPLE_ROUNDS = 8;      // kernels.metal:1416
constexpr uint32_t AM_BLOCK = 4096;        // kernels.metal:1413

// kernels.metal:1418-1420 `better`: ties go to the lowest id.
inline void better(float& bv, uint32_t& bi, float v, uint32_t i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

// kernels.metal:1430-1451 `argmax_partial` then :1525-1531: blocks of 4096, then over blocks.
// The order of the reductions does not matter: `better` is a total order on (value, id).
inline void argmax_row(const float* x, uint32_t vocab, float& lmax, uint32_t& tok) {
    lmax = -FLT_MAX;
    tok = 0xffffffffu;
    for (uint32_t i = 0; i < vocab; i++) better(lmax, tok, x[i], i);
}

// kernels.metal:1482-1501 `tg_scan`. in: v[1024] per-thread sums. out: ex[0..1024], ex[t] the
// sum over threads before t, ex[1024] the total. Association: 32 groups of 32 consecutive
// threads summed left to right from 0, then the group totals scanned left to right from 0,
// then each in-group prefix + its group's base.
inline void tg_scan(const float* v, float* ex) {
    float base[32];
    for (uint32_t g = 0; g < 32; g++) {
        float acc = 0.0f;
        for (uint32_t i = 32 * g; i < 32 * g + 32; i++) { ex[i] = acc; acc += v[i]; }
        base[g] = acc;
    }
    float acc = 0.0f;
    for (uint32_t g = 0; g < 32; g++) { float x = base[g]; base[g] = acc; acc += x; }
    ex[SAMPLE_THREADS] = acc;
    for (uint32_t t = 0; t < SAMPLE_THREADS; t++) ex[t] += base[t / 32];
}

// kernels.metal:1510-1576 `sample`, one row. `pos` is the position of the drawn token
// (kernels.metal:1524). exp2 is soft_exp2 (see bits.hpp for why).
inline uint32_t sample_row(const float* x, uint32_t vocab, const SampleRow& row, uint32_t pos) {
    float lmax;
    uint32_t tok;
    argmax_row(x, vocab, lmax, tok);
    if (!(row.temperature > 0.0f)) return tok;
    const float c = LOG2E / row.temperature;
    std::vector<float> s(SAMPLE_THREADS), ex(SAMPLE_THREADS + 1);
    for (uint32_t t = 0; t < SAMPLE_THREADS; t++) {
        float a = 0.0f;
        for (uint32_t i = t; i < vocab; i += SAMPLE_THREADS) a += soft_exp2((x[i] - lmax) * c);
        s[t] = a;
    }
    tg_scan(s.data(), ex.data());
    const float z = ex[SAMPLE_THREADS];
    float low = -INFINITY;
    for (uint32_t round = 0; round < SAMPLE_ROUNDS; round++) {
        const float target = uniform01(row.seed_lo, row.seed_hi, pos, round) * ex[SAMPLE_THREADS];
        uint32_t pick = 0xffffffffu;
        for (uint32_t t = 0; t < SAMPLE_THREADS; t++) {
            const float lo = ex[t];
            if (lo <= target && target < ex[t + 1]) {
                float acc = 0.0f;
                uint32_t j = 0xffffffffu;
                for (uint32_t i = t; i < vocab; i += SAMPLE_THREADS) {
                    float xi = x[i];
                    if (!(xi > low)) continue;
                    float e = soft_exp2((xi - lmax) * c);
                    acc += e;
                    if (e > 0.0f) j = i;
                    if (target - lo < acc) break;
                }
                pick = j;  // at most one thread's interval holds the target: ex never decreases
            }
        }
        const uint32_t j = pick;
        if (j == 0xffffffffu) break;
        const float xj = x[j];
        if (xj == lmax || row.top_p >= 1.0f) { tok = j; break; }
        for (uint32_t t = 0; t < SAMPLE_THREADS; t++) {
            float q = 0.0f;
            for (uint32_t i = t; i < vocab; i += SAMPLE_THREADS) {
                float xi = x[i];
                if (xi > xj) q += soft_exp2((xi - lmax) * c);
            }
            s[t] = q;
        }
        tg_scan(s.data(), ex.data());
        if (ex[SAMPLE_THREADS] < row.top_p * z) { tok = j; break; }
        low = xj;
    }
    return tok;
}

// kernels.metal:1605-1657 `accept`, one run. Arrays are the whole step's / engine's.
// `decided` (not in the reference): if not 0, a verify run's candidates were settled before this by the
// rejection-sampling rule (see spec_step_run): rows 0 .. decided - 1 are the path and out[head0 ..] already
// holds their tokens; everything from the stop-token scan on is the reference's.
inline void accept_run(uint32_t r, const RunIn* runs, const uint32_t* tokens, uint32_t* out, uint32_t* lens,
                       uint32_t* feed, GenState* gen, uint32_t* emitted, const uint32_t* tree, uint32_t* path,
                       uint32_t* path_len, uint32_t* on_path, uint32_t decided = 0) {
    const RunIn ru = runs[r];
    GenState& gs = gen[ru.slot];
    path_len[r] = 0;
    for (uint32_t j = 0; j < ru.count; j++) on_path[ru.first + j] = !ru.verify && !gs.done;
    if (gs.done) { emitted[r] = 0; return; }
    if (!ru.verify) lens[ru.slot] += ru.count;
    if (ru.nhead == 0) { emitted[r] = 0; return; }
    uint32_t first = ru.head0 + ru.nhead - 1, e = 1;
    uint32_t walk[FEED_W];
    walk[0] = 0;
    if (ru.verify && decided) {
        e = decided;
        for (uint32_t j = 0; j < e; j++) walk[j] = j;
        first = ru.head0;
    } else if (ru.verify) {
        const uint32_t* node = tree + ru.slot * FEED_W;
        for (uint32_t c = 1, at = 0; c < ru.count; c++) {
            if (node_parent(node[c]) == at && tokens[ru.first + c] == out[ru.head0 + at]) walk[e++] = at = c;
        }
        for (uint32_t j = 1; j < e; j++) out[ru.head0 + j] = out[ru.head0 + walk[j]];
        first = ru.head0;
    }
    bool stop = false;
    uint32_t k = 0;
    while (k < e && k < gs.remaining && !stop) {
        const uint32_t tok = out[first + k];
        for (uint32_t j = 0; j < gs.nstop; j++) stop = stop || tok == gs.stop[j];
        k++;
    }
    if (ru.verify) {
        lens[ru.slot] += k;
        path_len[r] = k;
        for (uint32_t j = 0; j < k; j++) {
            path[r * FEED_W + j] = walk[j];
            on_path[ru.first + walk[j]] = 1;
        }
    }
    feed[ru.slot * FEED_W] = out[first + k - 1];
    gs.remaining -= k;
    if (stop || gs.remaining == 0) gs.done = 1;
    emitted[r] = k;
}

// kernels.metal:1705-1724 `replay_draft`, one run.
struct ReplayArgs { uint32_t stride, seed; float rate; uint32_t vocab; };
inline void replay_draft_run(uint32_t r, const RunIn* runs, const uint32_t* lens, uint32_t* feed, const uint32_t* trace,
                             const uint32_t* trace_len, const ReplayArgs& ra, uint32_t* tree) {
    if (runs[r].nhead == 0) return;
    const uint32_t slot = runs[r].slot, n = trace_len[slot];
    if (n == 0) return;
    for (uint32_t i = 1; i < FEED_W; i++) {
        const uint32_t pos = lens[slot] + i;
        uint32_t tok = pos < n ? trace[uint64_t(slot) * ra.stride + pos] : 0u;
        const uint32_t h = philox(U4{pos, 0x5eed, 0, 0}, ra.seed, 0x0dd5u).x;
        if (float(h >> 8) * 0x1p-24f < ra.rate) tok = (tok + 1) % ra.vocab;
        feed[slot * FEED_W + i] = tok;
        tree[slot * FEED_W + i] = chain_node(i);
    }
}

// kernels.metal:1846-1889 `draft_top`, one row: the `ncand` best ids (ties to the lowest id)
// and their probabilities at temperature 1/inv_t. z's sum: thread t of 1024 adds ids
// t, t+1024, ... in turn; the reference then adds the threads' sums in simdgroup order
// (tg_sum, kernels.metal:40-48), which Metal's simd_sum leaves unpinned: here lanes are added
// left to right within a group of 32, then the 32 groups left to right. exp(x) is the shared
// soft_exp2(x * log2e), every operation a single IEEE one, so that the CUDA kernel can agree
// with this bit for bit (the reference's own tests pin the integers: candidates and tree).
constexpr uint32_t CANDS = 4;
inline void draft_top_row(const float* row, uint32_t nv, const uint32_t* vocab_ids, float inv_t, uint32_t ncand,
                          uint32_t* cand, float* cand_q) {
    float top_v[CANDS];
    uint32_t top_i[CANDS];
    for (uint32_t c = 0; c < ncand; c++) {
        float bv = -FLT_MAX;
        uint32_t bi = 0xffffffffu;
        for (uint32_t j = 0; j < nv; j++) {
            bool taken = false;
            for (uint32_t m = 0; m < c; m++) taken = taken || top_i[m] == j;
            if (!taken) better(bv, bi, row[j], j);
        }
        top_v[c] = bv;
        top_i[c] = bi;
    }
    float groups[32];
    for (uint32_t g = 0; g < 32; g++) {
        float acc = 0.0f;
        for (uint32_t l = 0; l < 32; l++) {
            float zt = 0.0f;
            for (uint32_t j = g * 32 + l; j < nv; j += 1024) zt += soft_exp2(((row[j] - top_v[0]) * inv_t) * LOG2E);
            acc += zt;
        }
        groups[g] = acc;
    }
    float z = 0.0f;
    for (uint32_t g = 0; g < 32; g++) z += groups[g];
    for (uint32_t c = 0; c < ncand; c++) {
        cand[c] = vocab_ids ? vocab_ids[top_i[c]] : top_i[c];
        cand_q[c] = soft_exp2(((top_v[c] - top_v[0]) * inv_t) * LOG2E) / z;
    }
}

// kernels.metal:1896-1934 `draft_tree`, one block of `rows` rows starting at step row `first`
// (cand/cand_q indexed by step row). VERIFY_T = 8 rows at most.
inline void draft_tree_block(uint32_t first, uint32_t rows, uint32_t slot, const uint32_t* cand, const float* cand_q,
                             uint32_t ncand, uint32_t* feed, uint32_t* tree) {
    float score[8] = {1.0f};
    uint32_t depth[8] = {0}, taken[8] = {0}, sees[8] = {1};
    uint32_t n = 1;
    for (; n < rows; n++) {
        float best = -1.0f;
        uint32_t p = 0;
        for (uint32_t i = 0; i < n; i++) {
            if (depth[i] + 1 == rows || taken[i] == ncand) continue;
            const float s = score[i] * cand_q[(first + depth[i] + 1) * CANDS + taken[i]];
            if (s > best) { best = s; p = i; }
        }
        if (best < 0.0f) break;
        const uint32_t d = depth[p] + 1;
        feed[slot * FEED_W + n] = cand[(first + d) * CANDS + taken[p]];
        taken[p]++;
        score[n] = best;
        depth[n] = d;
        taken[n] = 0;
        sees[n] = sees[p] | 1u << n;
        tree[slot * FEED_W + n] = tree_node(d, p, sees[n]);
    }
    for (; n < FEED_W; n++) tree[slot * FEED_W + n] = dead_node(n);
}

// ---------------------------------------------------------------------------------------
// Rejection-sampling acceptance: NOT in the reference, whose rule is "draw the target's token
// on every row, accept a draft that equals it" (kernels.metal:1578-1589). This is the
// textbook speculative-sampling rule, defined here so that a GPU kernel has something exact
// to be compared with. Per stream, with k drafts x_1..x_k drawn from q_1..q_k and target rows
// p_0..p_k (row i scores the token after draft i; row 0 the token after the stream's input):
//   P_i = softmax(p_{i-1} / T), Q_i = softmax(q_i / T) over bf16 logits widened to fp32;
//   e(x) = soft_exp2((x - max) * (log2e / T)); Z = sum of e in the sampler's thread-major
//   order (thread t of 1024 adds ids t, t+1024, ...; then tg_scan's association);
//   draft i is accepted iff u_i * eq(x_i) * Zp < ep(x_i) * Zq, the products taken left to
//   right in fp32, u_i = uniform01(seed, pos0 + i, round 0), pos0 the position of draft 1;
//   at the first rejected i the replacement is drawn from r(j) = max(0, ep_j * Zq - eq_j * Zp)
//   by the sampler's inverse CDF (same thread-major order, same scan) at
//   uniform01(seed, pos0 + i, round 1) * sum(r); if that sum is 0, the target's argmax;
//   with all k accepted the bonus token is drawn from P_{k+1} the same way, round 0 of
//   position pos0 + k.
// Outputs: accepted (0..k), the token that follows the accepted drafts, rollback = k - accepted.
inline float logit_of(uint16_t x) { return bf16_to_f32(x); }
inline float logit_of(float x) { return x; }
template <typename T>
inline void softmax_stats(const T* x, uint32_t vocab, float c, float& lmax, uint32_t& amax, float& z) {
    lmax = -FLT_MAX;
    amax = 0xffffffffu;
    for (uint32_t i = 0; i < vocab; i++) better(lmax, amax, logit_of(x[i]), i);
    std::vector<float> s(SAMPLE_THREADS), ex(SAMPLE_THREADS + 1);
    for (uint32_t t = 0; t < SAMPLE_THREADS; t++) {
        float a = 0.0f;
        for (uint32_t i = t; i < vocab; i += SAMPLE_THREADS) a += soft_exp2((logit_of(x[i]) - lmax) * c);
        s[t] = a;
    }
    tg_scan(s.data(), ex.data());
    z = ex[SAMPLE_THREADS];
}

// Inverse CDF over per-id weights w(i) >= 0 in the sampler's order; `fallback` if they sum to 0.
template <typename W>
inline uint32_t inverse_cdf(uint32_t vocab, W w, float u, uint32_t fallback) {
    std::vector<float> s(SAMPLE_THREADS), ex(SAMPLE_THREADS + 1);
    for (uint32_t t = 0; t < SAMPLE_THREADS; t++) {
        float a = 0.0f;
        for (uint32_t i = t; i < vocab; i += SAMPLE_THREADS) a += w(i);
        s[t] = a;
    }
    tg_scan(s.data(), ex.data());
    const float total = ex[SAMPLE_THREADS];
    if (!(total > 0.0f)) return fallback;
    const float target = u * total;
    for (uint32_t t = 0; t < SAMPLE_THREADS; t++) {
        const float lo = ex[t];
        if (lo <= target && target < ex[t + 1]) {
            float acc = 0.0f;
            uint32_t j = 0xffffffffu;
            for (uint32_t i = t; i < vocab; i += SAMPLE_THREADS) {
                float e = w(i);
                acc += e;
                if (e > 0.0f) j = i;
                if (target - lo < acc) break;
            }
            return j == 0xffffffffu ? fallback : j;
        }
    }
    return fallback;
}

struct SpecOut { uint32_t accepted, token, rollback; };
inline SpecOut spec_accept_stream(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t k,
                                  uint32_t vocab, float temperature, uint32_t seed_lo, uint32_t seed_hi, uint32_t pos0) {
    const float c = LOG2E / temperature;
    for (uint32_t i = 0; i < k; i++) {
        const uint16_t* pi = p + uint64_t(i) * vocab;
        const uint16_t* qi = q + uint64_t(i) * vocab;
        float pm, qm, zp, zq;
        uint32_t pa, qa;
        softmax_stats(pi, vocab, c, pm, pa, zp);
        softmax_stats(qi, vocab, c, qm, qa, zq);
        const uint32_t x = drafts[i];
        const float ep = soft_exp2((bf16_to_f32(pi[x]) - pm) * c), eq = soft_exp2((bf16_to_f32(qi[x]) - qm) * c);
        const float u = uniform01(seed_lo, seed_hi, pos0 + i, 0);
        const float lhs = (u * eq) * zp, rhs = ep * zq;
        if (lhs < rhs) continue;
        auto resid = [&](uint32_t j) {
            float a = soft_exp2((bf16_to_f32(pi[j]) - pm) * c) * zq;
            float b = soft_exp2((bf16_to_f32(qi[j]) - qm) * c) * zp;
            float d = a - b;
            return d > 0.0f ? d : 0.0f;
        };
        const uint32_t tok = inverse_cdf(vocab, resid, uniform01(seed_lo, seed_hi, pos0 + i, 1), pa);
        return SpecOut{i, tok, k - i};
    }
    const uint16_t* pk = p + uint64_t(k) * vocab;
    float pm, zp;
    uint32_t pa;
    softmax_stats(pk, vocab, c, pm, pa, zp);
    auto w = [&](uint32_t j) { return soft_exp2((bf16_to_f32(pk[j]) - pm) * c); };
    const uint32_t tok = inverse_cdf(vocab, w, uniform01(seed_lo, seed_hi, pos0 + k, 0), pa);
    return SpecOut{k, tok, 0};
}

// A draft token drawn from softmax(q / T) by the same inverse CDF, round 2 of its position
// (rounds 0 and 1 belong to the acceptance test and the residual draw).
inline uint32_t draw_draft(const uint16_t* q, uint32_t vocab, float temperature, uint32_t seed_lo, uint32_t seed_hi,
                           uint32_t pos) {
    const float c = LOG2E / temperature;
    float qm, zq;
    uint32_t qa;
    softmax_stats(q, vocab, c, qm, qa, zq);
    auto w = [&](uint32_t j) { return soft_exp2((bf16_to_f32(q[j]) - qm) * c); };
    return inverse_cdf(vocab, w, uniform01(seed_lo, seed_hi, pos, 2), qa);
}

// ---------------------------------------------------------------------------------------
// The same rule inside the engine's step (NOT in the reference either), for a verify run whose drafts the chain
// drafter drew in the step before. What differs from spec_accept_stream: the target's rows are the step's fp32
// logits over the whole vocabulary; a draft row q_i is fp32 over the draft vocabulary of `v` ids (id_of[index],
// index_of[id] or NO_TOK), its statistics and the draft's own draw taken in the sampler's order over draft
// indices, and Q is 0 for an id outside that vocabulary (such a draft is rejected); the uniforms are keyed by the
// position of the token they decide (pos[i] for draft i: round 0 the test, round 1 the replacement; the bonus
// token's position is pos[count - 1] + 1, round 0). p: rows 0 .. count - 1 (row i - 1 scores draft i);
// q: rows 1 .. count - 1 at q + (i - 1) * v; x: the run's tokens (x[i] is draft i). Returns the number of
// candidates e = accepted + 1 and leaves them in out[0 .. e): the accepted drafts, then the drawn token.
inline uint32_t spec_step_run(const float* p, uint32_t vocab, const float* q, uint32_t v, const uint32_t* index_of, const uint32_t* x, const uint32_t* pos,
                              uint32_t count, float temperature, uint32_t seed_lo, uint32_t seed_hi, uint32_t* out) {
    const float c = LOG2E / temperature;
    for (uint32_t i = 1; i < count; i++) {
        const float* pi = p + uint64_t(i - 1) * vocab;
        const float* qi = q + uint64_t(i - 1) * v;
        float pm, qm, zp, zq;
        uint32_t pa, qa;
        softmax_stats(pi, vocab, c, pm, pa, zp);
        softmax_stats(qi, v, c, qm, qa, zq);
        const uint32_t tok = x[i], idx = tok < vocab ? index_of[tok] : NO_TOK;
        bool ok = false;
        if (idx != NO_TOK) {
            const float ep = soft_exp2((pi[tok] - pm) * c), eq = soft_exp2((qi[idx] - qm) * c);
            const float u = uniform01(seed_lo, seed_hi, pos[i], 0);
            ok = (u * eq) * zp < ep * zq;
        }
        if (ok) { out[i - 1] = tok; continue; }
        auto resid = [&](uint32_t j) {
            const float a = soft_exp2((pi[j] - pm) * c) * zq;
            const float b = index_of[j] == NO_TOK ? 0.0f : soft_exp2((qi[index_of[j]] - qm) * c) * zp;
            const float d = a - b;
            return d > 0.0f ? d : 0.0f;
        };
        out[i - 1] = inverse_cdf(vocab, resid, uniform01(seed_lo, seed_hi, pos[i], 1), pa);
        return i;
    }
    const float* pk = p + uint64_t(count - 1) * vocab;
    float pm, zp;
    uint32_t pa;
    softmax_stats(pk, vocab, c, pm, pa, zp);
    auto w = [&](uint32_t j) { return soft_exp2((pk[j] - pm) * c); };
    out[count - 1] = inverse_cdf(vocab, w, uniform01(seed_lo, seed_hi, pos[count - 1] + 1, 0), pa);
    return count;
}

// The chain drafter's draw for that rule: draft index from softmax(q / T) over the draft vocabulary by the same
// inverse CDF, round 2 of the drafted token's position.
inline uint32_t draw_draft_index(const float* q, uint32_t v, float temperature, uint32_t seed_lo, uint32_t seed_hi, uint32_t pos) {
    const float c = LOG2E / temperature;
    float qm, zq;
    uint32_t qa;
    softmax_stats(q, v, c, qm, qa, zq);
    auto w = [&](uint32_t j) { return soft_exp2((q[j] - qm) * c); };
    return inverse_cdf(v, w, uniform01(seed_lo, seed_hi, pos, 2), qa);
}

}  // namespace orc
