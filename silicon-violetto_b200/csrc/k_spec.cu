// Rejection-sampling acceptance over draft and target logits (not in the reference, whose rule
// is "draw the target's token on every row and accept a draft that equals it",
// kernels.metal:1578-1589; this is the textbook speculative-sampling rule, built on the
// reference sampler's conventions so that it can be checked bit for bit).
//
// Per stream, with k drafts x_1..x_k drawn from q_1..q_k and target rows p_0..p_k (bf16 logits):
//   e(x) = 2^((x - max) log2(e) / T) with the sampler's exp2; Z = the sum of e in the sampler's
//   order (thread t of 1024 adds ids t, t + 1024, ...; then tg_scan's association);
//   draft i is accepted iff (u_i * eq(x_i)) * Zp < ep(x_i) * Zq, u_i = uniform01(seed, pos0 + i, 0);
//   at the first rejected i the replacement is drawn from max(0, ep_j Zq - eq_j Zp) by the sampler's
//   inverse CDF at uniform01(seed, pos0 + i, 1); with all accepted, the bonus token from p_k at
//   uniform01(seed, pos0 + k, 0). Outputs: accepted count, that token, rollback = k - accepted.
// Two kernels: per-row statistics (max, argmax, Z) for all S (2k + 1) rows at once -- one pass
// over the logits from HBM -- then a cluster of 8 blocks per stream that decides and draws (its two rows
// come from L2).
#include <cfloat>
#include <cmath>
#include <mutex>

#include "kernels.h"
#include "sampling.cuh"

namespace vlt {

namespace spec {

constexpr uint32_t THREADS = 1024;
__device__ __forceinline__ uint32_t ex_at(uint32_t t) { return t + t / 32; }

// kernels.metal:1482-1501 `tg_scan` (see k_small.cu).
__device__ void tg_scan(float v, float* ex, float* base, uint32_t tid) {
    ex[ex_at(tid)] = v;
    __syncthreads();
    if (tid < 32) {
        float acc = 0.0f;
        for (uint32_t i = 32 * tid; i < 32 * tid + 32; i++) {
            const float x = ex[ex_at(i)];
            ex[ex_at(i)] = acc;
            acc = __fadd_rn(acc, x);
        }
        base[tid] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        float acc = 0.0f;
        for (uint32_t g = 0; g < 32; g++) {
            const float x = base[g];
            base[g] = acc;
            acc = __fadd_rn(acc, x);
        }
        ex[ex_at(THREADS)] = acc;
    }
    __syncthreads();
    ex[ex_at(tid)] = __fadd_rn(ex[ex_at(tid)], base[tid / 32]);
    __syncthreads();
}

using vlt::SpecRowStats;
typedef SpecRowStats RowStats;

__device__ __forceinline__ float e_of(uint16_t x, float mx, float c) { return soft_exp2(__fmul_rn(__fsub_rn(bf16_to_f32(x), mx), c)); }

// One block per row of logits (p rows first, then q rows): max, argmax (ties to the lowest id), Z.
__global__ void __launch_bounds__(THREADS) stats_kernel(const uint16_t* __restrict__ p, const uint16_t* __restrict__ q, uint32_t p_rows, uint32_t vocab,
                                                        float c, RowStats* out) {
    __shared__ float ex[THREADS + THREADS / 32 + 1];
    __shared__ float base[32];
    __shared__ float bvs[32];
    __shared__ uint32_t bis[32];
    const uint32_t r = blockIdx.x, tid = threadIdx.x, lane = tid % 32;
    const uint16_t* x = r < p_rows ? p + size_t(r) * vocab : q + size_t(r - p_rows) * vocab;
    float mx = -FLT_MAX;
    uint32_t am = 0xffffffffu;
    {
        uint32_t i0 = tid;
        for (; i0 + 7 * THREADS < vocab; i0 += 8 * THREADS) {
            uint16_t v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = x[i0 + u * THREADS];
#pragma unroll
            for (int u = 0; u < 8; u++) better(mx, am, bf16_to_f32(v[u]), i0 + u * THREADS);
        }
        for (; i0 < vocab; i0 += THREADS) better(mx, am, bf16_to_f32(x[i0]), i0);
    }
    warp_best(mx, am);
    if (lane == 0) { bvs[tid / 32] = mx; bis[tid / 32] = am; }
    __syncthreads();
    mx = bvs[0];
    am = bis[0];
    for (uint32_t i = 1; i < 32; i++) better(mx, am, bvs[i], bis[i]);
    float s = 0.0f;
    uint32_t i0 = tid;
    for (; i0 + 7 * THREADS < vocab; i0 += 8 * THREADS) {  // eight loads in flight, the additions in id order
        uint16_t v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = x[i0 + u * THREADS];
#pragma unroll
        for (int u = 0; u < 8; u++) s = __fadd_rn(s, e_of(v[u], mx, c));
    }
    for (; i0 < vocab; i0 += THREADS) s = __fadd_rn(s, e_of(x[i0], mx, c));
    tg_scan(s, ex, base, tid);
    if (tid == 0) out[r] = RowStats{mx, am, ex[ex_at(THREADS)], 0};
}

// The sampler's inverse CDF (kernels.metal:1540-1559) over weights w(i) >= 0; `fallback` if they
// sum to 0 or the target falls past the last term.
template <typename W>
__device__ uint32_t inverse_cdf(uint32_t vocab, W w, float u, uint32_t fallback, float* ex, float* base, uint32_t* pick, uint32_t tid) {
    float a = 0.0f;
    for (uint32_t i = tid; i < vocab; i += THREADS) a = __fadd_rn(a, w(i));
    tg_scan(a, ex, base, tid);
    const float total = ex[ex_at(THREADS)];
    if (!(total > 0.0f)) return fallback;
    const float target = __fmul_rn(u, total);
    if (tid == 0) *pick = 0xffffffffu;
    __syncthreads();
    const float lo = ex[ex_at(tid)];
    // The one thread whose interval holds the target re-adds its terms in order until they pass it; its warp helps:
    // the lanes evaluate 32 of its ids at a time, and only the additions stay in the thread's order.
    const bool mine = lo <= target && target < ex[ex_at(tid + 1)];
    const uint32_t owners = __ballot_sync(0xffffffffu, mine);
    if (owners) {
        const uint32_t lane = tid % 32;
        const int src = __ffs(owners) - 1;
        const uint32_t first = __shfl_sync(0xffffffffu, tid, src);
        const float rest = __fsub_rn(target, __shfl_sync(0xffffffffu, lo, src));
        float acc = 0.0f;
        uint32_t j = 0xffffffffu;
        bool done = false;
        for (uint32_t i0 = first; i0 < vocab && !done; i0 += 32 * THREADS) {
            const uint32_t i = i0 + lane * THREADS;
            const float e = i < vocab ? w(i) : 0.0f;
            const uint32_t n_live = min(32u, (vocab - i0 + THREADS - 1) / THREADS);
            for (uint32_t l = 0; l < n_live && !done; l++) {
                const float el = __shfl_sync(0xffffffffu, e, l);
                acc = __fadd_rn(acc, el);
                if (el > 0.0f) j = i0 + l * THREADS;
                if (rest < acc) done = true;
            }
        }
        if (int(lane) == src) *pick = j;
    }
    __syncthreads();
    const uint32_t j = *pick;
    return j == 0xffffffffu ? fallback : j;
}

// The decision, a cluster of 8 blocks per stream: the 1024 "threads" of the sampler's order are the cluster's 8 x 128 (as
// in the sampler's cluster form), so every sum keeps its order and association while a stream's pass over its two rows
// runs on eight SMs (one block per stream left 116 of 148 SMs idle at 32 streams).
__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS) decide_cluster_kernel(const uint16_t* __restrict__ p, const uint16_t* __restrict__ q,
                                                                                                 const uint32_t* __restrict__ drafts, const RowStats* __restrict__ stats,
                                                                                                 uint32_t streams, uint32_t k, uint32_t vocab, float c,
                                                                                                 const uint64_t* __restrict__ seeds, const uint32_t* __restrict__ pos0,
                                                                                                 uint32_t* accepted, uint32_t* token, uint32_t* rollback) {
    __shared__ ScExchange xc;
    __shared__ float vals[SC_THREADS], pre[SC_THREADS], tot_all[32], base[33];
    __shared__ uint32_t first_reject;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const uint32_t s = blockIdx.x / SC_CTAS, tid = threadIdx.x;
    const uint32_t seed_lo = uint32_t(seeds[s]), seed_hi = uint32_t(seeds[s] >> 32);
    const RowStats* ps = stats + size_t(s) * (k + 1);
    const RowStats* qs = stats + size_t(streams) * (k + 1) + size_t(s) * k;
    const uint16_t* pp = p + size_t(s) * (k + 1) * vocab;
    const uint16_t* qq = q + size_t(s) * k * vocab;
    if (tid == 0) {  // every block runs the few tests itself: cheaper than sending the result round
        uint32_t i = 0;
        for (; i < k; i++) {
            const uint32_t x = drafts[s * k + i];
            const float ep = e_of(pp[size_t(i) * vocab + x], ps[i].max, c), eq = e_of(qq[size_t(i) * vocab + x], qs[i].max, c);
            const float u = uniform01(seed_lo, seed_hi, pos0[s] + i, 0);
            const float lhs = __fmul_rn(__fmul_rn(u, eq), ps[i].z), rhs = __fmul_rn(ep, qs[i].z);
            if (!(lhs < rhs)) break;
        }
        first_reject = i;
        xc.pick[0] = 0xffffffffu;
        xc.pick[1] = 0xffffffffu;
    }
    __syncthreads();
    const uint32_t i = first_reject;
    uint32_t tok;
    if (i < k) {
        const uint16_t* pi = pp + size_t(i) * vocab;
        const uint16_t* qi = qq + size_t(i) * vocab;
        const float pm = ps[i].max, qm = qs[i].max, zp = ps[i].z, zq = qs[i].z;
        auto resid = [&](uint32_t j) {
            const float a = __fmul_rn(e_of(pi[j], pm, c), zq), b = __fmul_rn(e_of(qi[j], qm, c), zp);
            const float d = __fsub_rn(a, b);
            return d > 0.0f ? d : 0.0f;
        };
        tok = sc_inverse_cdf(vocab, resid, uniform01(seed_lo, seed_hi, pos0[s] + i, 1), ps[i].argmax, &xc, 0, 0, vals, pre, tot_all, base, rank, tid);
    } else {
        const uint16_t* pk = pp + size_t(k) * vocab;
        const float pm = ps[k].max;
        auto w = [&](uint32_t j) { return e_of(pk[j], pm, c); };
        tok = sc_inverse_cdf(vocab, w, uniform01(seed_lo, seed_hi, pos0[s] + k, 0), ps[k].argmax, &xc, 0, 0, vals, pre, tot_all, base, rank, tid);
    }
    if (rank == 0 && tid == 0) {
        accepted[s] = i;
        token[s] = tok;
        rollback[s] = k - i;
    }
    sc_cluster_sync();  // nobody leaves while another block may still read its shared memory
}

}  // namespace spec

// p [S][k+1][V], q [S][k][V] bf16 on the device; stats: scratch for S (2k + 1) rows of 16 bytes.
void launch_spec_accept(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, uint32_t vocab, float temperature,
                        const uint64_t* seeds, const uint32_t* pos0, void* stats, uint32_t* accepted, uint32_t* token, uint32_t* rollback, cudaStream_t s) {
    const float c = LOG2E / temperature;  // the same IEEE division as the device's __fdiv_rn
    spec::stats_kernel<<<streams * (2 * k + 1), spec::THREADS, 0, s>>>(p, q, streams * (k + 1), vocab, c, static_cast<spec::RowStats*>(stats));
    launch_counter()++;
    spec::decide_cluster_kernel<<<streams * SC_CTAS, SC_THREADS, 0, s>>>(p, q, drafts, static_cast<const spec::RowStats*>(stats), streams, k, vocab, c, seeds, pos0,
                                                                        accepted, token, rollback);
    launch_counter()++;
}

// ------------------------------------------------ the rule inside the engine's step
// A verify run whose drafts the chain drafter drew (from softmax(q / T), keeping the q rows) in the step before is
// decided by the rule above instead of the reference's sample-then-match. What differs from the stand-alone form:
// the target's rows are the step's fp32 logits over the whole vocabulary; a q row is fp32 over the draft vocabulary
// (v ids, `index_of` maps a target id to its index or NO_TOK), its statistics taken in the sampler's order over
// draft indices, Q being 0 for an id outside it (such a draft is rejected); the uniforms are keyed by the position
// of the token they decide (round 0 the test, round 1 the replacement; the bonus token at the last row's position
// + 1, round 0). The kernels leave the run's candidates -- the accepted drafts, then the drawn token -- in
// out[head0 ..] and their number in spec_e[run]; `accept_kernel` then commits them exactly as it commits a walk
// of the reference's rule (lens, feed, path, on_path, gen, emitted), so rejected rows are rolled back the same
// way: the sequence advances by what was accepted and the K/V past it is overwritten by the next step.
namespace spec {

// Whether run r is decided by this rule: a verify run of a sequence that samples (temperature > 0, no top-p cut),
// whose rows are a plain chain and whose drafts all came with a kept q row. Uniform over a block.
__device__ bool step_applies(const SpecStepArgs& a, uint32_t r) {
    const RunIn ru = a.runs[r];
    if (!ru.verify || ru.count < 2 || ru.nhead != ru.count || ru.count > VERIFY_T) return false;
    const SampleRow sr = a.samples[ru.head0];
    if (!(sr.temperature > 0.0f) || sr.top_p < 1.0f) return false;
    if (a.q_rows[ru.slot] + 1 < ru.count) return false;
    for (uint32_t c = 1; c < ru.count; c++)
        if (a.tree[ru.slot * FEED_W + c] != d_chain_node(c)) return false;
    return true;
}

// One block per row: the step's head rows first, then VERIFY_T - 1 q rows per run. Rows of runs the rule does
// not decide are left alone (and marked for the sampler: row_skip 0); the others get (max, argmax, Z).
__global__ void __launch_bounds__(THREADS) step_stats_kernel(const SpecStepArgs a) {
    pdl_start();
    __shared__ float ex[THREADS + THREADS / 32 + 1];
    __shared__ float base[32];
    __shared__ float bvs[32];
    __shared__ uint32_t bis[32];
    const uint32_t b = blockIdx.x, tid = threadIdx.x, lane = tid % 32;
    const float* x;
    uint32_t n, r;
    RowStats* out;
    if (b < a.n_head) {
        for (r = 0; r < a.n_runs; r++)
            if (b >= a.runs[r].head0 && b < a.runs[r].head0 + a.runs[r].nhead) break;
        const bool on = r < a.n_runs && step_applies(a, r);
        if (tid == 0) a.row_skip[b] = on ? 1u : 0u;
        if (!on) return;
        x = a.logits + size_t(b) * a.vocab;
        n = a.vocab;
        out = a.stats + b;
    } else {
        r = (b - a.n_head) / (VERIFY_T - 1);
        const uint32_t i = (b - a.n_head) % (VERIFY_T - 1) + 1;
        if (!step_applies(a, r) || i >= a.runs[r].count) return;
        x = a.q_keep + (size_t(a.runs[r].slot) * (VERIFY_T - 1) + i - 1) * a.v;
        n = a.v;
        out = a.stats + a.max_head_rows + r * (VERIFY_T - 1) + i - 1;
    }
    const float c = __fdiv_rn(LOG2E, a.samples[a.runs[r].head0].temperature);
    float mx = -FLT_MAX;
    uint32_t am = 0xffffffffu;
    for (uint32_t i = tid; i < n; i += THREADS) better(mx, am, x[i], i);
    warp_best(mx, am);
    if (lane == 0) { bvs[tid / 32] = mx; bis[tid / 32] = am; }
    __syncthreads();
    mx = bvs[0];
    am = bis[0];
    for (uint32_t i = 1; i < 32; i++) better(mx, am, bvs[i], bis[i]);
    float s = 0.0f;
    uint32_t i0 = tid;
    for (; i0 + 7 * THREADS < n; i0 += 8 * THREADS) {  // eight loads in flight, the additions in id order
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = x[i0 + u * THREADS];
#pragma unroll
        for (int u = 0; u < 8; u++) s = __fadd_rn(s, soft_exp2(__fmul_rn(__fsub_rn(v[u], mx), c)));
    }
    for (; i0 < n; i0 += THREADS) s = __fadd_rn(s, soft_exp2(__fmul_rn(__fsub_rn(x[i0], mx), c)));
    tg_scan(s, ex, base, tid);
    if (tid == 0) *out = RowStats{mx, am, ex[ex_at(THREADS)], 0};
}

// A cluster of 8 blocks per run (the sampler's 1024 threads, see decide_cluster_kernel): the tests (a lane each, in
// every block), then the replacement or the bonus token (the cluster).
__global__ void __cluster_dims__(SC_CTAS, 1, 1) __launch_bounds__(SC_THREADS) step_decide_kernel(const SpecStepArgs a) {
    pdl_start();
    __shared__ ScExchange xc;
    __shared__ float vals[SC_THREADS], pre[SC_THREADS], tot_all[32], base[33];
    __shared__ uint32_t first_reject;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const uint32_t r = blockIdx.x / SC_CTAS, tid = threadIdx.x;
    const RunIn ru = a.runs[r];
    const bool on = step_applies(a, r);
    sc_cluster_sync();  // every thread of the cluster has read q_rows
    if (rank == 0 && tid == 0) {
        a.q_rows[ru.slot] = 0;  // a slot's kept rows serve one step
        if (!on) a.spec_e[r] = 0;
    }
    if (!on) return;  // the whole cluster leaves: no further cluster barrier
    const SampleRow sr = a.samples[ru.head0];
    const float c = __fdiv_rn(LOG2E, sr.temperature);
    const RowStats* ps = a.stats + ru.head0;
    const RowStats* qs = a.stats + a.max_head_rows + r * (VERIFY_T - 1);
    const float* pp = a.logits + size_t(ru.head0) * a.vocab;
    const float* qq = a.q_keep + size_t(ru.slot) * (VERIFY_T - 1) * a.v;
    auto e_of = [&](float x, float mx) { return soft_exp2(__fmul_rn(__fsub_rn(x, mx), c)); };
    // The tests, one lane each (every block of the cluster does them), so that the loads of all of them are in flight at
    // once; the first that fails, or whose draft is outside the draft vocabulary, is where the run stops.
    if (tid < 32) {
        bool fails = false;  // a lane without a test does not fail
        if (tid + 1 < ru.count) {
            const uint32_t i = tid + 1;
            const uint32_t tok = a.tokens[ru.first + i], idx = tok < a.vocab ? a.index_of[tok] : NO_TOK;
            fails = true;
            if (idx != NO_TOK) {
                const float ep = e_of(pp[size_t(i - 1) * a.vocab + tok], ps[i - 1].max), eq = e_of(qq[size_t(i - 1) * a.v + idx], qs[i - 1].max);
                const float u = uniform01(sr.seed_lo, sr.seed_hi, a.meta[2 * (ru.first + i) + 1], 0);
                const float lhs = __fmul_rn(__fmul_rn(u, eq), ps[i - 1].z), rhs = __fmul_rn(ep, qs[i - 1].z);
                fails = !(lhs < rhs);
            }
        }
        const uint32_t failed = __ballot_sync(0xffffffffu, fails);  // lane t holds test t + 1
        if (tid == 0) {
            first_reject = failed ? uint32_t(__ffs(failed)) : ru.count;
            xc.pick[0] = 0xffffffffu;
            xc.pick[1] = 0xffffffffu;
        }
    }
    __syncthreads();
    const uint32_t i = first_reject;
    uint32_t tok;
    if (i < ru.count) {
        const float* pi = pp + size_t(i - 1) * a.vocab;
        const float* qi = qq + size_t(i - 1) * a.v;
        const float pm = ps[i - 1].max, qm = qs[i - 1].max, zp = ps[i - 1].z, zq = qs[i - 1].z;
        const uint32_t* index_of = a.index_of;
        auto resid = [&](uint32_t j) {
            const uint32_t idx = index_of[j];
            const float qv = qi[idx == NO_TOK ? 0u : idx];  // an unconditional load: a batch's loads all go out before the arithmetic
            const float ea = __fmul_rn(e_of(pi[j], pm), zq), eb = idx == NO_TOK ? 0.0f : __fmul_rn(e_of(qv, qm), zp);
            const float d = __fsub_rn(ea, eb);
            return d > 0.0f ? d : 0.0f;
        };
        // A batch in three rounds of loads (draft index and p; q through the index), then the arithmetic.
        constexpr int B = 16;
        auto resid_batch = [&](uint32_t i0, float (&e)[B]) {
            uint32_t idx[B];
            float pv[B], qv[B];
#pragma unroll
            for (int u = 0; u < B; u++) {
                idx[u] = index_of[i0 + u * SAMPLE_THREADS];
                pv[u] = pi[i0 + u * SAMPLE_THREADS];
            }
#pragma unroll
            for (int u = 0; u < B; u++) qv[u] = qi[idx[u] == NO_TOK ? 0u : idx[u]];
#pragma unroll
            for (int u = 0; u < B; u++) {
                const float ea = __fmul_rn(e_of(pv[u], pm), zq), eb = idx[u] == NO_TOK ? 0.0f : __fmul_rn(e_of(qv[u], qm), zp);
                const float d = __fsub_rn(ea, eb);
                e[u] = d > 0.0f ? d : 0.0f;
            }
        };
        tok = sc_inverse_cdf_batched<B>(a.vocab, resid, resid_batch, uniform01(sr.seed_lo, sr.seed_hi, a.meta[2 * (ru.first + i) + 1], 1), ps[i - 1].argmax, &xc, 0, 0, vals, pre,
                                        tot_all, base, rank, tid);
    } else {
        const float* pk = pp + size_t(ru.count - 1) * a.vocab;
        const float pm = ps[ru.count - 1].max;
        auto w = [&](uint32_t j) { return e_of(pk[j], pm); };
        tok = sc_inverse_cdf<16>(a.vocab, w, uniform01(sr.seed_lo, sr.seed_hi, a.meta[2 * (ru.first + ru.count - 1) + 1] + 1, 0), ps[ru.count - 1].argmax, &xc, 0, 0, vals, pre, tot_all, base, rank, tid);
    }
    if (rank == 0 && tid == 0) {
        for (uint32_t j = 0; j + 1 < i; j++) a.out[ru.head0 + j] = a.tokens[ru.first + j + 1];
        a.out[ru.head0 + i - 1] = tok;
        a.spec_e[r] = i;
    }
    sc_cluster_sync();  // nobody leaves while another block may still read its shared memory
}

// The chain drafter's pick for pass i, one block per run: the draft vocabulary's argmax (ties to the lowest
// index), or -- under the rule, for a sequence that samples -- a draw from softmax(q / T) by the sampler's
// inverse CDF at round 2 of the drafted token's position, the row kept for the next step's test.
__global__ void __launch_bounds__(THREADS) draft_draw_kernel(const float* __restrict__ logits, uint32_t v, const uint32_t* __restrict__ vocab_ids,
                                                             const RunIn* __restrict__ runs, const SampleRow* __restrict__ samples,
                                                             const uint32_t* __restrict__ live, const uint32_t* __restrict__ lens, uint32_t i, uint32_t rule,
                                                             uint32_t* feed, uint32_t* tree, float* q_keep, uint32_t* q_rows) {
    pdl_start();
    __shared__ float ex[THREADS + THREADS / 32 + 1];
    __shared__ float base[32];
    __shared__ float bvs[32];
    __shared__ uint32_t bis[32];
    __shared__ uint32_t pick;
    const uint32_t r = blockIdx.x, tid = threadIdx.x, lane = tid % 32;
    if (!live[r]) return;
    const RunIn ru = runs[r];
    const float* row = logits + size_t(r) * v;
    float mx = -FLT_MAX;
    uint32_t am = 0xffffffffu;
    for (uint32_t j = tid; j < v; j += THREADS) better(mx, am, row[j], j);
    warp_best(mx, am);
    if (lane == 0) { bvs[tid / 32] = mx; bis[tid / 32] = am; }
    __syncthreads();
    mx = bvs[0];
    am = bis[0];
    for (uint32_t j = 1; j < 32; j++) better(mx, am, bvs[j], bis[j]);
    const SampleRow sr = samples[ru.head0];
    const bool draws = rule == 1 && sr.temperature > 0.0f && sr.top_p >= 1.0f;
    uint32_t idx = am;
    if (draws) {
        const float c = __fdiv_rn(LOG2E, sr.temperature);
        auto w = [&](uint32_t j) { return soft_exp2(__fmul_rn(__fsub_rn(row[j], mx), c)); };
        idx = inverse_cdf(v, w, uniform01(sr.seed_lo, sr.seed_hi, lens[ru.slot] + i, 2), am, ex, base, &pick, tid);
        float* keep = q_keep + (size_t(ru.slot) * (VERIFY_T - 1) + i - 1) * v;
        for (uint32_t j = tid; j < v; j += THREADS) keep[j] = row[j];
    }
    if (tid == 0) {
        feed[ru.slot * FEED_W + i] = vocab_ids[idx < v ? idx : 0];
        tree[ru.slot * FEED_W + i] = d_chain_node(i);
        if (draws) q_rows[ru.slot] = i;
        else if (i == 1) q_rows[ru.slot] = 0;
    }
}

}  // namespace spec

void launch_spec_step_stats(const SpecStepArgs& a, cudaStream_t s) {
    launch_pdl(spec::step_stats_kernel, a.n_head + a.n_runs * (VERIFY_T - 1), spec::THREADS, 0, s, a);
}
void launch_spec_step_decide(const SpecStepArgs& a, cudaStream_t s) {
    launch_pdl(spec::step_decide_kernel, a.n_runs * SC_CTAS, SC_THREADS, 0, s, a);
}
void launch_draft_draw(const float* logits, uint32_t v, const uint32_t* vocab_ids, const RunIn* runs, const SampleRow* samples, const uint32_t* live,
                       const uint32_t* lens, uint32_t n_runs, uint32_t i, uint32_t rule, uint32_t* feed, uint32_t* tree, float* q_keep, uint32_t* q_rows,
                       cudaStream_t s) {
    launch_pdl(spec::draft_draw_kernel, n_runs, spec::THREADS, 0, s, logits, v, vocab_ids, runs, samples, live, lens, i, rule, feed, tree, q_keep, q_rows);
}

// ------------------------------------------------ the same, with nothing allocated
// A variant for callers that cannot allocate device memory when they need an acceptance step:
// a serving loop that has handed every byte of the device to its own pools, or one that must not
// pay the device-wide synchronisation an allocation or a free can imply in the middle of decoding.
// Its scratch (the per-row statistics, and a bounds-checked copy of the draft ids) lives in
// file-scope device arrays of a fixed size, so a step may cover at most STATIC_MAX_ROWS rows of
// logits. The arrays' addresses are looked up once per device, on the first call made with that
// device current; that first call is set-up and belongs before the caller starts any stream
// capture. All calls on a device share the arrays: nothing in them has to start at zero (the first
// kernel overwrites every word the later ones read), but two calls in flight at once on one
// device race on them.
namespace spec {

constexpr uint32_t STATIC_MAX_ROWS = 2048;  // streams * (2 k + 1) rows of logits a call may cover
static __device__ __align__(256) RowStats static_stats[STATIC_MAX_ROWS];
static __device__ __align__(256) uint32_t static_drafts[STATIC_MAX_ROWS];

// The caller's draft ids cannot be checked on the host here; an id past the vocabulary is read as 0
// instead of indexing out of the logits (that stream's result then means nothing).
__global__ void copy_drafts_kernel(const uint32_t* __restrict__ drafts, uint32_t n, uint32_t vocab, uint32_t* out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = drafts[i] < vocab ? drafts[i] : 0u;
}

struct StaticScratch {
    RowStats* stats;
    uint32_t* drafts;
};

// The arrays' addresses on the current device; looked up (cudaGetSymbolAddress) on the first call per device.
static const char* static_scratch(StaticScratch* out) {
    constexpr int MAX_DEVICES = 64;
    static StaticScratch table[MAX_DEVICES] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return "spec_accept_static: no usable current device";
    std::lock_guard<std::mutex> lock(mu);
    if (!table[dev].stats) {
        void* ps = nullptr;
        void* pd = nullptr;
        if (cudaGetSymbolAddress(&ps, static_stats) != cudaSuccess || !ps) return "spec_accept_static: cudaGetSymbolAddress failed for the statistics array";
        if (cudaGetSymbolAddress(&pd, static_drafts) != cudaSuccess || !pd) return "spec_accept_static: cudaGetSymbolAddress failed for the draft array";
        table[dev].drafts = static_cast<uint32_t*>(pd);
        table[dev].stats = static_cast<RowStats*>(ps);
    }
    *out = table[dev];
    return nullptr;
}

}  // namespace spec

uint32_t spec_accept_static_max_rows() { return spec::STATIC_MAX_ROWS; }

// Every pointer is device memory of the current device. Returns NULL, or a message (a string literal:
// this path does not allocate on the host either).
const char* launch_spec_accept_static(const uint16_t* p, const uint16_t* q, const uint32_t* drafts, uint32_t streams, uint32_t k, uint32_t vocab,
                                      float temperature, const uint64_t* seeds, const uint32_t* pos0, uint32_t* accepted, uint32_t* token,
                                      uint32_t* rollback, cudaStream_t s) {
    if (!p || !q || !drafts || !seeds || !pos0 || !accepted || !token || !rollback) return "spec_accept_static: null pointer";
    if (streams == 0 || k == 0 || k > 15 || vocab == 0) return "spec_accept_static: needs at least one stream, 1..15 drafts and a vocabulary";
    if (!(std::isnormal(temperature) && temperature > 0.0f)) return "spec_accept_static: needs a normal positive temperature";
    if (uint64_t(streams) * (2 * k + 1) > spec::STATIC_MAX_ROWS)
        return "spec_accept_static: streams * (2 k + 1) exceeds the 2048 rows the static scratch holds; use vlt_spec_accept";
    spec::StaticScratch sc{};
    if (const char* e = spec::static_scratch(&sc)) return e;
    const uint32_t n = streams * k;
    spec::copy_drafts_kernel<<<(n + 255) / 256, 256, 0, s>>>(drafts, n, vocab, sc.drafts);
    launch_counter()++;
    launch_spec_accept(p, q, sc.drafts, streams, k, vocab, temperature, seeds, pos0, sc.stats, accepted, token, rollback, s);
    return cudaGetLastError() == cudaSuccess ? nullptr : "spec_accept_static: kernel launch failed";
}

}  // namespace vlt
