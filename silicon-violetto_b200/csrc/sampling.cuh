// Device helpers shared by the kernels that sum and invert a distribution in the reference sampler's order
// (kernels.metal:1482-1559): the padded scan index, and the scan over a cluster of 8 blocks that stands for the
// reference's 1024 threads.
#pragma once
#include "device.cuh"

namespace vlt {

constexpr uint32_t SAMPLE_THREADS = 1024;
__device__ __forceinline__ uint32_t ex_at(uint32_t t) { return t + t / 32; }

constexpr uint32_t SC_CTAS = 8, SC_THREADS = SAMPLE_THREADS / SC_CTAS, SC_WARPS = SC_THREADS / 32;
__device__ __forceinline__ void sc_cluster_sync() { asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t sc_remote(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(uint32_t(__cvta_generic_to_shared(p))), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t sc_ld_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

struct ScExchange {
    float tot[2][SC_WARPS];  // this block's group totals, double-buffered by scan
    uint32_t pick[2];        // the id a thread of this block picked (NO_TOK: none), double-buffered by round
    float bv;                // this block's best logit and its id
    uint32_t bi;
};

// tg_scan over the cluster. v: this thread's sum. Returns ex[t] (lo), ex[t + 1] (hi) and ex[1024] (total).
__device__ inline void sc_scan(float v, uint32_t buf, ScExchange* xc, float* vals, float* pre, float* tot_all, float* base, uint32_t rank, uint32_t tid, float& lo,
                        float& hi, float& total) {
    const uint32_t lane = tid % 32, warp = tid / 32;
    vals[tid] = v;
    __syncthreads();
    if (tid < SC_WARPS) {  // a group's exclusive prefixes, left to right from 0
        float acc = 0.0f;
        for (uint32_t i = 32 * tid; i < 32 * tid + 32; i++) {
            pre[i] = acc;
            acc = __fadd_rn(acc, vals[i]);
        }
        xc->tot[buf][tid] = acc;
    }
    sc_cluster_sync();
    if (tid < 32) tot_all[tid] = __uint_as_float(sc_ld_u32(sc_remote(&xc->tot[buf][tid % SC_WARPS], tid / SC_WARPS)));
    __syncthreads();
    if (tid == 0) {  // the group totals scanned left to right from 0
        float acc = 0.0f;
        for (uint32_t g = 0; g < 32; g++) {
            base[g] = acc;
            acc = __fadd_rn(acc, tot_all[g]);
        }
        base[32] = acc;
    }
    __syncthreads();
    const uint32_t group = rank * SC_WARPS + warp;
    lo = __fadd_rn(pre[tid], base[group]);
    hi = __shfl_down_sync(0xffffffffu, lo, 1);
    if (lane == 31) hi = base[group + 1];
    total = base[32];
}


// The sampler's inverse CDF (kernels.metal:1540-1559) over weights w(i) >= 0 across a cluster: thread vt of the cluster's
// 1024 owns ids vt, vt + 1024, ...; the one thread whose interval holds the target re-adds its terms in order until they
// pass it, its warp evaluating 32 of them at a time. `fallback` if the weights sum to 0 or the target falls past the last
// term. xc->pick[pb] must hold NO_TOK in every block on entry. Every block of the cluster returns the same id.
// This is the part after a thread's whole batches (sc_inverse_cdf and sc_inverse_cdf_batched below): `a` is its sum so
// far, `i0` its next id.
template <typename W>
__device__ inline uint32_t sc_inverse_cdf_rest(uint32_t vocab, W w, float a, uint32_t i0, float u, uint32_t fallback, ScExchange* xc, uint32_t buf, uint32_t pb, float* vals,
                                        float* pre, float* tot_all, float* base, uint32_t rank, uint32_t tid) {
    const uint32_t lane = tid % 32, vt = rank * SC_THREADS + tid;
    for (; i0 < vocab; i0 += SAMPLE_THREADS) a = __fadd_rn(a, w(i0));
    float lo, hi, total;
    sc_scan(a, buf, xc, vals, pre, tot_all, base, rank, tid, lo, hi, total);
    if (!(total > 0.0f)) return fallback;
    const float target = __fmul_rn(u, total);
    const uint32_t owners = __ballot_sync(0xffffffffu, lo <= target && target < hi);
    if (owners) {
        const int src = __ffs(owners) - 1;
        const uint32_t first = __shfl_sync(0xffffffffu, vt, src);
        const float rest = __fsub_rn(target, __shfl_sync(0xffffffffu, lo, src));
        float acc = 0.0f;
        uint32_t j = 0xffffffffu;
        bool done = false;
        for (uint32_t i0 = first; i0 < vocab && !done; i0 += 32 * SAMPLE_THREADS) {
            const uint32_t i = i0 + lane * SAMPLE_THREADS;
            const float e = i < vocab ? w(i) : 0.0f;
            const uint32_t n_live = min(32u, (vocab - i0 + SAMPLE_THREADS - 1) / SAMPLE_THREADS);
            for (uint32_t l = 0; l < n_live && !done; l++) {
                const float el = __shfl_sync(0xffffffffu, e, l);
                acc = __fadd_rn(acc, el);
                if (el > 0.0f) j = i0 + l * SAMPLE_THREADS;
                if (rest < acc) done = true;
            }
        }
        if (int(lane) == src) xc->pick[pb] = j;
    }
    sc_cluster_sync();
    uint32_t j = 0xffffffffu;
    for (uint32_t s = 0; s < SC_CTAS; s++) {
        const uint32_t pj = sc_ld_u32(sc_remote(&xc->pick[pb], s));
        if (pj != 0xffffffffu) j = pj;
    }
    return j == 0xffffffffu ? fallback : j;
}

template <int B = 8, typename W>
__device__ inline uint32_t sc_inverse_cdf(uint32_t vocab, W w, float u, uint32_t fallback, ScExchange* xc, uint32_t buf, uint32_t pb, float* vals, float* pre, float* tot_all,
                                   float* base, uint32_t rank, uint32_t tid) {
    float a = 0.0f;
    uint32_t i0 = rank * SC_THREADS + tid;
    for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {  // B weights' loads in flight, the additions in id order
        float e[B];
#pragma unroll
        for (int k = 0; k < B; k++) e[k] = w(i0 + k * SAMPLE_THREADS);
#pragma unroll
        for (int k = 0; k < B; k++) a = __fadd_rn(a, e[k]);
    }
    return sc_inverse_cdf_rest(vocab, w, a, i0, u, fallback, xc, buf, pb, vals, pre, tot_all, base, rank, tid);
}

// The same with the batches evaluated by `wb(i0, e)` -- the B weights of ids i0, i0 + 1024, ... into e -- which lets the
// caller issue a batch's loads in rounds of its own (a weight that needs a load through another load's result).
template <int B, typename W, typename WB>
__device__ inline uint32_t sc_inverse_cdf_batched(uint32_t vocab, W w, WB wb, float u, uint32_t fallback, ScExchange* xc, uint32_t buf, uint32_t pb, float* vals, float* pre,
                                           float* tot_all, float* base, uint32_t rank, uint32_t tid) {
    float a = 0.0f;
    uint32_t i0 = rank * SC_THREADS + tid;
    for (; i0 + (B - 1) * SAMPLE_THREADS < vocab; i0 += B * SAMPLE_THREADS) {
        float e[B];
        wb(i0, e);
#pragma unroll
        for (int k = 0; k < B; k++) a = __fadd_rn(a, e[k]);
    }
    return sc_inverse_cdf_rest(vocab, w, a, i0, u, fallback, xc, buf, pb, vals, pre, tot_all, base, rank, tid);
}

}  // namespace vlt
